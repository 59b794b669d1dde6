"""Reader and writer of the reference's on-disk model container ("NNM1"), so weights move between the
reference and this engine in both directions.

Container (src/format.rs:12-24, writer :286-330, reader :349-389, header check :417-430): little-endian
    magic u32 0x4E4E4D31 | version u8 (1 or 2) | kind u8 (0 flat, 1 hierarchical)
    hierarchical only: vocab u32, context u32, step u64, and from version 2 six u64 data counters
    n_sections u32, then per section: name (u32 byte count + UTF-8) and one layer-stack blob.
Stack blob (src/saving.rs:10-22,102-126; src/loading.rs:367-409):
    magic u32 0x4E4E4657 | version u8 (2) | n_layers u32 | per layer (tag u8, input u32, output u32) |
    per layer its weights, in the layer's own field order, with no shapes beyond what each field carries.
Fields: a vector is u32 count + f32s, a matrix is rows u32, cols u32 + a vector of rows*cols values,
row-major (src/saving.rs:58-69). Every weight matrix is [input, output].

The layer codecs below are one table: tag -> ordered (field, type) list, shared by reader and writer. A
layer in memory is a dict {"tag", "input", "output", <fields>} with numpy float32 arrays.

Nothing in the reference holds a byte-level fixture of this format (its tests are round trips,
src/format.rs:437-604) and the reference cannot be built here, so this codec follows the format's
source and documentation and is checked by hand-assembled byte strings and round trips only.
"""
import os
import struct

import numpy as np

MAGIC = 0x4E4E4D31        # "NNM1", src/format.rs:41
VERSION = 2               # src/format.rs:45
MIN_VERSION = 1           # src/format.rs:47
STACK_MAGIC = 0x4E4E4657  # "NNFW", src/saving.rs:35
STACK_VERSION = 2         # src/saving.rs:36
KIND_FLAT, KIND_HIERARCHICAL = 0, 1
SEEN_FIELDS = ("pretrain_chars", "pretrain_words", "sft_chars", "sft_words", "sft_resp_chars", "sft_resp_words")

TAG_LSTM, TAG_LINEAR_NB, TAG_LEGACY_SOFTMAX, TAG_SLSTM, TAG_DROPOUT, TAG_EMBEDDING = 0, 3, 4, 5, 6, 7
TAG_NORM, TAG_SILU_DENSE, TAG_SLSTM_BLOCK, TAG_LINEAR, TAG_MLSTM, TAG_MLSTM_BLOCK = 9, 10, 11, 12, 13, 14
TAG_CONV1D, TAG_SOFT_CAP = 15, 17


class FormatError(ValueError):
    """The bytes are not a container this reader accepts (the reference's io::ErrorKind::InvalidData /
    UnexpectedEof cases)."""


# field types: "m" matrix, "v" vector, "u" u32, "f" f32
_SLSTM_CELL = [("wz", "m"), ("wi", "m"), ("wf", "m"), ("wo", "m"), ("bz", "v"), ("bi", "v"), ("bf", "v"), ("bo", "v"),
               ("h_init", "v"), ("c_init", "v")]                                  # src/nn/slstm.rs:533-546
_MLSTM_CELL = [("num_heads", "u"), ("dqk", "u"), ("wq", "m"), ("wk", "m"), ("wv", "m"), ("wo", "m"), ("wi", "m"),
               ("wf", "m"), ("bq", "v"), ("bk", "v"), ("bv", "v"), ("bo", "v"), ("bi", "v"), ("bf", "v"),
               ("w_out", "m"), ("b_out", "v"), ("head_norm", "v")]                # src/nn/mlstm.rs:762-780
_FFN = [("w_gate", "m"), ("b_gate", "v"), ("w_value", "m"), ("b_value", "v"), ("w_down", "m"), ("b_down", "v")]


def _cell(fields):
    return [("cell." + n, t) for n, t in fields]


SCHEMA = {
    TAG_LSTM: [("wf", "m"), ("wi", "m"), ("wc", "m"), ("wo", "m"), ("b", "m"), ("h_init", "v"), ("c_init", "v")],
    TAG_LINEAR_NB: [("weights", "m")],                                            # src/nn/linear_nb.rs:174-176
    TAG_SLSTM: _SLSTM_CELL,
    TAG_DROPOUT: [("rate", "f")],
    TAG_EMBEDDING: [("weights", "m")],                                            # src/nn/embedding.rs:127-129
    TAG_NORM: [("gamma", "v")],                                                   # src/nn/rms_norm.rs:223-225
    TAG_SILU_DENSE: [("weights", "m"), ("biases", "v")],
    # src/nn/slstm_block.rs:305-317
    TAG_SLSTM_BLOCK: [("up_size", "u"), ("pre_norm1", "v"), ("post_cell_norm", "v"), ("pre_norm2", "v")]
                     + _cell(_SLSTM_CELL) + _FFN,
    # src/nn/linear.rs:211-217: a stand-alone Linear repeats its sizes before the weights
    TAG_LINEAR: [("in_dim", "u"), ("out_dim", "u"), ("weights", "m"), ("biases", "v")],
    TAG_MLSTM: _MLSTM_CELL,
    # src/nn/mlstm_block.rs:280-293
    TAG_MLSTM_BLOCK: [("up_size", "u"), ("pre_norm1", "v"), ("pre_norm2", "v")] + _cell(_MLSTM_CELL) + _FFN,
    TAG_CONV1D: [("kernel_size", "u"), ("weights", "m"), ("bias", "v")],
    TAG_SOFT_CAP: [("cap", "f")],                                                 # src/nn/soft_cap.rs:88-91
}


class _Out:
    def __init__(self):
        self.parts = []

    def u8(self, v):
        self.parts.append(struct.pack("<B", v))

    def u32(self, v):
        self.parts.append(struct.pack("<I", v))

    def u64(self, v):
        self.parts.append(struct.pack("<Q", v))

    def f32(self, v):
        self.parts.append(struct.pack("<f", v))

    def string(self, s):
        b = s.encode("utf-8")
        self.u32(len(b))
        self.parts.append(b)

    def vector(self, a):
        a = np.ascontiguousarray(a, dtype="<f4").reshape(-1)
        self.u32(a.size)
        self.parts.append(a.tobytes())

    def matrix(self, a):
        a = np.asarray(a)
        if a.ndim != 2:
            raise FormatError(f"a matrix field needs a 2-D array, got shape {a.shape}")
        self.u32(a.shape[0])
        self.u32(a.shape[1])
        self.vector(a)

    def bytes(self):
        return b"".join(self.parts)


class _In:
    def __init__(self, buf):
        self.buf, self.pos = memoryview(buf), 0

    def _take(self, n):
        if self.pos + n > len(self.buf):
            raise FormatError(f"unexpected end of file at byte {self.pos} (wanted {n} more)")
        s = self.buf[self.pos:self.pos + n]
        self.pos += n
        return s

    def u8(self):
        return struct.unpack("<B", self._take(1))[0]

    def u32(self):
        return struct.unpack("<I", self._take(4))[0]

    def u64(self):
        return struct.unpack("<Q", self._take(8))[0]

    def f32(self):
        return struct.unpack("<f", self._take(4))[0]

    def string(self):
        n = self.u32()
        try:
            return bytes(self._take(n)).decode("utf-8")
        except UnicodeDecodeError as e:
            raise FormatError(f"section name is not UTF-8: {e}") from None

    def vector(self):
        n = self.u32()
        return np.frombuffer(self._take(4 * n), dtype="<f4").astype(np.float32)

    def matrix(self):
        rows, cols = self.u32(), self.u32()
        flat = self.vector()
        if flat.size != rows * cols:
            raise FormatError(f"matrix says {rows} x {cols} but carries {flat.size} values")
        return flat.reshape(rows, cols)


_WRITE = {"m": _Out.matrix, "v": _Out.vector, "u": _Out.u32, "f": _Out.f32}
_READ = {"m": _In.matrix, "v": _In.vector, "u": _In.u32, "f": _In.f32}


def _write_stack(out, layers):
    """One layer-stack blob: architecture header for every layer, then every layer's weights."""
    out.u32(STACK_MAGIC)
    out.u8(STACK_VERSION)
    out.u32(len(layers))
    for l in layers:
        if l["tag"] not in SCHEMA:
            raise FormatError(f"Unknown layer tag {l['tag']}")
        out.u8(l["tag"])
        out.u32(l["input"])
        out.u32(l["output"])
    for l in layers:
        for name, kind in SCHEMA[l["tag"]]:
            if name not in l:
                raise FormatError(f"layer with tag {l['tag']} lacks field {name!r}")
            _WRITE[kind](out, l[name])


def _read_stack(inp):
    if inp.u32() != STACK_MAGIC:
        raise FormatError("Wrong stack magic number")
    if inp.u8() != STACK_VERSION:
        raise FormatError("Unknown stack version")
    n = inp.u32()
    arch = [(inp.u8(), inp.u32(), inp.u32()) for _ in range(n)]
    layers = []
    for tag, isz, osz in arch:
        if tag == TAG_LEGACY_SOFTMAX:  # consumed and dropped, src/loading.rs:337-340
            inp.u32()
            continue
        if tag not in SCHEMA:
            raise FormatError(f"Unknown layer tag {tag}")
        if tag == TAG_SLSTM_BLOCK and isz != osz:  # src/loading.rs:178-186
            raise FormatError(f"an sLSTM block needs input_size == output_size, got {isz} != {osz}")
        l = dict(tag=tag, input=isz, output=osz)
        for name, kind in SCHEMA[tag]:
            l[name] = _READ[kind](inp)
        layers.append(l)
    return layers


def new_meta(vocab_size=0, context_size=0, step=0, **seen):
    """The typed head of a hierarchical container (src/format.rs:77-84); the six data counters default to 0."""
    unknown = set(seen) - set(SEEN_FIELDS)
    if unknown:
        raise TypeError(f"unknown counters {sorted(unknown)}")
    return dict(vocab_size=vocab_size, context_size=context_size, step=step,
                seen={k: int(seen.get(k, 0)) for k in SEEN_FIELDS})


class Container:
    """kind, metadata and the named layer stacks in file order (src/format.rs:332-338)."""

    def __init__(self, kind=KIND_FLAT, meta=None, sections=None):
        self.kind = kind
        self.meta = meta if meta is not None else new_meta()
        self.sections = list(sections or [])  # [(name, [layer dict, ...])]

    def section(self, name, layers):
        """Appends a named stack; a single stand-alone layer is a one-layer stack (src/format.rs:266-283)."""
        self.sections.append((name, [layers] if isinstance(layers, dict) else list(layers)))
        return self

    def take(self, name):
        """Removes and returns the layers of section `name`; a missing section is an error
        (src/format.rs:394-401)."""
        for i, (n, _) in enumerate(self.sections):
            if n == name:
                return self.sections.pop(i)[1]
        raise FormatError(f"missing section {name!r}")


def dumps(c):
    out = _Out()
    out.u32(MAGIC)
    out.u8(VERSION)
    if c.kind not in (KIND_FLAT, KIND_HIERARCHICAL):
        raise FormatError(f"unknown model kind tag {c.kind}")
    out.u8(c.kind)
    if c.kind == KIND_HIERARCHICAL:
        out.u32(c.meta["vocab_size"])
        out.u32(c.meta["context_size"])
        out.u64(c.meta["step"])
        for k in SEEN_FIELDS:
            out.u64(c.meta["seen"][k])
    out.u32(len(c.sections))
    for name, layers in c.sections:
        out.string(name)
        _write_stack(out, layers)
    return out.bytes()


def _read_header(inp):
    if inp.u32() != MAGIC:
        raise FormatError("not an NNM1 model file (wrong magic)")
    version = inp.u8()
    if not MIN_VERSION <= version <= VERSION:
        raise FormatError(f"unsupported NNM1 version {version} (this build reads {MIN_VERSION}..={VERSION})")
    kind = inp.u8()
    if kind not in (KIND_FLAT, KIND_HIERARCHICAL):
        raise FormatError(f"unknown model kind tag {kind}")
    return version, kind


def loads(buf):
    inp = _In(buf)
    version, kind = _read_header(inp)
    meta = new_meta()
    if kind == KIND_HIERARCHICAL:
        meta = new_meta(inp.u32(), inp.u32(), inp.u64())
        if version >= 2:  # a version-1 head ends at `step`, src/format.rs:359-370
            for k in SEEN_FIELDS:
                meta["seen"][k] = inp.u64()
    c = Container(kind, meta)
    for _ in range(inp.u32()):
        name = inp.string()
        c.sections.append((name, _read_stack(inp)))
    return c


def save(path, c):
    """Writes to `path` through a temporary file and a rename, creating the folder (src/format.rs:317-329)."""
    folder = os.path.dirname(path)
    if folder:
        os.makedirs(folder, exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(dumps(c))
    os.replace(tmp, path)


def load(path):
    with open(path, "rb") as f:
        return loads(f.read())


def peek_kind(path):
    """The kind tag from the six header bytes alone (src/format.rs:343-346)."""
    with open(path, "rb") as f:
        return _read_header(_In(f.read(6)))[1]


def describe(c):
    """One line per section and layer: tag, sizes, parameter count (what the reference's `inspect` tool lists)."""
    lines = ["kind: " + ("flat" if c.kind == KIND_FLAT else "hierarchical")]
    if c.kind == KIND_HIERARCHICAL:
        m = c.meta
        lines.append(f"vocab {m['vocab_size']}  context {m['context_size']}  step {m['step']}  " +
                     "  ".join(f"{k} {m['seen'][k]}" for k in SEEN_FIELDS))
    for name, layers in c.sections:
        total = 0
        body = []
        for l in layers:
            n = sum(int(np.size(v)) for k, v in l.items() if isinstance(v, np.ndarray))
            total += n
            body.append(f"    tag {l['tag']:2d}  {l['input']} -> {l['output']}  {n} parameters")
        lines.append(f"  section {name!r}: {len(layers)} layers, {total} parameters")
        lines += body
    return "\n".join(lines)


# ---- the language model's host parameter dictionary <-> a flat container -------------------------------------
# The dictionary is the one `layers.build_lm` takes. The file keeps what the CPU layers keep: wk and bk
# unscaled (the 1/sqrt(dqk) of k is applied at run time here, folded and un-folded by the reference's GPU cell,
# src/gpu/mlstm.rs:241-247,285-322), and the sLSTM's four gates as separate [input + H, H] matrices whose top
# `input` rows act on x and whose last H rows on h (the reference's GPU cell packs and unpacks the same way,
# src/gpu/slstm.rs:389-407,567-582).

_F32 = np.float32


def _slstm_gates(cell, d):
    """wx [in, 4H], wh dense [H, 4H] or block-diagonal [nh, dh, 4dh], bcat [4H] -> the file's four gate matrices
    and biases (gate order z, i, f, o)."""
    wx, wh, b = (np.asarray(cell[k], _F32) for k in ("wx", "wh", "bcat"))
    H = wx.shape[1] // 4
    if wh.ndim == 3:  # heads: gate g of head h sits at columns g*dh.. of wh[h]; off-diagonal blocks are zero
        nh, dh = wh.shape[0], wh.shape[1]
        dense = np.zeros((H, 4 * H), _F32)
        for h in range(nh):
            for g in range(4):
                dense[h * dh:(h + 1) * dh, g * H + h * dh:g * H + (h + 1) * dh] = wh[h][:, g * dh:(g + 1) * dh]
        wh = dense
    out = {}
    for g, name in enumerate("zifo"):
        out["w" + name] = np.concatenate([wx[:, g * H:(g + 1) * H], wh[:, g * H:(g + 1) * H]], axis=0)
        out["b" + name] = b[g * H:(g + 1) * H].copy()
    out["h_init"] = np.zeros(H, _F32)  # always zero from a GPU model, src/gpu/slstm.rs:495-497
    out["c_init"] = np.zeros(H, _F32)
    return out


def _slstm_pack(l, d, nh):
    """Inverse of `_slstm_gates`. With nh > 1 the recurrent part must be block-diagonal: a checkpoint with
    weight between heads cannot run on the head-sharded kernels and is refused rather than truncated."""
    H = l["cell.wz"].shape[1]
    gates = [np.asarray(l["cell.w" + n], _F32) for n in "zifo"]
    for g in gates:
        if g.shape != (d + H, H):
            raise FormatError(f"sLSTM gate matrix is {g.shape}, expected {(d + H, H)}")
    wx = np.concatenate([g[:d] for g in gates], axis=1)
    wh = np.concatenate([g[d:] for g in gates], axis=1)
    bcat = np.concatenate([np.asarray(l["cell.b" + n], _F32) for n in "zifo"])
    if nh > 1:
        if H % nh:
            raise FormatError(f"{nh} heads do not divide the sLSTM width {H}")
        dh = H // nh
        heads = np.zeros((nh, dh, 4 * dh), _F32)
        mask = np.ones((H, 4 * H), bool)
        for h in range(nh):
            for g in range(4):
                rows, cols = slice(h * dh, (h + 1) * dh), slice(g * H + h * dh, g * H + (h + 1) * dh)
                heads[h][:, g * dh:(g + 1) * dh] = wh[rows, cols]
                mask[rows, cols] = False
        if np.any(wh[mask] != 0):
            raise FormatError("the checkpoint's sLSTM recurrence has weight between heads; load it with one head")
        wh = heads
    return dict(kind="slstm", wx=wx, wh=wh, bcat=bcat)


def _block_to_layer(bp, d, heads, dqk):
    """One block of the parameter dictionary as the file's block layer (tag 14 mLSTM, tag 11 sLSTM)."""
    c = bp["cell"]
    up = np.asarray(bp["w_gate"]).shape[1]
    l = dict(input=d, output=d, up_size=up, pre_norm1=bp["g1"], pre_norm2=bp["g2"])
    for k in ("w_gate", "b_gate", "w_value", "b_value", "w_down", "b_down"):
        l[k] = bp[k]
    if c["kind"] == "mlstm":
        if np.asarray(c["wv"]).shape[1] != d or np.asarray(c["wq"]).shape[1] != heads * dqk:
            raise FormatError("the format needs heads * dhv == hidden and wq [hidden, heads * dqk]")
        l["tag"] = TAG_MLSTM_BLOCK
        l["cell.num_heads"], l["cell.dqk"], l["cell.head_norm"] = heads, dqk, c["gamma"]
        for k in ("wq", "wk", "wv", "wo", "wi", "wf", "bq", "bk", "bv", "bo", "bi", "bf", "w_out", "b_out"):
            l["cell." + k] = c[k]
    else:
        l["tag"] = TAG_SLSTM_BLOCK
        l["post_cell_norm"] = bp["gpost"]
        for k, v in _slstm_gates(c, d).items():
            l["cell." + k] = v
    return l


def _layer_to_block(l, d, nh_s=1):
    """Inverse of `_block_to_layer`. Returns (block dictionary, (heads, dqk) or None for an sLSTM block)."""
    bp = dict(g1=l["pre_norm1"], g2=l["pre_norm2"])
    for k in ("w_gate", "b_gate", "w_value", "b_value", "w_down", "b_down"):
        bp[k] = l[k]
    if l["tag"] == TAG_MLSTM_BLOCK:
        shape = (int(l["cell.num_heads"]), int(l["cell.dqk"]))
        cell = dict(kind="mlstm", gamma=l["cell.head_norm"])
        for k in ("wq", "wk", "wv", "wo", "wi", "wf", "bq", "bk", "bv", "bo", "bi", "bf", "w_out", "b_out"):
            cell[k] = l["cell." + k]
    elif l["tag"] == TAG_SLSTM_BLOCK:
        shape = None
        cell = _slstm_pack(l, d, nh_s)
        bp["gpost"] = l["post_cell_norm"]
    else:
        raise FormatError(f"layer tag {l['tag']} is not a block")
    bp["cell"] = cell
    return bp, shape


def lm_to_container(params, heads, dqk, cap=30.0, head_w=None, head_b=None):
    """A flat container with the one section "model" (as `Sequential::save`, src/sequential.rs:90-94):
    Embedding, one block layer per block, RMSNorm, the head, SoftCap. A tied head (head_w None) is written as
    a bias-free projection holding the transposed table, since the format has no notion of tying; an untied
    head as a Linear."""
    table = np.asarray(params["table"], _F32)
    vocab, d = table.shape
    layers = [dict(tag=TAG_EMBEDDING, input=vocab, output=d, weights=table)]
    layers += [_block_to_layer(bp, d, heads, dqk) for bp in params["blocks"]]
    layers.append(dict(tag=TAG_NORM, input=d, output=d, gamma=params["gamma"]))
    if head_w is None:
        layers.append(dict(tag=TAG_LINEAR_NB, input=d, output=vocab, weights=np.ascontiguousarray(table.T)))
    else:
        layers.append(dict(tag=TAG_LINEAR, input=d, output=vocab, in_dim=d, out_dim=vocab, weights=head_w,
                           biases=head_b if head_b is not None else np.zeros(vocab, _F32)))
    layers.append(dict(tag=TAG_SOFT_CAP, input=vocab, output=vocab, cap=float(cap)))
    return Container(KIND_FLAT).section("model", layers)


def lm_from_container(c, nh_s=1, section="model"):
    """Inverse of `lm_to_container`. Returns (params, info): `params` for `layers.build_lm`, `info` with heads,
    dqk, dhv, up, cap, tied, head_w, head_b (head_* None when the head is the transposed table)."""
    layers = dict(c.sections).get(section)
    if layers is None:
        raise FormatError(f"missing section {section!r}")
    if not layers or layers[0]["tag"] != TAG_EMBEDDING:
        raise FormatError("the model section must start with an Embedding")
    table = layers[0]["weights"]
    d = table.shape[1]
    info = dict(heads=None, dqk=None, dhv=None, up=None, cap=30.0, tied=True, head_w=None, head_b=None)
    blocks, gamma = [], None
    for l in layers[1:]:
        tag = l["tag"]
        if tag in (TAG_MLSTM_BLOCK, TAG_SLSTM_BLOCK):
            if gamma is not None:
                raise FormatError("a block after the final norm")
            bp, shape = _layer_to_block(l, d, nh_s)
            info["up"] = int(l["up_size"])
            if shape is not None:
                if info["heads"] not in (None, shape[0]) or info["dqk"] not in (None, shape[1]):
                    raise FormatError("mLSTM blocks disagree on heads or dqk")
                info.update(heads=shape[0], dqk=shape[1], dhv=d // shape[0])
            blocks.append(bp)
        elif tag == TAG_NORM:
            gamma = l["gamma"]
        elif tag == TAG_LINEAR_NB:
            if not np.array_equal(l["weights"], table.T):
                info.update(tied=False, head_w=l["weights"], head_b=np.zeros(l["weights"].shape[1], _F32))
        elif tag == TAG_LINEAR:
            info.update(tied=False, head_w=l["weights"], head_b=l["biases"])
        elif tag == TAG_SOFT_CAP:
            info["cap"] = float(l["cap"])
        elif tag == TAG_DROPOUT:
            continue  # inactive outside CPU training
        else:
            raise FormatError(f"layer tag {tag} has no place in the language model")
    if gamma is None:
        raise FormatError("the model section is missing its final RMSNorm")
    return dict(table=table, blocks=blocks, gamma=gamma), info


def export_lm_params(lm):
    """The host parameter dictionary of a live `layers.Lm` (fp32 master weights, device -> host)."""
    from . import layers

    host = lambda p: p.w.detach().cpu().numpy()
    blocks = []
    for blk in lm.blocks:
        u = blk.up  # the projections may be stored padded with zero columns / rows; the file holds the model's width
        bp = dict(g1=host(blk.n1.gamma), g2=host(blk.n2.gamma), w_gate=host(blk.lg.w)[:, :u].copy(), b_gate=host(blk.lg.b)[:u].copy(),
                  w_value=host(blk.lv.w)[:, :u].copy(), b_value=host(blk.lv.b)[:u].copy(), w_down=host(blk.ld.w)[:u].copy(),
                  b_down=host(blk.ld.b))
        c = blk.cell
        if isinstance(c, layers.MLstm):
            cell = dict(kind="mlstm", w_out=host(c.lout.w), b_out=host(c.lout.b), gamma=host(c.hn.gamma))
            for n, lin in zip("qkvoif", (c.lq, c.lk, c.lv, c.lo, c.li, c.lf)):
                cell["w" + n], cell["b" + n] = host(lin.w), host(lin.b)
        else:
            cell = dict(kind="slstm", wx=host(c.wx), wh=host(c.wh), bcat=host(c.b))
            bp["gpost"] = host(blk.post.gamma)
        bp["cell"] = cell
        blocks.append(bp)
    return dict(table=host(lm.table), blocks=blocks, gamma=host(lm.norm.gamma))


def save_lm(path, lm, heads, dqk):
    """Writes a live model as a flat container the reference's `Sequential::load` opens."""
    head = (None, None) if lm.tied else (lm.head.w.w.detach().cpu().numpy(), lm.head.b.w.detach().cpu().numpy())
    save(path, lm_to_container(export_lm_params(lm), heads, dqk, lm.cap, *head))


def load_lm(path, nh_s=1, **build_kw):
    """Builds a `layers.Lm` on the current GPU from a flat container (AdamW moments start at zero: the format
    holds weights only, src/gpu/hierarchical.rs:1808-1811)."""
    from . import layers

    params, info = lm_from_container(load(path), nh_s)
    return layers.build_lm(params, info["heads"] or 1, info["dqk"] or 1, info["dhv"] or 1, nh_s=nh_s, cap=info["cap"],
                           tied=info["tied"], head_w=info["head_w"], head_b=info["head_b"], **build_kw)


# ---- the hierarchical model's parameter dictionary <-> a hierarchical container ------------------------------
# Sections and their layers as the reference's GPU model exports them (src/gpu/hierarchical.rs:1750-1806):
#   "encoder"      Embedding(tied table), encoder blocks
#   "word_model"   Linear(hc -> wh), backbone blocks, Linear(wh -> hc)
#   "char2_model"  decoder blocks, RMSNorm, bias-free head, SoftCap
# The typed head carries vocab, context_size = hc (the backbone's output width, :1815-1817), the step count and
# the data counters.

def hier_to_container(params, cfg, step=0, seen=None):
    """`cfg`: anything with vocab, hc, wh, heads, dqk, small_heads, cap (hier.HierCfg)."""
    hc, wh, sh = cfg.hc, cfg.wh, cfg.small_heads
    table = np.asarray(params["table"], _F32)
    lin = lambda w, b: dict(tag=TAG_LINEAR, input=np.asarray(w).shape[0], output=np.asarray(w).shape[1],
                            in_dim=np.asarray(w).shape[0], out_dim=np.asarray(w).shape[1], weights=w, biases=b)
    enc = [dict(tag=TAG_EMBEDDING, input=cfg.vocab, output=hc, weights=table)]
    enc += [_block_to_layer(bp, hc, sh, hc // sh) for bp in params["enc"]]
    wm = [lin(params["front_w"], params["front_b"])]
    wm += [_block_to_layer(bp, wh, cfg.heads, cfg.dqk) for bp in params["bb"]]
    wm.append(lin(params["back_w"], params["back_b"]))
    dec = [_block_to_layer(bp, hc, sh, hc // sh) for bp in params["dec"]]
    dec.append(dict(tag=TAG_NORM, input=hc, output=hc, gamma=params["dec_gamma"]))
    dec.append(dict(tag=TAG_LINEAR_NB, input=hc, output=cfg.vocab, weights=params["head_w"]))
    dec.append(dict(tag=TAG_SOFT_CAP, input=cfg.vocab, output=cfg.vocab, cap=float(cfg.cap)))
    meta = new_meta(cfg.vocab, hc, step, **(seen or {}))
    return Container(KIND_HIERARCHICAL, meta).section("encoder", enc).section("word_model", wm).section("char2_model", dec)


def hier_from_container(c):
    """Inverse of `hier_to_container`, with the checks of the reference's loader (src/gpu/hierarchical.rs:1838-1935):
    the encoder starts with an Embedding, the backbone starts and ends with a Linear, the decoder holds blocks, then
    an RMSNorm, a bias-free projection and a SoftCap. Returns (params, info) with info = vocab, hc, wh, block
    kinds per stage, heads, dqk, small_heads, cap, step, seen."""
    if c.kind != KIND_HIERARCHICAL:
        raise FormatError("not a hierarchical container")
    sec = dict(c.sections)
    for name in ("encoder", "word_model", "char2_model"):
        if name not in sec:
            raise FormatError(f"missing section {name!r}")
    enc, wm, dec = sec["encoder"], sec["word_model"], sec["char2_model"]
    if not enc or enc[0]["tag"] != TAG_EMBEDDING:
        raise FormatError("encoder must start with an Embedding")
    table = enc[0]["weights"]
    vocab, hc = table.shape
    if len(wm) < 2 or wm[0]["tag"] != TAG_LINEAR or wm[-1]["tag"] != TAG_LINEAR:
        raise FormatError("backbone must start and end with a Linear")
    wh = wm[0]["weights"].shape[1]
    info = dict(vocab=vocab, hc=hc, wh=wh, heads=None, dqk=None, small_heads=None, cap=30.0, step=c.meta["step"],
                seen=dict(c.meta["seen"]))

    def stage(layers, d, small):
        blocks, kinds = [], ""
        for l in layers:
            bp, shape = _layer_to_block(l, d)
            kinds += "s" if shape is None else "m"
            if shape is not None:
                key = ("small_heads",) if small else ("heads", "dqk")
                got = shape[:1] if small else shape
                if any(info[k] not in (None, v) for k, v in zip(key, got)):
                    raise FormatError("the mLSTM blocks of a stage disagree on heads or dqk")
                info.update(zip(key, got))
            blocks.append(bp)
        return blocks, kinds

    params = dict(table=table, front_w=wm[0]["weights"], front_b=wm[0]["biases"], back_w=wm[-1]["weights"],
                  back_b=wm[-1]["biases"])
    params["enc"], info["enc_kinds"] = stage(enc[1:], hc, True)
    params["bb"], info["bb_kinds"] = stage(wm[1:-1], wh, False)
    at = next((i for i, l in enumerate(dec) if l["tag"] == TAG_NORM), None)
    if at is None:
        raise FormatError("decoder is missing its RMSNorm")
    params["dec"], info["dec_kinds"] = stage(dec[:at], hc, True)
    params["dec_gamma"] = dec[at]["gamma"]
    heads_ = [l for l in dec[at + 1:] if l["tag"] == TAG_LINEAR_NB]
    if len(heads_) != 1:
        raise FormatError("decoder is missing its head")
    params["head_w"] = heads_[0]["weights"]
    for l in dec[at + 1:]:
        if l["tag"] == TAG_SOFT_CAP:
            info["cap"] = float(l["cap"])
    return params, info


def export_hier_params(model):
    """The host parameter dictionary of a live `hier.Hierarchical`."""
    host = lambda p: p.w.detach().cpu().numpy()

    class _Stack:  # the three block lists read like a flat model's
        def __init__(self, blocks):
            self.blocks, self.table, self.norm = blocks, model.table, model.dec_norm

    out = dict(table=host(model.table), front_w=host(model.front.w), front_b=host(model.front.b),
               back_w=host(model.back.w), back_b=host(model.back.b), dec_gamma=host(model.dec_norm.gamma),
               head_w=host(model.head))
    for name, blocks in (("enc", model.enc), ("bb", model.bb), ("dec", model.dec)):
        out[name] = export_lm_params(_Stack(blocks))["blocks"]
    return out


def save_hier(path, model, seen=None):
    """Writes a live hierarchical model as the container the reference's `Hierarchical::load` opens."""
    save(path, hier_to_container(export_hier_params(model), model.cfg, step=model.step_count, seen=seen))


def load_hier(path, w_token, **build_kw):
    """Builds a `hier.Hierarchical` on the current GPU from a container; `w_token` comes from the caller, the
    format does not store it (src/gpu/hierarchical.rs:1835-1838). AdamW moments start at zero."""
    from . import hier

    params, info = hier_from_container(load(path))
    sh = info["small_heads"] or 16
    cfg = hier.HierCfg(info["vocab"], info["hc"], info["wh"], len(params["enc"]), len(params["bb"]), len(params["dec"]),
                       info["heads"] or 8, info["dqk"] or info["wh"] // 8, w_token, cap=info["cap"], small_heads=sh,
                       enc_kinds=info["enc_kinds"], bb_kinds=info["bb_kinds"], dec_kinds=info["dec_kinds"])
    model = hier.Hierarchical(params, cfg, **build_kw)
    model.step_count = info["step"]
    return model
