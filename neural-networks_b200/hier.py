"""The reference's three-stage hierarchical model (gpu::Hierarchical, src/gpu/hierarchical.rs) on this
engine's blocks: the caller of the cells' carry API.

  encoder   every word as one row of a [words, tmax] rectangle (chars, then the [W] token), words being the
            batch axis: tied table -> blocks; e_w = the row at the [W] step. One rectangle per length group.
  backbone  Linear(hc->wh) -> blocks over a window's words as one sequence -> Linear(wh->hc). Swept in
            spans of the word axis: a span passes through all blocks with every cell's state carried in from
            the span before it, and the backward unwinds the spans right to left with the cells' BPTT state
            carried the other way. The arithmetic is that of one long call; only memory residency changes.
  decoder   word w+1 as one row: slot 0 = the backbone's output at word w, slot k = table[char k-1]; blocks
            -> RMSNorm -> bias-free fp32 head -> SoftCap -> masked cross-entropy scaled by 1/(valid rows of
            the whole call). Forward and backward per length group.
The encoder's backward re-runs each group's forward first (src/gpu/hierarchical.rs:1347-1407), so only one
group's activations are ever resident.

Beyond the reference: a call takes several windows with equally many words; their words share the encoder
and decoder rectangles and the backbone runs them as a batch (the reference's backbone is batch 1).
"""
import numpy as np
import torch

from . import layers, ops

BACKBONE_CHUNK = 512    # src/config.rs:96
# Row cap of one encoder/decoder rectangle. The reference's 2048 (src/config.rs:115) bounds the activations of a
# 16 GB card; it is a batching choice that does not change results, and here it costs a factor of two in step
# time at 16 x 8192 bytes (72 small rectangles per stage instead of one or two), so the default is sized for
# 180 GB: a 131072-row rectangle of width 256 holds about 20 GB of activations.
GROUP_MAX_ROWS = 131072


class HierCfg:
    """ModelCfg (src/gpu/hierarchical.rs:53-65). `small_heads`: heads of the encoder's and decoder's mLSTM
    blocks (16 in the reference). `*_kinds`: a string of "s"/"m" per stage overriding the reference's
    patterns (encoder and decoder alternate sLSTM, mLSTM; the backbone has an sLSTM at every eighth block)."""

    def __init__(self, vocab, hc, wh, enc_blocks, bb_blocks, dec_blocks, heads, dqk, w_token, cap=30.0, small_heads=16,
                 enc_kinds=None, bb_kinds=None, dec_kinds=None):
        self.vocab, self.hc, self.wh = vocab, hc, wh
        self.enc_blocks, self.bb_blocks, self.dec_blocks = enc_blocks, bb_blocks, dec_blocks
        self.heads, self.dqk, self.w_token, self.cap, self.small_heads = heads, dqk, w_token, cap, small_heads
        self.enc_kinds = enc_kinds or "".join("s" if i % 2 == 0 else "m" for i in range(enc_blocks))
        self.bb_kinds = bb_kinds or "".join("s" if i % 8 == 0 else "m" for i in range(bb_blocks))
        self.dec_kinds = dec_kinds or "".join("s" if i % 2 == 0 else "m" for i in range(dec_blocks))

    def stage(self, name):
        """(kinds, width, heads, dqk, dhv) of a stage's blocks."""
        if name == "bb":
            return self.bb_kinds, self.wh, self.heads, self.dqk, self.wh // self.heads
        sh = self.small_heads
        return (self.enc_kinds if name == "enc" else self.dec_kinds), self.hc, sh, self.hc // sh, self.hc // sh


def up_of(hidden):
    """SwiGLU inner width of a block, from its own width (src/gpu/hierarchical.rs:70-72)."""
    return hidden * 8 // 3


def init_hier_params(rng, cfg, std=0.02):
    """Seeded N(0, std) host weights (norm gains 1) in the dictionary `Hierarchical` takes."""
    def n(*shape):
        return rng.standard_normal(shape, dtype=np.float32) * np.float32(std)

    def blocks(name):
        kinds, d, heads, dqk, dhv = cfg.stage(name)
        sl = tuple(i for i, k in enumerate(kinds) if k == "s")
        return layers.init_lm_params(rng, 1, d, len(kinds), heads, dqk, dhv, up_of(d), std=std, slstm_at=sl)["blocks"]

    return dict(table=n(cfg.vocab, cfg.hc), enc=blocks("enc"), front_w=n(cfg.hc, cfg.wh), front_b=n(cfg.wh),
                bb=blocks("bb"), back_w=n(cfg.wh, cfg.hc), back_b=n(cfg.hc), dec=blocks("dec"),
                dec_gamma=np.ones(cfg.hc, np.float32), head_w=n(cfg.hc, cfg.vocab))


def group_by_len(lens, no_group=False, cap=None):
    """Word indices bucketed by the next power of two of their length, buckets in ascending order, each cut
    into pieces of at most `cap` rows (rows = words x (longest word + 1); cap 0 = no cut; None = GROUP_MAX_ROWS),
    the pieces after the first appended behind all buckets (src/gpu/hierarchical.rs:117-200). The order fixes
    the order in which losses are summed and gradients scattered."""
    cap = GROUP_MAX_ROWS if cap is None else cap
    lens = np.asarray(lens, np.int64)
    if no_group:
        return [list(range(len(lens)))]
    l1 = np.maximum(lens, 1)
    key = np.left_shift(1, np.ceil(np.log2(l1)).astype(np.int64))  # next power of two, exact for these sizes
    out = [np.nonzero(key == k)[0] for k in np.unique(key)]
    if cap:
        first = len(out)
        for g in range(first):
            per = max(cap // (int(l1[out[g]].max()) + 1), 1)
            if len(out[g]) > per:
                tail, out[g] = out[g][per:], out[g][:per]
                out += [tail[i:i + per] for i in range(0, len(tail), per)]
    return [g.tolist() for g in out]


def chunk_spans(n, chunk):
    """[(start, len)] covering n rows in near-equal pieces of at most `chunk`; one span when chunk >= n
    (src/gpu/hierarchical.rs:245-261)."""
    if chunk >= n:
        return [(0, n)]
    pieces = -(-n // chunk)
    base, extra = divmod(n, pieces)
    out, c0 = [], 0
    for i in range(pieces):
        ln = base + (1 if i < extra else 0)
        out.append((c0, ln))
        c0 += ln
    return out


def _build_blocks(plist, d, heads, dqk, dhv, bf16, chunk, recompute_states=False):
    t = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.float32)
    out = []
    for bp in plist:
        c = {k: (t(v) if k != "kind" else v) for k, v in bp["cell"].items()}
        bpt = {k: t(v) for k, v in bp.items() if k != "cell"}
        if c["kind"] == "mlstm":
            out.append(layers.Block(layers.MLstm(c, heads, dqk, dhv, bf16=bf16, chunk=chunk, recompute_states=recompute_states), bpt, bf16=bf16))
        else:
            out.append(layers.Block(layers.SLstm(c, d, 1, bf16=bf16), bpt, post_norm=True, bf16=bf16))
    return out


class Hierarchical:
    """gpu::Hierarchical (src/gpu/hierarchical.rs:460-1746): forward_backward over windows, then step."""

    def __init__(self, params, cfg, bf16=False, chunk=64, bb_chunk=None, group_cap=None, no_group=False, recompute_states=False):
        """recompute_states: the mLSTM cells keep no chunk-state record; their backward rebuilds the chunk-boundary states."""
        t = lambda a: torch.as_tensor(np.asarray(a), dtype=torch.float32)
        self.cfg, self.bf16 = cfg, bf16
        self.table = layers.Param(t(params["table"]), False)
        self.enc = _build_blocks(params["enc"], *cfg.stage("enc")[1:], bf16, chunk, recompute_states)
        self.front = layers.Linear(t(params["front_w"]), t(params["front_b"]), True, bf16)
        self.bb = _build_blocks(params["bb"], *cfg.stage("bb")[1:], bf16, chunk, recompute_states)
        self.back = layers.Linear(t(params["back_w"]), t(params["back_b"]), True, bf16)
        self.dec = _build_blocks(params["dec"], *cfg.stage("dec")[1:], bf16, chunk, recompute_states)
        self.dec_norm = layers.RmsNorm(t(params["dec_gamma"]))
        # fp32 whatever the blocks run in: the softmax exponentiates the head's output
        # (src/gpu/hierarchical.rs:626-635); bias-free, as the checkpoint stores it (:1797-1801)
        self.head = layers.Param(t(params["head_w"]), False)
        self.bb_chunk = bb_chunk      # None: BACKBONE_CHUNK; >= the window's words: one span
        self.group_cap = group_cap    # None: GROUP_MAX_ROWS; 0: no cap
        self.no_group = no_group      # every word in one rectangle per stage (the A/B baseline)
        self.loss = torch.zeros((1,), dtype=torch.float32, device="cuda")
        self.step_count = 0
        self.last_rows = 0
        self.last_word_loss = 0.0
        # data parallelism (dp.attach_hier): called with 0, 1, 2 when the decoder's, the backbone's and the
        # encoder's (and the table's) gradients are complete; `rows_of_all_ranks(valid)` returns the call's valid
        # decoder rows summed over the ranks, the loss normaliser of the global batch
        self.on_stage_backward = None
        self.check_status = True  # a step raises, before AdamW, if a kernel gave up on a bounded device-side wait
        self.rows_of_all_ranks = None

    def stage_params(self):
        """The parameters in the order their gradients complete in a backward: decoder stage, backbone stage,
        encoder stage with the tied table (which both the decoder and the encoder write)."""
        dec = [q for blk in self.dec for q in blk.params()] + self.dec_norm.params() + [self.head]
        bb = self.back.params() + [q for blk in self.bb for q in blk.params()] + self.front.params()
        enc = [q for blk in self.enc for q in blk.params()] + [self.table]
        return [dec, bb, enc]

    def params(self):
        out = [self.table]
        for blk in self.enc:
            out += blk.params()
        out += self.front.params()
        for blk in self.bb:
            out += blk.params()
        out += self.back.params()
        for blk in self.dec:
            out += blk.params()
        return out + self.dec_norm.params() + [self.head]

    def step(self, cfg):
        """One AdamW update of every tensor through the batched queue (src/gpu/hierarchical.rs:1696-1746)."""
        q = ops.AdamwQueue()
        for p in self.params():
            q.push(p.w, p.g, p.m, p.v, p.decay, p.wb)
        q.flush(cfg, zero_grad=True)
        self.step_count += 1

    # ---- host-side index plans ----------------------------------------------------------------------------
    def _cap(self):
        return GROUP_MAX_ROWS if self.group_cap is None else self.group_cap

    def _spans(self, dw):
        c = BACKBONE_CHUNK if self.bb_chunk is None else self.bb_chunk
        return chunk_spans(dw, dw if c == 0 else max(1, min(c, dw)))

    @staticmethod
    def _dev(a, dtype):
        return torch.from_numpy(np.ascontiguousarray(a)).to("cuda", dtype=dtype, non_blocking=False)

    def _enc_plan(self, tok, start, lens):
        """Per group: (word rows, n, tmax, ids [n * tmax], readout rows): the chars, then the [W] token, zero
        padded (src/gpu/hierarchical.rs:436-458). tok: all windows' tokens; start, lens: per word."""
        plan = []
        for grp in group_by_len(lens, self.no_group, self._cap()):
            grp = np.asarray(grp, np.int64)
            L = lens[grp]
            tmax = int(L.max()) + 1
            k = np.arange(tmax)[None, :]
            ids = np.where(k < L[:, None], tok[np.minimum(start[grp][:, None] + k, len(tok) - 1)], 0)
            ids[np.arange(len(grp)), L] = self.cfg.w_token
            readout = np.arange(len(grp)) * tmax + L
            # rows that hold a char or the [W] token; the padding behind them carries zero gradient and is kept out
            # of the embedding scatter (all of it would land on id 0 and be summed by a single CTA)
            live = np.flatnonzero((k <= L[:, None]).reshape(-1))
            live_dev = None if live.size == ids.size else self._dev(live, torch.int64)
            plan.append((self._dev(grp, torch.int64), len(grp), tmax, self._dev(ids.reshape(-1), torch.int64),
                         self._dev(readout, torch.int64), live_dev))
        return plan

    def _dec_plan(self, tok, start, lens, on):
        """Per group the id lists of src/gpu/hierarchical.rs:329-364: slot-0 rows, char rows and ids (slot k feeds
        char k-1), targets (the chars, then [W]) and the loss mask. on: 0/1 per word."""
        plan = []
        for grp in group_by_len(lens, self.no_group, self._cap()):
            grp = np.asarray(grp, np.int64)
            L = lens[grp]
            tmax = int(L.max()) + 1
            k = np.arange(tmax)[None, :]
            chars = tok[np.minimum(start[grp][:, None] + k, len(tok) - 1)]
            targets = np.where(k < L[:, None], chars, 0)
            targets[np.arange(len(grp)), L] = self.cfg.w_token
            mask = (k <= L[:, None]) * on[grp][:, None]
            fed = (k >= 1) & (k <= L[:, None])          # slots that take the previous char, row-major
            rows = (np.arange(len(grp))[:, None] * tmax + k)[fed]
            prev = tok[np.minimum(start[grp][:, None] + k - 1, len(tok) - 1)][fed]
            plan.append(dict(words=self._dev(grp, torch.int64), n=len(grp), tmax=tmax,
                             o_rows=self._dev(np.arange(len(grp)) * tmax, torch.int64),
                             char_rows=self._dev(rows, torch.int64), char_ids=self._dev(prev, torch.int64),
                             targets=self._dev(targets.reshape(-1), torch.int32),
                             mask=self._dev(mask.reshape(-1), torch.int32)))
        return plan, int(((lens + 1) * on).sum()), int(on.sum())

    # ---- stages ---------------------------------------------------------------------------------------------
    def _enc_stack(self, n_g, tmax, ids):
        h = self.table.w.index_select(0, ids)
        for blk in self.enc:
            h = blk.forward(h, n_g, tmax)
        return h

    def _backbone_forward(self, e_w, Bw, dw):
        """Chunk-major sweep (src/gpu/hierarchical.rs:959-1021). Returns o [Bw*dw, hc] and what the backward needs."""
        wh, hc = self.cfg.wh, self.cfg.hc
        bb_in = self.front.forward(e_w).view(Bw, dw, wh)
        spans = self._spans(dw)
        sweep = len(spans) > 1
        o = torch.empty((Bw, dw, hc), dtype=torch.float32, device=e_w.device)
        chunks, states = [], [None] * len(self.bb)
        for c0, ln in spans:
            blocks = [layers.shell(b) for b in self.bb] if sweep else self.bb
            back = layers.shell(self.back) if sweep else self.back
            h = bb_in[:, c0:c0 + ln].reshape(Bw * ln, wh)
            for i, blk in enumerate(blocks):
                cell = blk.cell
                cell.sweep = sweep
                if isinstance(cell, layers.MLstm):
                    cell.carry, cell.dcarry = states[i], None
                else:
                    cell.state, cell.dstate = states[i], None
                h = blk.forward(h, Bw, ln)
                states[i] = cell.carry if isinstance(cell, layers.MLstm) else cell.state
            o[:, c0:c0 + ln] = back.forward(h).view(Bw, ln, hc)
            chunks.append((blocks, back))
        return o.view(Bw * dw, hc), (spans, chunks, sweep)

    def _backbone_backward(self, d_o, saved, Bw, dw):
        """Spans right to left, each through all blocks, BPTT state handed leftwards (src/gpu/hierarchical.rs:1236-1295)."""
        wh, hc = self.cfg.wh, self.cfg.hc
        spans, chunks, sweep = saved
        d_o = d_o.view(Bw, dw, hc)
        d_in = torch.empty((Bw, dw, wh), dtype=torch.float32, device=d_o.device)
        dstates = [None] * len(self.bb)
        for (c0, ln), (blocks, back) in zip(reversed(spans), reversed(chunks)):
            d = back.backward(d_o[:, c0:c0 + ln].reshape(Bw * ln, hc))
            for i in range(len(blocks) - 1, -1, -1):
                cell = blocks[i].cell
                if isinstance(cell, layers.MLstm):
                    cell.dcarry = dstates[i]
                else:
                    cell.dstate = dstates[i]
                d = blocks[i].backward(d)
                dstates[i] = cell.dcarry if isinstance(cell, layers.MLstm) else cell.dstate
                blocks[i].release()
            d_in[:, c0:c0 + ln] = d.view(Bw, ln, wh)
        for blk in self.bb:  # leave the cells as plain training cells
            blk.cell.sweep = False
            if isinstance(blk.cell, layers.MLstm):
                blk.cell.carry = blk.cell.dcarry = None
            else:
                blk.cell.state = blk.cell.dstate = None
        return self.front.backward(d_in.view(Bw * dw, wh))

    def _decode_groups(self, plan, o, inv):
        """Forward and backward per length group; the loss accumulates on the device
        (src/gpu/hierarchical.rs:1029-1132). Returns d_o [words, hc]."""
        hc = self.cfg.hc
        d_o = torch.zeros_like(o)
        for g in plan:
            n_g, tmax = g["n"], g["tmax"]
            rows = n_g * tmax
            dec_in = torch.zeros((rows, hc), dtype=torch.float32, device=o.device)
            dec_in.index_copy_(0, g["o_rows"], o.index_select(0, g["words"]))
            if g["char_rows"].numel():
                dec_in.index_copy_(0, g["char_rows"], self.table.w.index_select(0, g["char_ids"]))
            h = dec_in
            for blk in self.dec:
                h = blk.forward(h, n_g, tmax)
            hdn = self.dec_norm.forward(h)
            pre = torch.mm(hdn, self.head.w)
            d_pre = pre  # the fused soft-cap + loss kernel writes the gradient over its input
            ops.softcap_cross_entropy(pre, g["targets"], d_pre, self.loss, self.cfg.cap, mask=g["mask"], inv=inv)
            self.head.g.addmm_(hdn.t(), d_pre)
            d = self.dec_norm.backward(torch.mm(d_pre, self.head.w.t()))
            for blk in reversed(self.dec):
                d = blk.backward(d)
                blk.release()
            self.dec_norm.release()
            # the decoder input's gradient goes to its two sources: slot 0 -> the backbone, char slots -> the table
            d_o.index_copy_(0, g["words"], d.index_select(0, g["o_rows"]))
            if g["char_rows"].numel():
                ops.embedding_scatter_add(self.table.g, g["char_ids"], d.index_select(0, g["char_rows"]))
        return d_o

    def _encoder_backward(self, plan, d_e_w):
        """Per group: forward again, then backward from the [W]-step rows (src/gpu/hierarchical.rs:1347-1407)."""
        hc = self.cfg.hc
        for words, n_g, tmax, ids, readout, live in plan:
            self._enc_stack(n_g, tmax, ids)
            d = torch.zeros((n_g * tmax, hc), dtype=torch.float32, device=d_e_w.device)
            d.index_copy_(0, readout, d_e_w.index_select(0, words))
            for blk in reversed(self.enc):
                d = blk.backward(d)
                blk.release()
            if live is None:
                ops.embedding_scatter_add(self.table.g, ids, d)
            else:
                ops.embedding_scatter_add(self.table.g, ids.index_select(0, live), d.index_select(0, live))

    def forward_backward(self, windows, word_loss=None):
        """windows: [(tokens, [(start, end), ...]), ...] with equally many words each; word 0 of a window is
        encode-only, words 1.. are decoded. word_loss (per window, one flag per decoded word; None = all on)
        keeps a word's rows out of the loss while the word is still encoded and decoded, as in supervised
        fine-tuning on the response only (src/gpu/hierarchical.rs:698-720). Accumulates every gradient and
        returns the mean cross-entropy over the unmasked decoder rows, read from the device once (under data
        parallelism: this rank's share of the global mean; the ranks' values add up to it)."""
        nw = len(windows[0][1])
        if any(len(w) != nw for _, w in windows):
            raise ValueError("the windows of one call must hold equally many words")
        dw, Bw = nw - 1, len(windows)
        if dw < 1:
            self.last_rows, self.last_word_loss = 0, 0.0
            return 0.0
        N = Bw * dw  # row i: window i // dw, word i % dw

        # all windows' tokens in one array; per row the start and length of the word it encodes and of the
        # word it decodes (the next one)
        tok = np.concatenate([np.asarray(t, np.int64).reshape(-1) for t, _ in windows] + [np.zeros(1, np.int64)])
        base = np.cumsum([0] + [len(t) for t, _ in windows[:-1]])
        se = np.stack([np.asarray(w, np.int64).reshape(nw, 2) + b for (_, w), b in zip(windows, base)])  # [Bw, nw, 2]
        enc_start, enc_len = se[:, :-1, 0].reshape(-1), (se[:, :-1, 1] - se[:, :-1, 0]).reshape(-1)
        dec_start, dec_len = se[:, 1:, 0].reshape(-1), (se[:, 1:, 1] - se[:, 1:, 0]).reshape(-1)
        on = np.ones(N, np.int64) if word_loss is None else np.asarray(word_loss).astype(bool).astype(np.int64).reshape(-1)
        if on.size != N:
            raise ValueError("word_loss needs one flag per decoded word of every window")
        enc_plan = self._enc_plan(tok, enc_start, enc_len)
        dec_plan, valid, scored = self._dec_plan(tok, dec_start, dec_len, on)
        total = valid if self.rows_of_all_ranks is None else self.rows_of_all_ranks(valid)
        inv = 1.0 / max(total, 1)

        e_w = torch.zeros((N, self.cfg.hc), dtype=torch.float32, device="cuda")
        for words, n_g, tmax, ids, readout, _live in enc_plan:
            h = self._enc_stack(n_g, tmax, ids)
            e_w.index_copy_(0, words, h.index_select(0, readout))
            for blk in self.enc:  # the backward re-runs this group, nothing of it is read again
                blk.release()
        o, saved = self._backbone_forward(e_w, Bw, dw)
        self.loss.zero_()
        done = self.on_stage_backward or (lambda i: None)
        d_o = self._decode_groups(dec_plan, o, inv)
        done(0)
        d_e_w = self._backbone_backward(d_o, saved, Bw, dw)
        done(1)
        self._encoder_backward(enc_plan, d_e_w)
        done(2)
        loss = float(self.loss.item())
        self.last_rows = valid
        self.last_word_loss = loss * valid / max(scored, 1)  # the same total re-averaged over words (:1124-1128)
        return loss
