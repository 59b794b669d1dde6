"""The NNM1 container codec (no GPU). The cases mirror the reference's own container tests
(src/format.rs:437-604: flat and hierarchical round trips, kind tag, version-1 head) and add what those leave
out: a byte string assembled by hand from the format's layout, every refusal the reader has, and the mapping
between the language model's parameter dictionary and the file's CPU-layer layout."""
import importlib.util
import os
import struct

import numpy as np
import pytest

from oracle import model as M

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    # The codec is numpy only; taking it from its file keeps this test independent of the CUDA library.
    spec = importlib.util.spec_from_file_location("xl_checkpoint", os.path.join(ROOT, "neural-networks_b200", "checkpoint.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


ck = _load()
r = np.random.default_rng(5)
f32 = lambda *s: r.standard_normal(s).astype(np.float32)


def emb(v, d):
    return dict(tag=ck.TAG_EMBEDDING, input=v, output=d, weights=f32(v, d))


def norm(d):
    return dict(tag=ck.TAG_NORM, input=d, output=d, gamma=f32(d))


def lin(i, o):
    return dict(tag=ck.TAG_LINEAR, input=i, output=o, in_dim=i, out_dim=o, weights=f32(i, o), biases=f32(o))


def test_bytes_of_a_small_flat_container_assembled_by_hand():
    w = np.array([[1.0], [-2.5]], np.float32)
    c = ck.Container(ck.KIND_FLAT).section("model", [
        dict(tag=ck.TAG_LINEAR, input=2, output=1, in_dim=2, out_dim=1, weights=w, biases=np.array([0.5], np.float32)),
        dict(tag=ck.TAG_SOFT_CAP, input=1, output=1, cap=30.0)])
    want = b"".join([
        b"\x31\x4d\x4e\x4e",              # 0x4E4E4D31 little-endian
        b"\x02", b"\x00",                 # version 2, flat: no typed head
        struct.pack("<I", 1),             # one section
        struct.pack("<I", 5), b"model",
        b"\x57\x46\x4e\x4e", b"\x02",     # stack magic 0x4E4E4657, stack version 2
        struct.pack("<I", 2),             # two layers
        b"\x0c", struct.pack("<II", 2, 1),
        b"\x11", struct.pack("<II", 1, 1),
        struct.pack("<II", 2, 1),         # Linear: its sizes again,
        struct.pack("<III", 2, 1, 2), struct.pack("<ff", 1.0, -2.5),   # matrix rows, cols, count, values
        struct.pack("<I", 1), struct.pack("<f", 0.5),                  # bias vector
        struct.pack("<f", 30.0),          # SoftCap
    ])
    assert ck.dumps(c) == want
    back = ck.loads(want)
    assert back.kind == ck.KIND_FLAT and [n for n, _ in back.sections] == ["model"]
    l0, l1 = back.sections[0][1]
    assert np.array_equal(l0["weights"], w) and l0["biases"].tolist() == [0.5] and l1["cap"] == 30.0


def test_flat_container_round_trips_to_identical_bytes():
    c = ck.Container(ck.KIND_FLAT).section("model", [emb(8, 16), norm(16), lin(16, 4)])
    b1 = ck.dumps(c)
    back = ck.loads(b1)
    assert back.kind == ck.KIND_FLAT and len(back.sections) == 1
    assert ck.dumps(ck.Container(ck.KIND_FLAT).section("model", back.take("model"))) == b1


def test_hierarchical_container_keeps_metadata_and_sections():
    meta = ck.new_meta(8, 16, 4242, pretrain_chars=12_345, pretrain_words=3_456, sft_chars=789, sft_words=210,
                       sft_resp_chars=456, sft_resp_words=120)
    c = (ck.Container(ck.KIND_HIERARCHICAL, meta).section("encoder", [emb(8, 16), norm(16)])
         .section("extra", lin(32, 16)).section("word_model", [norm(16), lin(16, 16)])
         .section("char2_model", [norm(16), lin(16, 8)]))
    back = ck.loads(ck.dumps(c))
    assert back.kind == ck.KIND_HIERARCHICAL
    assert (back.meta["vocab_size"], back.meta["context_size"], back.meta["step"]) == (8, 16, 4242)
    assert back.meta["seen"] == meta["seen"]
    for name in ("encoder", "word_model", "char2_model"):
        assert len(back.take(name)) == 2
    assert len(back.take("extra")) == 1  # a single stand-alone layer comes back as a one-layer stack
    with pytest.raises(ck.FormatError, match="missing section"):
        back.take("nope")


def test_version_1_head_ends_at_step_and_counters_read_zero():
    enc, wm, dec = [emb(8, 16)], [lin(16, 16)], [lin(16, 8)]
    out = ck._Out()
    out.u32(ck.MAGIC)
    out.u8(1)
    out.u8(ck.KIND_HIERARCHICAL)
    out.u32(8)
    out.u32(16)
    out.u64(99)
    out.u32(3)
    for name, layers in (("encoder", enc), ("word_model", wm), ("char2_model", dec)):
        out.string(name)
        ck._write_stack(out, layers)
    back = ck.loads(out.bytes())
    assert back.meta["step"] == 99 and all(v == 0 for v in back.meta["seen"].values())
    assert [n for n, _ in back.sections] == ["encoder", "word_model", "char2_model"]
    assert np.array_equal(back.sections[2][1][0]["weights"], dec[0]["weights"])


def test_kind_is_readable_from_the_header_alone(tmp_path):
    p = str(tmp_path / "sub" / "m.nnm")
    ck.save(p, ck.Container(ck.KIND_FLAT).section("model", [lin(4, 2)]))
    assert ck.peek_kind(p) == ck.KIND_FLAT
    assert not os.path.exists(p + ".tmp")
    assert "tag 12" in ck.describe(ck.load(p))


def test_reader_refusals():
    good = ck.dumps(ck.Container(ck.KIND_FLAT).section("model", [lin(4, 2)]))
    with pytest.raises(ck.FormatError, match="wrong magic"):
        ck.loads(b"\x00" + good[1:])
    with pytest.raises(ck.FormatError, match="unsupported NNM1 version 3"):
        ck.loads(good[:4] + b"\x03" + good[5:])
    with pytest.raises(ck.FormatError, match="unknown model kind tag 7"):
        ck.loads(good[:5] + b"\x07" + good[6:])
    at = good.index(b"\x57\x46\x4e\x4e")
    with pytest.raises(ck.FormatError, match="Wrong stack magic"):
        ck.loads(good[:at] + b"\x00" + good[at + 1:])
    with pytest.raises(ck.FormatError, match="Unknown stack version"):
        ck.loads(good[:at + 4] + b"\x09" + good[at + 5:])
    with pytest.raises(ck.FormatError, match="Unknown layer tag 99"):
        ck.loads(good[:at + 9] + b"\x63" + good[at + 10:])
    with pytest.raises(ck.FormatError, match="unexpected end of file"):
        ck.loads(good[:-3])
    with pytest.raises(ck.FormatError, match="lacks field"):
        ck.dumps(ck.Container(ck.KIND_FLAT).section("model", [dict(tag=ck.TAG_NORM, input=2, output=2)]))


def test_legacy_softmax_entry_is_consumed_and_dropped():
    out = ck._Out()
    out.u32(ck.STACK_MAGIC)
    out.u8(ck.STACK_VERSION)
    out.u32(2)
    out.u8(ck.TAG_LEGACY_SOFTMAX), out.u32(4), out.u32(4)
    out.u8(ck.TAG_NORM), out.u32(4), out.u32(4)
    out.u32(4)            # the softmax's size field
    out.vector(np.ones(4, np.float32))
    layers = ck._read_stack(ck._In(out.bytes()))
    assert len(layers) == 1 and layers[0]["tag"] == ck.TAG_NORM


def test_slstm_block_with_unequal_sizes_is_refused():
    out = ck._Out()
    out.u32(ck.STACK_MAGIC)
    out.u8(ck.STACK_VERSION)
    out.u32(1)
    out.u8(ck.TAG_SLSTM_BLOCK), out.u32(4), out.u32(8)
    with pytest.raises(ck.FormatError, match="input_size == output_size"):
        ck._read_stack(ck._In(out.bytes()))


CFG = dict(vocab=50, d=16, nb=3, heads=2, dqk=4, dhv=8, up=24)


def _params(slstm_at=(1,), nh_s=1, seed=3):
    c = CFG
    return M.init_lm_params(np.random.default_rng(seed), c["vocab"], c["d"], c["nb"], c["heads"], c["dqk"], c["dhv"], c["up"],
                            std=0.3, slstm_at=slstm_at, nh_s=nh_s)


def _same(a, b):
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_same(a[k], b[k]) for k in a)
    if isinstance(a, list):
        return len(a) == len(b) and all(_same(x, y) for x, y in zip(a, b))
    if isinstance(a, str):
        return a == b
    return np.array_equal(np.asarray(a), np.asarray(b))


@pytest.mark.parametrize("nh_s", [1, 2])
def test_lm_parameters_survive_the_file_bit_for_bit(nh_s):
    p = _params(nh_s=nh_s)
    c = ck.loads(ck.dumps(ck.lm_to_container(p, CFG["heads"], CFG["dqk"], cap=15.0)))
    q, info = ck.lm_from_container(c, nh_s=nh_s)
    assert _same(p, q)
    assert (info["heads"], info["dqk"], info["dhv"], info["up"], info["cap"], info["tied"]) == (2, 4, 8, 24, 15.0, True)
    # and the model built from the file computes what the original computes
    ids = np.random.default_rng(0).integers(0, CFG["vocab"], 2 * 6)
    a = M.build_lm(p, 2, 4, 8, nh_s=nh_s, cap=15.0).forward(ids, 2, 6)
    b = M.build_lm(q, info["heads"], info["dqk"], info["dhv"], nh_s=nh_s, cap=info["cap"]).forward(ids, 2, 6)
    assert np.array_equal(a, b)


def test_file_layout_is_the_cpu_layers_layout():
    p = _params(nh_s=2)
    layers = ck.lm_to_container(p, CFG["heads"], CFG["dqk"]).sections[0][1]
    d, H = CFG["d"], CFG["d"]
    assert [l["tag"] for l in layers] == [7, 14, 11, 14, 9, 3, 17]
    m = layers[1]
    assert np.array_equal(m["cell.wk"], p["blocks"][0]["cell"]["wk"])  # unscaled k projection
    assert m["cell.num_heads"] == 2 and m["cell.dqk"] == 4 and m["up_size"] == 24
    s, cell = layers[2], p["blocks"][1]["cell"]
    dh = H // 2
    for g, name in enumerate("zifo"):
        w = s["cell.w" + name]
        assert w.shape == (d + H, H)
        assert np.array_equal(w[:d], cell["wx"][:, g * H:(g + 1) * H])
        rec = w[d:]
        for h in range(2):
            assert np.array_equal(rec[h * dh:(h + 1) * dh, h * dh:(h + 1) * dh], cell["wh"][h][:, g * dh:(g + 1) * dh])
        assert not rec[:dh, dh:].any() and not rec[dh:, :dh].any()
        assert np.array_equal(s["cell.b" + name], cell["bcat"][g * H:(g + 1) * H])
    assert not s["cell.h_init"].any() and not s["cell.c_init"].any()
    assert np.array_equal(layers[5]["weights"], p["table"].T)


def test_dense_recurrence_is_not_cut_down_to_heads():
    c = ck.lm_to_container(_params(nh_s=1), CFG["heads"], CFG["dqk"])
    with pytest.raises(ck.FormatError, match="between heads"):
        ck.lm_from_container(c, nh_s=2)


def test_untied_head_round_trips_as_a_linear():
    p = _params(slstm_at=())
    hw, hb = f32(CFG["d"], CFG["vocab"]), f32(CFG["vocab"])
    c = ck.loads(ck.dumps(ck.lm_to_container(p, 2, 4, head_w=hw, head_b=hb)))
    q, info = ck.lm_from_container(c)
    assert _same(p, q) and not info["tied"]
    assert np.array_equal(info["head_w"], hw) and np.array_equal(info["head_b"], hb)


# ---- hierarchical model -------------------------------------------------------------------------------------
from oracle import hier as OH


def _hier():
    cfg = OH.HierCfg(vocab=12, hc=16, wh=24, enc_blocks=2, bb_blocks=3, dec_blocks=2, heads=2, dqk=8, w_token=11,
                     cap=20.0, small_heads=2)
    p = OH.init_hier_params(np.random.default_rng(4), cfg, std=0.3)
    p = {k: ([dict(b, cell=dict(b["cell"])) for b in v] if isinstance(v, list) else np.asarray(v, np.float32)) for k, v in p.items()}
    for k in ("enc", "bb", "dec"):
        for b in p[k]:
            for kk in list(b):
                if kk != "cell":
                    b[kk] = np.asarray(b[kk], np.float32)
            b["cell"] = {kk: (vv if kk == "kind" else np.asarray(vv, np.float32)) for kk, vv in b["cell"].items()}
    return cfg, p


def test_hierarchical_parameters_survive_the_file_and_keep_the_references_section_layout():
    cfg, p = _hier()
    c = ck.hier_to_container(p, cfg, step=77, seen=dict(pretrain_chars=1000, pretrain_words=200))
    assert [n for n, _ in c.sections] == ["encoder", "word_model", "char2_model"]
    tags = {n: [l["tag"] for l in ls] for n, ls in c.sections}
    assert tags == {"encoder": [7, 11, 14], "word_model": [12, 11, 14, 14, 12], "char2_model": [11, 14, 9, 3, 17]}
    back = ck.loads(ck.dumps(c))
    assert (back.meta["vocab_size"], back.meta["context_size"], back.meta["step"]) == (12, 16, 77)
    assert back.meta["seen"]["pretrain_chars"] == 1000 and back.meta["seen"]["sft_words"] == 0
    q, info = ck.hier_from_container(back)
    assert _same(p, q)
    assert (info["vocab"], info["hc"], info["wh"], info["heads"], info["dqk"], info["small_heads"], info["cap"]) == \
        (12, 16, 24, 2, 8, 2, 20.0)
    assert (info["enc_kinds"], info["bb_kinds"], info["dec_kinds"]) == ("sm", "smm", "sm")


def test_hierarchical_loader_checks_the_stage_layout():
    cfg, p = _hier()
    c = ck.hier_to_container(p, cfg)
    flat = ck.Container(ck.KIND_FLAT, sections=c.sections)
    with pytest.raises(ck.FormatError, match="not a hierarchical"):
        ck.hier_from_container(flat)
    sections = dict(c.sections)
    broken = ck.Container(ck.KIND_HIERARCHICAL, c.meta, [("encoder", sections["encoder"][1:]),
                                                         ("word_model", sections["word_model"]),
                                                         ("char2_model", sections["char2_model"])])
    with pytest.raises(ck.FormatError, match="start with an Embedding"):
        ck.hier_from_container(broken)
    broken = ck.Container(ck.KIND_HIERARCHICAL, c.meta, [("encoder", sections["encoder"]),
                                                         ("word_model", sections["word_model"][:-1]),
                                                         ("char2_model", sections["char2_model"])])
    with pytest.raises(ck.FormatError, match="start and end with a Linear"):
        ck.hier_from_container(broken)
    broken = ck.Container(ck.KIND_HIERARCHICAL, c.meta, [("encoder", sections["encoder"]),
                                                         ("word_model", sections["word_model"])])
    with pytest.raises(ck.FormatError, match="missing section 'char2_model'"):
        ck.hier_from_container(broken)
