"""GPU parity of the layer stack (cells, block, flat LM) against the CPU oracle stack, in the
manner of the reference's mlstm_matches_cpu / block tests / lm_matches_cpu (src/gpu/mlstm.rs:1004,
src/gpu/block.rs:1328-1447, src/gpu/lm.rs:187-286): forward, backward and one AdamW step from the
same host weights; compare loss, every gradient and every post-step weight.
fp32 bar: 1e-4 rel-to-max for the loss and every gradient. The optimizer step is checked exactly
(1e-6) by applying the oracle's AdamW to the GPU's own gradients: comparing post-step weights of
two independent pipelines is ill-conditioned at t = 1, where every element moves by
lr * g / (|g| + eps) and a 1e-9 difference on a near-zero gradient becomes a visible fraction of lr
(the reference's own post-step bar is 2e-2 for that reason, src/gpu/lm.rs:187-286).
With bf16 GEMM operands and bf16 q/k/v the whole-model gradients compound some twenty rounding
points per block: loss within 5e-3 (the reference's bar), gradient tensors above the noise floor
within 1.5e-1 rel-to-max (the worst tensor's single worst element; it moves between 0.10 and 0.13
with the rounding realisation, e.g. whether q/k/v are narrowed by the GEMM epilogue or by a cast) and the
full gradient direction within cos >= 0.995; the 2e-2 bar is held at the op level
(tests/test_gpu_mlstm.py)."""
import importlib

import numpy as np
import pytest
import torch

from oracle import model as M

pytestmark = pytest.mark.gpu


def _compare(cfg, bf16, tol, loss_tol, slstm_at=(), nh_s=1, seed=0, noise_floor=0.0, cos_min=0.999999):
    xl = importlib.import_module("neural-networks_b200")
    layers = importlib.import_module("neural-networks_b200.layers")
    vocab, d, nb, heads, dqk, dhv, up, B, T = cfg
    rng = np.random.default_rng(seed)
    p = M.init_lm_params(rng, vocab, d, nb, heads, dqk, dhv, up, std=0.02 if not slstm_at else 0.1, slstm_at=slstm_at, nh_s=nh_s)
    ids = rng.integers(0, vocab, B * T)
    tg = np.roll(ids.reshape(B, T), -1, axis=1).reshape(-1)
    ref = M.build_lm(p, heads, dqk, dhv, nh_s=nh_s, tied=True)
    loss_ref, grads_ref = ref.train_step(ids, tg, B, T, 1e-3, 0.1, 1)
    lm = layers.build_lm(p, heads, dqk, dhv, nh_s=nh_s, tied=True, bf16=bf16)
    tid = torch.tensor(ids, dtype=torch.int64, device="cuda")
    ttg = torch.tensor(tg.astype(np.int32), device="cuda")
    loss = lm.forward_backward(tid, ttg, B, T)
    grads = [q.g.clone() for q in lm.params()]
    w_before = [q.w.cpu().numpy().copy() for q in lm.params()]
    cfg_ = xl.ops.AdamCfg(1e-3, 0.1, t=1)
    lm.step(cfg_)
    torch.cuda.synchronize()
    assert xl._lib.lib.xlstm_device_status() == 0
    assert abs(loss.item() - loss_ref) <= loss_tol * max(1.0, abs(loss_ref)), (loss.item(), loss_ref)
    rp = ref.params()
    assert len(rp) == len(grads)
    from oracle import oracle as O
    dot = nn_ = nr_ = 0.0
    for i, (g, gr, q, r, w0) in enumerate(zip(grads, grads_ref, lm.params(), rp, w_before)):
        gg = g.cpu().numpy().astype(np.float64)
        dot += float((gg * gr).sum()); nn_ += float((gg * gg).sum()); nr_ += float((gr * gr).sum())
        if np.abs(gr).max() >= noise_floor:
            e = np.abs(gg - gr).max() / np.abs(gr).max()
            assert e <= tol, "grad %d %s: rel-to-max %.3e" % (i, gr.shape, e)
        # the optimizer step itself, checked exactly: AdamW(oracle) applied to the GPU's own gradient
        want = O.adamw(w0, g.cpu().numpy(), np.zeros_like(w0), np.zeros_like(w0), 1e-3, 0.1 if q.decay else 0.0, 1,
                       dtype=np.float32)[0]
        ew = np.abs(q.w.cpu().numpy() - want).max() / max(np.abs(want).max(), 1e-12)
        assert ew <= 1e-6, "post-step weight %d: rel-to-max %.3e" % (i, ew)
        assert float(q.g.abs().max()) == 0.0
        if q.wb is not None:
            assert torch.equal(q.wb, q.w.to(torch.bfloat16))  # the bf16 shadow follows the weight
    assert dot / np.sqrt(nn_ * nr_) >= cos_min


def test_config1_byte_lm_fp32():
    """BASELINE config 1: vocab 256, d=128, 2 mLSTM blocks of 4 heads x 32, up = 341, B8 x T256, fp32,
    tied head, one AdamW step (lr 1e-3, wd 0.1)."""
    _compare((256, 128, 2, 4, 32, 32, 341, 8, 256), False, 1e-4, 1e-4)


def test_toy_lm_fp32_with_slstm_blocks():
    _compare((13, 8, 2, 2, 4, 4, 12, 2, 12), False, 1e-4, 1e-4, slstm_at=(1,), nh_s=1)
    _compare((13, 16, 2, 2, 8, 8, 24, 2, 12), False, 1e-4, 1e-4, slstm_at=(0,), nh_s=2, seed=1)


def test_lm_bf16_operands_tensor_core_cells():
    """Two mLSTM blocks with 2 heads x 128 (tensor-core path), bf16 GEMM operands and q/k/v storage."""
    _compare((64, 256, 2, 2, 128, 128, 680, 2, 128), True, 1.5e-1, 5e-3, seed=2, noise_floor=1e-3, cos_min=0.995)


def test_remat_is_exact_and_row_chunked_head_agrees():
    """Re-running a block's forward before its backward changes memory only: loss and every gradient are
    bit-equal to the plain path's. The row-chunked head (fused soft-cap + loss kernel, head gradient summed
    chunk by chunk) agrees with the plain head to fp32 rounding."""
    layers = importlib.import_module("neural-networks_b200.layers")
    vocab, d, nb, heads, dqk, dhv, up, B, T = 97, 64, 3, 2, 32, 32, 176, 3, 50
    rng = np.random.default_rng(7)
    p = M.init_lm_params(rng, vocab, d, nb, heads, dqk, dhv, up, std=0.1, slstm_at=(1,), nh_s=2)
    ids = torch.tensor(rng.integers(0, vocab, B * T), dtype=torch.int64, device="cuda")
    tg = torch.tensor(rng.integers(0, vocab, B * T).astype(np.int32), device="cuda")
    out = []
    for kw in (dict(), dict(remat=True), dict(remat=[0, 2], head_rows=64), dict(head_rows=64, head_split=True),
               dict(head_rows=64, head_split=3)):
        lm = layers.build_lm(p, heads, dqk, dhv, nh_s=2, tied=True, **kw)
        loss = lm.forward_backward(ids, tg, B, T).item()
        out.append((loss, [q.g.clone() for q in lm.params()]))
    (l0, g0), (l1, g1), (l2, g2), (l3, g3), (l4, g4) = out
    assert l0 == l1
    for i, (a, b) in enumerate(zip(g0, g1)):
        assert torch.equal(a, b), i
    gmax = max(float(a.abs().max()) for a in g0)  # bias gradients are sums that nearly cancel: floor the bar
    for l, g in ((l2, g2), (l3, g3)):
        assert abs(l0 - l) <= 1e-6 * abs(l0)
        for i, (a, b) in enumerate(zip(g0, g)):
            assert float((a - b).abs().max()) <= 2e-5 * float(a.abs().max()) + 1e-6 * gmax, i
    # the three-product head: operands cut at 16 bits, so the bar is the fp32 parity bar, not round-off
    assert abs(l0 - l4) <= 1e-5 * abs(l0)
    for i, (a, b) in enumerate(zip(g0, g4)):
        assert float((a - b).abs().max()) <= 1e-4 * float(a.abs().max()) + 1e-5 * gmax, i


def test_split_bf16_product_is_fp32_accurate():
    """The head's split product (six bf16 tensor-core GEMMs on 3-way split operands) against an fp64 product:
    no worse than the plain fp32 GEMM it replaces."""
    layers = importlib.import_module("neural-networks_b200.layers")
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn((512, 768), device="cuda", generator=g)
    b = torch.randn((768, 640), device="cuda", generator=g) * 0.02
    ref = a.double() @ b.double()
    got = layers._mm_split(layers._split3(a), layers._split3(b))
    plain = a @ b
    scale = float(ref.abs().max())
    e_split = float((got.double() - ref).abs().max()) / scale
    e_plain = float((plain.double() - ref).abs().max()) / scale
    assert e_split <= max(2.0 * e_plain, 2e-6), (e_split, e_plain)
    # three products (hi*hi + hi*mid + mid*hi): 16 bits per operand, far inside TF32's 10 and bf16's 8
    got3 = layers._mm_split(layers._split3(a), layers._split3(b), terms=3)
    e3 = float((got3.double() - ref).abs().max()) / scale
    tf32 = float(((a.double() * (1 + 2.0 ** -11)) @ b.double() - ref).abs().max()) / scale  # one TF32 half-ulp on a
    assert e3 <= 1e-5 and e3 < tf32, (e3, tf32)
    into = torch.empty_like(got3)
    assert layers._mm_split(layers._split3(a), layers._split3(b), terms=3, into=into) is into and torch.equal(into, got3)


def test_recomputed_chunk_states_leave_the_step_bit_identical():
    """`recompute_states`: training keeps no chunk-state record and the backward rebuilds the chunk-boundary
    states (the reference stores them for every chunk, src/gpu/ops.rs:3955-3967). Loss and every gradient of a
    two-block bf16 LM on the tensor-core cells are bit-identical with the switch on."""
    layers = importlib.import_module("neural-networks_b200.layers")
    vocab, d, nb, heads, dqk, dhv, up, B, T = 64, 256, 2, 2, 128, 128, 680, 2, 200
    rng = np.random.default_rng(11)
    p = M.init_lm_params(rng, vocab, d, nb, heads, dqk, dhv, up, std=0.05)
    ids = torch.tensor(rng.integers(0, vocab, B * T), dtype=torch.int64, device="cuda")
    tg = torch.tensor(rng.integers(0, vocab, B * T).astype(np.int32), device="cuda")
    out = []
    for rec in (False, True):
        lm = layers.build_lm(p, heads, dqk, dhv, tied=True, bf16=True, recompute_states=rec)
        loss = lm.forward_backward(ids, tg, B, T).item()
        assert all((blk.cell.fused is None) for blk in lm.blocks)  # released after the backward
        out.append((loss, [q.g.clone() for q in lm.params()]))
    assert out[0][0] == out[1][0]
    for i, (a, b) in enumerate(zip(out[0][1], out[1][1])):
        assert torch.equal(a, b), i
