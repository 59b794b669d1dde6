"""GPU parity of RMSNorm, softmax-CE and AdamW against the CPU oracle, through the C ABI.
Shapes follow the reference's op tests (src/gpu/ops.rs:5527-5672, 4728-4808). Bars: 1e-4
rel-to-max for RMSNorm/CE, 1e-6 for AdamW."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,F,group", [(7 * 64, 1024, 1024), (3 * 512, 256, 256), (5 * 30, 300, 300), (5, 12, 4),
                                          (64, 2048, 2048), (100, 1024, 128), (33, 2048, 256), (9, 4096, 4096)])
def test_rmsnorm(rows, F, group):
    from gpu_util import ops, dev, host, rel_to_max
    r = np.random.default_rng(0)
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    x = f32(r.standard_normal((rows, F)) * 2); gamma = f32(1 + 0.1 * r.standard_normal(F)); dy = f32(r.standard_normal((rows, F)))
    y, xh, inv = O.rmsnorm_fw(x, gamma, group)
    dx, dgam = O.rmsnorm_bw(dy, xh, inv, gamma, group)
    dx_, dg_ = dev(x), dev(gamma)
    out = torch.full((rows, F), float("nan"), device="cuda"); inv_ = torch.empty((rows * (F // group),), device="cuda")
    xh_ = torch.empty((rows, F), device="cuda")
    ops.rms_norm_forward_into(dx_, dg_, group, out, inv_, x_hat=xh_)
    base = f32(r.standard_normal(F))
    dgam_ = dev(base)
    dxo = torch.full((rows, F), float("nan"), device="cuda")
    ops.rms_norm_backward_into(dev(dy), dx_, inv_, dg_, group, dxo, dgam_)
    torch.cuda.synchronize()
    assert rel_to_max(host(out), y) <= 1e-4
    assert rel_to_max(host(xh_), xh) <= 1e-4
    assert rel_to_max(host(inv_).reshape(inv.shape), inv) <= 1e-4
    assert rel_to_max(host(dxo), dx) <= 1e-4
    assert rel_to_max(host(dgam_), base + dgam) <= 1e-4  # accumulated onto what was there


@pytest.mark.parametrize("rows,C", [(6, 9), (2048, 256), (37, 1000), (64, 5000), (16, 50304), (3, 70001)])
@pytest.mark.parametrize("masked", [False, True])
def test_softmax_ce(rows, C, masked):
    from gpu_util import ops, dev, host, rel_to_max
    r = np.random.default_rng(1)
    z = (r.standard_normal((rows, C)) * 3).astype(np.float32).astype(np.float64)
    t = r.integers(0, C, rows)
    mask = None; inv = 1.0 / rows
    if masked:
        mask = (r.random(rows) > 0.3).astype(np.uint32); mask[0] = 1
        inv = 1.0 / float(mask.sum()) * 0.5  # a window-level scale, not 1/own rows
    loss, d = O.softmax_ce(z, t, mask=mask, inv=inv)
    logits = dev(z)
    acc = torch.full((1,), 2.5, device="cuda")
    tg = torch.tensor(t.astype(np.int32), device="cuda")
    mk = None if mask is None else torch.tensor(mask.astype(np.int32), device="cuda")
    ops.softmax_cross_entropy(logits, tg, logits, acc, mask=mk, inv=inv)  # in place
    torch.cuda.synchronize()
    assert abs(acc.item() - 2.5 - loss) <= 1e-4 * max(1.0, abs(loss))
    assert rel_to_max(host(logits), d) <= 1e-4


@pytest.mark.parametrize("rows,C", [(6, 9), (37, 1000), (64, 5000), (16, 50304), (3, 70001)])
def test_softcap_fused_into_ce(rows, C):
    """Loss of cap*tanh(x/cap) and its gradient with respect to x, against the oracle's CE composed with the
    soft-cap in float64 (src/nn2/ops.rs:25-42 then src/nn2/loss.rs:10-53)."""
    from gpu_util import ops, dev, host, rel_to_max
    r = np.random.default_rng(2)
    cap = 30.0
    x = (r.standard_normal((rows, C)) * 25).astype(np.float32).astype(np.float64)  # well into the cap's bend
    t = r.integers(0, C, rows)
    z = cap * np.tanh(x / cap)
    loss, dz = O.softmax_ce(z, t, inv=1.0 / rows)
    dx = dz * (1.0 - (z / cap) ** 2)
    pre = dev(x)
    acc = torch.zeros((1,), device="cuda")
    ops.softcap_cross_entropy(pre, torch.tensor(t.astype(np.int32), device="cuda"), pre, acc, cap)  # in place
    torch.cuda.synchronize()
    assert abs(acc.item() - loss) <= 1e-4 * max(1.0, abs(loss))
    assert rel_to_max(host(pre), dx) <= 1e-4


@pytest.mark.parametrize("n", [8, 4 * 1000 + 3, 1 << 20])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_swiglu_and_output_gate_glue(n, out_dtype):
    """SwiGLU and output-gate forward/backward against float64 formulas (src/nn2/block.rs:128-216,
    src/nn2/mlstm.rs:347-577); bf16 outputs within one rounding (2^-8 relative)."""
    from gpu_util import ops, dev, host
    r = np.random.default_rng(3)
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    g, v, d, y = (f32(r.standard_normal(n) * 2) for _ in range(4))
    sig = 1.0 / (1.0 + np.exp(-g))
    tol = 1e-6 if out_dtype == torch.float32 else 2.0 ** -8
    close = lambda got, ref: np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())
    assert close(host(ops.swiglu_forward(dev(g), dev(v), out_dtype).float()), g * sig * v)
    if n % 8 == 0:  # the projections' biases folded into the kernels: [rows, cols] with cols = 8
        bg, bv = f32(r.standard_normal(8)), f32(r.standard_normal(8))
        gb, vb = g.reshape(-1, 8) + bg, v.reshape(-1, 8) + bv
        sb = 1.0 / (1.0 + np.exp(-gb))
        g2, v2, d2 = dev(g).view(-1, 8), dev(v).view(-1, 8), dev(d).view(-1, 8)
        assert close(host(ops.swiglu_forward(g2, v2, out_dtype, dev(bg), dev(bv)).float()), gb * sb * vb)
        dgb, dvb = ops.swiglu_backward(d2, g2, v2, out_dtype, dev(bg), dev(bv))
        assert close(host(dgb.float()), d.reshape(-1, 8) * vb * sb * (1.0 + gb * (1.0 - sb)))
        assert close(host(dvb.float()), d.reshape(-1, 8) * gb * sb)
    dg, dv = ops.swiglu_backward(dev(d), dev(g), dev(v), out_dtype)
    assert close(host(dg.float()), d * v * sig * (1.0 + g * (1.0 - sig)))
    assert close(host(dv.float()), d * g * sig)
    # bf16 pre-activations (a bf16 layer's GEMM epilogues) and, in the backward, a bf16 upstream gradient: exact on
    # the rounded inputs
    gn, vn, dn = (dev(a).to(torch.bfloat16) for a in (g, v, d))
    g_, v_, d_ = (host(a.float()).astype(np.float64) for a in (gn, vn, dn))
    s_ = 1.0 / (1.0 + np.exp(-g_))
    assert close(host(ops.swiglu_forward(gn, vn, out_dtype).float()), g_ * s_ * v_)
    if out_dtype == torch.bfloat16:
        for dd, dref in ((dn, d_), (dev(d), d)):
            dg, dv = ops.swiglu_backward(dd, gn, vn, out_dtype)
            assert close(host(dg.float()), dref * v_ * s_ * (1.0 + g_ * (1.0 - s_)))
            assert close(host(dv.float()), dref * g_ * s_)
    else:
        with pytest.raises(Exception):
            ops.swiglu_backward(dn, gn, vn, out_dtype)
    o = dev(g)
    hc = ops.ogate_forward(o, dev(y), out_dtype)
    assert np.abs(host(o) - sig).max() <= (1e-6 if out_dtype == torch.float32 else 2e-6)  # bf16 layers: SFU sigmoid
    assert close(host(hc.float()), sig * y)
    do_pre, d_yhat = ops.ogate_backward(dev(d), o, dev(y), out_dtype)
    assert close(host(do_pre.float()), d * y * sig * (1.0 - sig))
    assert np.abs(host(d_yhat) - d * sig).max() <= 1e-6 * max(1.0, np.abs(d * sig).max())


@pytest.mark.parametrize("n", [8, 1003, 1 << 18])
def test_split3_bf16_carries_the_full_significand(n):
    """hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid): each term is a bf16 number and their sum is x to
    within 2^-24 relative (three 8-bit significands)."""
    from gpu_util import ops
    g = torch.Generator(device="cuda").manual_seed(9)
    x = torch.randn((n,), device="cuda", generator=g) * torch.exp(3.0 * torch.randn((n,), device="cuda", generator=g))
    hi, mid, lo = ops.split3_bf16(x)
    assert torch.equal(hi, x.to(torch.bfloat16))
    assert torch.equal(mid, (x - hi.float()).to(torch.bfloat16))
    back = hi.double() + mid.double() + lo.double()
    assert float(((back - x.double()).abs() / x.double().abs().clamp_min(1e-30)).max()) <= 2.0 ** -23


def test_embedding_scatter_add_is_exact_and_repeatable():
    """Token-row sums in position order: equal to a sequential float32 accumulation, bit for bit, on ids with
    heavy repeats (src/gpu/cuda/common.cu:127-168 is deterministic too, by slicing)."""
    from gpu_util import ops
    r = np.random.default_rng(4)
    n, dm, vocab = 3000, 96, 50
    ids = r.integers(0, vocab, n)
    d = r.standard_normal((n, dm)).astype(np.float32)
    g0 = r.standard_normal((vocab, dm)).astype(np.float32)
    want = g0.copy()
    for p in range(n):
        want[ids[p]] += d[p]
    outs = []
    for _ in range(2):
        g = torch.tensor(g0, device="cuda")
        ops.embedding_scatter_add(g, torch.tensor(ids, device="cuda"), torch.tensor(d, device="cuda"))
        outs.append(g.cpu().numpy())
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0], want)


@pytest.mark.parametrize("dm,vocab", [(256, 7), (128, 3), (1024, 5), (2048, 40)])
def test_embedding_scatter_add_wide_rows_fixed_lane_order(dm, vocab):
    """Rows that are a whole number of 16-byte pieces tiling the CTA: 256 / min(dm / 4, 256) row lanes each sum every
    RL-th row of an id's run in position order and the lane sums are added in lane order: a fixed order, reproduced here
    in float32, so the result is exact and repeatable (a byte vocabulary: runs of hundreds of rows)."""
    from gpu_util import ops
    r = np.random.default_rng(dm)
    n = 2500
    ids = r.integers(0, vocab, n)
    d = r.standard_normal((n, dm)).astype(np.float32)
    g0 = r.standard_normal((vocab, dm)).astype(np.float32)
    RL = 256 // min(dm // 4, 256)
    want = g0.copy()
    for i in range(vocab):
        rows = np.nonzero(ids == i)[0]
        parts = []
        for lane in range(RL):
            acc = np.zeros(dm, np.float32)
            for p in rows[lane::RL]:
                acc += d[p]
            parts.append(acc)
        if len(rows):
            for acc in parts:
                want[i] += acc
    outs = []
    for _ in range(2):
        g = torch.tensor(g0, device="cuda")
        ops.embedding_scatter_add(g, torch.tensor(ids, device="cuda"), torch.tensor(d, device="cuda"))
        outs.append(g.cpu().numpy())
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(outs[0], want)


@pytest.mark.parametrize("wd", [0.0, 0.01])
def test_adamw_single_and_batched(wd):
    from gpu_util import ops, dev, host, rel_to_max
    r = np.random.default_rng(2)
    sizes = [20, 4096, 4097, 12345, 1, 70000]
    f32 = lambda a: a.astype(np.float32)
    P = [f32(r.standard_normal(n)) for n in sizes]; M = [np.zeros(n, np.float32) for n in sizes]; V = [np.zeros(n, np.float32) for n in sizes]
    dP = [dev(p) for p in P]; dM = [dev(m) for m in M]; dV = [dev(v) for v in V]
    dPb = [torch.empty((n,), dtype=torch.bfloat16, device="cuda") for n in sizes]
    sP = [dev(p) for p in P]; sM = [dev(m) for m in M]; sV = [dev(v) for v in V]
    cfg = ops.AdamCfg(1e-3, wd)
    for t in range(1, 4):
        cfg.t = t
        G = [f32(r.standard_normal(n)) for n in sizes]
        dG = [dev(g) for g in G]
        q = ops.AdamwQueue()
        for i in range(len(sizes)):
            q.push(dP[i], dG[i], dM[i], dV[i], decay=(i % 2 == 0), p_bf16=dPb[i])
        q.flush(cfg)
        for i in range(len(sizes)):
            ops.adamw(sP[i], dev(G[i]), sM[i], sV[i], cfg, decay=(i % 2 == 0))
            P[i], M[i], V[i] = O.adamw(P[i], G[i], M[i], V[i], 1e-3, wd if i % 2 == 0 else 0.0, t, dtype=np.float32)
            assert float(dG[i].abs().max()) == 0.0  # flush clears the grads
    torch.cuda.synchronize()
    for i in range(len(sizes)):
        assert rel_to_max(host(dP[i]), P[i]) <= 1e-6
        assert rel_to_max(host(dM[i]), M[i]) <= 1e-6 and rel_to_max(host(dV[i]), V[i]) <= 1e-6
        assert torch.equal(dP[i], sP[i])  # batched == per-tensor, bit for bit
        assert torch.equal(dPb[i], dP[i].to(torch.bfloat16))  # the bf16 shadow is the RNE cast of the new weight


@pytest.mark.parametrize("rows,F,group", [(64, 2048, 256), (33, 1024, 1024), (5, 12, 4), (7, 300, 300)])
def test_rmsnorm_bf16_storage_and_residual(rows, F, group):
    """The norm reading a bf16 tensor (the mLSTM core's output), writing bf16 (what only GEMMs consume), and the
    backward adding the skip connection's gradient in the same pass: each equals the fp32 op applied to the
    bf16-rounded operand, to bf16 rounding of the result where the result is bf16."""
    from gpu_util import ops, dev, host, rel_to_max, bf16_round
    r = np.random.default_rng(3)
    f32 = lambda a: a.astype(np.float32).astype(np.float64)
    x = bf16_round(r.standard_normal((rows, F)) * 2); gamma = f32(1 + 0.1 * r.standard_normal(F))
    dy = f32(r.standard_normal((rows, F))); res = f32(r.standard_normal((rows, F)))
    y, xh, inv = O.rmsnorm_fw(x, gamma, group)
    dx, dgam = O.rmsnorm_bw(dy, xh, inv, gamma, group)
    xb, g_ = dev(x, torch.bfloat16), dev(gamma)
    inv_ = torch.empty((rows * (F // group),), device="cuda")
    for ydt, tol in ((torch.float32, 1e-4), (torch.bfloat16, 8e-3)):
        out = torch.empty((rows, F), dtype=ydt, device="cuda")
        ops.rms_norm_forward_into(xb, g_, group, out, inv_)
        assert rel_to_max(host(out), y) <= tol
    for ddt, tol in ((torch.float32, 1e-4), (torch.bfloat16, 8e-3)):
        dgam_ = torch.zeros(F, device="cuda")
        dxo = torch.empty((rows, F), dtype=ddt, device="cuda")
        ops.rms_norm_backward_into(dev(dy), xb, inv_, g_, group, dxo, dgam_, residual=dev(res))
        assert rel_to_max(host(dxo), dx + res) <= tol
        assert rel_to_max(host(dgam_), dgam) <= 1e-4


@pytest.mark.parametrize("rows,cols", [(1, 4), (37, 8), (1000, 2048), (4096, 5464), (333, 130), (64, 7)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_colsum_narrow(rows, cols, dtype):
    """Bias gradient (fixed-order column sum, accumulated) and the bf16 copy of the scaled tensor in one pass."""
    from gpu_util import ops, dev, host, rel_to_max, bf16_round
    r = np.random.default_rng(4)
    x = r.standard_normal((rows, cols)) + 0.3
    x = bf16_round(x) if dtype == torch.bfloat16 else x.astype(np.float32).astype(np.float64)
    base = r.standard_normal(cols).astype(np.float32).astype(np.float64)
    for scale, narrow in ((1.0, True), (0.125, True), (0.5, False)):
        acc = dev(base)
        xd = dev(x, dtype)
        out = ops.colsum_narrow(xd, acc, scale, narrow=narrow)
        assert rel_to_max(host(acc), base + scale * x.sum(0)) <= 1e-5
        if not narrow or (dtype == torch.bfloat16 and scale == 1.0):
            assert out is xd
        else:
            assert out.dtype == torch.bfloat16
            assert torch.equal(out, (xd.float() * scale).to(torch.bfloat16))
        again = dev(base)
        ops.colsum_narrow(xd, again, scale, narrow=narrow)
        assert torch.equal(acc, again)  # fixed summation order


@pytest.mark.parametrize("rows,cols", [(3, 5), (128, 2048), (77, 12)])
def test_bias_rows_and_ogate_bias(rows, cols):
    from gpu_util import ops, dev, host
    r = np.random.default_rng(5)
    f32 = lambda a: a.astype(np.float32)
    b, res = f32(r.standard_normal(cols)), f32(r.standard_normal((rows, cols)))
    assert torch.equal(ops.bias_rows(dev(b), rows), dev(np.broadcast_to(b, (rows, cols)).copy()))
    assert torch.equal(ops.bias_rows(dev(b), rows, dev(res)), dev(res + b))
    o, y = f32(r.standard_normal((rows, cols))), f32(r.standard_normal((rows, cols)))
    od = dev(o)
    hc = ops.ogate_forward(od, dev(y), torch.float32, bias=dev(b))
    sig = 1.0 / (1.0 + np.exp(-(o.astype(np.float64) + b)))
    assert np.abs(host(od) - sig).max() <= 1e-6
    assert np.abs(host(hc) - sig * y).max() <= 1e-5
