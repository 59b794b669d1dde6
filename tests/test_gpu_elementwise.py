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
