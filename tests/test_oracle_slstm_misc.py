"""Oracle checks for the sLSTM loop, grouped RMSNorm, softmax-CE and AdamW: each against
an independent torch float64 formulation (autograd for the backward passes), plus the
block-diagonal == masked-dense identity and carry == whole-sequence, as the reference
tests them (src/gpu/slstm.rs:1843-1938, src/nn2/rms_norm.rs:86-143, src/nn2/loss.rs:71-95,
src/gpu/ops.rs:5643)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O


def _torch_slstm(wh, g, bcat, B, H, T, state=None):
    c = torch.zeros(B, H, dtype=torch.float64); n = c.clone(); m = c.clone(); h = c.clone()
    if state is not None:
        c, n, m, h = state
    outs = []
    for t in range(T):
        pre = g[:, t] + h @ wh + bcat
        zp, ip_, fp_, op_ = pre.split(H, dim=-1)
        z = torch.tanh(zp); o = torch.sigmoid(op_)
        fm = torch.nn.functional.logsigmoid(fp_) + m
        with torch.no_grad():
            mm = torch.where(n == 0, ip_, torch.maximum(fm, ip_))
        ip = torch.exp(ip_ - mm).clamp(max=1.0)
        fp = torch.exp(fm - mm).clamp(max=1.0)
        c = fp * c + ip * z
        n = fp * n + ip
        m = mm
        h = o * c / n
        outs.append(h)
    return torch.stack(outs, 1), (c, n, m, h)


def _dense_from_blocks(wbd, NH, dh):
    H = NH * dh
    w = np.zeros((H, 4 * H))
    for hd in range(NH):
        for gt in range(4):
            w[hd * dh:(hd + 1) * dh, gt * H + hd * dh: gt * H + (hd + 1) * dh] = wbd[hd, :, gt * dh:(gt + 1) * dh]
    return w


@pytest.mark.parametrize("B,H,T", [(2, 6, 5), (2, 12, 40)])
def test_slstm_matches_autograd(B, H, T):
    r = np.random.default_rng(0)
    wh = r.standard_normal((H, 4 * H)) / np.sqrt(H)
    g = r.standard_normal((B, T, 4 * H))
    bcat = np.concatenate([np.zeros(2 * H), np.full(H, 4.5), np.zeros(H)]) * 0.2
    dy = r.standard_normal((B, T, H))
    fw = O.slstm_fw(wh, g, bcat, B, H, 1, T)
    bw = O.slstm_bw(wh, dy, fw, B, H, 1, T)
    tw = torch.tensor(wh); tb = torch.tensor(bcat)
    tg = torch.tensor(g, requires_grad=True)
    out, st = _torch_slstm(tw, tg, tb, B, H, T)
    np.testing.assert_allclose(fw["out"], out.detach().numpy(), rtol=1e-10, atol=1e-12)
    (out * torch.tensor(dy)).sum().backward()
    # the gate deltas ARE dL/dg (g enters the pre-activations additively)
    np.testing.assert_allclose(bw["dg"], tg.grad.numpy(), rtol=1e-8, atol=1e-10)


def test_slstm_block_diagonal_equals_masked_dense():
    B, NH, dh, T = 3, 4, 8, 17
    H = NH * dh
    r = np.random.default_rng(1)
    wbd = r.standard_normal((NH, dh, 4 * dh)) / np.sqrt(dh)
    wd = _dense_from_blocks(wbd, NH, dh)
    g = r.standard_normal((B, T, 4 * H)); bcat = r.standard_normal(4 * H) * 0.1
    dy = r.standard_normal((B, T, H))
    a = O.slstm_fw(wbd, g, bcat, B, H, NH, T); b = O.slstm_fw(wd, g, bcat, B, H, 1, T)
    np.testing.assert_allclose(a["out"], b["out"], rtol=1e-11, atol=1e-13)
    ga = O.slstm_bw(wbd, dy, a, B, H, NH, T); gb = O.slstm_bw(wd, dy, b, B, H, 1, T)
    np.testing.assert_allclose(ga["dg"], gb["dg"], rtol=1e-10, atol=1e-12)


def test_slstm_carry_matches_whole():
    B, H, T = 1, 12, 128
    r = np.random.default_rng(2)
    wh = r.standard_normal((H, 4 * H)) / np.sqrt(H)
    g = r.standard_normal((B, T, 4 * H)); bcat = np.zeros(4 * H); dy = r.standard_normal((B, T, H))
    whole = O.slstm_fw(wh, g, bcat, B, H, 1, T)
    wb = O.slstm_bw(wh, dy, whole, B, H, 1, T)
    cuts = [(0, 48), (48, 96), (96, 128)]
    st = None; parts = []
    for s, e in cuts:
        f = O.slstm_fw(wh, g[:, s:e], bcat, B, H, 1, e - s, state=st)
        st = f["state"]; parts.append(f)
    np.testing.assert_allclose(np.concatenate([p["out"] for p in parts], 1), whole["out"], rtol=1e-11, atol=1e-13)
    dst = None; dgs = []
    for (s, e), f in reversed(list(zip(cuts, parts))):
        b_ = O.slstm_bw(wh, dy[:, s:e], f, B, H, 1, e - s, dstate=dst)
        dst = b_["dstate"]; dgs.append(b_["dg"])
    np.testing.assert_allclose(np.concatenate(dgs[::-1], 1), wb["dg"], rtol=1e-9, atol=1e-11)


@pytest.mark.parametrize("rows,F,group", [(7, 32, 32), (5, 12, 4), (3, 64, 16)])
def test_rmsnorm_matches_autograd(rows, F, group):
    r = np.random.default_rng(3)
    x = r.standard_normal((rows, F)); gamma = r.standard_normal(F); dy = r.standard_normal((rows, F))
    y, xh, inv = O.rmsnorm_fw(x, gamma, group)
    dx, dgam = O.rmsnorm_bw(dy, xh, inv, gamma, group)
    tx = torch.tensor(x, requires_grad=True); tg = torch.tensor(gamma, requires_grad=True)
    xg = tx.view(rows, F // group, group)
    ty = (xg * torch.rsqrt((xg * xg).mean(-1, keepdim=True) + 1e-6)).view(rows, F) * tg
    np.testing.assert_allclose(y, ty.detach().numpy(), rtol=1e-12, atol=1e-13)
    (ty * torch.tensor(dy)).sum().backward()
    np.testing.assert_allclose(dx, tx.grad.numpy(), rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dgam, tg.grad.numpy(), rtol=1e-9, atol=1e-11)


def test_softmax_ce_matches_torch_and_mask():
    r = np.random.default_rng(4)
    rows, C = 9, 13
    z = r.standard_normal((rows, C)) * 3; t = r.integers(0, C, rows)
    loss, d = O.softmax_ce(z, t)
    tz = torch.tensor(z, requires_grad=True)
    tl = torch.nn.functional.cross_entropy(tz, torch.tensor(t))
    tl.backward()
    assert abs(loss - tl.item()) < 1e-12
    np.testing.assert_allclose(d, tz.grad.numpy(), rtol=1e-10, atol=1e-13)
    mask = (r.random(rows) > 0.4).astype(np.uint32); mask[0] = 1
    inv = 1.0 / mask.sum()
    loss_m, dm = O.softmax_ce(z, t, mask=mask, inv=inv)
    tz2 = torch.tensor(z, requires_grad=True)
    per = torch.nn.functional.cross_entropy(tz2, torch.tensor(t), reduction="none")
    lm = (per * torch.tensor(mask.astype(np.float64))).sum() * inv
    lm.backward()
    assert abs(loss_m - lm.item()) < 1e-12
    np.testing.assert_allclose(dm, tz2.grad.numpy(), rtol=1e-10, atol=1e-13)


@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_adamw_matches_torch(wd):
    r = np.random.default_rng(5)
    p0 = r.standard_normal(20)
    tp = torch.tensor(p0.copy(), requires_grad=True)
    opt = torch.optim.AdamW([tp], lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=wd)
    p, m, v = p0.copy(), np.zeros(20), np.zeros(20)
    for t in range(1, 4):
        g = r.standard_normal(20)
        tp.grad = torch.tensor(g.copy()); opt.step()
        p, m, v = O.adamw(p, g, m, v, 1e-3, wd, t)
    np.testing.assert_allclose(p, tp.detach().numpy(), rtol=1e-12, atol=1e-14)


def test_gemm_forms():
    r = np.random.default_rng(6)
    a = r.standard_normal((7, 5)); b = r.standard_normal((5, 9))
    np.testing.assert_allclose(O.gemm("nn", a, b), a @ b, rtol=1e-12)
    np.testing.assert_allclose(O.gemm("tn", a.T.copy(), b), a @ b, rtol=1e-12)
    np.testing.assert_allclose(O.gemm("nt", a, b.T.copy()), a @ b, rtol=1e-12)
