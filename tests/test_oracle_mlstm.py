"""The oracle's mLSTM core checked three ways, mirroring how the reference pins its own
CPU layer (src/nn2/mlstm.rs:910-971 directional finite differences; chunk-length
invariance src/gpu/mlstm.rs:1062-1191; carry == whole sequence :1337-1533), plus an
independent autograd cross-check in float64 with the stabiliser m detached."""
import numpy as np
import pytest
import torch

from oracle import oracle as O


def _inputs(B, H, T, dqk, dhv, seed, fbias=3.0):
    r = np.random.default_rng(seed)
    q = r.standard_normal((B * T, H * dqk))
    k = r.standard_normal((B * T, H * dqk)) / np.sqrt(dqk)
    v = r.standard_normal((B * T, H * dhv))
    ig = r.standard_normal((B * T, H))
    fg = r.standard_normal((B * T, H)) + fbias
    return q, k, v, ig, fg


def _torch_core(q, k, v, ig, fg, B, H, T, dqk, dhv, C0=None, n0=None, m0=None):
    """Recurrent form in torch float64; m is computed without grad."""
    q = q.view(B, T, H, dqk); k = k.view(B, T, H, dqk); v = v.view(B, T, H, dhv)
    ig = ig.view(B, T, H); fg = fg.view(B, T, H)
    lf = torch.nn.functional.logsigmoid(fg)
    C = torch.zeros(B, H, dhv, dqk, dtype=q.dtype) if C0 is None else C0.view(B, H, dhv, dqk)
    n = torch.zeros(B, H, dqk, dtype=q.dtype) if n0 is None else n0.view(B, H, dqk)
    m = torch.zeros(B, H, dtype=q.dtype) if m0 is None else m0.view(B, H)
    ys = []
    for t in range(T):
        with torch.no_grad():
            mh = torch.maximum(lf[:, t] + m, ig[:, t])
        ip = torch.exp(ig[:, t] - mh)
        fp = torch.exp(lf[:, t] + m - mh)
        m = mh
        n = fp[..., None] * n + ip[..., None] * k[:, t]
        C = fp[..., None, None] * C + ip[..., None, None] * (v[:, t][..., :, None] * k[:, t][..., None, :])
        nq = (n * q[:, t]).sum(-1)
        psi = torch.maximum(nq.abs(), torch.exp(-mh))
        ys.append((C @ q[:, t][..., None]).squeeze(-1) / psi[..., None])
    y = torch.stack(ys, 1)  # B,T,H,dhv
    return y.reshape(B * T, H * dhv), C, n, m


@pytest.mark.parametrize("shape", [(2, 2, 20, 4, 4), (1, 3, 37, 8, 16), (2, 1, 70, 16, 8)])
def test_recurrent_matches_autograd(shape):
    B, H, T, dqk, dhv = shape
    q, k, v, ig, fg = _inputs(*shape, seed=1)
    r = np.random.default_rng(2)
    dy = r.standard_normal((B * T, H * dhv))
    fw = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv)
    bw = O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, dqk, dhv)
    tq, tk, tv, ti, tf = (torch.tensor(a, dtype=torch.float64, requires_grad=True)
                          for a in (q, k, v, ig, fg))
    y, C, n, m = _torch_core(tq, tk, tv, ti, tf, B, H, T, dqk, dhv)
    np.testing.assert_allclose(fw["ytil"], y.detach().numpy(), rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(fw["C"].reshape(B, H, dhv, dqk), C.detach().numpy(), rtol=1e-10, atol=1e-12)
    (y * torch.tensor(dy)).sum().backward()
    for name, t in (("dq", tq), ("dk", tk), ("dv", tv), ("dig", ti), ("dfg", tf)):
        np.testing.assert_allclose(bw[name], t.grad.numpy(), rtol=1e-8, atol=1e-10, err_msg=name)


def test_carry_matches_whole_and_state_grads():
    B, H, T, dqk, dhv = 2, 2, 24, 8, 8
    q, k, v, ig, fg = _inputs(B, H, T, dqk, dhv, seed=3)
    r = np.random.default_rng(4)
    dy = r.standard_normal((B * T, H * dhv))
    whole_f = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv)
    whole_b = O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, dqk, dhv)

    def part(a, W, s, e):
        return np.ascontiguousarray(a.reshape(B, T, H * W)[:, s:e].reshape(B * (e - s), H * W))

    cuts = [(0, 10), (10, 17), (17, 24)]
    st = (None, None, None)
    saved = []
    ys = np.zeros((B, T, H * dhv))
    for s, e in cuts:
        args = (part(q, dqk, s, e), part(k, dqk, s, e), part(v, dhv, s, e), part(ig, 1, s, e), part(fg, 1, s, e))
        f = O.mlstm_core_fw(*args, B, H, e - s, dqk, dhv, C0=st[0], n0=st[1], m0=st[2])
        saved.append((args, st))
        ys[:, s:e] = f["ytil"].reshape(B, e - s, H * dhv)
        st = (f["C"], f["n"], f["mlast"])
    np.testing.assert_allclose(ys.reshape(B * T, -1), whole_f["ytil"], rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(st[0], whole_f["C"], rtol=1e-11, atol=1e-13)
    dst = (None, None)
    dq = np.zeros((B, T, H * dqk))
    dfg = np.zeros((B, T, H))
    for (s, e), (args, st0) in reversed(list(zip(cuts, saved))):
        b_ = O.mlstm_core_bw(*args, part(dy, dhv, s, e), B, H, e - s, dqk, dhv, C0=st0[0], n0=st0[1],
                             m0=st0[2], dC_in=dst[0], dn_in=dst[1])
        dq[:, s:e] = b_["dq"].reshape(B, e - s, -1)
        dfg[:, s:e] = b_["dfg"].reshape(B, e - s, -1)
        dst = (b_["dC"], b_["dn"])
    np.testing.assert_allclose(dq.reshape(B * T, -1), whole_b["dq"], rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(dfg.reshape(B * T, -1), whole_b["dfg"], rtol=1e-9, atol=1e-11)


@pytest.mark.parametrize("L", [1, 3, 8, 16, 32, 64, 200])
def test_chunkwise_equals_recurrent(L):
    B, H, T, dqk, dhv = 2, 2, 70, 8, 12
    q, k, v, ig, fg = _inputs(B, H, T, dqk, dhv, seed=5)
    rec = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv)
    ch = O.mlstm_chunkwise_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, L)
    np.testing.assert_allclose(ch["ytil"], rec["ytil"], rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(ch["m"], rec["m"], rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(ch["psi"], rec["psi"], rtol=1e-9, atol=1e-12)
    np.testing.assert_allclose(ch["Cst"][:, -1], rec["C"], rtol=1e-9, atol=1e-12)


def test_directional_finite_difference_f32():
    """The reference's own check on its CPU layer: step along the normalised analytic
    gradient, require |fd - ||G||| <= 0.3 ||G|| + 1e-3 (src/nn2/mlstm.rs:910-971)."""
    B, H, T, dqk, dhv = 2, 2, 6, 4, 4
    q, k, v, ig, fg = _inputs(B, H, T, dqk, dhv, seed=6, fbias=1.0)
    r = np.random.default_rng(7)
    w = r.standard_normal((B * T, H * dhv))

    def loss(q_, k_, v_, i_, f_):
        return float((O.mlstm_core_fw(q_, k_, v_, i_, f_, B, H, T, dqk, dhv, dtype=np.float32)["ytil"].astype(np.float64) * w).sum())

    g = O.mlstm_core_bw(q, k, v, ig, fg, w, B, H, T, dqk, dhv, dtype=np.float32)
    grads = [g["dq"], g["dk"], g["dv"], g["dig"], g["dfg"]]
    norm = np.sqrt(sum(float((x.astype(np.float64) ** 2).sum()) for x in grads))
    eps = 1e-2
    plus = [a + eps * x / norm for a, x in zip((q, k, v, ig, fg), grads)]
    minus = [a - eps * x / norm for a, x in zip((q, k, v, ig, fg), grads)]
    fd = (loss(*plus) - loss(*minus)) / (2 * eps)
    assert abs(fd - norm) <= 0.3 * norm + 1e-3, (fd, norm)


def test_f32_tracks_f64():
    B, H, T, dqk, dhv = 2, 2, 64, 16, 16
    q, k, v, ig, fg = _inputs(B, H, T, dqk, dhv, seed=8)
    a = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, dtype=np.float32)
    b = O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, dtype=np.float64)
    assert np.abs(a["ytil"] - b["ytil"]).max() <= 1e-4 * np.abs(b["ytil"]).max()


def test_random_seeded_range_and_determinism():
    a = O.random_seeded((1000,), 0.5, 0xA1)
    b = O.random_seeded((1000,), 0.5, 0xA1)
    assert (a == b).all() and a.min() >= -0.5 and a.max() < 0.5 and abs(a.mean()) < 0.05
    assert (O.random_seeded((10,), 0.5, 0xA2) != a[:10]).any()
