"""The oracle's layer stack (cells, block, flat LM) checked the way the reference checks its CPU
model: a directional finite-difference test of the whole backward (src/nn2/block.rs:266-327,
src/nn2/mlstm.rs:910-971) and "one AdamW step lowers the loss" (src/nn2/mod.rs:36-153)."""
import numpy as np
import pytest

from oracle import model as M
from oracle import oracle as O


def _lm(seed, slstm_at=(), nh_s=1, tied=True):
    rng = np.random.default_rng(seed)
    vocab, d, heads, dqk, dhv, up = 13, 8, 2, 4, 4, 12
    p = M.init_lm_params(rng, vocab, d, 2, heads, dqk, dhv, up, std=0.3, slstm_at=slstm_at, nh_s=nh_s)
    hw = hb = None
    if not tied:
        hw, hb = rng.standard_normal((d, vocab)) * 0.3, rng.standard_normal(vocab) * 0.1
    return M.build_lm(p, heads, dqk, dhv, nh_s=nh_s, tied=tied, head_w=hw, head_b=hb), vocab


@pytest.mark.parametrize("slstm_at,nh_s,tied", [((), 1, True), ((0,), 1, False), ((1,), 2, True)])
def test_lm_backward_matches_directional_finite_difference(slstm_at, nh_s, tied):
    lm, vocab = _lm(0, slstm_at, nh_s, tied)
    rng = np.random.default_rng(1)
    B, T = 2, 6
    ids = rng.integers(0, vocab, B * T); tg = rng.integers(0, vocab, B * T)

    def loss():
        return O.softmax_ce(lm.forward(ids, B, T), tg)[0]

    l0, d = O.softmax_ce(lm.forward(ids, B, T), tg)
    lm.backward(d)
    ps = lm.params()
    grads = [p.g.copy() for p in ps]
    norm = np.sqrt(sum((g * g).sum() for g in grads))
    eps = 1e-5
    base = [p.w.copy() for p in ps]
    for p, w0, g in zip(ps, base, grads):
        p.w = w0 + eps * g / norm
    lp = loss()
    for p, w0, g in zip(ps, base, grads):
        p.w = w0 - eps * g / norm
    lm_ = loss()
    fd = (lp - lm_) / (2 * eps)
    assert abs(fd - norm) <= 1e-4 * norm + 1e-7, (fd, norm)


def test_lm_step_lowers_loss():
    lm, vocab = _lm(2)
    rng = np.random.default_rng(3)
    B, T = 2, 8
    ids = rng.integers(0, vocab, B * T); tg = rng.integers(0, vocab, B * T)
    l0, _ = lm.train_step(ids, tg, B, T, 1e-2, 0.1, 1)
    l1 = O.softmax_ce(lm.forward(ids, B, T), tg)[0]
    assert l1 < l0
