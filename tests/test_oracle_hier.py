"""The oracle of the hierarchical window checks itself (no GPU): its hand-written backward against central
differences of its own loss, in the manner of the reference's finite-difference tests of every nn2 layer
(src/nn2/mlstm.rs:910-971), and the loss normalisation / masking rules of src/gpu/hierarchical.rs:1051-1060."""
import numpy as np

from oracle import hier as H


def _window(seed, lens, vocab=12):
    r = np.random.default_rng(seed)
    toks = r.integers(0, vocab - 1, sum(lens)).tolist()
    words, s = [], 0
    for l in lens:
        words.append((s, s + l))
        s += l
    return toks, words


def _model(seed=0):
    cfg = H.HierCfg(vocab=12, hc=8, wh=12, enc_blocks=2, bb_blocks=2, dec_blocks=2, heads=2, dqk=3, w_token=11, small_heads=2)
    return cfg, H.Hierarchical(H.init_hier_params(np.random.default_rng(seed), cfg, std=0.3), cfg)


WINS = [_window(1, [2, 3, 1, 4]), _window(2, [1, 2, 5, 2])]


def test_backward_matches_central_differences():
    cfg, m = _model()
    m.forward_backward(WINS)
    ps = m.params()
    grads = [p.g.copy() for p in ps]
    r = np.random.default_rng(3)
    for pi in r.choice(len(ps), 12, replace=False):
        P = ps[pi]
        idx = tuple(int(r.integers(0, s)) for s in P.w.shape)
        old, e = P.w[idx], 1e-5
        P.w[idx] = old + e
        lp = m.forward_backward(WINS)
        P.w[idx] = old - e
        lm = m.forward_backward(WINS)
        P.w[idx] = old
        fd, g = (lp - lm) / (2 * e), grads[pi][idx]
        assert abs(fd - g) <= 1e-5 * max(abs(fd), abs(g)) + 1e-9, (pi, P.w.shape, fd, g)


def test_rows_counted_and_masked_words_carry_no_gradient():
    cfg, m = _model(1)
    loss = m.forward_backward(WINS)
    # decoded words: 3 per window, each (length + 1) rows: (3+1)+(1+1)+(4+1) + (2+1)+(5+1)+(2+1)
    assert m.last_rows == 11 + 12 and loss > 0
    # all words masked out: no rows, no loss, no gradient anywhere
    cfg, m2 = _model(1)
    off = [[False] * 3, [False] * 3]
    assert m2.forward_backward(WINS, off) == 0.0 and m2.last_rows == 0
    assert all(not p.g.any() for p in m2.params())
    # masking the second window's words leaves exactly the first window's loss
    cfg, a = _model(1)
    cfg, b = _model(1)
    la = a.forward_backward(WINS, [[True] * 3, [False] * 3])
    lb = b.forward_backward(WINS[:1])
    assert abs(la - lb) <= 1e-12 * abs(lb)
