"""Host-side logic of context parallelism (no GPU): folding segment summaries reproduces the step-by-step
stabilised recurrence, and the exchange returns the ranks' tensors in rank order (2 gloo ranks)."""
import importlib
import os
import socket

import numpy as np
import torch

cp = importlib.import_module("neural-networks_b200.cp")


class _Shape:
    def __init__(self, b, h, dqk, dhv):
        self.b, self.h, self.dqk, self.dhv = b, h, dqk, dhv

    def bh(self):
        return self.b * self.h


def _recurrence(C, n, m, ig, fg, k, v):
    """The reference's stabilised step (src/nn2/mlstm.rs:483-541) for one (batch, head), float64."""
    for t in range(len(ig)):
        lf = -np.log1p(np.exp(-fg[t]))
        m2 = max(lf + m, ig[t])
        i_, f_ = np.exp(ig[t] - m2), np.exp(lf + m - m2)
        C, n, m = f_ * C + i_ * np.outer(v[t], k[t]), f_ * n + i_ * k[t], m2
    return C, n, m


def test_fold_of_segment_summaries_is_the_sequential_recurrence():
    r = np.random.default_rng(0)
    W, Ts, dqk, dhv = 4, 5, 3, 2
    for fbias in (3.0, -3.0):  # weak and strong forgetting: both branches of the max
        ig, fg = r.standard_normal((W, Ts)) * 2, r.standard_normal((W, Ts)) + fbias
        k, v = r.standard_normal((W, Ts, dqk)), r.standard_normal((W, Ts, dhv))
        sums = []
        for s in range(W):
            Cs, ns, Ms = _recurrence(np.zeros((dhv, dqk)), np.zeros(dqk), -1e30, ig[s], fg[s], k[s], v[s])
            F = float(np.sum(-np.log1p(np.exp(-fg[s]))))
            sums.append(torch.tensor(np.concatenate([Cs.reshape(-1), ns, [Ms, F]])[None, :], dtype=torch.float32))
        C, n, m = np.zeros((dhv, dqk)), np.zeros(dqk), 0.0
        assert cp.fold(sums, 0, _Shape(1, 1, dqk, dhv)) is None
        for rank in range(1, W + 1):
            C, n, m = _recurrence(C, n, m, ig[rank - 1], fg[rank - 1], k[rank - 1], v[rank - 1])
            if rank == W:
                break
            fC, fn, fm = cp.fold(sums, rank, _Shape(1, 1, dqk, dhv))
            assert abs(float(fm[0]) - m) <= 1e-5 * max(1.0, abs(m))
            assert np.allclose(fC[0].numpy(), C, rtol=1e-4, atol=1e-6) and np.allclose(fn[0].numpy(), n, rtol=1e-4, atol=1e-6)


def _rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    got = cp.dist_gather()(torch.full((2, 3), float(rank + 1)))
    torch.save([g.clone() for g in got], "%s.%d" % (out, rank))
    dist.destroy_process_group()


def test_exchange_returns_rank_order(tmp_path):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "g")
    mp.spawn(_rank, args=(2, port, out), nprocs=2, join=True)
    for r in range(2):
        got = torch.load("%s.%d" % (out, r), weights_only=False)
        assert [float(g[0, 0]) for g in got] == [1.0, 2.0]
