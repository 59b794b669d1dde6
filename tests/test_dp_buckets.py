"""Host logic of the data-parallel gradient buckets on CPU: two gloo ranks, each with its own
gradients; after the overlapped all-reduce every rank holds the sum, the parameters' `.g` are views
of the flat buckets, and a one-rank run is a no-op."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import importlib
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class P:
    def __init__(self, shape, val):
        self.w = torch.zeros(shape)
        self.g = torch.full(shape, float(val))


def _worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    spec = importlib.util.spec_from_file_location("dp", os.path.join(ROOT, "neural-networks_b200", "dp.py"))
    dp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dp)
    groups = [[P((3, 4), rank + 1), P((5,), 10 * (rank + 1))], [P((2, 2), -(rank + 1))], []]
    b = dp.GradBuckets(groups)
    for i in (1, 0, 2):  # reverse-layer order, as backward produces them
        b.reduce_async(i)
    b.wait()
    tot = sum(range(1, world + 1))
    assert torch.all(groups[0][0].g == tot) and torch.all(groups[0][1].g == 10 * tot) and torch.all(groups[1][0].g == -tot)
    assert groups[0][0].g.data_ptr() == b.flat[0].data_ptr()  # a view of the bucket, not a copy
    groups[0][1].g.add_(1.0)
    assert torch.all(b.flat[0][12:] == 10 * tot + 1)
    dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_rank_gloo_bucket_allreduce():
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_single_process_is_noop():
    spec = importlib.util.spec_from_file_location("dp", os.path.join(ROOT, "neural-networks_b200", "dp.py"))
    dp = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(dp)
    g = [[P((4,), 3.0)]]
    b = dp.GradBuckets(g)
    b.reduce_async(0)
    b.wait()
    assert torch.all(g[0][0].g == 3.0)


def test_all_reduces_gather_at_the_slstm_time_loops():
    """`attach` on a model with sLSTM blocks: a block's all-reduce is held until the next sLSTM backward time loop is
    launched (or the pass ends); without sLSTM blocks every block starts its own at once."""
    sys.path.insert(0, ROOT)
    dp = importlib.import_module("neural-networks_b200.dp")
    layers = importlib.import_module("neural-networks_b200.layers")

    class Rec:
        def __init__(self, groups, group=None):
            self.started, self.n = [], len(groups)

        def reduce_async(self, i):
            self.started.append(i)

    class Blk:
        def __init__(self, cell):
            self.cell = cell

        def params(self):
            return []

    class Norm:
        def params(self):
            return []

    class FakeLm:
        def __init__(self, kinds):
            self.blocks = [Blk(object.__new__(layers.SLstm) if k == "s" else object()) for k in kinds]
            for b in self.blocks:
                if isinstance(b.cell, layers.SLstm):
                    b.cell.before_time_loop = None
            self.table, self.norm, self.head, self.on_block_backward = object(), Norm(), None, None

    def backward(lm, buckets):
        log = []
        for i in range(len(lm.blocks) - 1, -1, -1):
            cell = lm.blocks[i].cell
            if isinstance(cell, layers.SLstm) and cell.before_time_loop is not None:
                cell.before_time_loop()
                log.append(("loop %d" % i, list(buckets.started)))
            lm.on_block_backward(i)
        getattr(buckets, "reduce_async_deferred", buckets.reduce_async)(len(lm.blocks))
        return log

    real = dp.GradBuckets
    dp.GradBuckets = Rec
    try:
        lm = FakeLm("smmsmm")
        b = dp.attach(lm)
        log = backward(lm, b)
        # at block 3's loop: blocks 5, 4 start; at block 0's loop: 3, 2, 1; then 0 and the table's bucket
        assert log == [("loop 3", [5, 4]), ("loop 0", [5, 4, 3, 2, 1])], log
        assert b.started == [5, 4, 3, 2, 1, 0, 6]
        lm = FakeLm("mmsm")  # the bottom block is not an sLSTM block: what is pending goes out with block 0
        b = dp.attach(lm)
        log = backward(lm, b)
        assert log == [("loop 2", [3])] and b.started == [3, 2, 1, 0, 4], (log, b.started)
        lm = FakeLm("mmm")
        b = dp.attach(lm)
        assert backward(lm, b) == [] and b.started == [2, 1, 0, 3]
        lm = FakeLm("smm")
        b = dp.attach(lm, gather_at_slstm=False)
        backward(lm, b)
        assert b.started == [2, 1, 0, 3] and lm.blocks[0].cell.before_time_loop is None
    finally:
        dp.GradBuckets = real
