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
