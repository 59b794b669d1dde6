"""Inference on the training kernels: greedy decoding with stateful (carried) cells gives exactly the token ids
the CPU oracle stack gives when it re-runs the whole sequence from scratch for every new token (the
reference's carry == whole property, src/gpu/mlstm.rs:1337-1533, src/gpu/slstm.rs:1843-1938, taken to the
model level), and head-sharded mLSTM blocks on 2 GPUs reproduce the unsharded model."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch

from oracle import model as M

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _params(seed, vocab, d, nb, heads, dqk, dhv, up, slstm_at=(), nh_s=1, std=0.2):
    return M.init_lm_params(np.random.default_rng(seed), vocab, d, nb, heads, dqk, dhv, up, std=std, slstm_at=slstm_at, nh_s=nh_s)


def _oracle_greedy(p, heads, dqk, dhv, nh_s, prompt, n_new):
    ids = prompt.copy()
    B = ids.shape[0]
    picked, seen = [], []
    for _ in range(n_new):
        T = ids.shape[1]
        ref = M.build_lm(p, heads, dqk, dhv, nh_s=nh_s, tied=True)
        logits = ref.forward(ids.reshape(-1), B, T).reshape(B, T, -1)[:, -1, :]
        seen.append(logits)
        nxt = logits.argmax(axis=1)
        picked.append(nxt)
        ids = np.concatenate([ids, nxt[:, None]], axis=1)
    return np.stack(picked, axis=1), np.stack(seen, axis=0)


@pytest.mark.parametrize("slstm_at,nh_s", [((), 1), ((1,), 2)])
def test_greedy_decoding_gives_the_oracles_token_ids(slstm_at, nh_s):
    layers = importlib.import_module("neural-networks_b200.layers")
    infer = importlib.import_module("neural-networks_b200.infer")
    vocab, d, nb, heads, dqk, dhv, up, B, Tp, n_new = 61, 32, 2, 2, 16, 16, 88, 3, 7, 9
    p = _params(11, vocab, d, nb, heads, dqk, dhv, up, slstm_at, nh_s)
    prompt = np.random.default_rng(5).integers(0, vocab, (B, Tp))
    want_ids, want_logits = _oracle_greedy(p, heads, dqk, dhv, nh_s, prompt, n_new)
    lm = layers.build_lm(p, heads, dqk, dhv, nh_s=nh_s, tied=True)
    got_ids, got_logits = infer.greedy_decode(lm, torch.tensor(prompt, device="cuda"), n_new)
    torch.cuda.synchronize()
    gl = got_logits.cpu().numpy().astype(np.float64)
    assert np.abs(gl - want_logits).max() <= 1e-4 * np.abs(want_logits).max()
    assert np.array_equal(got_ids.cpu().numpy(), want_ids)


def test_stateful_calls_continue_a_sequence_on_the_tensor_core_path():
    """bf16 storage, heads of 128: last-position logits after (prefill 100, then 3 x 1 position) against one
    stateless call over all 103 positions."""
    layers = importlib.import_module("neural-networks_b200.layers")
    infer = importlib.import_module("neural-networks_b200.infer")
    vocab, d, nb, heads, dqk, dhv, up, B = 64, 256, 2, 2, 128, 128, 680, 2
    p = _params(12, vocab, d, nb, heads, dqk, dhv, up, std=0.05)
    ids = torch.tensor(np.random.default_rng(6).integers(0, vocab, (B, 103)), device="cuda")
    lm = layers.build_lm(p, heads, dqk, dhv, tied=True, bf16=True)
    whole = infer.last_logits(lm, ids.reshape(-1), B, 103)
    infer.set_stateful(lm, True)
    infer.last_logits(lm, ids[:, :100].reshape(-1), B, 100)
    for t in range(100, 103):
        step = infer.last_logits(lm, ids[:, t].contiguous(), B, 1)
    infer.set_stateful(lm, False)
    torch.cuda.synchronize()
    xl = importlib.import_module("neural-networks_b200")
    assert xl._lib.lib.xlstm_device_status() == 0
    assert float((step - whole).abs().max()) <= 2e-2 * float(whole.abs().max())


CFG = dict(vocab=61, d=64, nb=2, heads=4, dqk=16, dhv=16, up=176, B=2, Tp=9, n_new=6)


def _shard_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    infer = importlib.import_module("neural-networks_b200.infer")
    c = CFG
    p = _params(13, c["vocab"], c["d"], c["nb"], c["heads"], c["dqk"], c["dhv"], c["up"], slstm_at=(1,), nh_s=2)
    lm = infer.build_lm_head_sharded(p, c["heads"], c["dqk"], c["dhv"], rank, world, nh_s=2, tied=True)
    prompt = torch.tensor(np.random.default_rng(8).integers(0, c["vocab"], (c["B"], c["Tp"])), device="cuda")
    ids, logits = infer.greedy_decode(lm, prompt, c["n_new"])
    torch.cuda.synchronize()
    if rank == 0:
        torch.save((ids.cpu(), logits.cpu()), out)
    dist.barrier()
    dist.destroy_process_group()


def test_head_sharded_mlstm_inference_on_two_gpus(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    layers = importlib.import_module("neural-networks_b200.layers")
    infer = importlib.import_module("neural-networks_b200.infer")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "ids.pt")
    mp.spawn(_shard_worker, args=(2, port, out), nprocs=2, join=True)
    got_ids, got_logits = torch.load(out)
    c = CFG
    p = _params(13, c["vocab"], c["d"], c["nb"], c["heads"], c["dqk"], c["dhv"], c["up"], slstm_at=(1,), nh_s=2)
    lm = layers.build_lm(p, c["heads"], c["dqk"], c["dhv"], nh_s=2, tied=True)
    prompt = torch.tensor(np.random.default_rng(8).integers(0, c["vocab"], (c["B"], c["Tp"])), device="cuda")
    ids, logits = infer.greedy_decode(lm, prompt, c["n_new"])
    assert float((got_logits - logits.cpu()).abs().max()) <= 1e-4 * float(logits.abs().max())
    assert torch.equal(got_ids, ids.cpu())
