"""Context parallelism of the mLSTM core: a sequence cut into W segments, each run as its own call with the
carry folded from the segments to its left and the BPTT state summed from the segments to its right, equals the
whole-sequence result of the oracle. The W ranks are emulated one after the other on one GPU (the exchange is a
list); the same functions run over NCCL in the two-GPU case below. Bars: 1e-4 (fp32 storage), 2e-2 (bf16)."""
import importlib
import os
import socket

import numpy as np
import pytest
import torch

from oracle import oracle as O

pytestmark = pytest.mark.gpu

NAMES = ("ytil", "dq", "dk", "dv", "dig", "dfg")


def _segments(a, B, T, W):
    """[B*T, w] -> W arrays [B*(T/W), w], rank r holding positions r*T/W .. of every sequence."""
    x = a.reshape(B, W, T // W, -1)
    return [np.ascontiguousarray(x[:, r]).reshape(B * (T // W), -1) for r in range(W)]


def _join(parts, B, T, W):
    return np.stack([p.reshape(B, T // W, -1) for p in parts], axis=1).reshape(B * T, -1)


def _emulate(shape, L, dtype, W, seed, fbias=3.0):
    from gpu_util import ops, dev, host, mlstm_inputs
    cp = importlib.import_module("neural-networks_b200.cp")
    B, H, T, dqk, dhv = shape
    q, k, v, ig, fg, dy = mlstm_inputs(*shape, seed=seed, fbias=fbias, bf16=dtype == torch.bfloat16)
    seg = [[dev(s, dt) for s in _segments(a, B, T, W)] for a, dt in
           ((q, dtype), (k, dtype), (v, dtype), (ig, torch.float32), (fg, torch.float32), (dy, torch.float32))]
    st = ops.MlstmShape(B, H, T // W, dqk, dhv, L, dtype, torch.float32)
    per = lambda r: [s[r] for s in seg]
    # exchange 1: every rank's summary
    sums = [cp.segment_summary(*per(r)[:5], st) for r in range(W)]
    fw = [cp.forward(*per(r)[:5], st, r, lambda t: sums) for r in range(W)]
    # exchange 2: a first round only records what each rank would send, the second round runs with all of it
    sent = []
    for r in range(W):
        cp.backward(fw[r][0], *per(r)[:5], per(r)[5], st, fw[r][1], r, W, lambda t: sent.append(t) or [t] * W)
    assert len(sent) == W
    bw = [cp.backward(fw[r][0], *per(r)[:5], per(r)[5], st, fw[r][1], r, W, lambda t: sent) for r in range(W)]
    torch.cuda.synchronize()
    got = dict(ytil=_join([host(f[0].ytil) for f in fw], B, T, W))
    for i, n in enumerate(NAMES[1:]):
        got[n] = _join([host(g[i]) for g in bw], B, T, W)
    got["state"] = [host(t) for t in fw[-1][0].state]
    ref = dict(O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, C0=None, n0=None, m0=None))
    ref.update(O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, dqk, dhv, C0=None, n0=None, m0=None, dC_in=None, dn_in=None))
    return got, ref


@pytest.mark.parametrize("shape,L,W,fbias", [((2, 2, 96, 8, 12), 16, 3, 3.0), ((1, 3, 64, 16, 16), 64, 4, 3.0),
                                            ((2, 2, 60, 8, 8), 8, 2, -2.0)])
def test_fp32_segments_equal_the_whole_sequence(shape, L, W, fbias):
    """fbias = -2: strong forgetting, where the carried stabiliser drops below the segment's own and the fold's
    max() picks the other branch."""
    from gpu_util import rel_to_max, xl
    got, ref = _emulate(shape, L, torch.float32, W, seed=41, fbias=fbias)
    assert xl._lib.lib.xlstm_device_status() == 0
    for n in NAMES:
        assert rel_to_max(got[n], ref[n]) <= 1e-4, n
    for a, b in zip(got["state"], (ref["C"], ref["n"], ref["mlast"])):
        assert rel_to_max(a, b) <= 1e-4  # the last rank ends in the whole sequence's final (C, n, m)


def test_bf16_tensor_core_segments_equal_the_whole_sequence():
    from gpu_util import rel_to_max, xl
    got, ref = _emulate((2, 2, 384, 128, 128), 64, torch.bfloat16, 3, seed=42)
    assert xl._lib.lib.xlstm_device_status() == 0
    for n in NAMES:
        assert rel_to_max(got[n], ref[n]) <= 2e-2, n


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from gpu_util import ops, dev, host, mlstm_inputs
    cp = importlib.import_module("neural-networks_b200.cp")
    B, H, T, d = 2, 2, 256, 128
    q, k, v, ig, fg, dy = mlstm_inputs(B, H, T, d, d, seed=43, bf16=True)
    mine = [dev(_segments(a, B, T, world)[rank], dt) for a, dt in
            ((q, torch.bfloat16), (k, torch.bfloat16), (v, torch.bfloat16), (ig, torch.float32), (fg, torch.float32), (dy, torch.float32))]
    st = ops.MlstmShape(B, H, T // world, d, d, 64, torch.bfloat16, torch.float32)
    gather = cp.dist_gather()
    fused, carry = cp.forward(*mine[:5], st, rank, gather)
    grads = cp.backward(fused, *mine[:5], mine[5], st, carry, rank, world, gather)
    torch.save([host(fused.ytil)] + [host(g) for g in grads], "%s.%d" % (out, rank))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpus_over_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from gpu_util import mlstm_inputs, rel_to_max
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = str(tmp_path / "cp")
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    B, H, T, d = 2, 2, 256, 128
    q, k, v, ig, fg, dy = mlstm_inputs(B, H, T, d, d, seed=43, bf16=True)
    ref = dict(O.mlstm_core_fw(q, k, v, ig, fg, B, H, T, d, d, C0=None, n0=None, m0=None))
    ref.update(O.mlstm_core_bw(q, k, v, ig, fg, dy, B, H, T, d, d, C0=None, n0=None, m0=None, dC_in=None, dn_in=None))
    parts = [torch.load("%s.%d" % (out, r), weights_only=False) for r in range(2)]
    for i, n in enumerate(NAMES):
        assert rel_to_max(_join([p[i] for p in parts], B, T, 2), ref[n]) <= 2e-2, n


class _ThreadRanks:
    """W host threads as W ranks on one GPU: the exchange is a list behind a barrier. All kernels go to the same
    stream in issue order and none waits on another, so this is a plain serialised run of the multi-rank code."""

    def __init__(self, world):
        import threading
        self.world, self.slots, self.bar = world, [None] * world, threading.Barrier(world)

    def gather_of(self, rank):
        def gather(t):
            self.slots[rank] = t
            self.bar.wait()
            out = list(self.slots)
            self.bar.wait()
            return out
        return gather


def test_language_model_over_three_segments_equals_the_whole_sequence():
    """Every rank runs the same model on its third of each sequence; the summed losses and the summed parameter
    gradients equal the single run on the whole sequences (fp32, 2e-4: two fp32 runs)."""
    import threading
    from gpu_util import xl
    layers = importlib.import_module("neural-networks_b200.layers")
    cp = importlib.import_module("neural-networks_b200.cp")
    vocab, d, nb, heads, dqk, dhv, up, B, T, W = 40, 32, 2, 2, 8, 16, 48, 2, 48, 3
    rng = np.random.default_rng(51)
    p = layers.init_lm_params(rng, vocab, d, nb, heads, dqk, dhv, up, std=0.2)
    ids = rng.integers(0, vocab, (B, T))
    tg = np.roll(ids, -1, axis=1)
    whole = layers.build_lm(p, heads, dqk, dhv, tied=True, chunk=8)
    dev_ids = lambda a: torch.tensor(np.ascontiguousarray(a).reshape(-1), dtype=torch.int64, device="cuda")
    dev_tg = lambda a: torch.tensor(np.ascontiguousarray(a).reshape(-1).astype(np.int32), device="cuda")
    loss0 = whole.forward_backward(dev_ids(ids), dev_tg(tg), B, T).item()
    ranks = _ThreadRanks(W)
    models = [layers.build_lm(p, heads, dqk, dhv, tied=True, chunk=8) for _ in range(W)]
    losses, errors = [None] * W, []

    def run(r):
        try:
            cp.enable(models[r], r, W, gather=ranks.gather_of(r))
            seg = slice(r * T // W, (r + 1) * T // W)
            losses[r] = models[r].forward_backward(dev_ids(ids[:, seg]), dev_tg(tg[:, seg]), B, T // W, inv=1.0 / (B * T))
        except Exception as e:  # a dead rank would leave the others at the barrier
            errors.append(e)
            ranks.bar.abort()

    threads = [threading.Thread(target=run, args=(r,)) for r in range(W)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    torch.cuda.synchronize()
    assert xl._lib.lib.xlstm_device_status() == 0
    assert abs(sum(l.item() for l in losses) - loss0) <= 2e-5 * abs(loss0)
    gmax = max(float(q.g.abs().max()) for q in whole.params())
    for i, q in enumerate(whole.params()):
        total = sum(m.params()[i].g for m in models)
        e = float((total - q.g).abs().max()) / max(float(q.g.abs().max()), 1e-2 * gmax)
        assert e <= 2e-4, (i, tuple(q.g.shape), e)
