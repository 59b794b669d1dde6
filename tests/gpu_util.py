"""Helpers shared by the GPU parity tests."""
import importlib

import numpy as np
import torch

xl = importlib.import_module("neural-networks_b200")
ops = xl.ops


def dev(a, dtype=torch.float32):
    return torch.tensor(np.ascontiguousarray(a), dtype=dtype, device="cuda")


def host(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rel_to_max(got, ref):
    ref = np.asarray(ref, np.float64)
    scale = max(np.abs(ref).max(), 1e-30)
    return float(np.abs(np.asarray(got, np.float64) - ref).max() / scale)


def bf16_round(a):
    """Round a float array to bf16 precision (so the oracle sees the same inputs the kernel does)."""
    return torch.tensor(np.asarray(a, np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


def mlstm_inputs(B, H, T, dqk, dhv, seed, fbias=3.0, bf16=False):
    r = np.random.default_rng(seed)
    q = r.standard_normal((B * T, H * dqk))
    k = r.standard_normal((B * T, H * dqk)) / np.sqrt(dqk)
    v = r.standard_normal((B * T, H * dhv))
    ig = r.standard_normal((B * T, H)).astype(np.float32).astype(np.float64)
    fg = (r.standard_normal((B * T, H)) + fbias).astype(np.float32).astype(np.float64)
    dy = r.standard_normal((B * T, H * dhv))
    if bf16:
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)
    else:
        q, k, v = (a.astype(np.float32).astype(np.float64) for a in (q, k, v))
    return q, k, v, ig, fg, dy
