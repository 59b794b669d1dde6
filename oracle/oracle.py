"""TEST INFRASTRUCTURE — numpy front end of the CPU oracle (liboracle.so).

The oracle restates the reference's CPU layer math (see xlstm_oracle_impl.h for the
file:line each function follows). PARITY UNPINNED at the bit level: the reference cannot
be built here and stores no golden vectors for these layers.

Only tests, the smoke check and the benchmark's cpu_baseline leg may import this module.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build():
    """Compile liboracle.so beside its sources (gcc, a few seconds)."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "liboracle.so"])


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _LIB = ctypes.CDLL(path)
    return _LIB


def _suf(dtype):
    return {np.dtype(np.float32): "_f32", np.dtype(np.float64): "_f64"}[np.dtype(dtype)]


def _p(a):
    if a is None:
        return ctypes.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def _real(dtype, x):
    return (ctypes.c_float if np.dtype(dtype) == np.float32 else ctypes.c_double)(x)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


def random_seeded(shape, scale, seed):
    """The reference's SplitMix64 generator (src/tensor/mod.rs:97-119)."""
    out = np.empty(shape, dtype=np.float32)
    f = lib().random_seeded_f32
    f.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_uint64]
    f(_p(out), out.size, scale, seed)
    return out


def mlstm_core_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, C0=None, n0=None, m0=None,
                  dtype=np.float64):
    """Recurrent mLSTM core. Returns dict(ytil, m, psi, nq, C, n, mlast)."""
    q, k, v, ig, fg = (_c(a, dtype) for a in (q, k, v, ig, fg))
    C0, n0, m0 = (_c(a, dtype) for a in (C0, n0, m0))
    BH = B * H
    o = dict(ytil=np.empty((B * T, H * dhv), dtype), m=np.empty((BH, T), dtype),
             psi=np.empty((BH, T), dtype), nq=np.empty((BH, T), dtype),
             C=np.empty((BH, dhv, dqk), dtype), n=np.empty((BH, dqk), dtype),
             mlast=np.empty((BH,), dtype))
    f = getattr(lib(), "mlstm_core_fw" + _suf(dtype))
    f.restype = None
    f(_p(q), _p(k), _p(v), _p(ig), _p(fg), _p(C0), _p(n0), _p(m0),
      B, H, T, dqk, dhv, _p(o["ytil"]), _p(o["m"]), _p(o["psi"]), _p(o["nq"]),
      _p(o["C"]), _p(o["n"]), _p(o["mlast"]))
    return o


def mlstm_core_bw(q, k, v, ig, fg, dytil, B, H, T, dqk, dhv, C0=None, n0=None, m0=None,
                  dC_in=None, dn_in=None, dtype=np.float64):
    """Backward of the recurrent core. Returns dict(dq, dk, dv, dig, dfg, dC, dn)."""
    q, k, v, ig, fg, dytil = (_c(a, dtype) for a in (q, k, v, ig, fg, dytil))
    C0, n0, m0, dC_in, dn_in = (_c(a, dtype) for a in (C0, n0, m0, dC_in, dn_in))
    BH = B * H
    o = dict(dq=np.empty((B * T, H * dqk), dtype), dk=np.empty((B * T, H * dqk), dtype),
             dv=np.empty((B * T, H * dhv), dtype), dig=np.empty((B * T, H), dtype),
             dfg=np.empty((B * T, H), dtype), dC=np.empty((BH, dhv, dqk), dtype),
             dn=np.empty((BH, dqk), dtype))
    f = getattr(lib(), "mlstm_core_bw" + _suf(dtype))
    f.restype = None
    f(_p(q), _p(k), _p(v), _p(ig), _p(fg), _p(C0), _p(n0), _p(m0), _p(dytil),
      _p(dC_in), _p(dn_in), B, H, T, dqk, dhv, _p(o["dq"]), _p(o["dk"]), _p(o["dv"]),
      _p(o["dig"]), _p(o["dfg"]), _p(o["dC"]), _p(o["dn"]))
    return o


SLSTM_SLABS = ("c_prev", "n_prev", "ipr", "fpr", "c", "n", "zt", "ot", "h_prev")


def slstm_fw(wh, g, bcat, B, H, NH, T, state=None, dtype=np.float64):
    """sLSTM forward loop. `g` [B,T,4H] is copied; returns dict(out, g (f block biased),
    slabs..., state=(c,n,m,h))."""
    wh, bcat = _c(wh, dtype), _c(bcat, dtype)
    g = np.array(g, dtype=dtype, order="C", copy=True)
    carry = state is not None
    if carry:
        c, n, m, h = (np.array(s, dtype=dtype, order="C", copy=True) for s in state)
    else:
        c, n, m, h = (np.zeros((B, H), dtype) for _ in range(4))
    o = {name: np.empty((B, T, H), dtype) for name in SLSTM_SLABS}
    o["out"] = np.empty((B, T, H), dtype)
    f = getattr(lib(), "slstm_fw" + _suf(dtype))
    f.restype = None
    f(_p(wh), _p(g), _p(bcat), _p(c), _p(n), _p(m), _p(h), int(carry), B, H, NH, T,
      _p(o["out"]), _p(o["c_prev"]), _p(o["n_prev"]), _p(o["ipr"]), _p(o["fpr"]),
      _p(o["c"]), _p(o["n"]), _p(o["zt"]), _p(o["ot"]), _p(o["h_prev"]))
    o["g"] = g
    o["state"] = (c, n, m, h)
    return o


def slstm_bw(wh, dy, fw, B, H, NH, T, dstate=None, dtype=np.float64):
    """sLSTM reverse loop on the records `fw` returned by slstm_fw. Returns
    dict(dg [B,T,4H], dstate=(dh,dc,dn))."""
    wh, dy = _c(wh, dtype), _c(dy, dtype)
    g = np.array(fw["g"], dtype=dtype, order="C", copy=True)
    carry = dstate is not None
    if carry:
        dh, dc, dn = (np.array(s, dtype=dtype, order="C", copy=True) for s in dstate)
    else:
        dh, dc, dn = (np.zeros((B, H), dtype) for _ in range(3))
    f = getattr(lib(), "slstm_bw" + _suf(dtype))
    f.restype = None
    s = {k_: _c(fw[k_], dtype) for k_ in SLSTM_SLABS}
    f(_p(wh), _p(dy), _p(g), _p(dh), _p(dc), _p(dn), int(carry), B, H, NH, T,
      _p(s["c_prev"]), _p(s["n_prev"]), _p(s["ipr"]), _p(s["fpr"]), _p(s["c"]), _p(s["n"]),
      _p(s["zt"]), _p(s["ot"]))
    return dict(dg=g, dstate=(dh, dc, dn))


def rmsnorm_fw(x, gamma, group, eps=1e-6, dtype=np.float64):
    x, gamma = _c(x, dtype), _c(gamma, dtype)
    rows, F = x.shape
    y, xh = np.empty_like(x), np.empty_like(x)
    inv = np.empty((rows, F // group), dtype)
    f = getattr(lib(), "rmsnorm_fw" + _suf(dtype))
    f.restype = None
    f(_p(x), _p(gamma), rows, F, group, _real(dtype, eps), _p(y), _p(xh), _p(inv))
    return y, xh, inv


def rmsnorm_bw(dy, x_hat, inv_rms, gamma, group, dtype=np.float64):
    dy, x_hat, inv_rms, gamma = (_c(a, dtype) for a in (dy, x_hat, inv_rms, gamma))
    rows, F = dy.shape
    dx = np.empty_like(dy)
    dgamma = np.zeros((F,), dtype)
    f = getattr(lib(), "rmsnorm_bw" + _suf(dtype))
    f.restype = None
    f(_p(dy), _p(x_hat), _p(inv_rms), _p(gamma), rows, F, group, _p(dx), _p(dgamma))
    return dx, dgamma


def softmax_ce(logits, targets, mask=None, inv=None, dtype=np.float64):
    logits = _c(logits, dtype)
    rows, C = logits.shape
    targets = np.ascontiguousarray(targets, dtype=np.uint32)
    mask = None if mask is None else np.ascontiguousarray(mask, dtype=np.uint32)
    if inv is None:
        inv = 1.0 / rows
    d = np.empty_like(logits)
    f = getattr(lib(), "softmax_ce" + _suf(dtype))
    f.restype = ctypes.c_float if np.dtype(dtype) == np.float32 else ctypes.c_double
    loss = f(_p(logits), _p(targets), _p(mask), rows, C, _real(dtype, inv), _p(d))
    return float(loss), d


def adamw(p, g, m, v, lr, wd, t, b1=0.9, b2=0.999, eps=1e-8, dtype=np.float64):
    """One AdamW step; returns new (p, m, v)."""
    p, m, v = (np.array(a, dtype=dtype, order="C", copy=True) for a in (p, m, v))
    g = _c(g, dtype)
    f = getattr(lib(), "adamw" + _suf(dtype))
    f.restype = None
    f(_p(p), _p(g), _p(m), _p(v), ctypes.c_size_t(p.size), _real(dtype, lr), _real(dtype, b1),
      _real(dtype, b2), _real(dtype, eps), _real(dtype, wd), int(t))
    return p, m, v


def gemm(kind, a, b, dtype=np.float64):
    """kind in nn|tn|nt, the reference's three GEMM forms (src/tensor/gemm.rs)."""
    a, b = _c(a, dtype), _c(b, dtype)
    if kind == "nn":
        m, k = a.shape; n = b.shape[1]
    elif kind == "tn":
        k, m = a.shape; n = b.shape[1]
    else:
        m, k = a.shape; n = b.shape[0]
    c = np.zeros((m, n), dtype)
    f = getattr(lib(), "gemm_" + kind + _suf(dtype))
    f.restype = None
    f(m, k, n, _p(a), _p(b), _p(c), _real(dtype, 0.0))
    return c


# --------------------------------------------------------------------------------------
# Chunkwise restatement of the mLSTM core in numpy float64, following the algebra the
# reference's fused kernels use (src/gpu/cuda/mlstm_fused.cu:12-19,118-125,494-500). It
# exists so kernel intermediates (fc, m, a, b, g, chunk states) can be compared one by
# one; its end results must equal the recurrent form for every chunk length.
# --------------------------------------------------------------------------------------
def log_sigmoid(x):
    return np.where(x >= 0, -np.log1p(np.exp(-np.abs(x))), x - np.log1p(np.exp(-np.abs(x))))


def mlstm_chunkwise_fw(q, k, v, ig, fg, B, H, T, dqk, dhv, L, C0=None, n0=None, m0=None):
    f8 = np.float64
    q = np.asarray(q, f8).reshape(B, T, H, dqk)
    k = np.asarray(k, f8).reshape(B, T, H, dqk)
    v = np.asarray(v, f8).reshape(B, T, H, dhv)
    ig = np.asarray(ig, f8).reshape(B, T, H)
    fg = np.asarray(fg, f8).reshape(B, T, H)
    NC = -(-T // L)
    ytil = np.zeros((B, T, H, dhv), f8)
    msv = np.zeros((B * H, T), f8); psi = np.zeros((B * H, T), f8); qnv = np.zeros((B * H, T), f8)
    Cst = np.zeros((B * H, NC + 1, dhv, dqk), f8); nst = np.zeros((B * H, NC + 1, dqk), f8)
    mst = np.zeros((B * H, NC + 1), f8)
    for b in range(B):
        for h in range(H):
            bh = b * H + h
            C = np.zeros((dhv, dqk), f8) if C0 is None else np.array(C0[bh], f8)
            n = np.zeros((dqk,), f8) if n0 is None else np.array(n0[bh], f8)
            mp = 0.0 if m0 is None else float(m0[bh])
            Cst[bh, 0], nst[bh, 0], mst[bh, 0] = C, n, mp
            for c in range(NC):
                s, e = c * L, min(T, (c + 1) * L)
                Q, K, V = q[b, s:e, h], k[b, s:e, h], v[b, s:e, h]
                fc = np.cumsum(log_sigmoid(fg[b, s:e, h]))
                ii = ig[b, s:e, h]
                logD = fc[:, None] - fc[None, :] + ii[None, :]
                mask = np.tril(np.ones((e - s, e - s), bool))
                logD = np.where(mask, logD, -np.inf)
                mt = np.maximum(logD.max(axis=1), fc + mp)
                D = np.exp(logD - mt[:, None])
                bt = np.exp(fc + mp - mt)
                S = (Q @ K.T) * D
                num = S @ V + bt[:, None] * (Q @ C.T)
                qn = S.sum(axis=1) + bt * (Q @ n)
                ps = np.maximum(np.abs(qn), np.exp(-mt))
                ytil[b, s:e, h] = num / ps[:, None]
                msv[bh, s:e], psi[bh, s:e], qnv[bh, s:e] = mt, ps, qn
                mL = mt[-1]
                a = np.exp(fc[-1] - fc + ii - mL)
                gk = np.exp(fc[-1] + mp - mL)
                C = gk * C + (a[:, None] * V).T @ K
                n = gk * n + (a[:, None] * K).sum(axis=0)
                mp = mL
                Cst[bh, c + 1], nst[bh, c + 1], mst[bh, c + 1] = C, n, mp
    return dict(ytil=ytil.reshape(B * T, H * dhv), m=msv, psi=psi, nq=qnv, Cst=Cst, nst=nst,
                mst=mst)
