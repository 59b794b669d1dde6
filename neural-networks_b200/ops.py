"""Host-side mirror of the reference's op seam (`gpu::ops`, src/gpu/ops.rs) over the C ABI.

Each function takes torch CUDA tensors the caller owns, passes their device pointers and the
current torch stream to libxlstm_b200.so, and returns. Names and argument meaning follow the
reference functions they stand in for; nothing here computes on the host.
"""
import ctypes
import math

import torch

from . import _lib
from ._lib import lib, check

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}
FORCE_SIMT, PACK_SHORT = _lib.FORCE_SIMT, _lib.PACK_SHORT  # MlstmShape flags

# ---- optional per-op device timing (benchmarks): CUDA events around the calls of the named ops -----------------------
_timing = None


def timing_start(names=None):
    """From now on every call of an op in `names` (all ops when None) is bracketed by two CUDA events on the current
    stream. Costs two event records per call; nothing is synchronised until timing_stop()."""
    global _timing
    _timing = {"names": None if names is None else set(names), "ev": {}}


def timing_stop():
    """Stops the recording and returns {op name: [milliseconds of each call]} (synchronises the device)."""
    global _timing
    t, _timing = _timing, None
    if t is None:
        return {}
    torch.cuda.synchronize()
    return {k: [a.elapsed_time(b) for a, b in v] for k, v in t["ev"].items()}


def timed(name):
    """Decorator (also usable on library GEMM wrappers in a benchmark): records the op's device time while timing is on."""
    def wrap(fn):
        def inner(*a, **kw):
            t = _timing
            if t is None or (t["names"] is not None and name not in t["names"]):
                return fn(*a, **kw)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            t["ev"].setdefault(name, []).append((e0, e1))
            return out
        inner.__name__, inner.__doc__, inner.__wrapped__ = fn.__name__, fn.__doc__, fn
        return inner
    return wrap


def _dt(t):
    return _DT[t]


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise _lib.XlstmError("xlstm_b200 ops take CUDA tensors only (there is no CPU path)")
    if not t.is_contiguous():
        raise _lib.XlstmError("xlstm_b200 ops take contiguous tensors")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_get_device = getattr(torch._C, "_cuda_getDevice", None)
_cuda_checked = False


def _stream():
    """The current torch stream's handle. Through torch's raw accessors where they exist: `torch.cuda.current_stream()`
    builds a Stream object behind several Python-level device lookups, 19 us a call, which at the hierarchical model's
    600 library calls per step was a fifth of a host-bound step."""
    global _cuda_checked
    if not _cuda_checked:
        if not torch.cuda.is_available():
            raise _lib.XlstmError("no CUDA device: xlstm_b200 has no CPU path")
        torch.cuda.current_stream()  # initialises the context on first use
        _cuda_checked = True
    if _raw_stream is not None and _get_device is not None:
        return _raw_stream(_get_device())
    return torch.cuda.current_stream().cuda_stream


class MlstmShape:
    """The logical shape of one fused mLSTM call (reference: MlstmShape, src/gpu/ops.rs:4368-4378)."""

    def __init__(self, b, h, t, dqk, dhv, l=64, dtype=torch.bfloat16, gdtype=torch.float32, flags=0):
        self.b, self.h, self.t, self.dqk, self.dhv, self.l = b, h, t, dqk, dhv, l
        self.dtype, self.gdtype, self.flags = dtype, gdtype, flags
        self.c = _lib.MlstmShape(b, h, t, dqk, dhv, l, _DT[dtype], _DT[gdtype], flags)

    def bh(self):
        return self.b * self.h


class MlstmFused:
    """What the fused forward leaves for the backward (reference: MlstmFused, src/gpu/ops.rs:3955-3967)."""

    def __init__(self, ytil, msv, psiv, qnv, saved, state):
        self.ytil, self.msv, self.psiv, self.qnv, self.saved, self.state = ytil, msv, psiv, qnv, saved, state


@timed("mlstm_fused_fw")
def mlstm_fused_fw(qh, kh, vh, igh, fgh, st, carry_in=None, save_states=True, want_state=True):
    """ops::mlstm_fused_fw (src/gpu/ops.rs:4380-4537). carry_in = (C [BH,dhv,dqk], n [BH,dqk], m [BH])."""
    dev = qh.device
    bh, n = st.bh(), st.b * st.t
    ytil = torch.empty((n, st.h * st.dhv), dtype=st.dtype, device=dev)
    msv, psiv, qnv = (torch.empty((bh, st.t), dtype=torch.float32, device=dev) for _ in range(3))
    saved = None
    if save_states:
        saved = torch.empty((lib.xlstm_mlstm_saved_bytes(ctypes.byref(st.c)),), dtype=torch.uint8, device=dev)
    state = None
    if want_state:
        state = (torch.empty((bh, st.dhv, st.dqk), dtype=torch.float32, device=dev),
                 torch.empty((bh, st.dqk), dtype=torch.float32, device=dev),
                 torch.empty((bh,), dtype=torch.float32, device=dev))
    wsb = lib.xlstm_mlstm_fw_workspace_bytes(ctypes.byref(st.c))
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=dev)
    cC, cn, cm = carry_in if carry_in is not None else (None, None, None)
    oC, on, om = state if state is not None else (None, None, None)
    check(lib.xlstm_mlstm_fw(_stream(), ctypes.byref(st.c), _ptr(qh), _ptr(kh), _ptr(vh), _ptr(igh), _ptr(fgh),
                             _ptr(cC), _ptr(cn), _ptr(cm), _ptr(ytil), _ptr(msv), _ptr(psiv), _ptr(qnv),
                             _ptr(saved), _ptr(oC), _ptr(on), _ptr(om), _ptr(ws), wsb), "mlstm_fused_fw")
    return MlstmFused(ytil, msv, psiv, qnv, saved, state)


@timed("mlstm_final_state")
def mlstm_final_state(qh, kh, vh, igh, fgh, st, carry_in=None):
    """The (C, n, m) a fused forward would end in, from the state recurrence alone (no outputs, no record)."""
    dev = qh.device
    bh = st.bh()
    state = (torch.empty((bh, st.dhv, st.dqk), dtype=torch.float32, device=dev),
             torch.empty((bh, st.dqk), dtype=torch.float32, device=dev),
             torch.empty((bh,), dtype=torch.float32, device=dev))
    cC, cn, cm = carry_in if carry_in is not None else (None, None, None)
    check(lib.xlstm_mlstm_final_state(_stream(), ctypes.byref(st.c), _ptr(qh), _ptr(kh), _ptr(vh), _ptr(igh), _ptr(fgh),
                                      _ptr(cC), _ptr(cn), _ptr(cm), _ptr(state[0]), _ptr(state[1]), _ptr(state[2])),
          "mlstm_final_state")
    return state


@timed("mlstm_fused_bw")
def mlstm_fused_bw(fused, qh, kh, vh, igh, fgh, d_ytil, st, carry_in=None, dstate_in=None, want_dstate=True):
    """ops::mlstm_fused_bw (src/gpu/ops.rs:4546-4707). dstate_in = (dC, dn) from the call to the right.
    Returns (dq, dk, dv, dig, dfg, (dC, dn))."""
    dev = qh.device
    bh, n = st.bh(), st.b * st.t
    dq = torch.empty((n, st.h * st.dqk), dtype=st.gdtype, device=dev)
    dk = torch.empty_like(dq)
    dv = torch.empty((n, st.h * st.dhv), dtype=st.gdtype, device=dev)
    dig = torch.empty((n, st.h), dtype=torch.float32, device=dev)
    dfg = torch.empty_like(dig)
    dstate = None
    if want_dstate:
        dstate = (torch.empty((bh, st.dhv, st.dqk), dtype=torch.float32, device=dev),
                  torch.empty((bh, st.dqk), dtype=torch.float32, device=dev))
    wsb = lib.xlstm_mlstm_bw_workspace_bytes(ctypes.byref(st.c), int(fused.saved is not None))
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=dev)
    cC, cn, cm = carry_in if carry_in is not None else (None, None, None)
    dC, dn = dstate_in if dstate_in is not None else (None, None)
    oC, on = dstate if dstate is not None else (None, None)
    check(lib.xlstm_mlstm_bw(_stream(), ctypes.byref(st.c), _ptr(qh), _ptr(kh), _ptr(vh), _ptr(igh), _ptr(fgh),
                             _ptr(cC), _ptr(cn), _ptr(cm), _ptr(fused.ytil), _ptr(fused.msv), _ptr(fused.psiv),
                             _ptr(fused.qnv), _ptr(fused.saved), _ptr(d_ytil), _ptr(dC), _ptr(dn), _ptr(dq), _ptr(dk),
                             _ptr(dv), _ptr(dig), _ptr(dfg), _ptr(oC), _ptr(on), _ptr(ws), wsb), "mlstm_fused_bw")
    return dq, dk, dv, dig, dfg, dstate


SLSTM_SLAB_NAMES = ("c_prev", "n_prev", "ipr", "fpr", "c", "n", "zt", "ot", "h_prev")


class SlstmSlabs:
    """The nine [B,T,H] records of the fused sLSTM loop (reference: SlstmSlabs, src/gpu/ops.rs:2206-2256)."""

    def __init__(self, b, t, h, device):
        self.t = {n: torch.empty((b, t, h), dtype=torch.float32, device=device) for n in SLSTM_SLAB_NAMES}
        self.c = _lib.SlstmSlabs(*[self.t[n].data_ptr() for n in SLSTM_SLAB_NAMES])


@timed("slstm_fused_time")
def slstm_fused_time(wh, g, bcat, state, out, slabs, nh=1, carry=False):
    """ops::slstm_fused_time (src/gpu/ops.rs:2787-2880). state = (c, n, m, h), each [B,H], updated in place.
    Raises Declined (nothing launched) where the reference would return false."""
    b, t, h4 = g.shape
    h = h4 // 4
    c, n, m, hh = state
    check(lib.xlstm_slstm_fw(_stream(), _ptr(wh), _ptr(g), _ptr(bcat), _ptr(c), _ptr(n), _ptr(m), _ptr(hh), _ptr(out),
                             ctypes.byref(slabs.c), b, h, nh, t, int(carry), 0), "slstm_fused_time")


@timed("slstm_fused_time_bwd")
def slstm_fused_time_bwd(wh, dy, g, dstate, slabs, nh=1, carry=False):
    """ops::slstm_fused_time_bwd (src/gpu/ops.rs:2712-2777). dstate = (dh, dc, dn), each [B,H], updated in place."""
    b, t, h4 = g.shape
    h = h4 // 4
    dh, dc, dn = dstate
    check(lib.xlstm_slstm_bw(_stream(), _ptr(wh), _ptr(dy), _ptr(g), _ptr(dh), _ptr(dc), _ptr(dn),
                             ctypes.byref(slabs.c), b, h, nh, t, int(carry), 0), "slstm_fused_time_bwd")


@timed("rms_norm_forward_into")
def rms_norm_forward_into(x, gamma, group, out, inv_rms, x_hat=None, eps=1e-6):
    """ops::rms_norm_forward_into (src/gpu/ops.rs:1601-1640). x may be fp32 or bf16; `out` fp32 or bf16."""
    rows, f = x.shape
    check(lib.xlstm_rmsnorm_fw(_stream(), _ptr(x), _dt(x.dtype), _ptr(gamma), _ptr(out), _dt(out.dtype), _ptr(inv_rms),
                               _ptr(x_hat), rows, f, group, eps), "rms_norm_forward_into")


@timed("rms_norm_backward_into")
def rms_norm_backward_into(dy, x, inv_rms, gamma, group, dx, dgamma, residual=None):
    """ops::rms_norm_backward_into + the dgamma column sum (src/gpu/ops.rs:1642-1685). dgamma is accumulated;
    `residual` (fp32, same shape) is added to dx in the same pass; x fp32 or bf16, dx fp32 or bf16."""
    rows, f = dy.shape
    wsb = lib.xlstm_rmsnorm_bw_workspace_bytes(rows, f)
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=dy.device)
    check(lib.xlstm_rmsnorm_bw(_stream(), _ptr(dy), _ptr(x), _dt(x.dtype), _ptr(inv_rms), _ptr(gamma), _ptr(residual),
                               _ptr(dx), _dt(dx.dtype), _ptr(dgamma), rows, f, group, _ptr(ws), wsb), "rms_norm_backward_into")


@timed("colsum_narrow")
def colsum_narrow(x, acc, scale=1.0, narrow=True):
    """acc += scale * x.sum(0) (a projection's bias gradient, add_col_sum of src/gpu/cuda/common.cu:49-124) and, with
    `narrow`, the bf16 copy of scale * x that the two weight-side GEMMs consume, in the same pass. Returns the
    bf16 tensor (x itself when it is bf16 already and scale == 1)."""
    rows, cols = x.shape
    out = None
    if narrow and (x.dtype != torch.bfloat16 or scale != 1.0):
        out = torch.empty((rows, cols), dtype=torch.bfloat16, device=x.device)
    wsb = lib.xlstm_colsum_workspace_bytes(rows, cols)
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=x.device)
    check(lib.xlstm_colsum_narrow(_stream(), _ptr(x), _dt(x.dtype), rows, cols, float(scale), _ptr(out), _ptr(acc), _ptr(ws), wsb),
          "colsum_narrow")
    return out if out is not None else x


@timed("bias_rows")
def bias_rows(bias, rows, residual=None):
    """broadcast_row / broadcast_row_resid (src/gpu/cuda/common.cu:20-48): a new [rows, cols] fp32 tensor holding
    bias (+ residual), the seed an output projection's GEMM accumulates into."""
    out = torch.empty((rows, bias.numel()), dtype=torch.float32, device=bias.device)
    check(lib.xlstm_bias_rows(_stream(), _ptr(residual), _ptr(bias), _ptr(out), rows, bias.numel()), "bias_rows")
    return out


def device_status_check():
    """Waits for the work enqueued so far and raises if a kernel gave up on a bounded device-side wait."""
    check(lib.xlstm_device_status(), "device status")


@timed("softmax_cross_entropy")
def softmax_cross_entropy(logits, targets, dlogits, loss_accum, mask=None, inv=None):
    """ops::softmax_cross_entropy / masked_softmax_ce_u32_into (src/gpu/ops.rs:1689-1714, 3567-3618).
    targets/mask are int32 tensors holding u32 values; loss_accum is a 1-element f32 device tensor (+=)."""
    rows, c = logits.shape
    if inv is None:
        inv = 1.0 / rows
    wsb = lib.xlstm_ce_workspace_bytes(rows)
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=logits.device)
    check(lib.xlstm_ce_fw_bw(_stream(), _ptr(logits), _ptr(targets), _ptr(mask), _ptr(dlogits), _ptr(loss_accum), rows, c,
                             inv, _ptr(ws), wsb), "softmax_cross_entropy")


@timed("softcap_cross_entropy")
def softcap_cross_entropy(pre_logits, targets, d_pre, loss_accum, cap, mask=None, inv=None):
    """Soft-cap (softcap_forward/backward, src/gpu/cuda/common.cu:4-12) fused into the loss: the loss of
    cap*tanh(pre/cap) and its gradient with respect to `pre_logits` (d_pre may alias pre_logits)."""
    rows, c = pre_logits.shape
    if inv is None:
        inv = 1.0 / rows
    wsb = lib.xlstm_ce_workspace_bytes(rows)
    ws = torch.empty((max(wsb, 1),), dtype=torch.uint8, device=pre_logits.device)
    check(lib.xlstm_softcap_ce_fw_bw(_stream(), _ptr(pre_logits), _ptr(targets), _ptr(mask), _ptr(d_pre), _ptr(loss_accum),
                                     rows, c, inv, float(cap), _ptr(ws), wsb), "softcap_cross_entropy")


@timed("swiglu_forward")
def swiglu_forward(gate_pre, value, out_dtype=torch.float32, bias_gate=None, bias_value=None):
    """swiglu_forward (src/gpu/cuda/block.cu:6-29): SiLU(gate_pre + bias_gate) * (value + bias_value), optionally
    narrowed to bf16. The biases are the two projections' (both or neither), folded in here. gate_pre / value: fp32, or
    bf16 as a bf16 layer's GEMM epilogues write them."""
    assert gate_pre.dtype == value.dtype
    out = torch.empty(gate_pre.shape, dtype=out_dtype, device=gate_pre.device)
    check(lib.xlstm_swiglu_fw(_stream(), _ptr(gate_pre), _ptr(value), _dt(gate_pre.dtype), _ptr(bias_gate), _ptr(bias_value),
                              gate_pre.shape[-1], _ptr(out), _dt(out_dtype), gate_pre.numel()), "swiglu_forward")
    return out


@timed("swiglu_backward")
def swiglu_backward(d_mixed, gate_pre, value, out_dtype=torch.float32, bias_gate=None, bias_value=None):
    """swiglu_backward: (d_gate_pre, d_value), optionally narrowed to bf16 for the GEMMs that consume them."""
    assert gate_pre.dtype == value.dtype
    dg = torch.empty(gate_pre.shape, dtype=out_dtype, device=gate_pre.device)
    dv = torch.empty(gate_pre.shape, dtype=out_dtype, device=gate_pre.device)
    check(lib.xlstm_swiglu_bw(_stream(), _ptr(d_mixed), _dt(d_mixed.dtype), _ptr(gate_pre), _ptr(value), _dt(gate_pre.dtype),
                              _ptr(bias_gate), _ptr(bias_value), gate_pre.shape[-1], _ptr(dg), _ptr(dv), _dt(out_dtype),
                              gate_pre.numel()), "swiglu_backward")
    return dg, dv


@timed("ogate_forward")
def ogate_forward(o, yhat, out_dtype=torch.float32, bias=None):
    """ogate_fwd (src/gpu/cuda/mlstm_ops.cu:147-153): o <- sigmoid(o + bias) in place; returns o * yhat. `bias` is the
    gate projection's, folded in here when its GEMM ran without one."""
    hc = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    check(lib.xlstm_ogate_fw(_stream(), _ptr(o), _ptr(yhat), _ptr(bias), o.shape[-1], _ptr(hc), _dt(out_dtype), o.numel()),
          "ogate_forward")
    return hc


@timed("ogate_backward")
def ogate_backward(d_hc, o, yhat, out_dtype=torch.float32):
    """ogate_bwd (src/gpu/cuda/mlstm_ops.cu:400-407): (do_pre [out_dtype], d_yhat [fp32])."""
    do_pre = torch.empty(o.shape, dtype=out_dtype, device=o.device)
    d_yhat = torch.empty(o.shape, dtype=torch.float32, device=o.device)
    check(lib.xlstm_ogate_bw(_stream(), _ptr(d_hc), _ptr(o), _ptr(yhat), _ptr(do_pre), _dt(out_dtype), _ptr(d_yhat), o.numel()),
          "ogate_backward")
    return do_pre, d_yhat


@timed("split3_bf16")
def split3_bf16(x):
    """fp32 tensor -> (hi, mid, lo) bf16 tensors with hi + mid + lo == x to 24 bits, in one pass."""
    x = x.contiguous()
    hi, mid, lo = (torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) for _ in range(3))
    check(lib.xlstm_split3_bf16(_stream(), _ptr(x), _ptr(hi), _ptr(mid), _ptr(lo), x.numel()), "split3_bf16")
    return hi, mid, lo


@timed("embedding_scatter_add")
def embedding_scatter_add(table_g, ids, d):
    """embedding_scatter_add (src/gpu/cuda/common.cu:127-168): table_g[ids[p]] += d[p], summed in position
    order for each token (deterministic; the sort is a library call, the accumulation is the kernel)."""
    sorted_ids, order = torch.sort(ids.reshape(-1), stable=True)
    sid, pos = sorted_ids.to(torch.int32), order.to(torch.int32)
    check(lib.xlstm_embedding_scatter_add(_stream(), _ptr(d), _ptr(sid), _ptr(pos), _ptr(table_g), ids.numel(), d.shape[1]),
          "embedding_scatter_add")


class AdamCfg:
    """reference: AdamCfg, src/nn2/optim.rs:12-33."""

    def __init__(self, lr, weight_decay, beta1=0.9, beta2=0.999, eps=1e-8, t=0):
        self.lr, self.weight_decay, self.beta1, self.beta2, self.eps, self.t = lr, weight_decay, beta1, beta2, eps, t


class AdamwQueue:
    """Collects (param, grad, m, v, decay) and applies them in one batched pass
    (reference: AdamwQueue::{push,flush}, src/gpu/ops.rs:1816-1933). flush clears the grads."""

    def __init__(self):
        self.items = []

    def push(self, p, g, m, v, decay, p_bf16=None):
        self.items.append((p, g, m, v, decay, p_bf16))

    def flush(self, cfg, zero_grad=True):
        if not self.items:
            return
        return self._flush(cfg, zero_grad)

    @timed("adamw_multi")
    def _flush(self, cfg, zero_grad):
        n = len(self.items)
        arr = (_lib.AdamwDesc * n)()
        for i, (p, g, m, v, decay, pb) in enumerate(self.items):
            arr[i] = _lib.AdamwDesc(_ptr(p), _ptr(g), _ptr(m), _ptr(v), _ptr(pb), p.numel(),
                                    cfg.weight_decay if decay else 0.0, 0.0)
        # bias corrections in f32, as the reference computes them on the host (powi)
        import numpy as np
        bc1 = float(np.float32(1.0) - np.float32(cfg.beta1) ** np.int32(cfg.t))
        bc2 = float(np.float32(1.0) - np.float32(cfg.beta2) ** np.int32(cfg.t))
        check(lib.xlstm_adamw_multi(_stream(), arr, n, cfg.lr, cfg.beta1, cfg.beta2, cfg.eps, bc1, bc2, int(zero_grad)),
              "adamw_multi")
        self.items = []


def adamw(p, g, m, v, cfg, decay, p_bf16=None, zero_grad=False):
    """ops::adamw (src/gpu/ops.rs:1775-1814): one tensor."""
    q = AdamwQueue()
    q.push(p, g, m, v, decay, p_bf16)
    q.flush(cfg, zero_grad=zero_grad)
