"""Host-side mirror of the reference's layer API above the op seam: `gpu::Linear`, `gpu::RmsNorm`,
`gpu::MLstm`, `gpu::SLstm`, `gpu::Block<C>` and `gpu::Lm` (src/gpu/linear.rs, rms_norm.rs,
mlstm.rs, slstm.rs, block.rs, lm.rs), with the same verbs: forward, backward (hand-written, no
autograd), zero_grad, step (AdamW through one batched queue).

The recurrent cores, RMSNorm, cross-entropy and AdamW run in libxlstm_b200.so through `ops`.
Plain projections are library GEMMs (torch.matmul -> cuBLAS/cuBLASLt), as they are in the
reference (src/gpu/ops.rs:186-441). Parameters of record are fp32; with `bf16=True` GEMM operands
are narrowed to bf16 (the per-layer bf16 weight shadow is written by the AdamW kernel in the same
pass that updates the weight, so it can never go stale) and q/k/v are stored as bf16.
In bf16 mode the element-wise glue between the GEMMs runs in the library too (SwiGLU, output gate, bias
gradients fused with the narrowing of the same tensor, residual gradients inside the norm's backward, bias +
residual seeds of the output GEMMs); what is left to torch tensor ops is the embedding gather, the sort in
front of the embedding scatter, and the fp32 reference mode of the small parity models.
"""
import copy
import math

import torch

from . import cp, ops


class Param:
    """One fp32 parameter with its gradient accumulator, AdamW moments and optional bf16 shadow."""

    def __init__(self, value, decay, shadow=False, grad=None):
        self.w = value.detach().to(torch.float32).contiguous().cuda()
        self.g = grad if grad is not None else torch.zeros_like(self.w)
        self.m = torch.zeros_like(self.w)
        self.v = torch.zeros_like(self.w)
        self.decay = decay
        self.wb = self.w.to(torch.bfloat16) if shadow else None


def _b16(a):
    return a if a.dtype == torch.bfloat16 else a.to(torch.bfloat16)


def _mm(a, b, bf16):
    """a @ b with fp32 result; bf16 operands when asked (fp32 accumulate inside the library)."""
    if bf16:
        try:
            return torch.mm(_b16(a), _b16(b), out_dtype=torch.float32)
        except TypeError:
            return torch.mm(_b16(a), _b16(b)).float()
    return torch.mm(a, b)


def _split3(a):
    """fp32 -> three bf16 terms whose sum carries the full 24-bit significand (one kernel pass)."""
    return ops.split3_bf16(a)


def _mm_split(a3, b3, accum=None, terms=6, into=None):
    """Product of two fp32 matrices given as bf16 triples, on the bf16 tensor cores with fp32 accumulation, smallest
    terms first, each accumulated into the result inside its GEMM (beta = 1). terms=6: every partial product whose
    weight is above 2^-24 (fp32-accurate). terms=3: hi*hi + hi*mid + mid*hi, 16 significand bits per operand (the
    dropped terms weigh 2^-16: 64 times finer than the TF32 mode the reference offers for its fp32 GEMMs,
    src/gpu/mod.rs:192-231) at half the cost. `accum`: add the product into this tensor; `into`: write it over this one."""
    (ah, am, al), (bh, bm, bl) = a3, b3
    pairs = ((al, bh), (ah, bl), (am, bm), (am, bh), (ah, bm), (ah, bh)) if terms == 6 else ((am, bh), (ah, bm), (ah, bh))
    out = accum
    for x, y in pairs:
        if out is None:
            out = torch.mm(x, y, out_dtype=torch.float32) if into is None else torch.mm(x, y, out_dtype=torch.float32, out=into)
        else:
            torch.addmm(out, x, y, out_dtype=torch.float32, out=out)
    return out


class Linear:
    """Y = X W + b (reference: gpu::Linear, src/gpu/linear.rs). W is [in, out]."""

    def __init__(self, w, b, decay=True, bf16=False):
        self.bf16 = bf16
        self.w = Param(w, decay, shadow=bf16)
        self.b = Param(b, False)

    def forward(self, x, bias=True, residual=None, narrow=False, scale=1.0):
        """x: fp32, or already narrowed to bf16 by a caller that feeds several projections from it.
        bias=False: the product alone (the consumer kernel adds the bias). residual: returns residual + x W + b,
        with one pass that seeds the output with residual + b and the product accumulated inside the GEMM (the
        reference's broadcast_row_resid seed, src/gpu/cuda/common.cu:20-48). narrow (bf16 layers): the result
        straight from the GEMM epilogue as bf16, scale * (x W + b), rounded once."""
        self.x = _b16(x) if self.bf16 else x
        w = self.w.wb if self.bf16 else self.w.w
        if narrow and self.bf16:
            if not bias:
                assert scale == 1.0
                return torch.mm(self.x, w)
            return torch.addmm(self.b.w.to(torch.bfloat16), self.x, w, beta=scale, alpha=scale)
        assert scale == 1.0, "scale is folded only into the narrowed epilogue"
        if residual is not None:
            out = ops.bias_rows(self.b.w, residual.shape[0], residual)
            if self.bf16:
                return torch.addmm(out, self.x, w, out_dtype=torch.float32, out=out)
            return out.addmm_(self.x, w)
        y = _mm(self.x, w, self.bf16)
        return y.add_(self.b.w) if bias else y

    def backward(self, dy, need_dx=True, accum=None, scale=1.0, narrow_dx=False):
        """Accumulates dW, db; returns dx, added into `accum` (inside the GEMM, beta = 1) when one is given.
        `scale`: the gradient that reaches this layer is scale * dy (the 1/sqrt(dqk) of the key projection).
        `narrow_dx` (bf16 layers, no `accum`): dx as bf16 from the GEMM epilogue, for an element-wise consumer."""
        if self.bf16:
            # bias gradient and the narrowing of dy for both products in one pass over dy; a dy that arrives in
            # bf16 is only summed, and the scale rides in the GEMMs' alpha
            was_narrow = dy.dtype == torch.bfloat16
            dy = ops.colsum_narrow(dy, self.b.g, scale, narrow=not was_narrow)
            alpha = scale if was_narrow else 1.0
            torch.addmm(self.w.g, self.x.t(), dy, out_dtype=torch.float32, out=self.w.g, alpha=alpha)
            if not need_dx:
                return None
            wt = self.w.wb.t()
            if accum is None:
                dx = torch.mm(dy, wt) if narrow_dx else torch.mm(dy, wt, out_dtype=torch.float32)
                return dx if alpha == 1.0 else dx.mul_(alpha)
            return torch.addmm(accum, dy, wt, out_dtype=torch.float32, out=accum, alpha=alpha)
        if scale != 1.0:
            dy = dy * scale
        self.b.g.add_(dy.sum(dim=0, dtype=torch.float32))
        self.w.g.addmm_(self.x.t(), dy)
        if not need_dx:
            return None
        wt = self.w.w.t()
        if accum is None:
            return torch.mm(dy, wt)
        return accum.addmm_(dy, wt)

    def params(self):
        return [self.w, self.b]

    def release(self):
        self.x = None


class RmsNorm:
    """Grouped RMSNorm, eps 1e-6, gamma undecayed (reference: gpu::RmsNorm, src/gpu/rms_norm.rs)."""

    def __init__(self, gamma, group=None):
        self.gamma = Param(gamma, False)
        self.group = group or gamma.numel()

    def forward(self, x, out_dtype=torch.float32):
        """x fp32 or bf16; the result in `out_dtype` (bf16 where only GEMMs consume it)."""
        self.x = x
        rows, f = x.shape
        y = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        self.inv = torch.empty((rows * (f // self.group),), dtype=torch.float32, device=x.device)
        ops.rms_norm_forward_into(x, self.gamma.w, self.group, y, self.inv)
        return y

    def backward(self, dy, residual=None, out_dtype=torch.float32):
        """Returns dx (+ residual, the gradient arriving over the skip connection, added in the same pass)."""
        dx = torch.empty(dy.shape, dtype=out_dtype, device=dy.device)
        ops.rms_norm_backward_into(dy, self.x, self.inv, self.gamma.w, self.group, dx, self.gamma.g, residual=residual)
        return dx

    def params(self):
        return [self.gamma]

    def release(self):
        self.x = self.inv = None


class MLstm:
    """gpu::MLstm (src/gpu/mlstm.rs:167-876): six projections -> fused chunkwise core -> head-wise
    RMSNorm -> output gate -> output projection. `p` holds wq,wk [in,H*dqk], wv,wo [in,H*dhv],
    wi,wf [in,H], their biases, w_out [d,d], b_out, gamma [d]."""

    def __init__(self, p, heads, dqk, dhv, bf16=False, chunk=64, recompute_states=False, grad_bf16=None):
        """recompute_states: training keeps no chunk-state record; the backward rebuilds the chunk-boundary states
        (the reference stores them for every chunk, src/gpu/ops.rs:3955-3967). grad_bf16 (default: as bf16): the
        core's gradient I/O (d_ytil in; dq, dk, dv out) is bf16, the width the GEMMs on either side consume."""
        self.h, self.dqk, self.dhv, self.bf16, self.chunk = heads, dqk, dhv, bf16, chunk
        self.recompute_states = recompute_states
        self.grad_bf16 = bf16 if grad_bf16 is None else (grad_bf16 and bf16)
        mk = lambda n: Linear(p["w" + n], p["b" + n], True, bf16)
        self.lq, self.lk, self.lv, self.lo, self.li, self.lf = (mk(n) for n in "qkvoif")
        self.lout = Linear(p["w_out"], p["b_out"], True, bf16)
        self.hn = RmsNorm(p["gamma"], group=dhv)
        self.inv_sqrt = 1.0 / math.sqrt(dqk)
        self.carry = None  # (C, n, m) when a call continues the previous one
        self.stateful = False  # inference: keep the state a call ends with as the next call's carry
        self.sweep = False  # training over a sequence cut into calls: `carry` in and out forwards, `dcarry` backwards
        self.dcarry = None  # (dC, dn) from the call to the right
        self.shard_group = None  # head-sharded inference: process group whose ranks split the heads
        self.cp = None  # context parallelism: (rank, world, gather) when the sequence is cut over the ranks (cp.enable)

    def forward(self, x, B, T, residual=None):
        """residual: when given, the call returns residual + cell(x) (the block's first residual add, done inside
        the output projection's GEMM)."""
        sdt = torch.bfloat16 if self.bf16 else torch.float32
        # short sequences that neither take nor leave a state (word rectangles): several to a chunk tile
        pack = T <= 32 and not (self.stateful or self.sweep) and self.carry is None and self.cp is None
        self.st = ops.MlstmShape(B, self.h, T, self.dqk, self.dhv, self.chunk, sdt,
                                 torch.bfloat16 if self.grad_bf16 else torch.float32, ops.PACK_SHORT if pack else 0)
        if self.bf16:
            x = _b16(x)  # one narrowing feeds all six projections
        if self.bf16:  # bf16 q, k, v straight from the GEMM epilogue (bias and the 1/sqrt(dqk) of k folded in)
            q = self.lq.forward(x, narrow=True)
            k = self.lk.forward(x, narrow=True, scale=self.inv_sqrt)
            v = self.lv.forward(x, narrow=True)
        else:
            q = self.lq.forward(x)
            k = self.lk.forward(x).mul_(self.inv_sqrt)
            v = self.lv.forward(x)
        self.o = self.lo.forward(x, bias=False)  # bias added and activated in place by the output-gate kernel below
        ig, fg = self.li.forward(x), self.lf.forward(x)
        self.core_in = (q, k, v, ig, fg)
        keep = self.stateful or self.sweep
        if self.cp is not None:  # this rank's segment inside the whole sequence: the carry comes from the ranks to the left
            self.fused, self.carry_in = cp.forward(q, k, v, ig, fg, self.st, self.cp[0], self.cp[2])
        else:
            self.carry_in = self.carry  # the backward needs the state this call entered with
            self.fused = ops.mlstm_fused_fw(q, k, v, ig, fg, self.st, carry_in=self.carry, want_state=keep,
                                            save_states=not (self.stateful or self.recompute_states))
        if keep:
            self.carry = self.fused.state
        self.yhat = self.hn.forward(self.fused.ytil)  # reads the core's bf16 output as it is
        hc = ops.ogate_forward(self.o, self.yhat, torch.bfloat16 if self.bf16 else torch.float32, bias=self.lo.b.w)
        if self.shard_group is None:
            return self.lout.forward(hc, residual=residual)
        # heads are split over the group's ranks: W_out's rows are too, and the partial products are summed
        # (the one exchange head sharding needs; the bias is added once, after the sum)
        import torch.distributed as dist
        y = _mm(hc, self.lout.w.wb if self.bf16 else self.lout.w.w, self.bf16)
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.shard_group)
        y.add_(self.lout.b.w)
        return y if residual is None else y.add_(residual)

    def backward(self, dy):
        d_hc = self.lout.backward(dy)
        do_pre, d_yhat = ops.ogate_backward(d_hc, self.o, self.yhat, torch.bfloat16 if self.bf16 else torch.float32)
        d_ytil = self.hn.backward(d_yhat, out_dtype=torch.bfloat16 if self.grad_bf16 else torch.float32)
        q, k, v, ig, fg = self.core_in
        if self.cp is not None:
            dq, dk, dv, dig, dfg = cp.backward(self.fused, q, k, v, ig, fg, d_ytil, self.st, self.carry_in, *self.cp)
        else:
            dq, dk, dv, dig, dfg, dstate = ops.mlstm_fused_bw(self.fused, q, k, v, ig, fg, d_ytil, self.st,
                                                              carry_in=self.carry_in,
                                                              dstate_in=self.dcarry if self.sweep else None,
                                                              want_dstate=self.sweep)
            if self.sweep:
                self.dcarry = dstate
        dx = self.lq.backward(dq)
        self.lk.backward(dk, accum=dx, scale=self.inv_sqrt)
        self.lv.backward(dv, accum=dx)
        self.lo.backward(do_pre, accum=dx)
        self.li.backward(dig, accum=dx)
        self.lf.backward(dfg, accum=dx)
        return dx

    def params(self):
        out = []
        for l in (self.lq, self.lk, self.lv, self.lo, self.li, self.lf, self.lout):
            out += l.params()
        return out + self.hn.params()

    def release(self):
        self.o = self.core_in = self.fused = self.yhat = None
        for l in (self.lq, self.lk, self.lv, self.lo, self.li, self.lf, self.lout, self.hn):
            l.release()


class SLstm:
    """gpu::SLstm (src/gpu/slstm.rs:91-1335): hoisted x.Wx GEMM -> fused recurrent loop; the
    post-cell norm is applied by the block. wh is dense [H,4H] (nh=1) or block-diagonal [nh,dh,4dh]."""

    def __init__(self, p, hidden, nh=1, bf16=False):
        self.H, self.nh, self.bf16 = hidden, nh, bf16
        self.wx = Param(p["wx"], True, shadow=bf16)
        self.wh = Param(p["wh"], True)
        self.b = Param(p["bcat"], False)
        self.stateful = False  # inference: (c, n, m, h) persists from call to call
        self.state = None
        self.sweep = False  # training over a sequence cut into calls: `state` forwards, `dstate` (dh, dc, dn) backwards
        self.dstate = None
        # hook() called right before the backward time loop is launched: a long, latency-bound kernel that leaves the
        # memory system and twenty SMs idle, so a data-parallel step starts its pending all-reduces here
        self.before_time_loop = None

    def forward(self, x, B, T):
        H = self.H
        self.B, self.T, self.x = B, T, (_b16(x) if self.bf16 else x)
        self.g = _mm(self.x, self.wx.wb if self.bf16 else self.wx.w, self.bf16).view(B, T, 4 * H)
        self.slabs = ops.SlstmSlabs(B, T, H, x.device)
        carry = (self.stateful or self.sweep) and self.state is not None
        # a sweep's calls each keep their own copy: the loop updates the state in place
        state = (tuple(t.clone() for t in self.state) if self.sweep else self.state) if carry else \
            tuple(torch.empty((B, H), dtype=torch.float32, device=x.device) for _ in range(4))
        out = torch.empty((B, T, H), dtype=torch.float32, device=x.device)
        ops.slstm_fused_time(self.wh.w, self.g, self.b.w, state, out, self.slabs, nh=self.nh, carry=carry)
        if self.stateful or self.sweep:
            self.state = state  # updated in place to the state after the last position
        return out.view(B * T, H)

    def backward(self, dy):
        B, T, H, nh = self.B, self.T, self.H, self.nh
        bptt = self.sweep and self.dstate is not None
        ds = tuple(t.clone() for t in self.dstate) if bptt else \
            tuple(torch.empty((B, H), dtype=torch.float32, device=dy.device) for _ in range(3))
        if self.before_time_loop is not None:
            self.before_time_loop()
        ops.slstm_fused_time_bwd(self.wh.w, dy.view(B, T, H).contiguous(), self.g, ds, self.slabs, nh=nh, carry=bptt)
        if self.sweep:
            self.dstate = ds  # now the gradient of the state this call entered with
        dg = self.g.view(B * T, 4 * H)  # the loop left the four gate deltas here
        if self.bf16:
            dgn = ops.colsum_narrow(dg, self.b.g)  # bias gradient and the bf16 copy in one pass
            torch.addmm(self.wx.g, self.x.t(), dgn, out_dtype=torch.float32, out=self.wx.g)
        else:
            dgn = dg
            self.wx.g.addmm_(self.x.t(), dgn)
            self.b.g.add_(dg.sum(dim=0))
        hp = self.slabs.t["h_prev"].view(B * T, H)
        if nh == 1:
            self.wh.g.add_(_mm(hp.t(), dgn, self.bf16))
        else:
            # one batched product over the heads: [nh, dh, rows] x [nh, rows, 4*dh]; the gate deltas are regrouped
            # head-major once (bf16 operands in bf16 mode, as the reference's h_prev^T dg, src/gpu/ops.rs:300-361)
            dh = H // nh
            dgh = dgn.view(B * T, 4, nh, dh).permute(2, 0, 1, 3).reshape(nh, B * T, 4 * dh)
            hph = (_b16(hp) if self.bf16 else hp).view(B * T, nh, dh).permute(1, 2, 0)
            if self.bf16:
                self.wh.g.add_(torch.bmm(hph, dgh, out_dtype=torch.float32))
            else:
                self.wh.g.baddbmm_(hph, dgh)
        return _mm(dgn, (self.wx.wb if self.bf16 else self.wx.w).t(), self.bf16)

    def params(self):
        return [self.wx, self.wh, self.b]

    def release(self):
        self.x = self.g = self.slabs = None


class Block:
    """gpu::Block<C> (src/gpu/block.rs:435-1185): z = x + [post](cell(norm1 x));
    y = z + down(SiLU(gate(norm2 z)) * value(norm2 z))."""

    # bf16 layers keep the SwiGLU pre-activations and the gradient of its output as bf16, written by the GEMM
    # epilogues (half the traffic and half the saved bytes); False keeps them fp32 between bf16 GEMMs
    narrow_ffn = True

    def __init__(self, cell, p, post_norm=False, bf16=False):
        self.cell = cell
        self.n1, self.n2 = RmsNorm(p["g1"]), RmsNorm(p["g2"])
        self.post = RmsNorm(p["gpost"]) if post_norm else None
        # The inner width as the model defines it (8h/3 in the reference's models: 682 at h = 256, 2730 at 1024).
        # A bf16 operand whose rows are not a multiple of 16 bytes sends the library to its slow unaligned GEMMs,
        # so in bf16 mode the three projections are stored padded to a multiple of 8 columns / rows of zeros. The
        # padding is exact: SiLU(0) * 0 = 0 feeds zero rows of w_down, every gradient of a padded entry is zero
        # and AdamW keeps a zero weight with a zero gradient at zero. `up` is what checkpoints see.
        self.up = p["w_gate"].shape[1]
        pad = (-self.up) % 8 if bf16 else 0
        wide = lambda w: torch.nn.functional.pad(torch.as_tensor(w, dtype=torch.float32), (0, pad))
        self.lg = Linear(wide(p["w_gate"]), wide(p["b_gate"]), True, bf16)
        self.lv = Linear(wide(p["w_value"]), wide(p["b_value"]), True, bf16)
        self.ld = Linear(torch.nn.functional.pad(torch.as_tensor(p["w_down"], dtype=torch.float32), (0, 0, 0, pad)), p["b_down"], True, bf16)

    def forward(self, x, B, T):
        nd_in = torch.bfloat16 if self.lg.bf16 else torch.float32  # the norms feed GEMMs only: narrowed as they are written
        if self.post is None:
            z = self.cell.forward(self.n1.forward(x, nd_in), B, T, residual=x)
        else:
            z = x + self.post.forward(self.cell.forward(self.n1.forward(x, nd_in), B, T))
        zn = self.n2.forward(z, nd_in)
        # the two projections without their biases: the SwiGLU kernels add them (forward and backward)
        # (bf16 layers: straight from the GEMM epilogues as bf16, which is also what the backward keeps)
        nf = self.narrow_ffn
        self.gate_pre, self.value = self.lg.forward(zn, bias=False, narrow=nf), self.lv.forward(zn, bias=False, narrow=nf)
        nd = torch.bfloat16 if self.ld.bf16 else torch.float32
        mixed = ops.swiglu_forward(self.gate_pre, self.value, nd, self.lg.b.w, self.lv.b.w)
        return self.ld.forward(mixed, residual=z)

    def backward(self, dy):
        d_mixed = self.ld.backward(dy, narrow_dx=self.ld.bf16 and self.narrow_ffn)
        d_gate, d_value = ops.swiglu_backward(d_mixed, self.gate_pre, self.value, torch.bfloat16 if self.lg.bf16 else torch.float32,
                                              self.lg.b.w, self.lv.b.w)
        d_zn = self.lg.backward(d_gate)
        self.lv.backward(d_value, accum=d_zn)
        d_z = self.n2.backward(d_zn, residual=dy)
        d_c = self.post.backward(d_z) if self.post is not None else d_z
        return self.n1.backward(self.cell.backward(d_c), residual=d_z)

    def params(self):
        out = self.n1.params() + self.cell.params() + self.n2.params()
        if self.post is not None:
            out += self.post.params()
        for l in (self.lg, self.lv, self.ld):
            out += l.params()
        return out

    def release(self):
        """Drops everything the forward saved for the backward."""
        self.gate_pre = self.value = None
        for l in (self.cell, self.n1, self.n2, self.lg, self.lv, self.ld):
            l.release()
        if self.post is not None:
            self.post.release()


def shell(obj):
    """A copy of a layer (or block) that shares every parameter with the original and owns its saved
    activations: the same weights can then hold several calls' forward records at once, which a sweep over a
    sequence cut into calls needs (all calls forward, then all calls backward, right to left). Gradients
    accumulate into the shared parameters."""
    new = copy.copy(obj)
    for k, v in vars(obj).items():
        if isinstance(v, (Linear, RmsNorm, MLstm, SLstm, Block)):
            setattr(new, k, shell(v))
    return new


class Lm:
    """gpu::Lm (src/gpu/lm.rs:25-163): embedding -> blocks -> RMSNorm -> head (fp32) -> SoftCap -> CE.
    `tied=True` uses the embedding table (transposed) as the head and sums its two gradients.

    Two memory levers for wide models, both exact: `remat` (True for every block, or the collection of
    block indices to treat so) keeps only a block's input and re-runs its forward right before its
    backward; `head_rows=n` (tied head, through
    `forward_backward`) walks the head GEMM, soft-cap and cross-entropy over n rows at a time, so the
    [rows, vocab] logits never exist as a whole."""

    def __init__(self, table, blocks, gamma, head_w=None, head_b=None, cap=30.0, tied=False, remat=False, head_rows=0,
                 head_split=False):
        self.table = Param(table, False)
        self.blocks = blocks
        self.norm = RmsNorm(gamma)
        self.tied = tied
        self.head = None if tied else Linear(head_w, head_b, decay=False, bf16=False)
        self.cap = cap
        self.loss = torch.zeros((1,), dtype=torch.float32, device="cuda")
        self.on_block_backward = None  # hook(i) called when block i's gradients are complete
        # train_step waits for the backward pass and raises if a kernel gave up on a bounded device-side wait, before
        # AdamW consumes the gradients; set False for a host that must stay fully asynchronous
        self.check_status = True
        self.remat = set(range(len(blocks))) if remat is True else set(remat or ())
        self.head_rows = head_rows
        # head_split: the fp32 head products (row-chunked path) run as bf16 tensor-core GEMMs on 3-way split
        # operands (see _mm_split): True or 6 keeps fp32 accuracy with six products, 3 keeps 16 bits per operand
        self.head_split = 6 if head_split is True else int(head_split or 0)
        assert self.head_split in (0, 3, 6)
        assert not head_rows or tied, "the row-chunked head is implemented for the tied head"

    def forward_hidden(self, ids, B, T):
        """Embedding, blocks and the final norm; returns the normed hidden state [rows, d]."""
        self.ids, self.B, self.T = ids.reshape(-1), B, T
        x = self.table.w.index_select(0, self.ids)
        self.block_in = [None] * len(self.blocks)
        for i, blk in enumerate(self.blocks):
            if i in self.remat:
                self.block_in[i] = x
            x = blk.forward(x, B, T)
            if i in self.remat:
                blk.release()
        self.normed = self.norm.forward(x)
        return self.normed

    def forward(self, ids, B, T):
        normed = self.forward_hidden(ids, B, T)
        pre = torch.mm(normed, self.table.w.t()) if self.tied else self.head.forward(normed)
        self.logits = torch.tanh_(pre.div_(self.cap)).mul_(self.cap)
        return self.logits

    def backward_hidden(self, d_n):
        d = self.norm.backward(d_n)
        for i in range(len(self.blocks) - 1, -1, -1):
            blk = self.blocks[i]
            if i in self.remat:
                blk.forward(self.block_in[i], self.B, self.T)
                self.block_in[i] = None
            d = blk.backward(d)
            blk.release()
            if self.on_block_backward is not None:
                self.on_block_backward(i)
        ops.embedding_scatter_add(self.table.g, self.ids, d)

    def backward(self, dlogits):
        t = self.logits / self.cap
        d_pre = dlogits * (1.0 - t * t)
        if self.tied:
            self.table.g.addmm_(d_pre.t(), self.normed)
            d_n = torch.mm(d_pre, self.table.w)
        else:
            d_n = self.head.backward(d_pre)
        self.backward_hidden(d_n)

    def params(self):
        out = [self.table]
        for blk in self.blocks:
            out += blk.params()
        out += self.norm.params()
        if self.head is not None:
            out += self.head.params()
        return out

    def step(self, cfg):
        q = ops.AdamwQueue()
        for p in self.params():
            q.push(p.w, p.g, p.m, p.v, p.decay, p.wb)
        q.flush(cfg, zero_grad=True)

    def forward_backward(self, ids, targets, B, T, inv=None):
        """Forward, fused CE (loss accumulated on the device), backward. Returns the device loss scalar."""
        self.loss.zero_()
        if not self.head_rows:
            logits = self.forward(ids, B, T)
            dlogits = torch.empty_like(logits)
            ops.softmax_cross_entropy(logits, targets, dlogits, self.loss, inv=inv)
            self.backward(dlogits)
            return self.loss
        normed = self.forward_hidden(ids, B, T)
        rows = normed.shape[0]
        inv = inv if inv is not None else 1.0 / rows
        d_n = torch.empty_like(normed)
        wt = self.table.w.t()
        if self.head_split:
            w3 = _split3(self.table.w)
            w3t = tuple(p.t() for p in w3)
        for lo in range(0, rows, self.head_rows):
            hi = min(rows, lo + self.head_rows)
            if self.head_split:
                n3 = _split3(normed[lo:hi])
                pre = _mm_split(n3, w3t, terms=self.head_split)
            else:
                pre = torch.mm(normed[lo:hi], wt)
            d_pre = pre  # the fused soft-cap + loss kernel writes the gradient over its input
            ops.softcap_cross_entropy(pre, targets[lo:hi], d_pre, self.loss, self.cap, inv=inv)
            if self.head_split:
                d3 = _split3(d_pre)
                _mm_split(tuple(p.t() for p in d3), n3, accum=self.table.g, terms=self.head_split)
                _mm_split(d3, w3, terms=self.head_split, into=d_n[lo:hi])
            else:
                self.table.g.addmm_(d_pre.t(), normed[lo:hi])
                torch.mm(d_pre, self.table.w, out=d_n[lo:hi])
        self.backward_hidden(d_n)
        return self.loss

    def train_step(self, ids, targets, B, T, cfg):
        loss = self.forward_backward(ids, targets, B, T)
        if self.check_status:
            ops.device_status_check()
        self.step(cfg)
        return loss


def init_lm_params(rng, vocab, d, n_blocks, heads, dqk, dhv, up, std=0.02, slstm_at=(), nh_s=1):
    """Seeded N(0, std) host weights (numpy Generator `rng`) in the dictionary layout `build_lm` takes: norm
    gains 1, every other tensor N(0, std) rounded to fp32. Blocks listed in `slstm_at` are sLSTM blocks with
    `nh_s` block-diagonal heads (dense recurrence when nh_s == 1)."""
    import numpy as np

    def n(*shape):
        return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std))

    blocks = []
    for i in range(n_blocks):
        blk = dict(g1=np.ones(d, np.float32), g2=np.ones(d, np.float32), w_gate=n(d, up), b_gate=n(up), w_value=n(d, up),
                   b_value=n(up), w_down=n(up, d), b_down=n(d))
        if i in slstm_at:
            dh = d // nh_s
            cell = dict(kind="slstm", wx=n(d, 4 * d), wh=n(nh_s, dh, 4 * dh) if nh_s > 1 else n(d, 4 * d), bcat=n(4 * d))
            blk["gpost"] = np.ones(d, np.float32)
        else:
            cell = dict(kind="mlstm", wq=n(d, heads * dqk), wk=n(d, heads * dqk), wv=n(d, heads * dhv), wo=n(d, heads * dhv),
                        wi=n(d, heads), wf=n(d, heads), bq=n(heads * dqk), bk=n(heads * dqk), bv=n(heads * dhv),
                        bo=n(heads * dhv), bi=n(heads), bf=n(heads), w_out=n(d, d), b_out=n(d), gamma=np.ones(d, np.float32))
        blk["cell"] = cell
        blocks.append(blk)
    return dict(table=n(vocab, d), blocks=blocks, gamma=np.ones(d, np.float32))


def build_lm(params, heads, dqk, dhv, nh_s=1, cap=30.0, tied=True, head_w=None, head_b=None, bf16=False, chunk=64,
             remat=False, head_rows=0, head_split=False, recompute_states=False, grad_bf16=None):
    """Builds an Lm from the host parameter dictionary `oracle.model.init_lm_params` produces."""
    t = lambda a: torch.as_tensor(a, dtype=torch.float32)
    d = params["table"].shape[1]
    blocks = []
    for bp in params["blocks"]:
        c = {k_: (t(v_) if k_ != "kind" else v_) for k_, v_ in bp["cell"].items()}
        bpt = {k_: t(v_) for k_, v_ in bp.items() if k_ != "cell"}
        if c["kind"] == "mlstm":
            blocks.append(Block(MLstm(c, heads, dqk, dhv, bf16=bf16, chunk=chunk, recompute_states=recompute_states,
                                      grad_bf16=grad_bf16), bpt, bf16=bf16))
        else:
            blocks.append(Block(SLstm(c, d, nh_s, bf16=bf16), bpt, post_norm=True, bf16=bf16))
    return Lm(t(params["table"]), blocks, t(params["gamma"]), None if head_w is None else t(head_w),
              None if head_b is None else t(head_b), cap=cap, tied=tied, remat=remat, head_rows=head_rows,
              head_split=head_split)
