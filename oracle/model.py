"""TEST INFRASTRUCTURE — CPU restatement of the reference's layer stack above the op seam.

Composes the oracle primitives (oracle.py / liboracle.so) into the reference's cells, block and
flat language model, with hand-written backward passes that follow the reference line by line:
  Linear        src/nn2/linear.rs:66-146
  RmsNorm       src/nn2/rms_norm.rs (eps 1e-6, gamma undecayed)
  MLstm cell    src/nn2/mlstm.rs:347-577 (forward), 580-839 (backward), 865-883 (AdamW grouping)
  SLstm cell    src/nn2/slstm.rs:205-453 with the hoisted x.Wx form of src/gpu/slstm.rs:640-732
  Block         src/nn2/block.rs:128-216 (pre-norm residual + SwiGLU; post-cell norm for sLSTM only)
  Lm            src/gpu/lm.rs:84-163 (embedding -> blocks -> RMSNorm -> head -> SoftCap -> CE)
PARITY UNPINNED at the bit level (see xlstm_oracle_impl.h). Only tests, the smoke check and the
benchmark's CPU legs may import this module.
"""
import numpy as np

from . import oracle as O

# Arithmetic width of everything built from this module. float64 is the low-noise comparison target the parity tests
# use; the benchmark's CPU legs set float32, the width of the reference's own CPU layers (src/nn2), before building.
DT = np.float64


class AdamState:
    def __init__(self, p):
        self.m = np.zeros_like(p)
        self.v = np.zeros_like(p)


class Param:
    """A parameter with its gradient accumulator and AdamW moments."""

    def __init__(self, value, decay):
        self.w = np.array(value, dtype=DT)
        self.g = np.zeros_like(self.w)
        self.decay = decay
        self.st = AdamState(self.w)

    def step(self, lr, wd, t):
        self.w, self.st.m, self.st.v = O.adamw(self.w, self.g, self.st.m, self.st.v, lr, wd if self.decay else 0.0, t, dtype=DT)
        self.g[...] = 0.0


class Linear:
    def __init__(self, w, b, decay=True):
        self.w = Param(w, decay)          # [in, out]
        self.b = Param(b, False)          # [out]

    def forward(self, x):
        self.x = x
        return x @ self.w.w + self.b.w

    def backward(self, dy):
        self.w.g += self.x.T @ dy
        self.b.g += dy.sum(axis=0)
        return dy @ self.w.w.T

    def params(self):
        return [self.w, self.b]


class RmsNorm:
    def __init__(self, gamma, group=None):
        self.gamma = Param(gamma, False)
        self.group = group or len(gamma)

    def forward(self, x):
        y, self.xh, self.inv = O.rmsnorm_fw(x, self.gamma.w, self.group, dtype=DT)
        return y

    def backward(self, dy):
        dx, dg = O.rmsnorm_bw(dy, self.xh, self.inv, self.gamma.w, self.group, dtype=DT)
        self.gamma.g += dg
        return dx

    def params(self):
        return [self.gamma]


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))  # numpy keeps the array's width (DT)


class MLstm:
    """Weights: wq, wk [in, H*dqk]; wv, wo [in, H*dhv]; wi, wf [in, H]; w_out [d, d]; gamma [d]."""

    def __init__(self, p, heads, dqk, dhv):
        self.h, self.dqk, self.dhv = heads, dqk, dhv
        self.lq, self.lk, self.lv, self.lo = (Linear(p["w" + n], p["b" + n]) for n in "qkvo")
        self.li, self.lf = Linear(p["wi"], p["bi"]), Linear(p["wf"], p["bf"])
        self.lout = Linear(p["w_out"], p["b_out"])
        self.hn = RmsNorm(p["gamma"], group=dhv)
        self.inv_sqrt = 1.0 / np.sqrt(dqk)

    def forward(self, x, B, T):
        self.B, self.T = B, T
        q = self.lq.forward(x)
        k = self.lk.forward(x) * self.inv_sqrt
        v = self.lv.forward(x)
        self.o = sigmoid(self.lo.forward(x))
        ig, fg = self.li.forward(x), self.lf.forward(x)
        self.core_in = (q, k, v, ig, fg)
        fw = O.mlstm_core_fw(q, k, v, ig, fg, B, self.h, T, self.dqk, self.dhv, dtype=DT)
        self.yhat = self.hn.forward(fw["ytil"])
        self.hc = self.o * self.yhat
        return self.lout.forward(self.hc)

    def backward(self, dy):
        d_hc = self.lout.backward(dy)
        do_pre = d_hc * self.yhat * self.o * (1.0 - self.o)
        d_ytil = self.hn.backward(d_hc * self.o)
        q, k, v, ig, fg = self.core_in
        g = O.mlstm_core_bw(q, k, v, ig, fg, d_ytil, self.B, self.h, self.T, self.dqk, self.dhv, dtype=DT)
        dx = self.lq.backward(g["dq"])
        dx += self.lk.backward(g["dk"] * self.inv_sqrt)
        dx += self.lv.backward(g["dv"])
        dx += self.lo.backward(do_pre)
        dx += self.li.backward(g["dig"])
        dx += self.lf.backward(g["dfg"])
        return dx

    def params(self):
        out = []
        for l in (self.lq, self.lk, self.lv, self.lo, self.li, self.lf, self.lout):
            out += l.params()
        return out + self.hn.params()


class SLstm:
    """Weights: wx [in, 4H] (gate blocks z,i,f,o), wh recurrent (dense [H,4H] or block-diagonal
    [NH, dh, 4*dh]), bcat [4H]. The post-cell RMSNorm lives in the block (src/nn2/block.rs:26-30)."""

    def __init__(self, p, hidden, nh=1):
        self.H, self.nh = hidden, nh
        self.wx = Param(p["wx"], True)
        self.wh = Param(p["wh"], True)
        self.b = Param(p["bcat"], False)

    def forward(self, x, B, T):
        self.B, self.T, self.x = B, T, x
        g = (x @ self.wx.w).reshape(B, T, 4 * self.H)
        self.fw = O.slstm_fw(self.wh.w, g, self.b.w, B, self.H, self.nh, T, dtype=DT)
        return self.fw["out"].reshape(B * T, self.H)

    def backward(self, dy):
        B, T, H, nh = self.B, self.T, self.H, self.nh
        bw = O.slstm_bw(self.wh.w, dy.reshape(B, T, H), self.fw, B, H, nh, T, dtype=DT)
        dg = bw["dg"].reshape(B * T, 4 * H)
        self.wx.g += self.x.T @ dg
        self.b.g += dg.sum(axis=0)
        hp = self.fw["h_prev"].reshape(B * T, H)
        if nh == 1:
            self.wh.g += hp.T @ dg
        else:
            dh = H // nh
            for hd in range(nh):
                cols = np.concatenate([np.arange(gt * H + hd * dh, gt * H + (hd + 1) * dh) for gt in range(4)])
                self.wh.g[hd] += hp[:, hd * dh:(hd + 1) * dh].T @ dg[:, cols]
        return dg @ self.wx.w.T

    def params(self):
        return [self.wx, self.wh, self.b]


def silu(x):
    return x * sigmoid(x)


def silu_prime(x):
    s = sigmoid(x)
    return s * (1.0 + x * (1.0 - s))


class Block:
    def __init__(self, cell, p, post_norm=False):
        self.cell = cell
        self.n1, self.n2 = RmsNorm(p["g1"]), RmsNorm(p["g2"])
        self.post = RmsNorm(p["gpost"]) if post_norm else None
        self.lg, self.lv, self.ld = Linear(p["w_gate"], p["b_gate"]), Linear(p["w_value"], p["b_value"]), Linear(p["w_down"], p["b_down"])

    def forward(self, x, B, T):
        c = self.cell.forward(self.n1.forward(x), B, T)
        if self.post is not None:
            c = self.post.forward(c)
        z = x + c
        zn = self.n2.forward(z)
        self.gate_pre, self.value = self.lg.forward(zn), self.lv.forward(zn)
        self.gate_act = silu(self.gate_pre)
        return z + self.ld.forward(self.gate_act * self.value)

    def backward(self, dy):
        d_mixed = self.ld.backward(dy)
        d_zn = self.lg.backward(d_mixed * self.value * silu_prime(self.gate_pre)) + self.lv.backward(d_mixed * self.gate_act)
        d_z = self.n2.backward(d_zn) + dy
        d_c = self.post.backward(d_z) if self.post is not None else d_z
        return self.n1.backward(self.cell.backward(d_c)) + d_z

    def params(self):
        out = self.n1.params() + self.cell.params() + self.n2.params()
        if self.post is not None:
            out += self.post.params()
        for l in (self.lg, self.lv, self.ld):
            out += l.params()
        return out


class Lm:
    """Flat LM. `tied`: the embedding table also serves (transposed) as the logit head, its two
    gradient contributions summed (no head bias)."""

    def __init__(self, table, blocks, gamma, head_w=None, head_b=None, cap=30.0, tied=False):
        self.table = Param(table, False)
        self.blocks = blocks
        self.norm = RmsNorm(gamma)
        self.tied = tied
        self.head = None if tied else Linear(head_w, head_b, decay=False)
        self.cap = cap

    def forward(self, ids, B, T):
        self.ids, self.B, self.T = np.asarray(ids).reshape(-1), B, T
        x = self.table.w[self.ids]
        for blk in self.blocks:
            x = blk.forward(x, B, T)
        self.normed = self.norm.forward(x)
        pre = self.normed @ self.table.w.T if self.tied else self.head.forward(self.normed)
        self.logits = self.cap * np.tanh(pre / self.cap)
        return self.logits

    def backward(self, dlogits):
        t = self.logits / self.cap
        d_pre = dlogits * (1.0 - t * t)
        if self.tied:
            self.table.g += d_pre.T @ self.normed
            d_n = d_pre @ self.table.w
        else:
            d_n = self.head.backward(d_pre)
        d = self.norm.backward(d_n)
        for blk in reversed(self.blocks):
            d = blk.backward(d)
        np.add.at(self.table.g, self.ids, d)

    def params(self):
        out = [self.table]
        for blk in self.blocks:
            out += blk.params()
        out += self.norm.params()
        if self.head is not None:
            out += self.head.params()
        return out

    def train_step(self, ids, targets, B, T, lr, wd, t):
        logits = self.forward(ids, B, T)
        loss, dlogits = O.softmax_ce(logits, targets, dtype=DT)
        self.backward(dlogits)
        grads = [p.g.copy() for p in self.params()]
        for p in self.params():
            p.step(lr, wd, t)
        return loss, grads


def init_lm_params(rng, vocab, d, n_blocks, heads, dqk, dhv, up, std=0.02, slstm_at=(), nh_s=1):
    """Seeded N(0, std) weights in the layout the Lm classes take (gamma = 1)."""
    def n(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32).astype(np.float64)
    blocks = []
    for i in range(n_blocks):
        blk = dict(g1=np.ones(d), g2=np.ones(d), w_gate=n(d, up), b_gate=n(up), w_value=n(d, up), b_value=n(up),
                   w_down=n(up, d), b_down=n(d))
        if i in slstm_at:
            dh = d // nh_s
            cell = dict(kind="slstm", wx=n(d, 4 * d), wh=n(nh_s, dh, 4 * dh) if nh_s > 1 else n(d, 4 * d), bcat=n(4 * d))
            blk["gpost"] = np.ones(d)
        else:
            cell = dict(kind="mlstm", wq=n(d, heads * dqk), wk=n(d, heads * dqk), wv=n(d, heads * dhv), wo=n(d, heads * dhv),
                        wi=n(d, heads), wf=n(d, heads), bq=n(heads * dqk), bk=n(heads * dqk), bv=n(heads * dhv),
                        bo=n(heads * dhv), bi=n(heads), bf=n(heads), w_out=n(d, d), b_out=n(d), gamma=np.ones(d))
        blk["cell"] = cell
        blocks.append(blk)
    return dict(table=n(vocab, d), blocks=blocks, gamma=np.ones(d))


def build_lm(params, heads, dqk, dhv, nh_s=1, cap=30.0, tied=True, head_w=None, head_b=None):
    blocks = []
    d = params["table"].shape[1]
    for bp in params["blocks"]:
        c = bp["cell"]
        if c["kind"] == "mlstm":
            blocks.append(Block(MLstm(c, heads, dqk, dhv), bp))
        else:
            blocks.append(Block(SLstm(c, d, nh_s), bp, post_norm=True))
    return Lm(params["table"], blocks, params["gamma"], head_w, head_b, cap=cap, tied=tied)
