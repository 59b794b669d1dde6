"""TEST INFRASTRUCTURE - CPU restatement (numpy, float64) of the reference's three-stage hierarchical model.
PARITY UNPINNED at the bit level: the reference cannot be built here and holds no fixtures for this model;
the restatement follows the reference's source.

One call = one or more windows of words (src/gpu/hierarchical.rs:725-778, phases in order):
  encoder   every word w < n-1 as one row of a [words, tmax] rectangle: its chars, then the [W] token, zero
            padded; Embedding(tied table) -> blocks; e_w = the row at the [W] step (:436-458, :899-956)
  backbone  Linear(hc->wh) -> blocks over the words of a window as one sequence -> Linear(wh->hc)
            (:959-1021); position w has read words 0..w and its output o_w conditions word w+1
  decoder   word w+1 as one row: slot 0 = o_w, slot k = table[char k-1]; blocks -> RMSNorm -> bias-free head
            -> SoftCap; targets = the chars then [W]; masked CE scaled by 1/valid rows of the whole call
            (:329-364, :1029-1132, :1142-1230)
Everything here is the plainest form: one rectangle per stage (the reference's own `no_group` baseline,
:117-134) and an unchunked backbone. Grouping by length and the chunked carry sweep are the product's batching
choices and must not change the result, which is what the tests compare against this file.
"""
import numpy as np

from . import model as M
from . import oracle as O


class HierCfg:
    """ModelCfg (src/gpu/hierarchical.rs:53-65). `small_heads`: heads of the encoder's and decoder's mLSTM
    blocks (16 in the reference, :88, :602-607)."""

    def __init__(self, vocab, hc, wh, enc_blocks, bb_blocks, dec_blocks, heads, dqk, w_token, cap=30.0, small_heads=16,
                 enc_kinds=None, bb_kinds=None, dec_kinds=None):
        self.vocab, self.hc, self.wh = vocab, hc, wh
        self.enc_blocks, self.bb_blocks, self.dec_blocks = enc_blocks, bb_blocks, dec_blocks
        self.heads, self.dqk, self.w_token, self.cap, self.small_heads = heads, dqk, w_token, cap, small_heads
        # block kinds: encoder and decoder alternate sLSTM, mLSTM (:88-108, :595-612); the backbone has an
        # sLSTM block at every eighth position (:576-594). A string of "s"/"m" overrides a stage's pattern.
        self.enc_kinds = enc_kinds or "".join("s" if i % 2 == 0 else "m" for i in range(enc_blocks))
        self.bb_kinds = bb_kinds or "".join("s" if i % 8 == 0 else "m" for i in range(bb_blocks))
        self.dec_kinds = dec_kinds or "".join("s" if i % 2 == 0 else "m" for i in range(dec_blocks))

    def stage(self, name):
        """(kinds, width, heads, dqk, dhv) of a stage's blocks."""
        if name == "bb":
            return self.bb_kinds, self.wh, self.heads, self.dqk, self.wh // self.heads
        sh = self.small_heads
        return (self.enc_kinds if name == "enc" else self.dec_kinds), self.hc, sh, self.hc // sh, self.hc // sh


def up_of(hidden):
    return hidden * 8 // 3  # src/gpu/hierarchical.rs:70-72


def init_hier_params(rng, cfg, std=0.02):
    """Seeded N(0, std) weights, norm gains 1: table, enc/bb/dec block lists, the two backbone projections, the
    decoder's norm and bias-free head."""
    def n(*shape):
        return (rng.standard_normal(shape) * std).astype(np.float32).astype(np.float64)

    def blocks(name):
        kinds, d, heads, dqk, dhv = cfg.stage(name)
        sl = tuple(i for i, k in enumerate(kinds) if k == "s")
        return M.init_lm_params(rng, 1, d, len(kinds), heads, dqk, dhv, up_of(d), std=std, slstm_at=sl)["blocks"]

    return dict(table=n(cfg.vocab, cfg.hc), enc=blocks("enc"), front_w=n(cfg.hc, cfg.wh), front_b=n(cfg.wh),
                bb=blocks("bb"), back_w=n(cfg.wh, cfg.hc), back_b=n(cfg.hc), dec=blocks("dec"),
                dec_gamma=np.ones(cfg.hc), head_w=n(cfg.hc, cfg.vocab))


def _build_blocks(plist, d, heads, dqk, dhv):
    out = []
    for bp in plist:
        c = bp["cell"]
        if c["kind"] == "mlstm":
            out.append(M.Block(M.MLstm(c, heads, dqk, dhv), bp))
        else:
            out.append(M.Block(M.SLstm(c, d, 1), bp, post_norm=True))
    return out


class Hierarchical:
    def __init__(self, params, cfg):
        self.cfg = cfg
        self.table = M.Param(params["table"], False)
        self.enc = _build_blocks(params["enc"], *cfg.stage("enc")[1:])
        self.front = M.Linear(params["front_w"], params["front_b"])
        self.bb = _build_blocks(params["bb"], *cfg.stage("bb")[1:])
        self.back = M.Linear(params["back_w"], params["back_b"])
        self.dec = _build_blocks(params["dec"], *cfg.stage("dec")[1:])
        self.dec_norm = M.RmsNorm(params["dec_gamma"])
        self.head = M.Param(params["head_w"], False)

    def params(self):
        out = [self.table]
        for blk in self.enc:
            out += blk.params()
        out += self.front.params()
        for blk in self.bb:
            out += blk.params()
        out += self.back.params()
        for blk in self.dec:
            out += blk.params()
        return out + self.dec_norm.params() + [self.head]

    def forward_backward(self, windows, word_loss=None):
        """windows: [(tokens, [(start, end), ...]), ...], every window with the same number of words.
        word_loss: per window one flag per decoded word (None = all on). Returns the mean CE over the
        unmasked decoder rows; gradients accumulate in the parameters."""
        cfg, hc = self.cfg, self.cfg.hc
        nw = len(windows[0][1])
        assert all(len(w) == nw for _, w in windows), "windows of one call must hold equally many words"
        dw, Bw = nw - 1, len(windows)
        if dw < 1:
            return 0.0
        N = Bw * dw  # row i = window i // dw, word i % dw

        def word(i, shift):
            tok, words = windows[i // dw]
            s, e = words[i % dw + shift]
            return tok[s:e]

        # encoder
        te = max(len(word(i, 0)) for i in range(N)) + 1
        ids = np.zeros((N, te), np.int64)
        readout = np.zeros(N, np.int64)
        for i in range(N):
            w = word(i, 0)
            ids[i, :len(w)] = w
            ids[i, len(w)] = cfg.w_token
            readout[i] = i * te + len(w)
        h = self.table.w[ids.reshape(-1)]
        for blk in self.enc:
            h = blk.forward(h, N, te)
        e_w = h[readout]
        # backbone
        hb = self.front.forward(e_w)
        for blk in self.bb:
            hb = blk.forward(hb, Bw, dw)
        o = self.back.forward(hb)
        # decoder
        td = max(len(word(i, 1)) for i in range(N)) + 1
        rows = N * td
        dec_in = np.zeros((rows, hc))
        targets = np.zeros(rows, np.uint32)
        mask = np.zeros(rows, np.uint32)
        char_rows, char_ids = [], []
        for i in range(N):
            w = word(i, 1)
            m = len(w)
            on = 1 if word_loss is None or word_loss[i // dw][i % dw] else 0
            dec_in[i * td] = o[i]
            for k in range(1, m + 1):
                char_rows.append(i * td + k)
                char_ids.append(w[k - 1])
            targets[i * td:i * td + m] = w
            targets[i * td + m] = cfg.w_token
            mask[i * td:i * td + m + 1] = on
        char_rows, char_ids = np.array(char_rows, np.int64), np.array(char_ids, np.int64)
        dec_in[char_rows] = self.table.w[char_ids]
        hd = dec_in
        for blk in self.dec:
            hd = blk.forward(hd, N, td)
        hdn = self.dec_norm.forward(hd)
        pre = hdn @ self.head.w
        capped = cfg.cap * np.tanh(pre / cfg.cap)
        valid = int(mask.sum())
        loss, d_capped = O.softmax_ce(capped, targets, mask=mask, inv=1.0 / max(valid, 1))
        self.last_rows = valid
        # decoder backward
        t = capped / cfg.cap
        d_pre = d_capped * (1.0 - t * t)
        self.head.g += hdn.T @ d_pre
        d = self.dec_norm.backward(d_pre @ self.head.w.T)
        for blk in reversed(self.dec):
            d = blk.backward(d)
        d_o = d[np.arange(N) * td]
        np.add.at(self.table.g, char_ids, d[char_rows])
        # backbone backward
        d = self.back.backward(d_o)
        for blk in reversed(self.bb):
            d = blk.backward(d)
        d_e_w = self.front.backward(d)
        # encoder backward
        d = np.zeros((N * te, hc))
        d[readout] = d_e_w
        for blk in reversed(self.enc):
            d = blk.backward(d)
        np.add.at(self.table.g, ids.reshape(-1), d)
        return loss
