"""Inference on the same kernels as training: stateful calls (a call's final recurrent state is the next
call's carry, the reference's chunked-carry API: src/gpu/mlstm.rs:598-623, src/gpu/slstm.rs:755-771),
greedy decoding, and head-sharded mLSTM blocks across the GPUs of one box.

Head sharding: in an mLSTM cell everything up to the output projection is local to a head (the q/k/v/i/f/o
projection columns, the state C, n, m, the head-wise norm and the output gate), so rank r keeps heads
[r*H/W, (r+1)*H/W) of every mLSTM block, runs the fused core on those alone, multiplies by its rows of W_out
and the partial [rows, d] products are summed with one all-reduce per block. Norms, SwiGLU, sLSTM blocks, the
embedding and the head are replicated. The reference has no multi-GPU path; this is new.
"""
import torch

from . import layers


def set_stateful(lm, on=True):
    """Switches every cell between training calls (zero state in, nothing kept) and inference calls."""
    for blk in lm.blocks:
        blk.cell.stateful = on
    reset_state(lm)


def reset_state(lm):
    for blk in lm.blocks:
        if isinstance(blk.cell, layers.MLstm):
            blk.cell.carry = None
        else:
            blk.cell.state = None


def last_logits(lm, ids, B, T):
    """Soft-capped logits [B, vocab] of the last of T positions; with stateful cells the call continues the
    sequences the previous calls left off."""
    normed = lm.forward_hidden(ids, B, T)
    last = normed.view(B, T, -1)[:, T - 1, :].contiguous()
    pre = torch.mm(last, lm.table.w.t()) if lm.tied else lm.head.forward(last)
    for blk in lm.blocks:
        blk.release()
    return torch.tanh_(pre.div_(lm.cap)).mul_(lm.cap)


@torch.no_grad()
def greedy_decode(lm, prompt_ids, n_new):
    """prompt_ids: int64 [B, Tp] on the GPU. Feeds the prompt in one call, then one position per call, always
    taking the arg-max token. Returns (new ids [B, n_new], the logits [n_new, B, vocab] they were picked from)."""
    B, Tp = prompt_ids.shape
    set_stateful(lm, True)
    out, seen = [], []
    logits = last_logits(lm, prompt_ids.reshape(-1), B, Tp)
    for _ in range(n_new):
        seen.append(logits)
        nxt = torch.argmax(logits, dim=1)
        out.append(nxt)
        logits = last_logits(lm, nxt, B, 1)
    set_stateful(lm, False)
    return torch.stack(out, dim=1), torch.stack(seen, dim=0)


def shard_mlstm_params(cell, heads, dqk, dhv, rank, world):
    """The slice of one mLSTM cell's host parameters that rank `rank` of `world` needs: its heads' columns of
    the six input projections, its heads' gains of the head-wise norm, its rows of W_out (b_out whole)."""
    assert heads % world == 0, "heads must divide evenly over the ranks"
    hl = heads // world
    h0, h1 = rank * hl, (rank + 1) * hl
    out = dict(kind="mlstm")
    for n, w in (("q", dqk), ("k", dqk), ("v", dhv), ("o", dhv), ("i", 1), ("f", 1)):
        out["w" + n] = cell["w" + n][:, h0 * w:h1 * w]
        out["b" + n] = cell["b" + n][h0 * w:h1 * w]
    out["gamma"] = cell["gamma"][h0 * dhv:h1 * dhv]
    out["w_out"] = cell["w_out"][h0 * dhv:h1 * dhv, :]
    out["b_out"] = cell["b_out"]
    return out


def build_lm_head_sharded(params, heads, dqk, dhv, rank, world, group=None, **kw):
    """`layers.build_lm` with every mLSTM block holding only this rank's heads (inference only: the backward of
    the sharded output projection is not wired)."""
    sharded = dict(params)
    sharded["blocks"] = []
    for bp in params["blocks"]:
        bp = dict(bp)
        if bp["cell"]["kind"] == "mlstm":
            bp["cell"] = shard_mlstm_params(bp["cell"], heads, dqk, dhv, rank, world)
        sharded["blocks"].append(bp)
    lm = layers.build_lm(sharded, heads // world, dqk, dhv, **kw)
    for blk in lm.blocks:
        if isinstance(blk.cell, layers.MLstm):
            blk.cell.shard_group = group if group is not None else torch.distributed.group.WORLD
    return lm
