"""Context parallelism for the mLSTM core: one sequence cut into W consecutive segments, one per GPU, on the
call-level carry API (carry (C, n, m) in, state out; BPTT state (dC, dn) in, gradient of the carry out). The
reference is single-GPU; this is new.

The recurrence is linear in (C, n) once the gates are known, so a segment is summarised by what it does to an
incoming state. With F = sum of log sigmoid(f) over the segment and, from a pass that enters with an empty state
and m = -inf, the segment's own (C_s, n_s, M_s) (M_s = max_t (i_t + sum of later log f), exactly the recurrent
stabiliser when nothing precedes):
    m' = max(F + m, M_s),   C' = e^(F + m - m') C + e^(M_s - m') C_s,   n' likewise.
m' is the recurrent m the single-GPU run has at the segment's end, so psi = max(|q.n|, e^-m) sees the same floor.
Forward per rank: summary pass -> all-gather of the summaries -> fold the ranks to the left -> the real pass
with that carry. Backward: the gradient of a segment's carry is (its own, with nothing coming from the right) +
t * (what comes from the right), t = e^(F + m_in - m_out) per (batch, head), because m is a constant of the
backward. So: one backward with no BPTT state gives the local term, an all-gather of those and of t, a suffix sum
gives each rank the BPTT state it must enter with, and the real backward runs with it. Two forward and two
backward passes per layer instead of one; what it buys is a sequence W times longer than one GPU holds, and
per-GPU time that does not grow with W.

The functions take `gather(tensor) -> [tensor of rank 0, ..., tensor of rank W-1]`, so the same code runs over
`torch.distributed` (`dist_gather(group)`) and, for tests on one GPU, over a list filled rank by rank.
"""
import torch

from . import ops

NO_HISTORY = -1.0e30  # m of "nothing precedes": e^(log f + m - m_1) underflows to exactly 0, so m_1 = i_1


def _flat(parts):
    return torch.cat([p.reshape(p.shape[0], -1) for p in parts], dim=1)


def _log_forget_sum(fg, st):
    """F = sum over the segment of log sigmoid(f), [BH, 1] (summed in fp64: T terms of either sign of rounding)."""
    return torch.nn.functional.logsigmoid(fg).view(st.b, st.t, st.h).sum(dim=1, dtype=torch.float64).float().reshape(st.bh(), 1)


def segment_summary(q, k, v, ig, fg, st):
    """[BH, dhv*dqk + dqk + 2]: the segment's own (C_s, n_s, M_s) and F, one row per (batch, head)."""
    bh = st.bh()
    dev = q.device
    empty = (torch.zeros((bh, st.dhv, st.dqk), dtype=torch.float32, device=dev),
             torch.zeros((bh, st.dqk), dtype=torch.float32, device=dev),
             torch.full((bh,), NO_HISTORY, dtype=torch.float32, device=dev))
    own = ops.mlstm_final_state(q, k, v, ig, fg, st, carry_in=empty)
    return _flat([own[0], own[1], own[2].reshape(bh, 1), _log_forget_sum(fg, st)])


def fold(summaries, rank, st):
    """The state rank `rank` enters with: the whole-sequence start (C = 0, n = 0, m = 0) pushed through the
    summaries of ranks 0..rank-1. None for rank 0."""
    if rank == 0:
        return None
    bh, dc, dn = st.bh(), st.dhv * st.dqk, st.dqk
    C = torch.zeros((bh, dc), dtype=torch.float32, device=summaries[0].device)
    n = torch.zeros((bh, dn), dtype=torch.float32, device=C.device)
    m = torch.zeros((bh, 1), dtype=torch.float32, device=C.device)
    for s in summaries[:rank]:
        Cs, ns, Ms, F = s[:, :dc], s[:, dc:dc + dn], s[:, dc + dn:dc + dn + 1], s[:, dc + dn + 1:]
        m2 = torch.maximum(F + m, Ms)
        a, b = torch.exp(F + m - m2), torch.exp(Ms - m2)
        C, n, m = a * C + b * Cs, a * n + b * ns, m2
    return C.view(bh, st.dhv, st.dqk).contiguous(), n.contiguous(), m.reshape(bh).contiguous()


def forward(q, k, v, ig, fg, st, rank, gather):
    """The fused forward of this rank's segment inside the whole sequence. Returns (fused, carry_in)."""
    mine = segment_summary(q, k, v, ig, fg, st)
    carry = fold(gather(mine), rank, st)
    fused = ops.mlstm_fused_fw(q, k, v, ig, fg, st, carry_in=carry, save_states=True, want_state=True)
    fused.log_forget_sum = mine[:, -1:]  # the backward's transport factor needs it again
    return fused, carry


def backward(fused, q, k, v, ig, fg, d_ytil, st, carry, rank, world, gather):
    """The fused backward of this rank's segment. Returns (dq, dk, dv, dig, dfg)."""
    bh, dc = st.bh(), st.dhv * st.dqk
    if world == 1:
        return ops.mlstm_fused_bw(fused, q, k, v, ig, fg, d_ytil, st, carry_in=carry, want_dstate=False)[:5]
    # the local term: what this segment's own outputs send into its carry
    own = ops.mlstm_fused_bw(fused, q, k, v, ig, fg, d_ytil, st, carry_in=carry, want_dstate=True)
    F = fused.log_forget_sum if hasattr(fused, "log_forget_sum") else _log_forget_sum(fg, st)
    m_in = carry[2].reshape(bh, 1) if carry is not None else torch.zeros_like(F)
    t = torch.exp(F + m_in - fused.state[2].reshape(bh, 1))
    parts = gather(_flat([own[5][0], own[5][1], t]))
    if rank == world - 1:
        return own[:5]  # nothing comes from the right: the first pass already is the answer
    # G_r = own_{r+1} + t_{r+1} G_{r+1}, G_{W-1} = 0
    G = torch.zeros_like(parts[0][:, :-1])
    for s in range(world - 1, rank, -1):
        G = parts[s][:, :-1] + parts[s][:, -1:] * G
    dstate = (G[:, :dc].reshape(bh, st.dhv, st.dqk).contiguous(), G[:, dc:].contiguous())
    return ops.mlstm_fused_bw(fused, q, k, v, ig, fg, d_ytil, st, carry_in=carry, dstate_in=dstate, want_dstate=False)[:5]


def dist_gather(group=None):
    """`gather` over a torch.distributed process group (NCCL all-gather of equally shaped tensors)."""
    import torch.distributed as dist

    def gather(t):
        out = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
        dist.all_gather(out, t.contiguous(), group=group)
        return out

    return gather


def enable(lm, rank, world, group=None, gather=None):
    """Turns a model's mLSTM cells into context-parallel ones: every call then treats its [B, T] input as segment
    `rank` of `world` of a sequence `world` times as long. Everything else in a block is position-wise and needs
    nothing. Gradients of the parameters are partial sums over this rank's positions: add them over the ranks as
    data parallelism does (`dp.attach`, whose loss scale 1/(B T world) is the whole sequence's). An sLSTM cell is
    refused: its recurrence is not linear in its state, so there is no summary to fold; it needs the state handed
    from rank to rank."""
    from . import layers

    g = gather if gather is not None else dist_gather(group)
    for blk in lm.blocks:
        if not isinstance(blk.cell, layers.MLstm):
            raise ValueError("context parallelism covers mLSTM blocks; this model has an sLSTM block")
        blk.cell.cp = (rank, world, g)
