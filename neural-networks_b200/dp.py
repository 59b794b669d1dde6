"""Data parallelism over batch: gradient buckets and their all-reduce, overlapped with backward.

The reference has no multi-GPU code (one `CudaContext::new(0)`, src/gpu/mod.rs:134); this is the
new piece the training step needs on N GPUs. Every rank holds a full replica and its own batch
shard; the only exchange is one SUM all-reduce of the gradients per step. Gradients live in flat
fp32 buckets (one per block, plus one for the embedding / final norm / head) so that a bucket can be
reduced with a single NCCL call as soon as the backward pass has finished writing it, while the
blocks below it are still computing. With the loss scaled by 1 / (rows * world) on every rank the
summed gradient is the gradient of the global mean loss, so N ranks reproduce one rank on the
concatenated batch.

Works on any torch.distributed backend (NCCL on GPUs; gloo in the CPU tests of the bucket logic).
"""
import torch
import torch.distributed as dist


class GradBuckets:
    def __init__(self, groups, group=None):
        """`groups`: list of lists of objects with `.w` (parameter) and `.g` (gradient) tensors. The
        gradients are re-homed into one flat buffer per group; `.g` becomes a view into it."""
        self.pg = group
        self.flat = []
        self.handles = []
        for params in groups:
            n = sum(p.g.numel() for p in params)
            if n == 0:
                self.flat.append(None)
                continue
            ref = params[0].g
            buf = torch.zeros((n,), dtype=ref.dtype, device=ref.device)
            off = 0
            for p in params:
                k = p.g.numel()
                view = buf[off:off + k].view_as(p.g)
                view.copy_(p.g)
                p.g = view
                off += k
            self.flat.append(buf)

    def world(self):
        return dist.get_world_size(self.pg) if dist.is_available() and dist.is_initialized() else 1

    def reduce_async(self, i):
        """Start the SUM all-reduce of bucket i (call when its gradients are complete)."""
        if self.world() == 1 or self.flat[i] is None:
            return
        self.handles.append(dist.all_reduce(self.flat[i], op=dist.ReduceOp.SUM, group=self.pg, async_op=True))

    def wait(self):
        """Block the current stream until every started reduction has finished."""
        for h in self.handles:
            h.wait()
        self.handles = []


def attach(lm, group=None):
    """Buckets for an `Lm`: one per block (reduced as soon as that block's backward is done) and a
    last one for the table, final norm and head (reduced after the embedding scatter)."""
    groups = [blk.params() for blk in lm.blocks]
    rest = [lm.table] + lm.norm.params() + (lm.head.params() if lm.head is not None else [])
    buckets = GradBuckets(groups + [rest], group)
    lm.on_block_backward = buckets.reduce_async
    return buckets


def train_step(lm, buckets, ids, targets, B, T, cfg):
    """One data-parallel step: local forward/backward with the loss scaled for the global batch,
    bucket all-reduces overlapped with backward, identical AdamW on every rank."""
    world = buckets.world()
    loss = lm.forward_backward(ids, targets, B, T, inv=1.0 / (B * T * world))
    buckets.reduce_async(len(lm.blocks))
    buckets.wait()
    lm.step(cfg)
    return loss


def attach_hier(model, group=None):
    """Buckets for a `hier.Hierarchical`: decoder stage, backbone stage, encoder stage + tied table, each reduced
    as soon as its part of the window's backward is done. The loss normaliser becomes the valid decoder rows of
    all ranks (the ranks' windows differ in length), one small all-reduce per call."""
    buckets = GradBuckets(model.stage_params(), group)
    model.on_stage_backward = buckets.reduce_async

    def rows_of_all_ranks(valid):
        if buckets.world() == 1:
            return valid
        t = torch.tensor([valid], dtype=torch.int64, device=model.loss.device)
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
        return int(t.item())

    model.rows_of_all_ranks = rows_of_all_ranks
    return buckets


def train_step_hier(model, buckets, windows, cfg, word_loss=None):
    """One data-parallel step of the hierarchical model: every rank its own windows, gradients summed, identical
    AdamW everywhere. Returns this rank's share of the global mean loss."""
    loss = model.forward_backward(windows, word_loss)
    buckets.wait()
    model.step(cfg)
    return loss
