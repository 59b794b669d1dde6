"""Data parallelism over batch: gradient buckets and their all-reduce, overlapped with backward.

The reference has no multi-GPU code (one `CudaContext::new(0)`, src/gpu/mod.rs:134); this is the
new piece the training step needs on N GPUs. Every rank holds a full replica and its own batch
shard; the only exchange is one SUM all-reduce of the gradients per step. Gradients live in flat
fp32 buckets (one per block, plus one for the embedding / final norm / head) so that a bucket can be
reduced with a single NCCL call as soon as the backward pass has finished writing it, while the
blocks below it are still computing. With the loss scaled by 1 / (rows * world) on every rank the
summed gradient is the gradient of the global mean loss, so N ranks reproduce one rank on the
concatenated batch.

On GPUs the buckets go through the library's own entry points (xlstm_dp_*, include/xlstm_b200.h): the
communicator is created inside libxlstm_b200.so from a unique id that rank 0 hands out over torch.distributed,
each bucket's all-reduce is ordered behind the backward pass on the library's side stream, and the optimizer's
stream waits for them before AdamW. On CPU tensors (the gloo tests of the bucket logic) the same class issues
torch.distributed all-reduces.
"""
import importlib

import torch
import torch.distributed as dist


def _native_lib():
    return importlib.import_module("neural-networks_b200")._lib


class GradBuckets:
    def __init__(self, groups, group=None, native=None):
        """`groups`: list of lists of objects with `.w` (parameter) and `.g` (gradient) tensors. The
        gradients are re-homed into one flat buffer per group; `.g` becomes a view into it.
        `native`: reduce through xlstm_dp_* (default: whenever the gradients are CUDA tensors, the default
        process group is NCCL and there is more than one rank)."""
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
        on_gpu = any(b is not None and b.is_cuda for b in self.flat)
        if native is None:
            native = on_gpu and group is None and self.world() > 1 and dist.get_backend() == "nccl"
        self.native = bool(native)
        self.index = [None] * len(self.flat)
        self.exposed = None  # (event before, event after) of the last wait(), when `time_wait` is set
        self.time_wait = False
        if self.native:
            self._init_native()

    def _init_native(self):
        L = _native_lib()
        lib = L.lib
        world, rank = self.world(), dist.get_rank()
        if lib.xlstm_dp_world() == 0:
            uid = torch.zeros(128, dtype=torch.uint8)
            if rank == 0:
                L.check(lib.xlstm_dp_unique_id(uid.data_ptr()), "dp_unique_id")
            dev = uid.cuda()
            dist.broadcast(dev, src=0)
            uid = dev.cpu()
            L.check(lib.xlstm_dp_init(world, rank, uid.data_ptr()), "dp_init")
        elif lib.xlstm_dp_world() != world:
            raise L.XlstmError("xlstm_dp: the library's communicator has %d ranks, the process group %d" % (lib.xlstm_dp_world(), world))
        for i, buf in enumerate(self.flat):
            if buf is None:
                continue
            if buf.dtype != torch.float32:
                raise L.XlstmError("xlstm_dp buckets are fp32")
            idx = lib.xlstm_dp_bucket_register(buf.data_ptr(), buf.numel())
            if idx < 0:
                L.check(idx, "dp_bucket_register")
            self.index[i] = idx

    def world(self):
        return dist.get_world_size(self.pg) if dist.is_available() and dist.is_initialized() else 1

    def reduce_async(self, i):
        """Start the SUM all-reduce of bucket i (call when its gradients are complete)."""
        if self.world() == 1 or self.flat[i] is None:
            return
        if self.native:
            L = _native_lib()
            L.check(L.lib.xlstm_dp_bucket_start(self.index[i], torch.cuda.current_stream().cuda_stream), "dp_bucket_start")
            return
        self.handles.append(dist.all_reduce(self.flat[i], op=dist.ReduceOp.SUM, group=self.pg, async_op=True))

    def wait(self):
        """Make the current stream wait until every started reduction has finished."""
        timed = self.time_wait and any(b is not None and b.is_cuda for b in self.flat)
        if timed:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        if self.native and self.world() > 1:
            L = _native_lib()
            L.check(L.lib.xlstm_dp_wait(torch.cuda.current_stream().cuda_stream), "dp_wait")
        for h in self.handles:
            h.wait()
        self.handles = []
        if timed:
            e1.record()
            self.exposed = (e0, e1)

    def exposed_ms(self):
        """Device time the stream spent stalled in the last wait() (needs `time_wait`; synchronises)."""
        if self.exposed is None:
            return 0.0
        self.exposed[1].synchronize()
        return self.exposed[0].elapsed_time(self.exposed[1])


def attach(lm, group=None, gather_at_slstm=None):
    """Buckets for an `Lm`: one per block and a last one for the table, final norm and head (reduced after the
    embedding scatter). A block's all-reduce starts as soon as its backward is done, or, with `gather_at_slstm`
    (default: on when the model has sLSTM blocks), when the next sLSTM backward time loop is launched: that kernel
    is latency-bound on 128 SMs and leaves HBM and NVLink idle, whereas an all-reduce beside the backward's GEMMs
    takes SMs from kernels sized for all 148 (measured at N = 2: 246 against 237 ms of GEMMs per step)."""
    from . import layers
    groups = [blk.params() for blk in lm.blocks]
    rest = [lm.table] + lm.norm.params() + (lm.head.params() if lm.head is not None else [])
    buckets = GradBuckets(groups + [rest], group)
    cells = [blk.cell for blk in lm.blocks if isinstance(blk.cell, layers.SLstm)]
    if gather_at_slstm is None:
        gather_at_slstm = bool(cells)
    if not gather_at_slstm or not cells:
        lm.on_block_backward = buckets.reduce_async
        return buckets
    pending = []

    def flush():
        for i in pending:
            buckets.reduce_async(i)
        del pending[:]

    def done(i):
        if i >= len(lm.blocks) or i == 0:  # the last block of the backward pass, or the table's bucket: nothing left to wait for
            flush()
            buckets.reduce_async(i)
        else:
            pending.append(i)

    for c in cells:
        c.before_time_loop = flush
    lm.on_block_backward = done
    buckets.reduce_async_deferred = done
    return buckets


def train_step(lm, buckets, ids, targets, B, T, cfg):
    """One data-parallel step: local forward/backward with the loss scaled for the global batch,
    bucket all-reduces overlapped with backward, identical AdamW on every rank."""
    world = buckets.world()
    loss = lm.forward_backward(ids, targets, B, T, inv=1.0 / (B * T * world))
    getattr(buckets, "reduce_async_deferred", buckets.reduce_async)(len(lm.blocks))
    buckets.wait()
    if getattr(lm, "check_status", False):  # waits for the backward pass; raises before the update is applied
        from . import ops
        ops.device_status_check()
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
    loss = model.forward_backward(windows, word_loss)  # reads the loss back: the backward pass has finished
    buckets.wait()
    if getattr(model, "check_status", False):
        from . import ops
        ops.device_status_check()
    model.step(cfg)
    return loss
