#!/usr/bin/env python
"""Benchmark of the xLSTM hot path on B200.

Default workload: the mLSTM layer kernel, forward + backward, at B=16 H=8 S=2048
d_qk=d_v=128 chunk 64, q/k/v bf16 ~N(0,1) (k pre-scaled by 1/sqrt(d_qk), the contract of the
op), gate logits fp32 (input N(0,1), forget N(3,1)), zero initial state, upstream grad N(0,1).
One "step" is one forward + backward over that batch. With N GPUs every rank runs the same
per-GPU batch (the path shards over batch with no data-path collective): weak scaling.

Prints ONE JSON line (rank 0). `value` is device-timed with inputs resident in HBM; `e2e` is
the same step through the public op API starting from pinned HOST buffers, host<->device
copies inside the timed region. `--impl reference` times the CPU restatement of the
reference's layer math (the reference itself is a Rust crate that cannot be built here) on
the host cores, on a bounded sample of the same workload.
"""
import argparse
import ctypes
import importlib
import json
import math
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(B=16, H=8, T=2048, dqk=128, dhv=128, L=64)


def flops_fwd_bwd(B, H, T, dqk, dhv, L):
    """Causal-exact contraction FLOPs of one forward + backward (L^2 terms counted as L(L+1)/2)."""
    nchunks = B * H * (T // L)
    fwd = L * (L + 1) * (dqk + dhv) + 4 * L * dqk * dhv
    bwd = L * (L + 1) * (3 * dqk + 2 * dhv) + 8 * L * dqk * dhv
    return nchunks * fwd, nchunks * bwd


def algorithmic_bytes(B, H, T, dqk, dhv, gbytes):
    """Compulsory HBM traffic of the op: inputs once, outputs once; chunk states excluded."""
    n = B * T * H
    qkv = n * (2 * dqk + dhv) * 2
    gates = n * 2 * 4
    ytil = n * dhv * 2
    scal = n * 2 * 4  # m, psi
    fwd = qkv + gates + ytil + scal
    bwd = qkv + gates + ytil + scal + n * dhv * gbytes + n * (2 * dqk + dhv) * gbytes + gates
    return fwd, bwd


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=d["hbm_gbs"], tensor=d["bf16_tflops"], src="measured")
    return dict(hbm=6650.0, tensor=1590.0, src="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks while the timed region runs."""

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def make_inputs(cfg, seed):
    """Seeded synthetic inputs of the workload on the host (numpy)."""
    r = np.random.default_rng(seed)
    B, H, T, dqk, dhv = cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"]
    n = B * T
    q = r.standard_normal((n, H * dqk), dtype=np.float32)
    k = r.standard_normal((n, H * dqk), dtype=np.float32) / np.float32(np.sqrt(dqk))
    v = r.standard_normal((n, H * dhv), dtype=np.float32)
    ig = r.standard_normal((n, H), dtype=np.float32)
    fg = r.standard_normal((n, H), dtype=np.float32) + np.float32(3.0)
    dy = r.standard_normal((n, H * dhv), dtype=np.float32)
    return q, k, v, ig, fg, dy


def cpu_sample(seconds_target=15.0, threads=None):
    """Times the CPU restatement (f32) on a slice of the workload: Bs sequences of the full length."""
    from oracle import oracle as O
    cfg = dict(CFG)
    ncores = os.cpu_count() or 1
    threads = threads or min(ncores, 64)  # each worker holds ~134 MB of per-step records
    os.environ["OMP_NUM_THREADS"] = str(threads)
    Bs = max(1, min(cfg["B"], (4 * threads + cfg["H"] - 1) // cfg["H"]))
    cfg["B"] = Bs
    q, k, v, ig, fg, dy = make_inputs(cfg, 0)
    args = (cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"])
    t0 = time.perf_counter()
    O.mlstm_core_fw(q, k, v, ig, fg, *args, dtype=np.float32)
    O.mlstm_core_bw(q, k, v, ig, fg, dy, *args, dtype=np.float32)
    dt = time.perf_counter() - t0
    f, b = flops_fwd_bwd(**cfg)
    return dict(seconds=dt, flops=f + b, tokens=Bs * cfg["T"], Bs=Bs, threads=threads)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    times = []
    for i in range(args.warmup + args.steps):
        s = cpu_sample()
        if i >= args.warmup:
            times.append(s["seconds"])
    t = float(np.mean(times))
    val = s["flops"] / t / 1e12
    line = {
        "impl": "reference", "metric": "mlstm_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "mlstm_layer_fwd_bwd B16 H8 S2048 dqk128 dv128 chunk64 (configs[1])",
                   "sample": "B=%d of 16 sequences, full length" % s["Bs"]},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": s["threads"], "kind": "port",
                         "sample": "%d of 16 sequences x 2048 positions x 8 heads, recurrent f32 oracle, OpenMP over (batch, head)" % s["Bs"]},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": s["tokens"] / t,
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    ops = xl.ops
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = dict(CFG)
    gd = torch.bfloat16 if args.grad_dtype == "bf16" else torch.float32
    st = ops.MlstmShape(cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], cfg["L"], torch.bfloat16, gd, 0)
    hq, hk, hv, hig, hfg, hdy = make_inputs(cfg, 1000 + rank)
    pin = lambda a, dt: torch.from_numpy(a).to(dt).pin_memory()
    host_in = [pin(hq, torch.bfloat16), pin(hk, torch.bfloat16), pin(hv, torch.bfloat16), pin(hig, torch.float32),
               pin(hfg, torch.float32), pin(hdy, gd)]
    dev_in = [t.cuda(non_blocking=True) for t in host_in]
    torch.cuda.synchronize()
    q, k, v, ig, fg, dy = dev_in

    marks = []  # (before forward, between, after backward) events of every timed step

    def step(timed=False):
        if timed:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            marks.append(ev)
            ev[0].record()
        fused = ops.mlstm_fused_fw(q, k, v, ig, fg, st, save_states=not args.recompute, want_state=False)
        if timed:
            ev[1].record()
        g = ops.mlstm_fused_bw(fused, q, k, v, ig, fg, dy, st, want_dstate=False)
        if timed:
            ev[2].record()
        return fused, g

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()

    # ---- device-timed steps (inputs resident) -------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step(timed=True)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = xl._lib.lib.xlstm_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps

    # ---- per-kernel durations for the roofline: CUDA events around each op inside the timed region above.
    # The device runs behind the host there, so the gap between two marks is the op's kernels and nothing else.
    fw_t = float(np.median([m[0].elapsed_time(m[1]) for m in marks]))
    bw_t = float(np.median([m[1].elapsed_time(m[2]) for m in marks]))

    # ---- end to end from pinned host buffers ----------------------------------------------
    # Every step copies its inputs from pinned host memory, runs forward + backward through `ops`, and copies every
    # result back to pinned host memory; all of it is inside the timed region. The three stages run on three
    # streams with double-buffered device inputs, so step i+1's upload and step i-1's download overlap step i
    # (PCIe is full duplex): steady state is the slower of the two copy directions, not their sum.
    s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
    dbuf = [[torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in host_in] for _ in range(2)]
    outs_host = None
    free_ev = [None, None]  # compute finished reading device-input set j

    def e2e_run(nsteps):
        nonlocal outs_host
        last_out = None
        for i in range(nsteps):
            j = i & 1
            with torch.cuda.stream(s_in):
                if free_ev[j] is not None:
                    s_in.wait_event(free_ev[j])
                for dst, src in zip(dbuf[j], host_in):
                    dst.copy_(src, non_blocking=True)
                ev_in = torch.cuda.Event(); ev_in.record(s_in)
            s_cmp.wait_event(ev_in)
            d = dbuf[j]
            fused = ops.mlstm_fused_fw(d[0], d[1], d[2], d[3], d[4], st, save_states=not args.recompute, want_state=False)
            g = ops.mlstm_fused_bw(fused, d[0], d[1], d[2], d[3], d[4], d[5], st, want_dstate=False)
            res = [fused.ytil, g[0], g[1], g[2], g[3], g[4]]
            ev_c = torch.cuda.Event(); ev_c.record(s_cmp)
            free_ev[j] = ev_c
            if outs_host is None:
                outs_host = [[torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res] for _ in range(2)]
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                for h, r in zip(outs_host[j], res):
                    r.record_stream(s_out)
                    h.copy_(r, non_blocking=True)
                last_out = torch.cuda.Event(); last_out.record(s_out)
        s_cmp.wait_event(last_out)  # the timed region ends when the last result is on the host

    e2e_steps = max(2, min(args.steps, 6))
    e2e_run(2)
    barrier()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_ms /= e2e_steps
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in outs_host[0])

    if rank == 0:
        ff, fb = flops_fwd_bwd(**cfg)
        gb = 2 if gd == torch.bfloat16 else 4
        bf, bb = algorithmic_bytes(cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], gb)
        pk = peaks()
        tokens = cfg["B"] * cfg["T"]
        value = (ff + fb) * world / (ms_per_step * 1e-3) / 1e12
        achieved = bb / (bw_t * 1e-3) / 1e9
        # dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of this workload at its default
        # settings (profiles/mlstm_tc_cfg2.md); includes the 138 MB chunk-state record, which the algorithmic bytes
        # leave out. Other settings were not captured.
        default_cfg = args.grad_dtype == "f32" and not args.recompute and cfg["B"] == 16
        traffic = {"bw": 545305088 + 368029952, "fw": 203553280 + 163480320} if default_cfg else {"bw": None, "fw": None}
        cpu = cpu_sample() if world == 1 and not args.no_cpu else None
        line = {
            "metric": "mlstm_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlstm_layer_fwd_bwd B16 H8 S2048 dqk128 dv128 chunk64 (configs[1])",
                       "per_gpu_batch": cfg["B"], "grad_dtype": args.grad_dtype,
                       "chunk_states": "recomputed in backward" if args.recompute else "saved by forward",
                       "l2": "inputs (%.0f MB) larger than L2" % ((bf + bb) / 1e6), "parallelism": "dp%d (batch shards, no collective)" % world},
            "tokens_per_s": tokens * world / (ms_per_step * 1e-3),
            "frac_of_bf16_peak": value / world / pk["tensor"],
            "roofline": {"kernel": "mlstm backward", "bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                         "frac": achieved / pk["hbm"], "traffic": traffic["bw"], "peak_source": pk["src"],
                         "algorithmic_bytes": bb, "launch_ms": bw_t,
                         "forward": {"achieved": bf / (fw_t * 1e-3) / 1e9, "frac": bf / (fw_t * 1e-3) / 1e9 / pk["hbm"],
                                     "algorithmic_bytes": bf, "launch_ms": fw_t, "traffic": traffic["fw"]}},
            "e2e": {"value": (ff + fb) * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if cpu is not None:
            line["cpu_baseline"] = {"value": cpu["flops"] / cpu["seconds"] / 1e12, "unit": "TFLOP/s", "cores": cpu["threads"],
                                    "kind": "port", "seconds": cpu["seconds"],
                                    "sample": "%d of 16 sequences x 2048 positions x 8 heads, recurrent f32 oracle, OpenMP over (batch, head)" % cpu["Bs"]}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


LM_CFG = dict(vocab=50304, d=1024, blocks=24, heads=8, dqk=128, dhv=128, slstm_every=8, slstm_heads=4, B=8, T=4096)
# configs[3] at its own widths: d = 2048, mLSTM 8 heads x 256, sLSTM 4 heads x 512
LM_CFG_FULL = dict(vocab=50304, d=2048, blocks=24, heads=8, dqk=256, dhv=256, slstm_every=8, slstm_heads=4, B=8, T=4096)


def run_lm(args):
    """Secondary workload: a data-parallel training step of an xLSTM LM with configs[3]'s structure
    (24 blocks, one sLSTM per 8, vocab 50304, per-GPU batch 8 x 4096, bf16 GEMM operands, fp32 master
    weights, AdamW) at d = 1024 with mLSTM heads of 128 and sLSTM heads of 256 -- the widths the
    kernels cover today (configs[3] itself asks for d = 2048 with heads of 256 / 512)."""
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    layers = importlib.import_module("neural-networks_b200.layers")
    dp = importlib.import_module("neural-networks_b200.dp")
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    c = dict(LM_CFG_FULL if args.lm_full else LM_CFG)
    if args.lm_blocks:
        c["blocks"] = args.lm_blocks
    up = (8 * c["d"] // 3 + 7) // 8 * 8
    rng = np.random.default_rng(0)  # identical replicas on every rank
    slstm_at = tuple(i for i in range(c["blocks"]) if i % c["slstm_every"] == 0)
    p = layers.init_lm_params(rng, c["vocab"], c["d"], c["blocks"], c["heads"], c["dqk"], c["dhv"], up, std=0.02, slstm_at=slstm_at,
                         nh_s=c["slstm_heads"])
    # full widths: the first `--lm-remat` mLSTM blocks keep only their input and re-run their forward in the
    # backward, so that 24 blocks fit in HBM; sLSTM blocks (the long sequential loops) are never re-run
    remat = [i for i in range(c["blocks"]) if i not in slstm_at][:args.lm_remat] if args.lm_full else ()
    # (the reduced model needs none); the head runs row-chunked with fp32-accurate split-bf16 products in both
    lm = layers.build_lm(p, c["heads"], c["dqk"], c["dhv"], nh_s=c["slstm_heads"], tied=True, bf16=True,
                         remat=remat, head_rows=4096, head_split=True)
    nparams = sum(q.w.numel() for q in lm.params())
    buckets = dp.attach(lm)
    B, T = c["B"], c["T"]
    g = torch.Generator().manual_seed(1234 + rank)
    host_ids = torch.randint(0, c["vocab"], (B, T + 1), generator=g).pin_memory()
    cfg = xl.ops.AdamCfg(1e-3, 0.1, t=0)

    def step():
        cfg.t += 1
        d = host_ids.cuda(non_blocking=True)
        ids = d[:, :-1].reshape(-1)
        tg = d[:, 1:].reshape(-1).to(torch.int32)
        return dp.train_step(lm, buckets, ids, tg, B, T, cfg)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        loss = step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step()
        lv = loss.item()  # the step's result read back on the host, as a training loop does
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = xl._lib.lib.xlstm_launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms /= args.steps
    if rank == 0:
        tokens = B * T
        pk = peaks()
        sustained = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained", pk["tensor"]) \
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1400.0
        flops = 6.0 * nparams * tokens
        val = tokens * world / (ms * 1e-3)
        line = {"metric": "train_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": ("xlstm_lm_train_step (configs[3] widths: d=%d, mLSTM %dx%d, sLSTM %dx%d)" if args.lm_full else
                                        "xlstm_lm_train_step (reduced stand-in for configs[3]: d=%d, mLSTM %dx%d, sLSTM %dx%d)")
                                       % (c["d"], c["heads"], c["dqk"], c["slstm_heads"], c["d"] // c["slstm_heads"]),
                           "blocks": c["blocks"], "vocab": c["vocab"], "params": nparams, "per_gpu_batch": [B, T],
                           "parallelism": "dp%d (gradient all-reduce per block, overlapped with backward)" % world,
                           "l2": "activations far larger than L2"},
                "loss": lv, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
                "roofline": {"kernel": "whole step (6*P*tokens dense FLOPs)", "bound": "tensor", "achieved": flops / (ms * 1e-3) / 1e12,
                             "peak": sustained, "unit": "TFLOP/s", "frac": flops / (ms * 1e-3) / 1e12 / sustained, "traffic": None,
                             "peak_source": pk["src"] + " (sustained)"},
                "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": host_ids.numel() * 8, "d2h_bytes_per_step": 4,
                        "note": "the timed step already starts from pinned host ids and reads the loss back"},
                "gpu_launches": int(launches), "clocks": clocks}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_ops(args):
    """Secondary workload: each remaining hot-path kernel on its own, at the sizes of configs[2] and
    configs[3]: HBM-bound kernels as achieved GB/s against the measured copy peak, the sLSTM loops as
    microseconds per timestep. One JSON line."""
    import torch
    xl = importlib.import_module("neural-networks_b200")
    ops = xl.ops
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if int(os.environ.get("RANK", "0")) != 0:
        return
    pk = peaks()
    n_it, warm = max(args.steps, 5), max(args.warmup, 3)

    def timeit(fn, n=n_it, w=warm):
        for _ in range(w):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    res = {}

    def hbm(name, nbytes, ms):
        gbs = nbytes / (ms * 1e-3) / 1e9
        res[name] = {"ms": ms, "algorithmic_bytes": nbytes, "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / pk["hbm"]}

    l0 = xl._lib.lib.xlstm_launch_count()
    rows, F = 32768, 2048
    for group in (2048, 256):
        x = torch.randn(rows, F, device="cuda"); gam = torch.ones(F, device="cuda"); y = torch.empty_like(x)
        inv = torch.empty(rows * F // group, device="cuda"); dy = torch.randn_like(x); dx = torch.empty_like(x); dg = torch.zeros(F, device="cuda")
        hbm("rmsnorm_fw_%dx%d_g%d" % (rows, F, group), 8 * rows * F, timeit(lambda: ops.rms_norm_forward_into(x, gam, group, y, inv)))
        hbm("rmsnorm_bw_%dx%d_g%d" % (rows, F, group), 12 * rows * F, timeit(lambda: ops.rms_norm_backward_into(dy, x, inv, gam, group, dx, dg)))
        del x, y, dy, dx
    for r_, C in ((8192, 50304), (65536, 256)):
        z = torch.randn(r_, C, device="cuda"); t = torch.randint(0, C, (r_,), device="cuda", dtype=torch.int32)
        d = torch.empty_like(z); acc = torch.zeros(1, device="cuda")
        hbm("ce_fw_bw_%dx%d" % (r_, C), 8 * r_ * C, timeit(lambda: ops.softmax_cross_entropy(z, t, d, acc)))
        del z, d
    n = 256 * 1024 * 1024
    p_ = torch.randn(n, device="cuda"); g_ = torch.randn(n, device="cuda"); m_ = torch.zeros(n, device="cuda"); v_ = torch.zeros(n, device="cuda")
    pb = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    cfg = ops.AdamCfg(1e-3, 0.1, t=1)
    hbm("adamw_%d" % n, 28 * n, timeit(lambda: ops.adamw(p_, g_, m_, v_, cfg, True)))
    hbm("adamw_shadow_zero_%d" % n, 34 * n, timeit(lambda: ops.adamw(p_, g_, m_, v_, cfg, True, p_bf16=pb, zero_grad=True)))
    del p_, g_, m_, v_, pb
    B, H, NH, T = 32, 1024, 4, 1024
    wh = torch.randn(NH, H // NH, 4 * H // NH, device="cuda") / 16; g = torch.randn(B, T, 4 * H, device="cuda"); bc = torch.zeros(4 * H, device="cuda")
    st = tuple(torch.zeros(B, H, device="cuda") for _ in range(4)); out = torch.empty(B, T, H, device="cuda"); slabs = ops.SlstmSlabs(B, T, H, "cuda")
    dy = torch.randn(B, T, H, device="cuda"); ds = tuple(torch.zeros(B, H, device="cuda") for _ in range(3))
    tf = timeit(lambda: ops.slstm_fused_time(wh, g, bc, st, out, slabs, nh=NH), n=10, w=20)
    tb = timeit(lambda: ops.slstm_fused_time_bwd(wh, dy, g, ds, slabs, nh=NH), n=10, w=20)
    res["slstm_fw_B32_H1024_NH4_T1024"] = {"ms": tf, "us_per_timestep": tf * 1e3 / T}
    res["slstm_bw_B32_H1024_NH4_T1024"] = {"ms": tb, "us_per_timestep": tb * 1e3 / T}
    launches = xl._lib.lib.xlstm_launch_count() - l0
    worst = min(v["frac_of_hbm_peak"] for k, v in res.items() if "frac_of_hbm_peak" in v and not k.startswith("ce_fw_bw_65536"))
    print(json.dumps({"metric": "op_microbench_min_hbm_fraction", "value": worst, "unit": "fraction of measured HBM peak", "n_gpus": 1,
                      "steps": n_it, "warmup": warm, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "rmsnorm / cross-entropy / adamw / slstm kernels alone", "l2": "tensors larger than L2"},
                      "peak": pk, "kernels": res, "gpu_launches": int(launches)}))


def run_hier(args):
    """Secondary workload: configs[4], one training step of the three-stage hierarchical model: bytes [16, 8192] in
    words of 8, lower stacks 2 mLSTM blocks of width 256, backbone 8 mLSTM blocks of width 1024 (8 x 128), bf16 GEMM
    operands, fp32 master weights, AdamW. The timed step starts from host token arrays (planning and id uploads
    inside) and reads the loss back. One process per GPU, each its own windows; gradients are summed over the ranks
    in three buckets (decoder, backbone, encoder + table) as the window's backward completes them."""
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    H = importlib.import_module("neural-networks_b200.hier")
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    B, T, S = 16, 8192, 8
    cfg = H.HierCfg(vocab=257, hc=256, wh=1024, enc_blocks=2, bb_blocks=8, dec_blocks=2, heads=8, dqk=128, w_token=256,
                    small_heads=2, enc_kinds="mm", bb_kinds="m" * 8, dec_kinds="mm")
    model = H.Hierarchical(H.init_hier_params(np.random.default_rng(0), cfg, std=0.02), cfg, bf16=True)
    nparams = sum(q.w.numel() for q in model.params())
    r = np.random.default_rng(1234 + rank)
    words = [(i * S, (i + 1) * S) for i in range(T // S)]
    wins = [(r.integers(0, 256, T), words) for _ in range(B)]
    acfg = xl.ops.AdamCfg(1e-3, 0.1, t=0)
    dp = importlib.import_module("neural-networks_b200.dp")
    buckets = dp.attach_hier(model)

    def step():
        acfg.t += 1
        return dp.train_step_hier(model, buckets, wins, acfg)  # reads the loss back

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        loss = step()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = xl._lib.lib.xlstm_launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    ms /= args.steps
    if rank == 0:
        val = B * T * world / (ms * 1e-3)
        ids_bytes = B * (T // S - 1) * (S + 1) * (8 + 8 + 4 + 4)  # encoder ids, decoder char ids, targets, mask (plus row lists)
        print(json.dumps({
            "metric": "train_bytes_per_s", "value": val, "unit": "bytes/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "hierarchical_train_step (configs[4]: bytes 16x8192 in words of 8, 2+2 blocks of 256, backbone 8 blocks of 1024 = 8x128)",
                       "params": nparams, "parallelism": "dp%d (gradient all-reduce per stage, overlapped with the window's backward)" % world, "l2": "activations far larger than L2"},
            "loss": loss, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            "e2e": {"value": val, "unit": "bytes/s", "h2d_bytes_per_step": ids_bytes, "d2h_bytes_per_step": 4,
                    "note": "the timed step already starts from host token arrays and reads the loss back"},
            "gpu_launches": int(launches), "clocks": clocks}))


def run_cp(args):
    """Secondary workload: the configs[1] mLSTM layer kernel pair with ONE sequence set cut over the GPUs (context
    parallelism): every rank holds a [16, 2048] segment of sequences world x 2048 long. Strong in the sequence,
    weak per GPU; each rank runs two forward and two backward passes plus two all-gathers of segment summaries."""
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    cp = importlib.import_module("neural-networks_b200.cp")
    ops = xl.ops
    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    c = CFG
    B, H, T, dqk, dhv = c["B"], c["H"], c["T"], c["dqk"], c["dhv"]
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    rnd = lambda *sh: torch.randn(sh, device="cuda", generator=g)
    q, k, v = (rnd(B * T, H * d).to(torch.bfloat16) for d in (dqk, dqk, dhv))
    k = (k.float() / math.sqrt(dqk)).to(torch.bfloat16)
    ig, fg, dy = rnd(B * T, H), rnd(B * T, H) + 3.0, rnd(B * T, H * dhv)
    st = ops.MlstmShape(B, H, T, dqk, dhv, c["L"], torch.bfloat16, torch.float32)
    gather = cp.dist_gather() if world > 1 else (lambda t: [t])

    def step():
        fused, carry = cp.forward(q, k, v, ig, fg, st, rank, gather) if world > 1 else \
            (ops.mlstm_fused_fw(q, k, v, ig, fg, st, save_states=True, want_state=False), None)
        return cp.backward(fused, q, k, v, ig, fg, dy, st, carry, rank, world, gather)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    l0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = xl._lib.lib.xlstm_launch_count() - l0
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    ms /= args.steps
    if rank == 0:
        print(json.dumps({
            "metric": "mlstm_layer_tokens_per_s", "value": B * T * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlstm_layer_fwd_bwd, sequences of %d positions cut over %d GPUs (B16 H8 S2048 per GPU, dqk128 dv128 chunk64)" % (T * world, world),
                       "parallelism": "cp%d (segment summaries all-gathered, carry folded, BPTT state suffix-summed)" % world,
                       "l2": "tensors larger than L2"},
            "gpu_launches": int(launches)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--grad-dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--recompute", action="store_true", help="backward recomputes chunk-boundary states")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--workload", default="mlstm", choices=["mlstm", "lm", "ops", "hier", "cp"],
                    help="mlstm: configs[1] layer kernel (headline); lm: training step; ops: the other hot-path kernels alone; "
                         "hier: configs[4] hierarchical training step; cp: the layer kernel with sequences cut over the GPUs")
    ap.add_argument("--lm-blocks", type=int, default=0, help="override the LM depth (development)")
    ap.add_argument("--lm-remat", type=int, default=2, help="blocks rematerialised in the full-width LM workload")
    ap.add_argument("--lm-full", action="store_true", help="LM workload at the full widths of configs[3] (d=2048, heads of 256 / 512)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "lm":
        run_lm(args)
    elif args.workload == "ops":
        run_ops(args)
    elif args.workload == "hier":
        run_hier(args)
    elif args.workload == "cp":
        run_cp(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
