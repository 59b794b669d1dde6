#!/usr/bin/env python
"""Benchmark of the xLSTM hot path on B200.

Default workload (every N): one data-parallel TRAINING STEP of the xLSTM language model of BASELINE.json configs[3] at
its own widths: 24 blocks (one sLSTM per 8, the rest mLSTM), d = 2048, mLSTM 8 heads x 256, sLSTM 4 heads x 512, vocab
50304, bf16 GEMM operands with fp32 master weights, AdamW, per-GPU batch 8 x 4096 of uniform-random token ids. A step
starts from pinned HOST token ids and ends with the loss read back on the host, so the device-timed `value` (train
tokens/s, whole job) and `e2e` are the same measurement. With N GPUs every rank holds a replica and its own batch
(weak scaling); gradients are summed with one NCCL all-reduce per block, started through the library's xlstm_dp_*
entry points the moment the block's backward is done and waited for in front of AdamW.

The same JSON line carries: `mlstm_fwd_bwd_tflops` (the configs[1] mLSTM layer kernel pair, B16 H8 S2048 d128 chunk 64,
measured in this process before the model is built), `roofline` (the mLSTM backward op at the model's shape, CUDA
events around every call inside the timed steps), `kernels` (device time of every library op and of the library GEMMs
in one extra instrumented step), `cpu_baseline` (N = 1), and for N > 1 `allreduce_exposed_ms` and `dp_parity_max_rel`
(a small model's N-rank gradients against one rank on the concatenated batch, checked before the timed region).

`--impl reference` times the CPU restatement of the reference's layers (the reference is a Rust crate that cannot be
built here) on the host cores, on a fixed sample of the same workload; the line states the sample and the
extrapolation. `--workload mlstm|ops|hier|cp` run the secondary workloads.
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


def _limit_threads(n):
    """Context manager: BLAS and OpenMP pools set to n threads; None = every host core, set explicitly because a
    launcher may have exported OMP_NUM_THREADS=1 for its ranks (torch.distributed.run does)."""
    from threadpoolctl import threadpool_limits
    return threadpool_limits(limits=n if n is not None else (os.cpu_count() or 1))


MLSTM_CPU_SEQS = 8  # sequences (of the 16) in the all-core CPU sample of the configs[1] kernel pair: fixed, not core-count dependent


def cpu_mlstm_sample(seqs=MLSTM_CPU_SEQS, threads=None):
    """Times the CPU restatement (f32) of the configs[1] kernel pair on `seqs` sequences of the full length."""
    from oracle import oracle as O
    cfg = dict(CFG)
    cfg["B"] = seqs
    q, k, v, ig, fg, dy = make_inputs(cfg, 0)
    args = (cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"])
    with _limit_threads(threads):
        t0 = time.perf_counter()
        O.mlstm_core_fw(q, k, v, ig, fg, *args, dtype=np.float32)
        O.mlstm_core_bw(q, k, v, ig, fg, dy, *args, dtype=np.float32)
        dt = time.perf_counter() - t0
    f, b = flops_fwd_bwd(**cfg)
    return dict(seconds=dt, flops=f + b, tokens=seqs * cfg["T"], seqs=seqs, threads=threads or (os.cpu_count() or 1))


# ---- the LM workload (configs[3]) -----------------------------------------------------------------------------------
LM_CFG_FULL = dict(vocab=50304, d=2048, blocks=24, heads=8, dqk=256, dhv=256, slstm_every=8, slstm_heads=4, B=8, T=4096)
# development stand-in with the same structure at half the width (`--lm-reduced`)
LM_CFG_REDUCED = dict(vocab=50304, d=1024, blocks=24, heads=8, dqk=128, dhv=128, slstm_every=8, slstm_heads=4, B=8, T=4096)
LM_CPU_SAMPLE = dict(B=8, T=64)       # all-core CPU sample: sequences x positions run through one block of each kind + the head
LM_CPU_SAMPLE_1CORE = dict(B=1, T=64)


def lm_cfg(args):
    c = dict(LM_CFG_REDUCED if args.lm_reduced else LM_CFG_FULL)
    if args.lm_blocks:
        c["blocks"] = args.lm_blocks
    c["up"] = (8 * c["d"] // 3 + 7) // 8 * 8
    c["slstm_at"] = tuple(i for i in range(c["blocks"]) if i % c["slstm_every"] == 0)
    return c


def lm_config_dict(args, world):
    """The `config` object of the LM line: identical for the engine's arm and the reference arm."""
    c = lm_cfg(args)
    return {"workload": "xlstm_lm_train_step (configs[3]%s: %d blocks, sLSTM at %s, d=%d, mLSTM %dx%d, sLSTM %dx%d, vocab %d, AdamW)"
                        % (" widths" if not args.lm_reduced else " structure, reduced widths", c["blocks"], list(c["slstm_at"]), c["d"],
                           c["heads"], c["dqk"], c["slstm_heads"], c["d"] // c["slstm_heads"], c["vocab"]),
            "per_gpu_batch": [c["B"], c["T"]], "global_batch_tokens": c["B"] * c["T"] * world,
            "parallelism": "dp%d (one NCCL gradient all-reduce per block through xlstm_dp_*, overlapped with backward)" % world,
            "chunk_states": "recomputed in backward" if args.recompute else "saved by forward",
            "rematerialised_blocks": args.lm_remat,
            "head": "fp32 logits; operands as bf16 triples, %d tensor-core products per GEMM" % args.lm_head_terms,
            "l2": "activations far larger than L2"}


def lm_param_count(c):
    d, up, H = c["d"], c["up"], c["heads"]
    ffn = 3 * d * up + 2 * up + d + 2 * d  # gate, value, down (+ biases) and the two norm gains
    m = 2 * (d * H * c["dqk"] + H * c["dqk"]) + 2 * (d * H * c["dhv"] + H * c["dhv"]) + 2 * (d * H + H) + d * d + d + d
    dh = d // c["slstm_heads"]
    s_ = d * 4 * d + c["slstm_heads"] * dh * 4 * dh + 4 * d + d  # wx, wh, bias, post-norm gain
    ns = len(c["slstm_at"])
    return c["vocab"] * d + d + (c["blocks"] - ns) * (m + ffn) + ns * (s_ + ffn), m + ffn, s_ + ffn


def _cpu_lm_params(rng, c):
    """Seeded N(0, 0.02) f32 host weights of one sLSTM block, one mLSTM block and the table at the model's widths, in the
    dictionary layout the CPU restatement's `build_lm` takes (numpy only: the CPU legs never load the engine)."""
    d, up, H, dqk, dhv, nh = c["d"], c["up"], c["heads"], c["dqk"], c["dhv"], c["slstm_heads"]
    n = lambda *shape: rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02)
    one = lambda k: np.ones(k, np.float32)
    ffn = lambda: dict(g1=one(d), g2=one(d), w_gate=n(d, up), b_gate=n(up), w_value=n(d, up), b_value=n(up), w_down=n(up, d), b_down=n(d))
    dh = d // nh
    sblk = dict(ffn(), gpost=one(d), cell=dict(kind="slstm", wx=n(d, 4 * d), wh=n(nh, dh, 4 * dh), bcat=n(4 * d)))
    mblk = dict(ffn(), cell=dict(kind="mlstm", wq=n(d, H * dqk), wk=n(d, H * dqk), wv=n(d, H * dhv), wo=n(d, H * dhv), wi=n(d, H),
                                 wf=n(d, H), bq=n(H * dqk), bk=n(H * dqk), bv=n(H * dhv), bo=n(H * dhv), bi=n(H), bf=n(H),
                                 w_out=n(d, d), b_out=n(d), gamma=one(d)))
    return dict(table=n(c["vocab"], d), blocks=[sblk, mblk], gamma=one(d))


_cpu_lm_cache = {}


def cpu_lm_sample(args, sample, threads=None):
    """Times the CPU restatement (f32, the width of the reference's src/nn2 layers) of the LM's three kinds of work at
    the model's full widths on a small batch: one sLSTM block, one mLSTM block, and embedding + final norm + tied fp32
    head + soft-cap + cross-entropy, each forward + backward, plus AdamW over one block's tensors. The full model's
    step on the full per-GPU batch is extrapolated: every per-token cost scales with the token count, AdamW with the
    parameter count. Returns the pieces and the extrapolated step."""
    from oracle import model as M
    from oracle import oracle as O
    c = lm_cfg(args)
    B, T = sample["B"], sample["T"]
    rows = B * T
    M.DT = np.float32
    try:
        if "lm" not in _cpu_lm_cache:
            _cpu_lm_cache["lm"] = M.build_lm(_cpu_lm_params(np.random.default_rng(0), c), c["heads"], c["dqk"], c["dhv"],
                                             nh_s=c["slstm_heads"], tied=True)
        lm = _cpu_lm_cache["lm"]
        ids = np.random.default_rng(1).integers(0, c["vocab"], (B, T + 1))
        x_ids, tg = ids[:, :-1].reshape(-1), ids[:, 1:].reshape(-1)
        with _limit_threads(threads):
            x = lm.table.w[x_ids]
            t = {}
            t0 = time.perf_counter(); y_s = lm.blocks[0].forward(x, B, T); t["slstm_fw"] = time.perf_counter() - t0
            t0 = time.perf_counter(); y_m = lm.blocks[1].forward(y_s, B, T); t["mlstm_fw"] = time.perf_counter() - t0
            t0 = time.perf_counter()
            normed = lm.norm.forward(y_m)
            pre = normed @ lm.table.w.T
            logits = lm.cap * np.tanh(pre / lm.cap)
            loss, dlogits = O.softmax_ce(logits, tg, dtype=np.float32)
            d_pre = dlogits * (1.0 - (logits / lm.cap) ** 2)
            lm.table.g += d_pre.T @ normed
            d = lm.norm.backward(d_pre @ lm.table.w)
            t["head"] = time.perf_counter() - t0
            t0 = time.perf_counter(); d = lm.blocks[1].backward(d); t["mlstm_bw"] = time.perf_counter() - t0
            t0 = time.perf_counter(); d = lm.blocks[0].backward(d); t["slstm_bw"] = time.perf_counter() - t0
            t0 = time.perf_counter(); np.add.at(lm.table.g, x_ids, d); t["embed_bw"] = time.perf_counter() - t0
            t0 = time.perf_counter()
            nstep = 0
            for q in lm.blocks[1].params():
                q.step(1e-3, 0.1, 1); nstep += q.w.size
            t["adamw"] = time.perf_counter() - t0
    finally:
        M.DT = np.float64
    total, _, _ = lm_param_count(c)
    nm, ns = c["blocks"] - len(c["slstm_at"]), len(c["slstm_at"])
    per_rows = nm * (t["mlstm_fw"] + t["mlstm_bw"]) + ns * (t["slstm_fw"] + t["slstm_bw"]) + t["head"] + t["embed_bw"]
    full_rows = c["B"] * c["T"]
    step_s = per_rows * (full_rows / rows) + t["adamw"] * (total / nstep)
    measured_s = sum(t.values())
    return dict(pieces=t, rows=rows, measured_s=measured_s, step_s=step_s, tokens_per_s=full_rows / step_s, loss=float(loss),
                threads=threads or (os.cpu_count() or 1),
                formula="step = (%d/%d rows) * (%d*(mlstm_fw+bw) + %d*(slstm_fw+bw) + head + embed_bw) + adamw * (%d/%d params)"
                        % (full_rows, rows, nm, ns, total, nstep))


def lm_cpu_baseline(args, with_one_core=True):
    s = cpu_lm_sample(args, LM_CPU_SAMPLE)
    out = {"value": s["tokens_per_s"], "unit": "tokens/s", "cores": s["threads"], "kind": "port",
           "sample": "f32 CPU restatement of the reference's layers at the model's full widths: one mLSTM block, one sLSTM block and "
                     "embedding + norm + tied head + soft-cap + CE, forward + backward + AdamW, on %d sequences x %d positions "
                     "(%.1f s measured); %s" % (LM_CPU_SAMPLE["B"], LM_CPU_SAMPLE["T"], s["measured_s"], s["formula"]),
           "seconds_measured": s["measured_s"], "extrapolated_step_s": s["step_s"], "pieces_s": s["pieces"]}
    if with_one_core:
        s1 = cpu_lm_sample(args, LM_CPU_SAMPLE_1CORE, threads=1)
        out["one_core"] = {"value": s1["tokens_per_s"], "unit": "tokens/s", "cores": 1,
                           "sample": "same pieces on %d x %d, BLAS and OpenMP limited to one thread (%.1f s measured)"
                                     % (LM_CPU_SAMPLE_1CORE["B"], LM_CPU_SAMPLE_1CORE["T"], s1["measured_s"])}
    return out, s


def run_reference(args):
    """The reference arm: the CPU restatement on the host cores (rank 0 only), same config / metric / unit as the engine's arm."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    if args.workload == "mlstm":
        times = []
        for i in range(args.warmup + args.steps):
            s = cpu_mlstm_sample()
            if i >= args.warmup:
                times.append(s["seconds"])
        t = float(np.mean(times))
        val = s["flops"] / t / 1e12
        one = cpu_mlstm_sample(seqs=1, threads=1)
        sample = "%d of 16 sequences x 2048 positions x 8 heads, recurrent f32 restatement, OpenMP over (batch, head)" % s["seqs"]
        line = {"impl": "reference", "metric": "mlstm_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": mlstm_config_dict(args, world),
                "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": s["threads"], "kind": "port", "sample": sample,
                                 "one_core": {"value": one["flops"] / one["seconds"] / 1e12, "unit": "TFLOP/s", "cores": 1,
                                              "sample": "1 of 16 sequences, one thread"}},
                "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return
    vals, secs = [], []
    for i in range(args.warmup + args.steps):
        s = cpu_lm_sample(args, LM_CPU_SAMPLE)
        if i >= args.warmup:
            vals.append(s["tokens_per_s"]); secs.append(s["measured_s"])
    val = float(np.mean(vals))
    cb, _ = lm_cpu_baseline(args, with_one_core=True)
    cb["value"] = val
    line = {"impl": "reference", "metric": "train_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(secs)) * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": lm_config_dict(args, world),
            "cpu_baseline": cb,
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "each step runs the fixed sample (ms_per_step is the sample's wall time); value is the full model's "
                    "tokens/s on the full per-GPU batch extrapolated from it on one host (the reference has no multi-GPU path)"}
    print(json.dumps(line))


def mlstm_cfg(args):
    """configs[1], or the shape `--mlstm-shape B,H,S,d` asks for (kernel studies: e.g. 2,8,4096,256 is a quarter of the
    batch the configs[3] model hands its mLSTM core)."""
    cfg = dict(CFG)
    shape = getattr(args, "mlstm_shape", None)
    if shape:
        B, H, T, d = (int(x) for x in shape.split(","))
        cfg.update(B=B, H=H, T=T, dqk=d, dhv=d)
    return cfg


# DRAM bytes per launch (read + written) from one ncu capture of each kernel at configs[1], fp32 gradients, states saved
MLSTM_TRAFFIC = {"fw": 203.5e6 + 163.4e6, "bw": 545.4e6 + 366.3e6}
# The configs[3] model's core ops (B8 H8 S4096, heads of 256 as four 128 x 128 sub-heads, bf16 gradients, states
# saved): DRAM bytes of every kernel of one op call, captured at a quarter of the batch (B = 2) and multiplied by four
# (each kernel's traffic is proportional to the batch). Backward: row-dot pass 67.1 MB, sub-head kernel 328.5 + 366.0 MB
# (the fp32 partial planes are its writes), three plane sums 3 x 140 MB; forward: sub-head kernel 101.3 + 212.3 MB,
# combine 140.8 MB. 4.4 and 3.4 times the algorithmic bytes: the price of the sub-head decomposition.
LM_CORE_TRAFFIC = {"fw": 4 * 454.4e6, "bw": 4 * 1183.7e6}


def mlstm_config_dict(args, world):
    cfg = mlstm_cfg(args)
    gb = 2 if args.grad_dtype == "bf16" else 4
    bf, bb = algorithmic_bytes(cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], gb)
    name = "mlstm_layer_fwd_bwd B%d H%d S%d dqk%d dv%d chunk%d" % (cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], cfg["L"])
    return {"workload": name + (" (configs[1])" if cfg == CFG else ""), "per_gpu_batch": cfg["B"],
            "grad_dtype": args.grad_dtype, "chunk_states": "recomputed in backward" if args.recompute else "saved by forward",
            "l2": "inputs (%.0f MB) larger than L2" % ((bf + bb) / 1e6), "parallelism": "dp%d (batch shards, no collective)" % world}


def _dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def measure_mlstm_pair(args, steps, warmup=3, with_e2e=False):
    """The configs[1] kernel pair on this rank's GPU: device-timed steps with inputs resident (CUDA events around the
    whole run and around each op), optionally the same step end to end from pinned host buffers. Returns a dict of
    this rank's figures (no collectives)."""
    import torch
    xl = importlib.import_module("neural-networks_b200")
    ops = xl.ops
    rank, world, local = _dist_env()
    cfg = mlstm_cfg(args)
    gd = torch.bfloat16 if args.grad_dtype == "bf16" else torch.float32
    st = ops.MlstmShape(cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], cfg["L"], torch.bfloat16, gd, 0)
    hq, hk, hv, hig, hfg, hdy = make_inputs(cfg, 1000 + rank)
    pin = lambda a, dt: torch.from_numpy(a).to(dt).pin_memory()
    host_in = [pin(hq, torch.bfloat16), pin(hk, torch.bfloat16), pin(hv, torch.bfloat16), pin(hig, torch.float32),
               pin(hfg, torch.float32), pin(hdy, gd)]
    dev_in = [t.cuda(non_blocking=True) for t in host_in]
    torch.cuda.synchronize()
    q, k, v, ig, fg, dy = dev_in

    def step():
        fused = ops.mlstm_fused_fw(q, k, v, ig, fg, st, save_states=not args.recompute, want_state=False)
        return fused, ops.mlstm_fused_bw(fused, q, k, v, ig, fg, dy, st, want_dstate=False)

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    launches0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops.timing_start(("mlstm_fused_fw", "mlstm_fused_bw"))
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    per_op = ops.timing_stop()  # synchronises
    ms_per_step = e0.elapsed_time(e1) / steps
    launches = xl._lib.lib.xlstm_launch_count() - launches0
    # the device runs behind the host here, so the gap between an op's two events is its kernels and nothing else
    fw_t, bw_t = float(np.median(per_op["mlstm_fused_fw"])), float(np.median(per_op["mlstm_fused_bw"]))
    ff, fb = flops_fwd_bwd(**cfg)
    gb = 2 if gd == torch.bfloat16 else 4
    bf, bb = algorithmic_bytes(cfg["B"], cfg["H"], cfg["T"], cfg["dqk"], cfg["dhv"], gb)
    pk = peaks()
    out = dict(ms_per_step=ms_per_step, fw_ms=fw_t, bw_ms=bw_t, flops=ff + fb, bytes_fw=bf, bytes_bw=bb, launches=int(launches),
               tflops=(ff + fb) / (ms_per_step * 1e-3) / 1e12, tokens=cfg["B"] * cfg["T"],
               bw_gbs=bb / (bw_t * 1e-3) / 1e9, fw_gbs=bf / (fw_t * 1e-3) / 1e9, peaks=pk,
               traffic=MLSTM_TRAFFIC if (cfg == CFG and args.grad_dtype == "f32" and not args.recompute) else {"fw": None, "bw": None})
    if with_e2e:
        # Every step copies its inputs from pinned host memory, runs forward + backward through `ops`, and copies every
        # result back to pinned host memory; all of it is inside the timed region. The three stages run on three
        # streams with double-buffered device inputs, so step i+1's upload and step i-1's download overlap step i
        # (PCIe is full duplex): steady state is the slower of the two copy directions, not their sum.
        s_in, s_out, s_cmp = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        dbuf = [[torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in host_in] for _ in range(2)]
        state = {"outs_host": None, "free": [None, None]}

        def e2e_run(nsteps):
            last_out = None
            for i in range(nsteps):
                j = i & 1
                with torch.cuda.stream(s_in):
                    if state["free"][j] is not None:
                        s_in.wait_event(state["free"][j])
                    for dst, src in zip(dbuf[j], host_in):
                        dst.copy_(src, non_blocking=True)
                    ev_in = torch.cuda.Event(); ev_in.record(s_in)
                s_cmp.wait_event(ev_in)
                d = dbuf[j]
                fused = ops.mlstm_fused_fw(d[0], d[1], d[2], d[3], d[4], st, save_states=not args.recompute, want_state=False)
                g = ops.mlstm_fused_bw(fused, d[0], d[1], d[2], d[3], d[4], d[5], st, want_dstate=False)
                res = [fused.ytil, g[0], g[1], g[2], g[3], g[4]]
                ev_c = torch.cuda.Event(); ev_c.record(s_cmp)
                state["free"][j] = ev_c
                if state["outs_host"] is None:
                    state["outs_host"] = [[torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res] for _ in range(2)]
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_c)
                    for h, r in zip(state["outs_host"][j], res):
                        r.record_stream(s_out)
                        h.copy_(r, non_blocking=True)
                    last_out = torch.cuda.Event(); last_out.record(s_out)
            s_cmp.wait_event(last_out)  # the timed region ends when the last result is on the host

        e2e_steps = max(2, min(steps, 6))
        e2e_run(2)
        torch.cuda.synchronize()
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        torch.cuda.synchronize()
        out["e2e_ms"] = e0.elapsed_time(e1) / e2e_steps
        out["h2d"] = sum(t.numel() * t.element_size() for t in host_in)
        out["d2h"] = sum(t.numel() * t.element_size() for t in state["outs_host"][0])
    return out


def mlstm_pair_summary(m):
    """The sub-object the LM line carries for the configs[1] kernel pair."""
    pk = m["peaks"]
    return {"value": m["tflops"], "unit": "TFLOP/s", "workload": "mlstm_layer_fwd_bwd B16 H8 S2048 dqk128 dv128 chunk64 (configs[1]), this rank",
            "ms_per_step": m["ms_per_step"], "frac_of_bf16_peak": m["tflops"] / pk["tensor"],
            "forward": {"launch_ms": m["fw_ms"], "algorithmic_bytes": m["bytes_fw"], "achieved_gbs": m["fw_gbs"], "frac_of_hbm_peak": m["fw_gbs"] / pk["hbm"],
                        "traffic": m["traffic"]["fw"]},
            "backward": {"launch_ms": m["bw_ms"], "algorithmic_bytes": m["bytes_bw"], "achieved_gbs": m["bw_gbs"], "frac_of_hbm_peak": m["bw_gbs"] / pk["hbm"],
                         "traffic": m["traffic"]["bw"]},
            "tokens_per_s": m["tokens"] / (m["ms_per_step"] * 1e-3), "peak_source": pk["src"]}


def run_mlstm(args):
    """Secondary workload: the configs[1] kernel pair as the whole line (device-timed, end to end from pinned host buffers,
    CPU baseline)."""
    import torch
    import torch.distributed as dist
    rank, world, local = _dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    m = measure_mlstm_pair(args, args.steps, args.warmup, with_e2e=True)
    clocks = sampler.stop() if rank == 0 else None
    ms, e2e_ms = m["ms_per_step"], m["e2e_ms"]
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0].item()), float(t[1].item())
    if rank == 0:
        pk = m["peaks"]
        traffic = m["traffic"]
        value = m["flops"] * world / (ms * 1e-3) / 1e12
        line = {"metric": "mlstm_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": mlstm_config_dict(args, world),
                "tokens_per_s": m["tokens"] * world / (ms * 1e-3), "frac_of_bf16_peak": value / world / pk["tensor"],
                "roofline": {"kernel": "mlstm backward", "bound": "hbm", "achieved": m["bw_gbs"], "peak": pk["hbm"], "unit": "GB/s",
                             "frac": m["bw_gbs"] / pk["hbm"], "traffic": traffic["bw"], "peak_source": pk["src"],
                             "algorithmic_bytes": m["bytes_bw"], "launch_ms": m["bw_ms"],
                             "forward": {"achieved": m["fw_gbs"], "frac": m["fw_gbs"] / pk["hbm"], "algorithmic_bytes": m["bytes_fw"],
                                         "launch_ms": m["fw_ms"], "traffic": traffic["fw"]}},
                "e2e": {"value": m["flops"] * world / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": m["h2d"],
                        "d2h_bytes_per_step": m["d2h"], "ms_per_step": e2e_ms},
                "gpu_launches": m["launches"], "clocks": clocks}
        if world == 1 and not args.no_cpu:
            cpu = cpu_mlstm_sample()
            one = cpu_mlstm_sample(seqs=1, threads=1)
            line["cpu_baseline"] = {"value": cpu["flops"] / cpu["seconds"] / 1e12, "unit": "TFLOP/s", "cores": cpu["threads"], "kind": "port",
                                    "seconds": cpu["seconds"],
                                    "sample": "%d of 16 sequences x 2048 positions x 8 heads, recurrent f32 restatement, OpenMP over (batch, head)" % cpu["seqs"],
                                    "one_core": {"value": one["flops"] / one["seconds"] / 1e12, "unit": "TFLOP/s", "cores": 1,
                                                 "sample": "1 of 16 sequences, one thread"}}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def mlstm_op_bytes(B, H, T, dqk, dhv, gbytes):
    """Compulsory HBM traffic of the fused forward and backward ops at a shape (chunk states excluded)."""
    return algorithmic_bytes(B, H, T, dqk, dhv, gbytes)


DP_CHECK_CFG = dict(vocab=64, d=256, blocks=2, heads=2, dqk=128, dhv=128, up=256, B=2, T=128)


def dp_parity_check(world, rank):
    """A small bf16 model's gradients after the bucketed all-reduce over `world` ranks against one rank on the
    concatenated batch (same kernels per sequence; only the fp32 summation order over the batch differs). Returns the
    largest error relative to each tensor's largest gradient, maximised over tensors and ranks."""
    import torch
    import torch.distributed as dist
    layers = importlib.import_module("neural-networks_b200.layers")
    dp = importlib.import_module("neural-networks_b200.dp")
    c = DP_CHECK_CFG

    def build():
        p = layers.init_lm_params(np.random.default_rng(0), c["vocab"], c["d"], c["blocks"], c["heads"], c["dqk"], c["dhv"], c["up"], std=0.05)
        return layers.build_lm(p, c["heads"], c["dqk"], c["dhv"], tied=True, bf16=True)

    ids = torch.tensor(np.random.default_rng(7).integers(0, c["vocab"], (world * c["B"], c["T"] + 1)), device="cuda")
    lm = build()
    buckets = dp.attach(lm)
    mine = ids[rank * c["B"]:(rank + 1) * c["B"]]
    lm.forward_backward(mine[:, :-1].reshape(-1), mine[:, 1:].reshape(-1).to(torch.int32), c["B"], c["T"], inv=1.0 / (c["B"] * c["T"] * world))
    buckets.reduce_async(len(lm.blocks))
    buckets.wait()
    one = build()
    one.forward_backward(ids[:, :-1].reshape(-1), ids[:, 1:].reshape(-1).to(torch.int32), world * c["B"], c["T"])
    worst = 0.0
    for a, b in zip(lm.params(), one.params()):
        scale = max(b.g.abs().max().item(), 1e-12)
        worst = max(worst, (a.g - b.g).abs().max().item() / scale)
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()), bool(buckets.native)


def head_sharding_check(world, rank):
    """Greedy decoding with every mLSTM block's heads split over the `world` ranks (one all-reduce of the W_out partials
    per block) against the same model unsharded on this rank: identical token ids, logits within 1e-4."""
    import torch
    import torch.distributed as dist
    layers = importlib.import_module("neural-networks_b200.layers")
    infer = importlib.import_module("neural-networks_b200.infer")
    heads = max(4, world)
    vocab, dh, nb, up, B, Tp, n_new = 61, 16, 2, 176, 2, 9, 6
    d = heads * dh
    p = layers.init_lm_params(np.random.default_rng(13), vocab, d, nb, heads, dh, dh, up, std=0.1, slstm_at=(1,), nh_s=2)
    prompt = torch.tensor(np.random.default_rng(8).integers(0, vocab, (B, Tp)), device="cuda")
    lm = infer.build_lm_head_sharded(p, heads, dh, dh, rank, world, nh_s=2, tied=True)
    ids, logits = infer.greedy_decode(lm, prompt, n_new)
    one = layers.build_lm(p, heads, dh, dh, nh_s=2, tied=True)
    ids1, logits1 = infer.greedy_decode(one, prompt, n_new)
    same = float(torch.equal(ids, ids1))
    err = float((logits - logits1).abs().max()) / max(float(logits1.abs().max()), 1e-30)
    t = torch.tensor([1.0 - same, err], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"ids_equal": bool(t[0].item() == 0.0), "logits_max_rel": float(t[1].item()), "heads": heads}


def context_parallel_check(world, rank):
    """The mLSTM layer kernel pair with each sequence cut into `world` segments, one per rank (segment summaries
    all-gathered over NCCL, carry folded, BPTT state suffix-summed) against the whole sequence run on this rank
    (bf16 tensor-core path). Returns the largest error relative to each tensor's largest element over
    ytil, dq, dk, dv, di, df of this rank's segment, maximised over ranks."""
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    cp = importlib.import_module("neural-networks_b200.cp")
    ops = xl.ops
    B, H, Ts, d = 2, 2, 128, 128
    T = Ts * world
    g = torch.Generator(device="cuda").manual_seed(43)
    rnd = lambda *sh: torch.randn(sh, device="cuda", generator=g)
    q, k, v = (rnd(B, T, H * d).to(torch.bfloat16) for _ in range(3))
    k = (k.float() / math.sqrt(d)).to(torch.bfloat16)
    ig, fg, dy = rnd(B, T, H), rnd(B, T, H) + 3.0, rnd(B, T, H * d)
    whole = ops.MlstmShape(B, H, T, d, d, 64, torch.bfloat16, torch.float32)
    flat = lambda a: a.reshape(B * a.shape[1], -1).contiguous()
    fw = ops.mlstm_fused_fw(flat(q), flat(k), flat(v), flat(ig), flat(fg), whole, want_state=False)
    ref = [fw.ytil.float()] + [a.float() for a in ops.mlstm_fused_bw(fw, flat(q), flat(k), flat(v), flat(ig), flat(fg), flat(dy), whole, want_dstate=False)[:5]]
    seg = lambda a: flat(a[:, rank * Ts:(rank + 1) * Ts])
    st = ops.MlstmShape(B, H, Ts, d, d, 64, torch.bfloat16, torch.float32)
    gather = cp.dist_gather()
    fused, carry = cp.forward(seg(q), seg(k), seg(v), seg(ig), seg(fg), st, rank, gather)
    grads = cp.backward(fused, seg(q), seg(k), seg(v), seg(ig), seg(fg), seg(dy), st, carry, rank, world, gather)
    got = [fused.ytil.float()] + [a.float() for a in grads[:5]]
    worst = 0.0
    for a, r in zip(got, ref):
        r = r.view(B, T, -1)[:, rank * Ts:(rank + 1) * Ts].reshape(B * Ts, -1)
        worst = max(worst, float((a - r).abs().max()) / max(float(r.abs().max()), 1e-30))
    t = torch.tensor([worst], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_lm(args):
    """Default workload: the data-parallel training step of the configs[3] language model (see the module docstring)."""
    import torch
    import torch.distributed as dist
    xl = importlib.import_module("neural-networks_b200")
    layers = importlib.import_module("neural-networks_b200.layers")
    dp = importlib.import_module("neural-networks_b200.dp")
    ops = xl.ops
    rank, world, local = _dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- the configs[1] kernel pair, in this process, before the model takes the memory ---------------------------------
    pair = measure_mlstm_pair(args, 20, 3) if not args.no_pair else None
    torch.cuda.empty_cache()
    # ---- multi-GPU correctness carried in the record: N-rank gradients against one rank -------------------------------
    parity = dp_parity_check(world, rank) if world > 1 else None
    shard_check = head_sharding_check(world, rank) if world > 1 else None
    cp_check = context_parallel_check(world, rank) if world > 1 else None

    c = lm_cfg(args)
    rng = np.random.default_rng(0)  # identical replicas on every rank
    p = layers.init_lm_params(rng, c["vocab"], c["d"], c["blocks"], c["heads"], c["dqk"], c["dhv"], c["up"], std=0.02,
                              slstm_at=c["slstm_at"], nh_s=c["slstm_heads"])
    # the first `--lm-remat` mLSTM blocks keep only their input and re-run their forward in the backward (a memory
    # lever: none is needed at 8 x 4096 per GPU); sLSTM blocks (the long sequential loops) are never re-run. The head runs
    # row-chunked on split-bf16 operands (`--lm-head-terms`: 6 = fp32-accurate, 3 = 16 bits per operand).
    remat = [i for i in range(c["blocks"]) if i not in c["slstm_at"]][:args.lm_remat] if not args.lm_reduced else ()
    lm = layers.build_lm(p, c["heads"], c["dqk"], c["dhv"], nh_s=c["slstm_heads"], tied=True, bf16=True, remat=remat,
                         head_rows=4096, head_split=args.lm_head_terms, recompute_states=args.recompute)
    del p
    nparams = sum(q.w.numel() for q in lm.params())
    buckets = dp.attach(lm)
    B, T = c["B"], c["T"]
    g = torch.Generator().manual_seed(1234 + rank)
    host_ids = torch.randint(0, c["vocab"], (B, T + 1), generator=g).pin_memory()
    cfg = ops.AdamCfg(1e-3, 0.1, t=0)

    def step():
        cfg.t += 1
        d = host_ids.cuda(non_blocking=True)
        ids = d[:, :-1].reshape(-1)
        tg = d[:, 1:].reshape(-1).to(torch.int32)
        return dp.train_step(lm, buckets, ids, tg, B, T, cfg)

    loss_step1 = None
    for i in range(max(args.warmup, 3)):
        loss = step()
        if i == 0:
            loss_step1 = float(loss.item()) * world  # each rank holds its share of the global mean
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    buckets.time_wait = world > 1
    exposed = []
    l0 = xl._lib.lib.xlstm_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ops.timing_start(("mlstm_fused_fw", "mlstm_fused_bw", "slstm_fused_time", "slstm_fused_time_bwd"))
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step()
        lv = loss.item()  # the step's result read back on the host, as a training loop does
        if world > 1:
            exposed.append(buckets.exposed_ms())
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    launches = xl._lib.lib.xlstm_launch_count() - l0
    per_op = ops.timing_stop()
    clocks = sampler.stop() if rank == 0 else None
    buckets.time_wait = False
    exposed_ms = float(np.mean(exposed)) if exposed else 0.0
    if world > 1:
        t = torch.tensor([ms, exposed_ms, lv], device="cuda")
        mx = t.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = t.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms, exposed_ms, lv = float(mx[0].item()), float(mx[1].item()), float(sm[2].item())
    ms /= args.steps

    # ---- one extra instrumented step: device time of every library op and of the library GEMMs ---------------------------
    kernels = None
    if not args.no_kernels:
        saved = (torch.mm, torch.addmm, torch.bmm)
        torch.mm, torch.addmm, torch.bmm = (ops.timed("library_gemm")(f) for f in saved)
        try:
            ops.timing_start(None)
            es0, es1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            es0.record()
            step().item()
            es1.record()
            table = ops.timing_stop()
        finally:
            torch.mm, torch.addmm, torch.bmm = saved
        step_ms = es0.elapsed_time(es1)
        kernels = {k: {"calls": len(v), "ms": float(np.sum(v))} for k, v in sorted(table.items())}
        acc = sum(v["ms"] for v in kernels.values())
        kernels["other (eager element-wise, copies, gaps)"] = {"calls": None, "ms": max(step_ms - acc, 0.0)}
        kernels["instrumented_step_ms"] = step_ms
    barrier()

    if rank == 0:
        tokens = B * T
        pk = peaks()
        val = tokens * world / (ms * 1e-3)
        gbytes = 2  # bf16 gradient I/O of the core in bf16 mode
        bfw, bbw = mlstm_op_bytes(B, c["heads"], T, c["dqk"], c["dhv"], gbytes)
        bw_calls = per_op.get("mlstm_fused_bw", [])
        fw_calls = per_op.get("mlstm_fused_fw", [])
        bw_ms = float(np.mean(bw_calls)) if bw_calls else None
        fw_ms = float(np.mean(fw_calls)) if fw_calls else None
        ff, fb = flops_fwd_bwd(B, c["heads"], T, c["dqk"], c["dhv"], 64)
        captured = (B, c["heads"], T, c["dqk"], c["dhv"]) == (8, 8, 4096, 256, 256) and not args.recompute
        roof = {"kernel": "mlstm backward op at the model's shape (B%d H%d S%d dqk%d dv%d chunk 64, bf16 gradient I/O)" % (B, c["heads"], T, c["dqk"], c["dhv"]),
                "bound": "hbm", "achieved": bbw / (bw_ms * 1e-3) / 1e9 if bw_ms else None, "peak": pk["hbm"], "unit": "GB/s",
                "frac": bbw / (bw_ms * 1e-3) / 1e9 / pk["hbm"] if bw_ms else None,
                "traffic": LM_CORE_TRAFFIC["bw"] if captured else None, "peak_source": pk["src"],
                "algorithmic_bytes": bbw, "launch_ms": bw_ms, "launches_timed": len(bw_calls),
                "tflops": fb / (bw_ms * 1e-3) / 1e12 if bw_ms else None,
                "forward": {"launch_ms": fw_ms, "algorithmic_bytes": bfw, "achieved": bfw / (fw_ms * 1e-3) / 1e9 if fw_ms else None,
                            "frac": bfw / (fw_ms * 1e-3) / 1e9 / pk["hbm"] if fw_ms else None, "launches_timed": len(fw_calls),
                            "traffic": LM_CORE_TRAFFIC["fw"] if captured else None,
                            "tflops": ff / (fw_ms * 1e-3) / 1e12 if fw_ms else None}}
        sl = {k: float(np.mean(per_op[k])) * 1e3 / T for k in ("slstm_fused_time", "slstm_fused_time_bwd") if per_op.get(k)}
        sustained = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained", pk["tensor"]) \
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1400.0
        dense = 6.0 * nparams * tokens / (ms * 1e-3) / 1e12
        line = {"metric": "train_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "config": lm_config_dict(args, world),
                "params": nparams, "loss_step1": loss_step1, "loss_expected_at_init": math.log(c["vocab"]), "loss": lv,
                "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
                "roofline": roof,
                "slstm_us_per_timestep": sl,
                "dense_equivalent": {"tflops_per_gpu": dense, "frac_of_sustained_bf16_peak": dense / sustained, "formula": "6 * params * tokens / step time"},
                "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": host_ids.numel() * 8, "d2h_bytes_per_step": 4,
                        "note": "the timed step starts from pinned host ids and reads the loss back: value and e2e are the same measurement"},
                "gpu_launches": int(launches), "clocks": clocks}
        if kernels is not None:
            line["kernels"] = kernels
        if pair is not None:
            line["mlstm_fwd_bwd_tflops"] = mlstm_pair_summary(pair)
        if world > 1:
            line["allreduce_exposed_ms"] = exposed_ms
            line["dp_parity_max_rel"] = parity[0]
            line["dp_native_buckets"] = parity[1]
            # the multi-GPU paths a one-GPU test box cannot show, checked here before the timed region
            line["head_sharded_inference_check"] = shard_check
            line["context_parallel_max_rel"] = cp_check
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _ = lm_cpu_baseline(args)
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
    # configs[4] asks for chunk-state recomputation: on unless --hier-saved-states
    recompute = not args.hier_saved_states
    model = H.Hierarchical(H.init_hier_params(np.random.default_rng(0), cfg, std=0.02), cfg, bf16=True, recompute_states=recompute)
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
    xl.ops.timing_start(("mlstm_fused_fw", "mlstm_fused_bw"))
    barrier()
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    per_op = xl.ops.timing_stop()
    launches = xl._lib.lib.xlstm_launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.destroy_process_group()
    ms /= args.steps
    if rank == 0:
        pk = peaks()
        sustained = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained", pk["tensor"]) \
            if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else 1400.0
        # dense-equivalent work of a step: 6 x (a stage's parameters) x (the rows that stage processes)
        words = B * (T // S)
        stage_rows = {"enc": words * (S + 1), "bb": words, "dec": (words - B) * (S + 1)}
        stage_params = {"enc": sum(q.w.numel() for b_ in model.enc for q in b_.params()),
                        "bb": sum(q.w.numel() for b_ in model.bb for q in b_.params()) + sum(q.w.numel() for l in (model.front, model.back) for q in l.params()),
                        "dec": sum(q.w.numel() for b_ in model.dec for q in b_.params())}
        dense = sum(6.0 * stage_params[k] * stage_rows[k] for k in stage_rows) / (ms * 1e-3) / 1e12
        mcore_ms = (sum(per_op.get("mlstm_fused_fw", [])) + sum(per_op.get("mlstm_fused_bw", []))) / args.steps
        val = B * T * world / (ms * 1e-3)
        ids_bytes = B * (T // S - 1) * (S + 1) * (8 + 8 + 4 + 4)  # encoder ids, decoder char ids, targets, mask (plus row lists)
        cpu = None
        if not args.no_cpu:
            _limit_threads(None)
            v, dt = cpu_hier_sample()
            cpu = {"value": v, "unit": "bytes/s", "cores": os.cpu_count(), "kind": "port",
                   "sample": "CPU restatement of the reference's hierarchical model at configs[4]'s widths (float64 numpy), one window of "
                             "512 bytes in words of 8: forward + backward + AdamW (%.1f s)" % dt}
        print(json.dumps({
            "metric": "train_bytes_per_s", "value": val, "unit": "bytes/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "hierarchical_train_step (configs[4]: bytes 16x8192 in words of 8, 2+2 blocks of 256, backbone 8 blocks of 1024 = 8x128)",
                       "params": nparams, "parallelism": "dp%d (gradient all-reduce per stage, overlapped with the window's backward)" % world, "l2": "activations far larger than L2",
                       "chunk_states": "recomputed in backward" if recompute else "saved by forward"},
            "loss": loss, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            "roofline": {"kernel": "whole step, dense-equivalent work (6 x stage parameters x stage rows)", "bound": "tensor", "achieved": dense,
                         "peak": sustained, "unit": "TFLOP/s", "frac": dense / sustained, "traffic": None, "peak_source": pk["src"] + " (sustained)",
                         "mlstm_core_ms_per_step": mcore_ms, "mlstm_core_share": mcore_ms / ms},
            "e2e": {"value": val, "unit": "bytes/s", "h2d_bytes_per_step": ids_bytes, "d2h_bytes_per_step": 4,
                    "note": "the timed step already starts from host token arrays and reads the loss back"},
            "gpu_launches": int(launches), "clocks": clocks, "cpu_baseline": cpu}))


def cpu_hier_sample(seed=0, nbytes=512, S=8):
    """The CPU restatement of the hierarchical model at configs[4]'s widths on one short window (`nbytes` bytes in
    words of S): forward, backward and AdamW. Every stage's cost is linear in the bytes it sees, so bytes/s of the
    sample is the figure for the full batch. Returns (bytes_per_s, seconds)."""
    from oracle import hier as OH
    cfg = OH.HierCfg(vocab=257, hc=256, wh=1024, enc_blocks=2, bb_blocks=8, dec_blocks=2, heads=8, dqk=128, w_token=256,
                     small_heads=2, enc_kinds="mm", bb_kinds="m" * 8, dec_kinds="mm")
    model = OH.Hierarchical(OH.init_hier_params(np.random.default_rng(seed), cfg, std=0.02), cfg)
    r = np.random.default_rng(seed + 1)
    wins = [(r.integers(0, 256, nbytes), [(i * S, (i + 1) * S) for i in range(nbytes // S)])]
    model.forward_backward(wins)  # first call: allocations, BLAS start-up
    t0 = time.perf_counter()
    model.forward_backward(wins)
    for q in model.params():
        q.step(1e-3, 0.1, 1)
    dt = time.perf_counter() - t0
    return nbytes / dt, dt


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
        line = {
            "metric": "mlstm_layer_tokens_per_s", "value": B * T * world / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "mlstm_layer_fwd_bwd, sequences of %d positions cut over %d GPUs (B16 H8 S2048 per GPU, dqk128 dv128 chunk64)" % (T * world, world),
                       "parallelism": "cp%d (segment summaries all-gathered, carry folded, BPTT state suffix-summed)" % world,
                       "l2": "tensors larger than L2"},
            "gpu_launches": int(launches)}
        bf, bb = algorithmic_bytes(B, H, T, dqk, dhv, 4)
        pk = peaks()
        gbs = (bf + bb) / (ms * 1e-3) / 1e9
        line["roofline"] = {"kernel": "forward + backward of one segment, everything a rank runs for it (summary pass, exchanges, fold included)",
                            "bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"], "traffic": None,
                            "peak_source": pk["src"], "algorithmic_bytes": bf + bb}
        if world == 1 and not args.no_cpu:
            cpu = cpu_mlstm_sample()
            line["cpu_baseline"] = {"value": cpu["tokens"] / cpu["seconds"], "unit": "tokens/s", "cores": cpu["threads"], "kind": "port",
                                    "sample": "%d of 16 sequences x 2048 positions x 8 heads, recurrent f32 restatement, OpenMP over (batch, head)" % cpu["seqs"]}
        print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="lm", choices=["lm", "mlstm", "ops", "hier", "cp"],
                    help="lm: data-parallel training step of the configs[3] model (headline); mlstm: the configs[1] layer kernel pair; "
                         "ops: the other hot-path kernels alone; hier: configs[4] hierarchical training step; cp: the layer kernel "
                         "with sequences cut over the GPUs")
    ap.add_argument("--grad-dtype", default="f32", choices=["f32", "bf16"], help="mlstm workload: width of d_ytil, dq, dk, dv")
    ap.add_argument("--mlstm-shape", default=None, help="mlstm workload: B,H,S,d instead of configs[1] (kernel studies)")
    ap.add_argument("--recompute", action="store_true", help="backward recomputes chunk-boundary states instead of reading a saved record")
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-pair", action="store_true", help="lm workload: skip the configs[1] kernel-pair measurement")
    ap.add_argument("--no-kernels", action="store_true", help="lm workload: skip the instrumented step behind `kernels`")
    ap.add_argument("--hier-saved-states", action="store_true", help="hier workload: keep the chunk-state records instead of recomputing them")
    ap.add_argument("--lm-blocks", type=int, default=0, help="override the LM depth (development)")
    ap.add_argument("--lm-remat", type=int, default=0,
                    help="mLSTM blocks rematerialised in the LM workload (0: all 24 blocks' activations fit, 127 GB peak)")
    ap.add_argument("--lm-head-terms", type=int, default=3, choices=(3, 6),
                    help="LM head GEMMs: bf16 products per fp32 product (6: fp32-accurate; 3: 16 significand bits per operand)")
    ap.add_argument("--lm-reduced", action="store_true", help="LM workload at half width (d=1024, heads of 128 / 256): development stand-in")
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
        run_mlstm(args)


if __name__ == "__main__":
    main()
