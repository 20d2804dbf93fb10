#!/usr/bin/env python
"""Benchmark of the quantized-weight matrix-product path on B200.

Default workload ("c1"): AWQ W4A16 batched decode GEMV, K=4096, N=14336,
group 128, swept over M in {1, 2, 4, 8, 16, 32}. One step = that sweep over
LAYERS distinct weight copies (LAYERS x 30.5 MB > the 126 MB L2, so every
launch streams its weights from HBM), replayed from one CUDA graph.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints one JSON line (rank 0). ``value`` is algorithmic GB/s over all GPUs
with inputs resident in HBM; ``e2e`` is the same metric through the public
operator (``PackedQuantLinear.forward``) with pinned host activations copied
in and results copied out inside the timed region. ``--impl reference`` times
the CPU restatement of the reference's path (dequantize at load, untimed, then
dense f32 matmul per forward; linear.rs:582-601) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

K, N, G = 4096, 14336, 128
M_SWEEP = (1, 2, 4, 8, 16, 32)
LAYERS = 12
WEIGHT_BYTES = K * N // 2 + (K // G) * (N // 8) * 4 + (K // G) * N * 2  # qweight + qzeros + f16 scales
METRIC = "Quant GEMV HBM GB/s (AWQ W4A16 decode, algorithmic bytes / time)"


def algo_bytes(m: int) -> int:
    """Every operand counted once: packed weights, zeros, scales, bf16 x and bf16 y."""
    return WEIGHT_BYTES + m * (K * 2 + N * 2)


BYTES_PER_STEP = LAYERS * sum(algo_bytes(m) for m in M_SWEEP)
LAUNCHES_PER_STEP = LAYERS * len(M_SWEEP)


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi polling in the background while the timed region runs (read-only queries)."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "nvidia-smi unavailable"}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1])); mx.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- GPU arm
def run_gpu(args):
    import torch
    import torch.distributed as dist

    from oxydllm_b200 import linear as L
    from oxydllm_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # LAYERS distinct packed layers per GPU (different seeds), resident in HBM.
    layers = []
    for l in range(LAYERS):
        qw, qz, sc = synth.awq_layer(K, N, G, seed=1000 * rank + l)
        raw = L.QuantWeight.new_awq(4, torch.from_numpy(qw.view(np.int32)).cuda(),
                                    torch.from_numpy(qz.view(np.int32)).cuda(), torch.from_numpy(sc).cuda())
        layers.append(L.PackedQuantLinear(raw))
    xs_host = {m: torch.from_numpy(synth.activations(m, K, seed=m)).to(torch.bfloat16).pin_memory() for m in M_SWEEP}
    xs = {m: xs_host[m].cuda() for m in M_SWEEP}
    ys = {m: torch.empty((m, N), dtype=torch.bfloat16, device="cuda") for m in M_SWEEP}
    ys_host = {m: torch.empty((m, N), dtype=torch.bfloat16).pin_memory() for m in M_SWEEP}

    def sweep(ms=M_SWEEP):
        for m in ms:
            for lin in layers:
                lin._gemv(xs[m], ys[m], m)

    def make_graph(fn):
        fn()
        torch.cuda.synchronize()
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            return g.replay, "cuda_graph"
        except Exception as e:  # capture unsupported: launch directly on the stream
            sys.stderr.write(f"[bench] graph capture failed ({e}); using stream launches\n")
            torch.cuda.synchronize()
            return fn, "stream"

    step, launch_mode = make_graph(sweep)

    def timed(fn, iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_wall0 = time.time()
    for _ in range(max(args.warmup, 3)):
        step()
    total_ms = timed(step, args.steps)
    ms_per_step = total_ms / args.steps
    value = world * BYTES_PER_STEP / (ms_per_step * 1e-3) / 1e9

    # Per-M breakdown (one graph per M over all layers) for the roofline of each launch shape.
    per_m = []
    for m in M_SWEEP:
        fn, _ = make_graph(lambda m=m: sweep((m,)))
        for _ in range(3):
            fn()
        reps = 20
        us = timed(fn, reps) * 1e3 / (reps * LAYERS)
        per_m.append({"m": m, "us_per_launch": round(us, 3), "gbs": round(algo_bytes(m) / us / 1e3, 1)})

    # End to end through the public operator with host buffers.
    def e2e_step():
        for m in M_SWEEP:
            for lin in layers:
                xd = xs_host[m].to("cuda", non_blocking=True)
                y = lin.forward(xd)
                ys_host[m].copy_(y, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    e2e_iters = max(3, min(args.steps, 10))
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_iters):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * BYTES_PER_STEP * e2e_iters / e2e_s / 1e9

    # Keep the same work running until the clock sampler has seen it under load.
    while rank == 0 and time.time() - t_wall0 < 2.5:
        step()
        torch.cuda.synchronize()
    clocks = sampler.stop() if rank == 0 else None

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(budget_s=12.0)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak, peak_kind = measured_peak()
    avg_launch_s = ms_per_step * 1e-3 / LAUNCHES_PER_STEP
    achieved = (BYTES_PER_STEP / LAUNCHES_PER_STEP) / avg_launch_s / 1e9
    for r in per_m:
        r["frac_of_peak"] = round(r["gbs"] / peak, 4)
    out = {
        "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights x bf16 activations, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": f"C1: AWQ W4A16 decode GEMV K={K} N={N} g={G}, M sweep {list(M_SWEEP)} over {LAYERS} "
                               f"distinct layers per GPU (weights {LAYERS * WEIGHT_BYTES / 1e6:.0f} MB > L2, no flush needed)",
                   "launch": launch_mode, "parallelism": "independent layers per GPU (no collective on this path)"},
        "pct_of_8tbs": round(100.0 * value / world / 8000.0, 2),
        "gpu_launches": args.steps * LAUNCHES_PER_STEP,
        "e2e": {"value": round(e2e_value, 1), "unit": "GB/s",
                "h2d_bytes_per_step": LAYERS * sum(m * K * 2 for m in M_SWEEP),
                "d2h_bytes_per_step": LAYERS * sum(m * N * 2 for m in M_SWEEP)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": None, "kernel": "awq_gemv_kernel",
                     "peak_kind": f"{peak_kind} copy bandwidth", "per_m": per_m},
        "clocks": clocks,
    }
    if cpu is not None:
        out["cpu_baseline"] = cpu
    print(json.dumps(out), flush=True)


# --------------------------------------------------------------------------- CPU arm
def cpu_sweep_once(w_f32, xs):
    import oracle
    for m in M_SWEEP:
        oracle.linear(xs[m], w_f32)


def cpu_prepare():
    import oracle
    from oxydllm_b200 import synth
    qw, qz, sc = synth.awq_layer(K, N, G, seed=0)
    w = oracle.awq_dequant(qw, qz, sc)  # at load, untimed: what the reference does off Metal
    xs = {m: synth.activations(m, K, seed=m) for m in M_SWEEP}
    return w, xs, oracle.num_threads()


def cpu_baseline(budget_s: float):
    """The reference's CPU path restated (dense f32 matmul on the load-time dequantized weight), bounded sample."""
    w, xs, threads = cpu_prepare()
    cpu_sweep_once(w, xs)
    t0 = time.perf_counter()
    n = 0
    while True:
        cpu_sweep_once(w, xs)
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 50:
            break
    dt = time.perf_counter() - t0
    gbs = n * sum(algo_bytes(m) for m in M_SWEEP) / dt / 1e9
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"{n} sweeps of M {list(M_SWEEP)} over 1 layer (dequantized once, untimed) in {dt:.1f} s; "
                      "GB/s counts the same algorithmic bytes as the GPU arm"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w, xs, threads = cpu_prepare()
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_sweep_once(w, xs)
    steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_sweep_once(w, xs)
    dt = time.perf_counter() - t0
    per_step_bytes = sum(algo_bytes(m) for m in M_SWEEP)
    gbs = steps * per_step_bytes / dt / 1e9
    sample = (f"each step = one M sweep {list(M_SWEEP)} over 1 of the {LAYERS} layers (1/{LAYERS} of the GPU arm's step); "
              f"{steps} steps timed")
    out = {"impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": "GB/s",
           "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": max(1, min(args.warmup, 2)),
           "ms_per_step": round(dt / steps * 1e3, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32 (dequantized at load)", "data": "synthetic",
           "config": {"workload": f"C1: AWQ W4A16 decode GEMV K={K} N={N} g={G}, M sweep {list(M_SWEEP)}; CPU restatement "
                                  "of the reference's non-Metal path (linear.rs:582-601), cargo/candle unavailable"},
           "cpu_baseline": {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
           "e2e": {"value": round(gbs, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(out), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
