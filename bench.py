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
# dram__bytes_read.sum + dram__bytes_write.sum of one m = 2 launch of awq_gemv_tma_kernel on this layer shape,
# recorded from an ncu capture (not measured by this script; algorithmic bytes of that launch: algo_bytes(2)).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 30_560_768


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

    def sweep(ms=M_SWEEP):
        for m in ms:
            for lin in layers:
                lin.forward(xs[m], out=ys[m])  # the operator's own dispatch: split-k GEMV up to 16 tokens, fused tcgen05 kernel at 32

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
    # Device staging buffers are allocated once (as a serving loop would); every call still copies its input from
    # pinned host memory and its result back. Calls alternate between two streams, each with its own staging and
    # host result buffers, so the copies of one call overlap the kernel of the other.
    NSTREAMS = 2
    e2e_streams = [torch.cuda.Stream() for _ in range(NSTREAMS)]
    xd = {(m, i): torch.empty_like(xs[m]) for m in M_SWEEP for i in range(NSTREAMS)}
    yd = {(m, i): torch.empty_like(ys[m]) for m in M_SWEEP for i in range(NSTREAMS)}
    yh = {(m, i): torch.empty((m, N), dtype=torch.bfloat16).pin_memory() for m in M_SWEEP for i in range(NSTREAMS)}

    def e2e_step():
        call = 0
        for m in M_SWEEP:
            for lin in layers:
                i = call % NSTREAMS
                call += 1
                with torch.cuda.stream(e2e_streams[i]):
                    xd[m, i].copy_(xs_host[m], non_blocking=True)
                    lin.forward(xd[m, i], out=yd[m, i])
                    yh[m, i].copy_(yd[m, i], non_blocking=True)
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

    extras, sharded = None, None
    if not args.no_extras:
        extras, sharded = run_extras(args, world, rank, layers[0])

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
                     "frac": round(achieved / peak, 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                     "traffic_source": "recorded ncu capture of one m = 2 launch of awq_gemv_tma_kernel (dram read + write bytes)",
                     "kernel": "awq_gemv_tma_kernel (m <= 8), awq_gemv_group_kernel (m = 16), awq_fused_tc_kernel (m = 32)",
                     "peak_kind": f"{peak_kind} copy bandwidth", "per_m": per_m},
        "clocks": clocks,
    }
    if cpu is not None:
        out["cpu_baseline"] = cpu
    if extras is not None:
        out["other_configs"] = extras
    if sharded:
        out["sharded"] = sharded
    print(json.dumps(out), flush=True)



# --------------------------------------------------------------------------- other configurations
def _timed_ms(torch, dist, world, fn, iters):
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
    ms = e0.elapsed_time(e1) / iters
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


class _NotSelected(Exception):
    pass


def run_extras(args, world, rank, c1_layer):
    """The benchmark configurations next to the headline one: Q4_K/Q8_0 GEMV, AWQ prefill GEMM, FP8 block GEMV/GEMM, MXFP4 MoE
    (single-GPU legs on every rank's own GPU; tensor- and expert-parallel legs when world > 1)."""
    import torch
    import torch.distributed as dist

    from oxydllm_b200 import formats as F
    from oxydllm_b200 import gemm, moe, parallel, synth
    from oxydllm_b200 import linear as L

    peaks = {}
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
    except Exception:
        pass
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    tf_burst = float(peaks.get("bf16_tflops", 1590.0))
    out = {}
    sharded = {}  # legs that split one operator over the ranks (tensor / expert parallel), with parity against one GPU
    dev = lambda a, dt=None: (torch.from_numpy(np.ascontiguousarray(a)).to(dt) if dt else torch.from_numpy(np.ascontiguousarray(a))).cuda()

    def graph_us(fn_once, launches, reps=20):
        fn_once(); torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn_once()
        for _ in range(3):
            g.replay()
        return _timed_ms(torch, dist, world, g.replay, reps) * 1e3 / launches

    want = {c.strip() for c in args.configs.split(",")}

    # ---- C0: GGUF Q4_K GEMV, N = K = 4096, M = 1 (16 distinct copies: 151 MB > L2)
    try:
        if "c0" not in want:
            raise _NotSelected()
        n = k = 4096
        copies = [L.QLinear(F.GGML_Q4_K, dev(synth.gguf_layer(F.GGML_Q4_K, n, k, seed=100 * rank + i)), n, k) for i in range(2)]
        base = copies[0].blocks
        lins = copies + [L.QLinear(F.GGML_Q4_K, torch.roll(base, 144 * (i + 1)), n, k) for i in range(14)]
        x = dev(synth.activations(1, k, seed=1), torch.bfloat16)
        us = graph_us(lambda: [lin.forward(x) for lin in lins], len(lins))
        b = n * (k // 256) * 144 + k * 2 + n * 2
        out["c0_q4k_gemv_m1"] = {"us_per_launch": round(us, 2), "gbs": round(b / us / 1e3, 1),
                                  "frac_of_hbm_peak": round(b / us / 1e3 / hbm, 4), "algorithmic_bytes": b}
        del lins, copies
        # the same layer shape as Q8_0 (34-byte blocks): 16 rolled copies of one encoded matrix
        base = dev(synth.gguf_layer(F.GGML_Q8_0, n, k, seed=200 + rank))
        lins = [L.QLinear(F.GGML_Q8_0, torch.roll(base, 34 * 2 * i), n, k) for i in range(16)]
        us = graph_us(lambda: [lin.forward(x) for lin in lins], len(lins))
        b = n * (k // 32) * 34 + k * 2 + n * 2
        out["c0_q8_0_gemv_m1"] = {"us_per_launch": round(us, 2), "gbs": round(b / us / 1e3, 1),
                                   "frac_of_hbm_peak": round(b / us / 1e3 / hbm, 4), "algorithmic_bytes": b}
        del lins, base
    except _NotSelected:
        pass
    except Exception as e:  # keep the headline line alive
        out["c0_q4k_gemv_m1"] = {"error": str(e)[:200]}

    # ---- C1 shape beyond the sweep: continuous-batching sizes through the operator (tensor-core GEMM on dequantized slabs
    #      above 32 tokens), the tcgen05 decode matmul on one-byte weights (opt-in entry point), and the GPTQ 4-bit GEMV
    try:
        if "c1x" not in want:
            raise _NotSelected()
        lins = [c1_layer] + [L.PackedQuantLinear(L.QuantWeight.new_awq(4, torch.roll(c1_layer.qweight, 64 * (i + 1), 0),
                                                                       c1_layer.qzeros, c1_layer.scales)) for i in range(5)]
        res = {}
        for m in (64, 128, 256):
            x = dev(synth.activations(m, K, seed=m), torch.bfloat16)
            y = torch.empty((m, N), dtype=torch.bfloat16, device="cuda")
            us = graph_us(lambda: [lin.forward(x, out=y) for lin in lins], len(lins), reps=10)
            res[f"operator_m{m}"] = {"us_per_call": round(us, 2), "gbs": round(algo_bytes(m) / us / 1e3, 1),
                                     "frac_of_hbm_peak": round(algo_bytes(m) / us / 1e3 / hbm, 4),
                                     "tflops": round(2.0 * m * N * K / us / 1e6, 1)}
        for m in (1, 8, 16, 32):
            x = dev(synth.activations(m, K, seed=m), torch.bfloat16)
            y = torch.empty((m, N), dtype=torch.bfloat16, device="cuda")
            us = graph_us(lambda: [gemm.awq_decode_matmul(lin, x, y) for lin in lins], len(lins), reps=10)
            res[f"tcgen05_decode_matmul_m{m}"] = {"us_per_call": round(us, 2), "gbs": round(algo_bytes(m) / us / 1e3, 1),
                                                  "frac_of_hbm_peak": round(algo_bytes(m) / us / 1e3 / hbm, 4)}
        gemm.check(gemm.decode_workspace(32, K, N, "cuda"))
        rng = np.random.default_rng(11)
        glins = []
        for i in range(4):
            gq = dev(rng.integers(0, 2 ** 32, size=(K // 8, N), dtype=np.uint64).astype(np.uint32).view(np.int32))
            gz = dev(rng.integers(0, 2 ** 32, size=(K // G, N // 8), dtype=np.uint64).astype(np.uint32).view(np.int32))
            glins.append(L.PackedQuantLinear(L.QuantWeight.new_gptq(4, False, gq, gz, c1_layer.scales)))
        for m in (1, 8, 64):  # GPTQ 4-bit through the operator: GEMV up to 2 tokens, fused tcgen05 kernel above
            x = dev(synth.activations(m, K, seed=m), torch.bfloat16)
            us = graph_us(lambda: [lin.forward(x) for lin in glins], len(glins), reps=10)
            res[f"gptq4_operator_m{m}"] = {"us_per_call": round(us, 2), "gbs": round(algo_bytes(m) / us / 1e3, 1),
                                           "frac_of_hbm_peak": round(algo_bytes(m) / us / 1e3 / hbm, 4)}
        # narrow layers of the same model family (attention projection 4096 x 4096, down projection 14336 -> 4096): the fused
        # kernel splits k over the SMs
        for (kk, nn, tag) in ((4096, 4096, "attn_4096x4096"), (14336, 4096, "down_4096x14336")):
            nl = []
            for i in range(6):
                nqw, nqz, nsc = synth.awq_layer(kk, nn, G, seed=700 + i)
                nl.append(L.PackedQuantLinear(L.QuantWeight.new_awq(4, dev(nqw.view(np.int32)), dev(nqz.view(np.int32)), dev(nsc))))
            for m in (1, 32, 128):
                x = dev(synth.activations(m, kk, seed=m), torch.bfloat16)
                us = graph_us(lambda: [lin.forward(x) for lin in nl], len(nl), reps=10)
                nb = kk * nn // 2 + (kk // G) * (nn // 2) + (kk // G) * nn * 2 + m * (2 * kk + 2 * nn)
                res[f"{tag}_operator_m{m}"] = {"us_per_call": round(us, 2), "gbs": round(nb / us / 1e3, 1),
                                               "frac_of_hbm_peak": round(nb / us / 1e3 / hbm, 4)}
            del nl
        # gated FFN projection of the same family at decode batches: fused [gate | up] weight 4096 -> 2 x 14336, SiLU
        fqw, fqz, fsc = synth.awq_layer(K, 2 * N, G, seed=770)
        fq = dev(fqw.view(np.int32))
        fl = [L.GatedFfnProjection(L.PackedQuantLinear(L.QuantWeight.new_awq(4, torch.roll(fq, 64 * i, 0), dev(fqz.view(np.int32)),
                                                                              dev(fsc))), "silu") for i in range(3)]
        for m in (1, 32, 128):
            x = dev(synth.activations(m, K, seed=m), torch.bfloat16)
            us = graph_us(lambda: [f.forward(x) for f in fl], len(fl), reps=10)
            nb = K * N + (K // G) * N + (K // G) * 2 * N * 2 + m * (2 * K + 2 * N)
            res[f"ffn_gate_up_silu_i14336_m{m}"] = {"us_per_call": round(us, 2), "gbs": round(nb / us / 1e3, 1),
                                                    "frac_of_hbm_peak": round(nb / us / 1e3 / hbm, 4)}
        del fl, fq
        out["c1_shape_other_batches_and_layouts"] = res
        del lins, glins
    except _NotSelected:
        pass
    except Exception as e:
        out["c1_shape_other_batches_and_layouts"] = {"error": str(e)[:200]}

    # ---- C2: AWQ prefill GEMM M = 2048, K = 4096, N in {4096, 14336}
    try:
        if "c2" not in want:
            raise _NotSelected()
        m = 2048
        x = dev(synth.activations(m, K, seed=2), torch.bfloat16)
        res = {}
        for n in (4096, 14336):
            a, b_ = 0, n
            qw, qz, sc = parallel.ColumnParallelLinear.slice_awq(c1_layer.qweight, c1_layer.qzeros, c1_layer.scales, a, b_)
            lin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, qw, qz, sc))
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            for _ in range(3):
                gemm.awq_matmul(lin, x, y)
            ms = _timed_ms(torch, dist, world, lambda: gemm.awq_matmul(lin, x, y), 10)
            tf = 2.0 * m * n * K / ms / 1e9
            res[f"n{n}"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_bf16_burst_peak": round(tf / tf_burst, 4)}
        # gated FFN projection on the fused [gate | up] weight (intermediate 14336): activation in the GEMM epilogue
        inter = 14336
        from oxydllm_b200 import formats as F2
        fused = F2.concat_awq_along_out([(c1_layer.qweight.cpu().numpy().view(np.uint32), c1_layer.qzeros.cpu().numpy().view(np.uint32),
                                          c1_layer.scales.cpu().numpy())] * 2)
        glin = L.PackedQuantLinear(L.QuantWeight.new_awq(4, dev(fused[0].view(np.int32)), dev(fused[1].view(np.int32)), dev(fused[2])))
        ffn = L.GatedFfnProjection(glin, "silu")
        for _ in range(3):
            ffn.forward(x)
        ms = _timed_ms(torch, dist, world, lambda: ffn.forward(x), 10)
        tf = 2.0 * m * 2 * inter * K / ms / 1e9
        res["ffn_gate_up_silu_i14336"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_bf16_burst_peak": round(tf / tf_burst, 4)}
        del glin, ffn, fused
        gemm.check(gemm.workspace(1, 8, "cuda"))
        # lm_head-class width (src/common/block.rs:598): the C1 layer's packed columns tiled to N = 128256 (throughput is
        # data-independent; parity at this width is covered by the tests)
        n_big = 128256
        reps = -(-n_big // N)
        big = [torch.cat([t] * reps, dim=1)[:, :w].contiguous() for t, w in
               ((c1_layer.qweight, n_big // 8), (c1_layer.qzeros, n_big // 8), (c1_layer.scales, n_big))]
        lin_big = L.PackedQuantLinear(L.QuantWeight.new_awq(4, *big))
        y_big = torch.empty((m, n_big), dtype=torch.bfloat16, device="cuda")
        for _ in range(2):
            gemm.awq_matmul(lin_big, x, y_big)
        ms_big = _timed_ms(torch, dist, world, lambda: gemm.awq_matmul(lin_big, x, y_big), 5)
        tf = 2.0 * m * n_big * K / ms_big / 1e9
        res[f"n{n_big}"] = {"ms": round(ms_big, 4), "tflops": round(tf, 1), "frac_of_bf16_burst_peak": round(tf / tf_burst, 4),
                            "note": "weight cut into 8 dequantization slabs of 128 MiB"}
        gemm.check(gemm.workspace(1, 8, "cuda"))
        if world > 1:  # tensor-parallel column split, checked against the single-GPU result of this rank
            # every rank must hold the SAME layer here (the headline layers differ per rank): one common seed
            cqw, cqz, csc = synth.awq_layer(K, N, G, seed=4242)
            common = [dev(cqw.view(np.int32)), dev(cqz.view(np.int32)), dev(csc)]
            lin_c = L.PackedQuantLinear(L.QuantWeight.new_awq(4, *common))
            big_c = [torch.cat([t] * reps, dim=1)[:, :w].contiguous() for t, w in
                     ((common[0], n_big // 8), (common[1], n_big // 8), (common[2], n_big))]
            lin_big_c = L.PackedQuantLinear(L.QuantWeight.new_awq(4, *big_c))
            y_c = torch.empty((m, N), dtype=torch.bfloat16, device="cuda")
            for n, lin_full, y_full, ms_1gpu in ((14336, lin_c, y_c, res["n14336"]["ms"]), (n_big, lin_big_c, y_big, ms_big)):
                a, b_ = parallel.column_shard(n, world, rank)
                qw, qz, sc = parallel.ColumnParallelLinear.slice_awq(lin_full.qweight, lin_full.qzeros, lin_full.scales, a, b_)
                shard = L.PackedQuantLinear(L.QuantWeight.new_awq(4, qw, qz, sc))
                tp = parallel.ColumnParallelLinear(shard.forward, n, chunks=1)  # one call: the shard is dequantized once
                for _ in range(3):
                    y_tp = tp.forward(x)
                ms = _timed_ms(torch, dist, world, lambda: tp.forward(x), 10 if n == 14336 else 5)
                gemm.awq_matmul(lin_full, x, y_full)
                ref = y_full.float()
                ok = bool(((y_tp.float() - ref).abs() <= 2e-2 * ref.abs().amax(dim=1, keepdim=True) + 1e-6).all().item())
                tf = 2.0 * m * n * K / ms / 1e9
                sharded[f"tp{world}_c2_awq_gemm_n{n}_allgather"] = {
                    "ms": round(ms, 4), "tflops_whole_job": round(tf, 1), "ms_1gpu": round(ms_1gpu, 4),
                    "speedup_vs_1gpu": round(ms_1gpu / ms, 3), "parity_ok": ok,
                    "gathered_bytes_per_rank": int(m * n * 2 * (world - 1) / world)}
                try:  # direct placement: the GEMM epilogue stores each tile into every rank's output (no gather, no re-layout)
                    ps = parallel.PeerStoreColumnLinear(shard, n, m_max=m)
                    for _ in range(3):
                        y_ps = ps.forward(x)
                    ms_ps = _timed_ms(torch, dist, world, lambda: ps.forward(x), 10 if n == 14336 else 5)
                    ok_ps = bool(((y_ps.float() - ref).abs() <= 2e-2 * ref.abs().amax(dim=1, keepdim=True) + 1e-6).all().item())
                    sharded[f"tp{world}_c2_awq_gemm_n{n}_peer_store"] = {
                        "ms": round(ms_ps, 4), "tflops_whole_job": round(2.0 * m * n * K / ms_ps / 1e9, 1),
                        "ms_1gpu": round(ms_1gpu, 4), "speedup_vs_1gpu": round(ms_1gpu / ms_ps, 3), "parity_ok": ok_ps,
                        "stored_to_peers_bytes_per_rank": int(m * (b_ - a) * 2 * (world - 1))}
                    del ps, y_ps
                except Exception as e:
                    sharded[f"tp{world}_c2_awq_gemm_n{n}_peer_store"] = {"error": str(e)[:200]}
                if n == 14336:  # the same split at a decode batch: the fused unpack + tcgen05 kernel on the shard, then the peer stores
                    try:
                        for md in (32, 256):
                            xdec = x[:md].contiguous()
                            y1 = torch.empty((md, n), dtype=torch.bfloat16, device="cuda")
                            for _ in range(3):
                                gemm.awq_matmul(lin_full, xdec, y1)
                            ms1 = _timed_ms(torch, dist, world, lambda: gemm.awq_matmul(lin_full, xdec, y1), 20)
                            psd = parallel.PeerStoreColumnLinear(shard, n, m_max=md)
                            for _ in range(3):
                                y_pd = psd.forward(xdec)
                            msd = _timed_ms(torch, dist, world, lambda: psd.forward(xdec), 20)
                            refd = y1.float()
                            okd = bool(((y_pd.float() - refd).abs() <= 2e-2 * refd.abs().amax(dim=1, keepdim=True) + 1e-6).all().item())
                            sharded[f"tp{world}_c1_awq_m{md}_peer_store"] = {
                                "ms": round(msd, 4), "ms_1gpu": round(ms1, 4), "speedup_vs_1gpu": round(ms1 / msd, 3), "parity_ok": okd,
                                "stored_to_peers_bytes_per_rank": int(md * (b_ - a) * 2 * (world - 1))}
                            del psd, y_pd
                    except Exception as e:
                        sharded[f"tp{world}_c1_awq_decode_peer_store"] = {"error": str(e)[:200]}
                del tp, shard
            del lin_c, lin_big_c, big_c, common, y_c
        del lin_big, y_big, big
        out["c2_awq_gemm_m2048"] = res
    except _NotSelected:
        pass
    except Exception as e:
        out["c2_awq_gemm_m2048"] = {"error": str(e)[:200]}

    # ---- C3: FP8 E4M3 128x128-block GEMV (M = 1, 32) and GEMM (M = 2048), N = 14336, K = 4096
    try:
        if "c3" not in want:
            raise _NotSelected()
        n = 14336
        q, s_ = synth.fp8_layer(n, K, seed=3 + rank)
        base = dev(q)
        lins = [L.Fp8Linear(base, dev(s_))] + [L.Fp8Linear(torch.roll(base, 4096 * (i + 1), 0), dev(s_)) for i in range(3)]
        res = {}
        for m in (1, 16, 32, 128):  # through the operator: GEMV up to 16 tokens, fused widen + tcgen05 kernel up to 256
            x = dev(synth.activations(m, K, seed=m), torch.bfloat16)
            us = graph_us(lambda: [lin.forward(x) for lin in lins], len(lins))
            b = n * K + (n // 128) * (K // 128) * 4 + m * (2 * K + 2 * n)
            res[f"gemv_m{m}" if m <= 16 else f"operator_m{m}"] = {"us_per_launch": round(us, 2), "gbs": round(b / us / 1e3, 1),
                                                                  "frac_of_hbm_peak": round(b / us / 1e3 / hbm, 4)}
        x = dev(synth.activations(2048, K, seed=5), torch.bfloat16)
        for _ in range(3):
            lins[0].forward(x)
        ms = _timed_ms(torch, dist, world, lambda: lins[0].forward(x), 10)
        tf = 2.0 * 2048 * n * K / ms / 1e9
        res["gemm_m2048"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_bf16_burst_peak": round(tf / tf_burst, 4)}
        out["c3_fp8_block"] = res
        del lins, base
    except _NotSelected:
        pass
    except Exception as e:
        out["c3_fp8_block"] = {"error": str(e)[:200]}

    # ---- C4: GPT-OSS-20B-shaped MXFP4 MoE layer, 32 experts, top-4, 4096 tokens
    try:
        if "c4" not in want:
            raise _NotSelected()
        e, hidden, inter, tokens = 32, 2880, 2880, 4096
        d = synth.gptoss_moe(4, hidden, inter, tokens, seed=4)  # 4 distinct experts, tiled 8x (throughput is data-independent)
        rep = lambda a: np.concatenate([a] * (e // 4), axis=0)
        layer = moe.GptOssMoe(dev(rep(d["gu_blocks"])), dev(rep(d["gu_scales"])), dev(rep(d["gu_bias"]), torch.bfloat16),
                              dev(rep(d["dn_blocks"])), dev(rep(d["dn_scales"])), dev(rep(d["dn_bias"]), torch.bfloat16),
                              hidden=hidden, inter=inter, top_k=4)
        lg = dev(np.random.default_rng(6).standard_normal((tokens, e)).astype(np.float32))
        x = dev(d["x"], torch.bfloat16)
        for _ in range(2):
            layer.forward_with_logits(x, lg)
        layer.check()
        ms = _timed_ms(torch, dist, world, lambda: layer.forward_with_logits(x, lg), 5)
        fl = tokens * 4 * (2.0 * hidden * 2 * inter + 2.0 * inter * hidden)
        res = {"ms": round(ms, 3), "tflops": round(fl / ms / 1e9, 1), "tokens_per_s": round(tokens / ms * 1e3, 0),
               "frac_of_bf16_burst_peak": round(fl / ms / 1e9 / tf_burst, 4),
               "note": "4 distinct experts tiled to 32; router logits N(0,1) given, router GEMM not timed"}
        # one expert's gate_up projection as a plain MXFP4 linear, decode-sized (8 rolled copies)
        gub, gus = layer.gu_blocks[0].reshape(-1), layer.gu_scales[0].reshape(-1)
        mx = [L.Mxfp4Linear(torch.roll(gub, 16 * (hidden // 32) * i).reshape(2 * inter, hidden // 32, 16),
                            torch.roll(gus, (hidden // 32) * i).reshape(2 * inter, hidden // 32), None, hidden, 2 * inter) for i in range(8)]
        x1 = x[:1].contiguous()
        us = graph_us(lambda: [lin.forward(x1) for lin in mx], len(mx))
        b = 2 * inter * hidden // 2 + 2 * inter * hidden // 32 + hidden * 2 + 2 * inter * 2
        res["mxfp4_gemv_m1_5760x2880"] = {"us_per_launch": round(us, 2), "gbs": round(b / us / 1e3, 1),
                                          "frac_of_hbm_peak": round(b / us / 1e3 / hbm, 4)}
        del mx
        # decode-sized batches: only the selected experts' packed weights are streamed (batched GEMVs)
        per_pair_bytes = (2 * inter * hidden + hidden * inter) // 2 + (2 * inter * hidden + hidden * inter) // 32
        for t_dec in (1, 8):
            xd, ld = x[:t_dec].contiguous(), lg[:t_dec].contiguous()
            us = graph_us(lambda: layer.forward_with_logits(xd, ld), 1)
            res[f"decode_tokens{t_dec}"] = {"us": round(us, 2), "gbs_upper_bound_distinct_experts": round(
                t_dec * 4 * per_pair_bytes / us / 1e3, 1), "note": "bytes counted as if every (token, slot) pair hit a distinct expert"}
        # batches between decode and the headline size: the grouped kernel reads every routed expert's packed weights once per
        # token block, no expert is dequantized to a dense copy
        for t_mid in (32, 128, 512):
            xm, lm = x[:t_mid].contiguous(), lg[:t_mid].contiguous()
            for _ in range(2):
                layer.forward_with_logits(xm, lm)
            ms_mid = _timed_ms(torch, dist, world, lambda: layer.forward_with_logits(xm, lm), 5)
            res[f"tokens{t_mid}"] = {"ms": round(ms_mid, 4), "tokens_per_s": round(t_mid / ms_mid * 1e3, 0)}
        if world > 1:  # expert parallel: tokens data-parallel, all-to-all dispatch and combine
            t_local = tokens // world
            sl = slice(rank * t_local, (rank + 1) * t_local)
            ep = parallel.ExpertParallelMoe(e, lambda l_: moe.route(l_, 4, True), parallel.gptoss_local_experts(layer))
            xl, ll = x[sl].contiguous(), lg[sl].contiguous()
            for _ in range(2):
                y_ep = ep.forward(xl, ll)
            ms_ep = _timed_ms(torch, dist, world, lambda: ep.forward(xl, ll), 5)
            ref = layer.forward_with_logits(xl, ll).float()  # the same tokens through all experts on this GPU
            ok = bool(((y_ep.float() - ref).abs() <= 2e-2 * ref.abs().amax(dim=1, keepdim=True) + 1e-3).all().item())
            sharded[f"ep{world}_c4_mxfp4_moe_all_to_all"] = {
                "ms": round(ms_ep, 3), "tflops_whole_job": round(fl / ms_ep / 1e9, 1),
                "tokens_per_s_whole_job": round(tokens / ms_ep * 1e3, 0), "ms_1gpu": round(ms, 3),
                "speedup_vs_1gpu": round(ms / ms_ep, 3), "parity_ok": ok}
        out["c4_mxfp4_moe"] = res
    except _NotSelected:
        pass
    except Exception as e:
        out["c4_mxfp4_moe"] = {"error": str(e)[:200]}
    return out, sharded

# --------------------------------------------------------------------------- CPU arm
def cpu_sweep_once(w_f32, xs):
    import oracle
    for m in M_SWEEP:
        oracle.linear(xs[m], w_f32)


def cpu_prepare():
    import oracle
    from oxydllm_b200 import synth
    # torchrun exports OMP_NUM_THREADS=1: take every core this process may run on
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    oracle.set_num_threads(cores)
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
    ap.add_argument("--no-extras", action="store_true", help="skip configurations 0, 2, 3, 4 (headline C1 line only)")
    ap.add_argument("--configs", default="c0,c1x,c2,c3,c4",
                    help="which of the other configurations to run, e.g. 'c3' (used to keep profiler captures small)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
