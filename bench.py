#!/usr/bin/env python
"""Benchmark of the affine-Q4 matmul path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # the CPU path, host cores

Workload (BASELINE.json configs[2]/[4]): the 27B-shape layer set of Q4
projections (q 5120->6144, k/v 5120->1024, o 6144->5120, fused gate/up
5120->17408 with SiLU, down 17408->5120) at decode (M rows = 1 by default),
looped over 64 layers with independent seeds (seed = layer index), so one step
streams 12.27 GB of distinct weights -- far more than L2.  With N > 1 every
projection is column-sharded over the ranks and the output slices are gathered.

One JSON line on stdout (rank 0).  `value` is algorithmic bytes of the whole job
per second of device time (max over ranks); `e2e` repeats the measurement with
the activations starting in pinned host memory and the outputs read back.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "q4_gemv_hbm_gbs"
UNIT = "GB/s"
LAYERS = 64


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.process = None
        self.path = None

    def start(self):
        try:
            handle = tempfile.NamedTemporaryFile(prefix="q4b_clocks_", suffix=".csv", delete=False)
            self.path = handle.name
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "100"], stdout=handle, stderr=subprocess.DEVNULL)
            handle.close()
        except OSError:
            self.process = None

    def stop(self):
        if self.process is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.process.terminate()
        try:
            self.process.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as handle:
            for line in handle:
                parts = [part.strip() for part in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    clocks.append(float(parts[1]))
                    maxima.append(float(parts[2]))
                except ValueError:
                    continue
                for name, flag in zip(names, parts[5:9]):
                    if flag.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(clocks), "sm_max_mhz": max(maxima), "samples": len(clocks),
                "reasons": sorted(reasons)}


def layer_work(q4b, m_rows):
    layer = q4b.LAYER_27B
    return q4b.layer_bytes(layer, m_rows), q4b.layer_flops(layer, m_rows)


# ----------------------------------------------------------------------------
# the CPU path (oracle port), timed on the host cores
# ----------------------------------------------------------------------------
def cpu_layer_pass(orc, q4b, m_rows, seed, row_fraction=1.0):
    """One layer of the workload through the CPU restatement of the reference's
    scalar loop, rows split over all host threads.  Returns (seconds, bytes)."""
    total_seconds, total_bytes, index = 0.0, 0, 0
    for p in q4b.LAYER_27B:
        groups = p.k // 64
        rows = max(16, int(p.n * row_fraction) // 16 * 16)
        x = orc.synth_x(seed, 0, m_rows, p.k)
        mats = []
        for _ in range(2 if p.fused else 1):
            mats.append(orc.synth_weight(seed, index, rows, groups))
            index += 1
        start = time.perf_counter()
        if p.fused:
            orc.gate_up_silu(mats[0][0], mats[0][1], mats[1][0], mats[1][1], groups, x, want64=False)
        else:
            orc.matmul(mats[0][0], mats[0][1], groups, x, want64=False)
        total_seconds += time.perf_counter() - start
        part = q4b.Projection(p.name, p.k, rows, p.fused)
        total_bytes += q4b.algorithmic_bytes(part, m_rows)
    return total_seconds, total_bytes


def cpu_baseline(q4b, m_rows, budget_seconds=12.0):
    from oracle import q4_oracle as orc
    threads = orc.max_threads()
    seconds, nbytes, passes = 0.0, 0, 0
    while seconds < budget_seconds and passes < 64:
        s, b = cpu_layer_pass(orc, q4b, m_rows, passes)
        seconds += s
        nbytes += b
        passes += 1
    return {"value": nbytes / seconds / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{passes} of {LAYERS} layers of the same workload (M={m_rows}), fp32 scalar loop, "
                      f"OpenMP over rows, {seconds:.1f} s of CPU time"}


def run_reference(args):
    """`--impl reference`: the reference's CPU formulation of the path on the host
    cores.  The reference's own functions are static code inside Objective-C files
    and a packer that only computes 8 rows, so the timed code is the C restatement
    (oracle/q4_oracle.c), all host threads, on whole layers of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    from oracle import q4_oracle as orc
    threads = orc.max_threads()
    layer_bytes, _ = layer_work(q4b, args.m)
    for step in range(args.warmup):
        cpu_layer_pass(orc, q4b, args.m, step, row_fraction=0.125)
    seconds, nbytes = 0.0, 0
    for step in range(args.steps):
        s, b = cpu_layer_pass(orc, q4b, args.m, step)
        seconds += s
        nbytes += b
    value = nbytes / seconds / 1e9
    sample = (f"each step = 1 of the {LAYERS} layers of the workload (M={args.m}); fp32 scalar loop, "
              f"OpenMP rows over {threads} threads")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u4*f16->f32",
            "data": "synthetic", "config": workload_config(args, 1),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def workload_config(args, world):
    return {"workload": f"27B-shape Q4 layer set (q,k,v,o,gate+up SiLU,down) x {LAYERS} layers, M={args.m}, "
                        f"seed=layer index (BASELINE configs[2]/[4])",
            "m_rows": args.m, "layers": LAYERS, "group": 64,
            "parallelism": ("single GPU" if world == 1 else
                            f"column-parallel N/{world} + all-gather ({args.gather})"),
            "l2": "inputs_exceed_l2 (12.27 GB of distinct weights per step)"}


# ----------------------------------------------------------------------------
# this library
# ----------------------------------------------------------------------------
def run_ours(args):
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N > 1 with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N")
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_module
        torch.cuda.set_device(local_rank)
        dist_module.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_module

    from importlib import import_module
    sharded = import_module("cpu-llms-in-c_b200.sharded")
    ctx = q4b.Q4Context(local_rank)
    model = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, LAYERS, args.m, rank, world, dist, gather=args.gather,
                                      mode=args.mode)
    layer_bytes, layer_flops = layer_work(q4b, args.m)
    step_bytes = layer_bytes * LAYERS

    def barrier():
        ctx.sync()
        if dist is not None:
            import torch
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(value):
        if dist is None:
            return value
        import torch
        tensor = torch.tensor([value], dtype=torch.float64, device="cuda")
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    # ---- device-resident measurement ----
    for _ in range(max(args.warmup, 3)):
        model.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = ctx.launches
    barrier()
    ctx.timer_start()
    for _ in range(args.steps):
        model.step()
    device_ms = ctx.sync(timed=True)
    barrier()
    launches = ctx.launches - launches_before
    device_ms = max_over_ranks(device_ms)
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = device_ms / args.steps
    value = step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: activations start in pinned host memory, outputs read back ----
    for _ in range(2):
        model.step_from_host()
    barrier()
    start = time.perf_counter()
    ctx.timer_start()
    for _ in range(args.steps):
        model.step_from_host()
    e2e_ms = ctx.sync(timed=True)
    wall_ms = (time.perf_counter() - start) * 1e3
    barrier()
    e2e_ms = max_over_ranks(max(e2e_ms, wall_ms)) / args.steps
    e2e = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": model.h2d_bytes_per_step, "d2h_bytes_per_step": model.d2h_bytes_per_step,
           "ms_per_step": e2e_ms}

    # ---- dominant kernel alone: fused gate/up over the 64 layers' distinct weights ----
    peaks = measured_peaks()
    reps = 5
    model.dominant_kernel_pass()
    barrier()
    ctx.timer_start()
    for _ in range(reps):
        model.dominant_kernel_pass()
    kernel_ms = max_over_ranks(ctx.sync(timed=True)) / (reps * LAYERS)
    gate_up = next(p for p in q4b.LAYER_27B if p.fused)
    kernel_bytes = q4b.algorithmic_bytes(gate_up, args.m) / world  # one launch, this rank's slice
    achieved = kernel_bytes / (kernel_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "gemv_kernel (fused gate/up + SiLU, 5120->17408)",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_source": f"of {peaks['source']}", "frac_of_8TBs": achieved / 8000.0,
                "us_per_launch": kernel_ms * 1e3, "traffic": model.ncu_traffic_bytes()}

    prefill = []
    if world == 1 and not args.no_prefill:
        prefill = prefill_gemm(q4b, ctx, model, peaks)
    elif not args.no_prefill:
        prefill = sharded_prefill(q4b, sharded, ctx, rank, world, dist, peaks, barrier, max_over_ranks, args.gather)
    h3 = h3_bf16_gemm(q4b, ctx, peaks) if world == 1 and not args.no_prefill else None
    extras = {"prefill_gemm": prefill, "h3_bf16_gemm": h3,
              "whole_step_frac_of_measured_hbm": value / world / peaks["hbm_gbs"],
              "whole_step_frac_of_8TBs": value / world / 8000.0,
              "tflops": layer_flops * LAYERS / (ms_per_step * 1e-3) / 1e12}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "u4*f16->f32", "data": "synthetic",
                "config": workload_config(args, world), "roofline": roofline, "e2e": e2e,
                "gpu_launches": launches, "clocks": clocks, "extra": extras}
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(q4b, args.m, args.cpu_seconds)
        print(json.dumps(line), flush=True)
    model.free()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()


def prefill_gemm(q4b, ctx, model, peaks, layers=8):
    """BASELINE configs[3]: the same layer set at M in {512, 2048, 8192} on the tcgen05 GEMM, rotating over
    `layers` layers of distinct weights; TFLOP/s = 2*M*N*K (x2 fused) over device time (CUDA events)."""
    results = []
    layer_set = q4b.LAYER_27B
    for m in (512, 2048, 8192):
        xs = {k: ctx.synth_x(m, 0, m, k) for k in sorted({p.k for p in layer_set})}
        ys = {p.name: ctx.alloc(m * p.n * 2) for p in layer_set}
        x_ptrs = {k: b.ptr for k, b in xs.items()}
        y_ptrs = {name: b.ptr for name, b in ys.items()}

        def run():
            for layer in model.layers[:layers]:
                layer.forward(x_ptrs, y_ptrs, m)
        run()
        ctx.sync()
        reps = 3 if m <= 2048 else 2
        ctx.timer_start()
        for _ in range(reps):
            run()
        ms = ctx.sync(timed=True) / (reps * layers)
        tflops = q4b.layer_flops(layer_set, m) / (ms * 1e-3) / 1e12
        results.append({"m_rows": m, "ms_per_layer": ms, "tflops": tflops,
                        "frac_of_measured_bf16_burst": tflops / peaks["bf16_tflops"],
                        "frac_of_measured_bf16_sustained": tflops / peaks["bf16_tflops_sustained"],
                        "frac_of_nominal_2250": tflops / 2250.0})
        for b in list(xs.values()) + list(ys.values()):
            b.free()
    return results


def h3_bf16_gemm(q4b, ctx, peaks, blocks=2, m=2048):
    """The four Q4 projections of a MiniMax-H3 block (qkv 5376->21504, out 7168->5376, fc1 5376->28672,
    fc2 14336->5376; compiler/minimax-h3/apple-m3-pro/minimax_h3_q4_layer.c:15-20) with bf16 activations and
    outputs, weights rounded to bf16, M = 2048 rows per call, rotating over `blocks` blocks of distinct weights
    (432 MB, larger than L2); TFLOP/s = 2*M*N*K over device time (CUDA events)."""
    import numpy as np
    shapes = [("qkv_proj", 21504, 5376), ("out_proj", 5376, 7168), ("fc1", 28672, 5376), ("fc2", 5376, 14336)]
    rng = np.random.default_rng(0)
    weights = [[ctx.synth_weight(100 + b, i, n, k // 64) for i, (_, n, k) in enumerate(shapes)] for b in range(blocks)]
    xs, ys = {}, {}
    for name, n, k in shapes:
        values = rng.standard_normal((m, k), dtype=np.float32)
        xs[name] = ctx.to_device((values.view(np.uint32) >> 16).astype(np.uint16))  # bf16 bits (truncated)
        ys[name] = ctx.alloc(m * n * 2)

    def run():
        for block in weights:
            for weight, (name, _, _) in zip(block, shapes):
                ctx.matmul(weight, xs[name].ptr, q4b.BF16, m, ys[name].ptr, q4b.BF16)
    run()
    ctx.sync()
    reps = 3
    ctx.timer_start()
    for _ in range(reps):
        run()
    ms = ctx.sync(timed=True) / (reps * blocks)
    flops = sum(2.0 * m * n * k for _, n, k in shapes)
    tflops = flops / (ms * 1e-3) / 1e12
    for block in weights:
        for weight in block:
            weight.free()
    for b in list(xs.values()) + list(ys.values()):
        b.free()
    return {"m_rows": m, "ms_per_block": ms, "tflops": tflops, "dtype": "u4*bf16->f32->bf16",
            "frac_of_measured_bf16_burst": tflops / peaks["bf16_tflops"],
            "frac_of_measured_bf16_sustained": tflops / peaks["bf16_tflops_sustained"]}


def sharded_prefill(q4b, sharded, ctx, rank, world, dist, peaks, barrier, max_over_ranks, gather, layers=8, m=512):
    """BASELINE configs[4] at M = 512: every rank runs the tensor-core GEMM on its N-slices of the 27B layer
    set and the slices are all-gathered (NCCL on the context's stream); device time, max over ranks."""
    stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, layers, m, rank, world, dist, gather=gather)
    for _ in range(2):
        stack.step()
    barrier()
    reps = 3
    ctx.timer_start()
    for _ in range(reps):
        stack.step()
    ms = max_over_ranks(ctx.sync(timed=True)) / (reps * layers)
    barrier()
    tflops = q4b.layer_flops(q4b.LAYER_27B, m) / (ms * 1e-3) / 1e12
    stack.free()
    return [{"m_rows": m, "ms_per_layer": ms, "tflops": tflops,
             "gather": ("slices stored into every rank's output by the GEMM epilogue + rank barrier" if gather == "push"
                        else "nccl all-gather per projection"),
             "frac_of_measured_bf16_burst_per_gpu": tflops / world / peaks["bf16_tflops"]}]


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=100)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--m", type=int, default=1, help="activation rows (1 decode, 4 verify)")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM section")
    parser.add_argument("--gather", default="push", choices=["push", "nccl"],
                        help="N > 1: slices stored into every rank's y by the kernel, or NCCL all-gather per projection")
    parser.add_argument("--mode", default="graph", choices=["graph", "sequence"],
                        help="N = 1: one launch per projection group replayed from a graph, or one persistent launch")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
