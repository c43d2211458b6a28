#!/usr/bin/env python
"""Benchmark of the affine-Q4 matmul path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # the CPU path, host cores
    python bench.py --case decode:gate_up:1                  # a small self-ending case of one kernel (profiling)

Workload: the 27B-shape layer set of Q4 projections (q 5120->6144, k/v
5120->1024, o 6144->5120, fused gate/up 5120->17408 with SiLU, down
17408->5120) at decode (M rows = 1 by default), looped over 64 layers with
independent seeds (seed = layer index), so one step streams 12.27 GB of distinct
weights -- far more than L2.  With N > 1 every projection is column-sharded over
the ranks and the output slices are gathered.  Every projection is queued as
depending on the one before it (stream order), as the projections of a real
token do.

One JSON line on stdout (rank 0).  `value` is algorithmic bytes of the whole job
per second of device time (max over ranks); `e2e` repeats the measurement with
the activations starting in pinned host memory and the outputs read back.
After the timed regions every rank compares sampled rows of its outputs with the
CPU oracle (`parity_max_rel_err`); a result outside 2e-3 makes the run fail.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "q4_gemv_hbm_gbs"
UNIT = "GB/s"
LAYERS = 64
TOLERANCE = 2e-3


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return {"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads() -> int:
    """Cores this process may run on (a launcher may have set OMP_NUM_THREADS=1: the affinity mask is what counts)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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


def layer_work(q4b, m_rows, layer_set=None):
    layer = layer_set if layer_set is not None else q4b.LAYER_27B
    return q4b.layer_bytes(layer, m_rows), q4b.layer_flops(layer, m_rows)


# ----------------------------------------------------------------------------
# the CPU path (oracle port), timed on the host cores
# ----------------------------------------------------------------------------
def cpu_layer_pass(orc, q4b, m_rows, seed, threads, row_fraction=1.0):
    """One layer of the workload through the CPU restatement of the reference's
    scalar loop, rows split over `threads` host threads.  Returns (seconds, bytes)."""
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
            orc.gate_up_silu(mats[0][0], mats[0][1], mats[1][0], mats[1][1], groups, x, want64=False, threads=threads)
        else:
            orc.matmul(mats[0][0], mats[0][1], groups, x, want64=False, threads=threads)
        total_seconds += time.perf_counter() - start
        part = q4b.Projection(p.name, p.k, rows, p.fused)
        total_bytes += q4b.algorithmic_bytes(part, m_rows)
    return total_seconds, total_bytes


def cpu_baseline(q4b, m_rows, budget_seconds=12.0):
    from oracle import q4_oracle as orc
    threads = host_threads()
    seconds, nbytes, passes = 0.0, 0, 0
    while seconds < budget_seconds and passes < 64:
        s, b = cpu_layer_pass(orc, q4b, m_rows, passes, threads)
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
    threads = host_threads()
    for step in range(args.warmup):
        cpu_layer_pass(orc, q4b, args.m, step, threads, row_fraction=0.125)
    seconds, nbytes = 0.0, 0
    for step in range(args.steps):
        s, b = cpu_layer_pass(orc, q4b, args.m, step, threads)
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


def workload_config(args, world, mode=None):
    how = {"graph": "every launch stores its slice into all ranks' outputs, a barrier between the ranks after it, "
                    "the pass replayed from a graph",
           "sequence": "one persistent launch per pass whose epilogue stores into all ranks' outputs"}
    gather = "NCCL all-gather per projection" if args.gather == "nccl" else how.get(mode, args.gather)
    return {"workload": f"27B-shape Q4 layer set (q,k,v,o,gate+up SiLU,down) x {LAYERS} layers, M={args.m}, "
                        f"seed=layer index",
            "m_rows": args.m, "layers": LAYERS, "group": 64,
            "parallelism": ("single GPU" if world == 1 else f"column-parallel N/{world}: {gather}"),
            "l2": "inputs_exceed_l2 (12.27 GB of distinct weights per step)"}


# ----------------------------------------------------------------------------
# parity of what was just timed, against the CPU oracle on sampled rows
# ----------------------------------------------------------------------------
def sample_indices(count, rng, picks):
    edges = [0, 1, 15, 16, 63, 64, 127, 128, count - 129, count - 128, count - 65, count - 64, count - 17,
             count - 16, count - 2, count - 1]
    chosen = [e for e in edges if 0 <= e < count]
    return np.unique(np.concatenate([np.array(chosen, dtype=np.int64), rng.integers(0, count, picks)]))


def layer_parity(orc, layer_set, seed, outputs, x_of, picks=16):
    """max over the projections of max|y - ref| / max|y| on sampled weight rows (and, for many activation rows,
    sampled activation rows).  `outputs[name]` is the device's whole [M, N]; x_of(k) the [M, K] it multiplied."""
    worst, index = 0.0, 0
    rng = np.random.default_rng(1000 + seed)
    for p in layer_set:
        groups = p.k // 64
        y = outputs[p.name]
        m = y.shape[0]
        rows = sample_indices(p.n, rng, picks)
        acts = np.arange(m) if m <= 16 else sample_indices(m, rng, 6)
        x = np.ascontiguousarray(x_of(p.k)[acts])
        if p.fused:
            gq, gm = orc.synth_weight_rows(seed, index, groups, rows)
            uq, um = orc.synth_weight_rows(seed, index + 1, groups, rows)
            ref = orc.gate_up_silu(gq, gm, uq, um, groups, x, want32=False)[1]
            index += 2
        else:
            q, mt = orc.synth_weight_rows(seed, index, groups, rows)
            ref = orc.matmul(q, mt, groups, x, want32=False)[1]
            index += 1
        y32 = y.astype(np.float32)
        if not np.isfinite(y32).all():
            return float("inf")
        scale = float(np.max(np.abs(y32)))
        error = float(np.max(np.abs(y32[np.ix_(acts, rows)].astype(np.float64) - ref))) / max(scale, 1e-30)
        worst = max(worst, error)
    return worst


def stack_parity(orc, stack, layer_set, layer_indices):
    """Parity of a ShardedLayerStack's gathered outputs (every rank holds the whole [M, N])."""
    worst = 0.0
    for index in layer_indices:
        outputs = stack.outputs(index)
        worst = max(worst, layer_parity(orc, layer_set, index, outputs,
                                        lambda k, index=index: orc.synth_x(index, 0, stack.m, k)))
    return worst


# ----------------------------------------------------------------------------
# this library
# ----------------------------------------------------------------------------
def timed_steps(ctx, barrier, max_over_ranks, step, steps, repeats=1):
    """Device milliseconds (max over ranks) of `repeats` x `steps` calls of step() inside one event pair."""
    barrier()
    ctx.timer_start()
    for _ in range(steps * repeats):
        step()
    ms = ctx.sync(timed=True)
    barrier()
    return max_over_ranks(ms)


def run_ours(args):
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    from oracle import q4_oracle as orc
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

    sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
    ctx = q4b.Q4Context(local_rank)
    peaks = measured_peaks()
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

    # One launch per projection group replayed from a graph, or the whole pass as one persistent launch: on one
    # GPU both are measured (same weights) and the faster one is the headline; ranks that share outputs use the
    # persistent launch, whose epilogue does the gather.
    mode = args.mode
    model = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, LAYERS, args.m, rank, world, dist, gather=args.gather,
                                      mode="sequence" if mode == "auto" else mode)
    modes = {}
    if world == 1 and mode == "auto":
        for candidate in ("sequence", "graph"):
            model.mode = candidate
            for _ in range(3):
                model.step()
            modes[candidate] = timed_steps(ctx, barrier, max_over_ranks, model.step, 5) / 5
        model.mode = min(modes, key=modes.get)
    elif mode == "auto" and args.gather == "push":
        # ranks that push: the persistent launch against a recorded graph of launches with barriers between the
        # ranks (the same weights); every rank takes the same decision from the max-over-ranks times
        other = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, LAYERS, args.m, rank, world, dist, gather=args.gather,
                                          mode="graph", layers=model.layers)
        for name, candidate in (("sequence", model), ("graph", other)):
            for _ in range(3):
                candidate.step()
            modes[name] = timed_steps(ctx, barrier, max_over_ranks, candidate.step, 5) / 5
        if modes["graph"] < modes["sequence"]:
            model.owns_layers, other.owns_layers = False, True
            model, other = other, model
        other.free()
    mode = model.mode

    # ---- device-resident measurement ----
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        model.step()
    probe_ms = timed_steps(ctx, barrier, max_over_ranks, model.step, 1)
    # a timed region of about a second: `repeats` times the K steps inside one event pair
    repeats = max(1, min(200, math.ceil(1000.0 / max(probe_ms * args.steps, 1e-3))))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = ctx.launches
    device_ms = timed_steps(ctx, barrier, max_over_ranks, model.step, args.steps, repeats)
    launches = ctx.launches - launches_before  # kernels of this library inside the timed region
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = device_ms / (args.steps * repeats)
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    parity = {"decode": stack_parity(orc, model, q4b.LAYER_27B, (0, LAYERS - 1))}

    # ---- end to end: activations start in pinned host memory, outputs read back ----
    for _ in range(2):
        model.step_from_host()
    barrier()
    e2e_steps = max(args.steps, 5)
    start = time.perf_counter()
    ctx.timer_start()
    for _ in range(e2e_steps):
        model.step_from_host()
    e2e_ms = ctx.sync(timed=True)
    wall_ms = (time.perf_counter() - start) * 1e3
    barrier()
    e2e_ms = max_over_ranks(max(e2e_ms, wall_ms)) / e2e_steps
    e2e = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
           "h2d_bytes_per_step": model.h2d_bytes_per_step, "d2h_bytes_per_step": model.d2h_bytes_per_step,
           "ms_per_step": e2e_ms, "steps": e2e_steps}

    # ---- every launch group alone over the 64 layers' distinct weights: one launch per layer, the 64 launches
    # replayed from a graph like the whole pass (issued one by one from Python the short ones would wait for the host)
    per_projection = {}
    for kind, members in model.layers[0].launch_plan():
        name = members[0].name
        model.projection_pass(name)
        ctx.sync()
        ctx.graph_begin()
        model.projection_pass(name)
        chain = ctx.graph_end()
        chain.launch()
        reps = 10
        ms = timed_steps(ctx, barrier, max_over_ranks, chain.launch, reps) / (reps * LAYERS)
        chain.free()
        nbytes = sum(q4b.algorithmic_bytes(p, args.m) for p in members) / world
        per_projection["+".join(p.name for p in members)] = {
            "us_per_launch": ms * 1e3, "algorithmic_bytes": nbytes, "gbs": nbytes / (ms * 1e-3) / 1e9,
            "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    gate_up = next(p for p in q4b.LAYER_27B if p.fused)
    dominant = per_projection[gate_up.name]
    roofline = {"bound": "hbm", "kernel": "decode_kernel (fused gate/up + SiLU, 5120->17408)",
                "achieved": dominant["gbs"], "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": dominant["frac_of_measured_hbm"], "peak_source": f"of {peaks['source']}",
                "frac_of_8TBs": dominant["gbs"] / 8000.0, "us_per_launch": dominant["us_per_launch"],
                "traffic": model.ncu_traffic_bytes()}

    # ---- where the persistent launch spends its time, as one consumer warp per thread block sees it ----
    phases = None
    if model.sequence is not None:
        model.mode = "sequence"
        model.sequence.profile()          # clocks on
        for _ in range(3):
            model.step()
        ticks = model.sequence.profile()  # [thread blocks, 6] SM clock ticks of the three launches
        total = np.maximum(ticks[:, 5].astype(np.float64), 1.0)
        names = model.sequence.PROFILE_PHASES
        sm_mhz = (clocks or {}).get("sm_mhz") or 1965.0
        phases = {"share_of_launch_median_over_thread_blocks":
                      {name: float(np.median(ticks[:, i] / total)) for i, name in enumerate(names[:5])},
                  "us_per_layer_median_over_thread_blocks":
                      {name: float(np.median(ticks[:, i])) / 3 / LAYERS / sm_mhz for i, name in enumerate(names)},
                  "note": "SM clock ticks x sampled median SM MHz; dependency = waiting for the previous projection's "
                          "outputs, entries = activations into tensor-pipe operands, weights = waiting for HBM, "
                          "tiles = multiplying, finish = split sums, epilogue, publishing"}
        model.mode = mode

    extras = {"mode": mode, "ms_per_step_by_mode": modes, "per_projection": per_projection, "sequence_phases": phases,
              "whole_step_frac_of_measured_hbm": value / world / peaks["hbm_gbs"],
              "whole_step_frac_of_8TBs": value / world / 8000.0, "us_per_layer": ms_per_step * 1e3 / LAYERS,
              "tflops": layer_flops * LAYERS / (ms_per_step * 1e-3) / 1e12}

    if not args.no_extras:
        if world == 1:
            extras["verify_m4"] = other_batch(q4b, sharded, orc, ctx, model, peaks, barrier, max_over_ranks, 4, parity)
            extras["small_layer"] = small_layer(q4b, sharded, orc, ctx, peaks, barrier, max_over_ranks, parity)
            extras["config0"] = config0(q4b, orc, ctx, peaks, barrier, max_over_ranks, parity)
    if not args.no_prefill:
        if world == 1:
            extras["prefill_gemm"] = prefill_gemm(q4b, orc, ctx, model, peaks, parity)
            extras["h3_bf16_gemm"] = h3_bf16_gemm(q4b, ctx, peaks)
            extras["h3_f16_large_m"] = h3_large_m(q4b, ctx, peaks)
        else:
            extras["prefill_gemm"] = sharded_prefill(q4b, sharded, orc, ctx, rank, world, dist, peaks, barrier,
                                                     max_over_ranks, args.gather, parity)

    worst = max_over_ranks(max(parity.values()))
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": warmup, "repeats": repeats, "timed_region_ms": device_ms, "ms_per_step": ms_per_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u4*f16->f32",
                "data": "synthetic", "config": workload_config(args, world, mode), "roofline": roofline, "e2e": e2e,
                "gpu_launches": launches, "clocks": clocks, "parity_max_rel_err": worst,
                "parity": {**parity, "tolerance": TOLERANCE,
                           "how": "every rank, sampled weight rows of layers 0 and 63 (first and last rows of the "
                                  "matrix and of its blocks, plus random ones) against the CPU oracle's double sum, "
                                  "relative to the largest |y| of the projection; max over ranks"},
                "extra": extras}
        if world == 1:
            line["cpu_baseline"] = cpu_baseline(q4b, args.m, args.cpu_seconds)
        print(json.dumps(line), flush=True)
    model.free()
    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    if not (worst <= TOLERANCE):
        raise SystemExit(f"parity check failed: max relative error {worst:.3e} > {TOLERANCE}")


def other_batch(q4b, sharded, orc, ctx, model, peaks, barrier, max_over_ranks, m, parity):
    """The same 64 layers (same weights) at another number of activation rows: M = 4 is the verify step of
    speculative decoding (3 draft tokens + 1)."""
    stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, LAYERS, m, mode=model.mode, layers=model.layers)
    for _ in range(3):
        stack.step()
    reps = 10
    ms = timed_steps(ctx, barrier, max_over_ranks, stack.step, reps) / reps
    nbytes = q4b.layer_bytes(q4b.LAYER_27B, m) * LAYERS
    parity[f"decode_m{m}"] = stack_parity(orc, stack, q4b.LAYER_27B, (0, LAYERS - 1))
    stack.free()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"m_rows": m, "ms_per_step": ms, "us_per_layer": ms * 1e3 / LAYERS, "gbs": gbs,
            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"], "mode": stack.mode}


def small_layer(q4b, sharded, orc, ctx, peaks, barrier, max_over_ranks, parity):
    """The small-model layer set (hidden 1024: q 1024->2048, k/v 1024->512, o 2048->1024, gate/up 1024->3072,
    down 3072->1024) at M = 1 and 4, rotating over 64 layers of distinct weights (528 MB, four times L2)."""
    results = []
    first = None
    for m in (1, 4):
        for mode in ("sequence", "graph"):
            stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_SMALL, LAYERS, m, mode=mode,
                                              layers=first.layers if first is not None else None)
            if first is None:
                first = stack
            for _ in range(3):
                stack.step()
            reps = 20
            ms = timed_steps(ctx, barrier, max_over_ranks, stack.step, reps) / reps
            nbytes = q4b.layer_bytes(q4b.LAYER_SMALL, m) * LAYERS
            parity[f"small_m{m}_{mode}"] = stack_parity(orc, stack, q4b.LAYER_SMALL, (0, LAYERS - 1))
            gbs = nbytes / (ms * 1e-3) / 1e9
            results.append({"m_rows": m, "mode": mode, "us_per_layer": ms * 1e3 / LAYERS, "gbs": gbs,
                            "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                            "l2": "64 rotating layers of distinct weights, 528 MB"})
            if stack is not first:
                stack.free()
    first.free()
    return results


def config0(q4b, orc, ctx, peaks, barrier, max_over_ranks, parity):
    """A single 1024 -> 3072 GEMV (M = 1, seed 0), one launch per call, rotating over 128 copies of distinct
    weights (226 MB, larger than L2); the weights of copy 0 are the seed-0 matrix the CPU runs."""
    copies, n, k = 128, 3072, 1024
    weights = [ctx.synth_weight(seed, 0, n, k // 64) for seed in range(copies)]
    x = ctx.synth_x(0, 0, 1, k)
    ys = ctx.alloc(copies * n * 2)

    def run():
        for index, weight in enumerate(weights):
            ctx.matmul(weight, x.ptr, q4b.F16, 1, ys.ptr + index * n * 2)
    run()
    reps = 10
    ms = timed_steps(ctx, barrier, max_over_ranks, run, reps) / (reps * copies)
    nbytes = q4b.algorithmic_bytes(q4b.Projection("config0", k, n), 1)
    y = ys.download(np.float16, (copies, n))
    quants, meta = orc.synth_weight(0, 0, n, k // 64)
    ref = orc.matmul(quants, meta, k // 64, orc.synth_x(0, 0, 1, k), want32=False)[1]
    parity["config0"] = float(np.max(np.abs(y[0].astype(np.float64) - ref[0])) / np.max(np.abs(ref)))
    for weight in weights:
        weight.free()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return {"us_per_launch": ms * 1e3, "gbs": gbs, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
            "note": "1.77 MB per launch: launch-latency bound, 128 rotating copies of distinct weights"}


def prefill_gemm(q4b, orc, ctx, model, peaks, parity, layers=8):
    """The same layer set at M in {512, 2048, 8192} on the tcgen05 GEMM, rotating over `layers` layers of
    distinct weights; TFLOP/s = 2*M*N*K (x2 fused) over device time (CUDA events).  The last layer's outputs
    are then checked against the oracle on sampled weight rows x sampled activation rows."""
    results = []
    layer_set = q4b.LAYER_27B
    for m in (512, 2048, 8192):
        seed_x = 100 + m
        xs = {k: ctx.synth_x(seed_x, 0, m, k) for k in sorted({p.k for p in layer_set})}
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
        outputs = {p.name: ys[p.name].download(np.float16, (m, p.n)) for p in layer_set}
        x_host = {k: xs[k].download(np.float16, (m, k)) for k in xs}
        parity[f"prefill_m{m}"] = layer_parity(orc, layer_set, layers - 1, outputs, lambda k: x_host[k], picks=8)
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


def h3_large_m(q4b, ctx, peaks):
    """The reference's largest measured affine-Q4 GEMM: 5376 -> 14336, fp16 in and out, M = 15,485 and its
    4,646-row sample (models/minimax-h3/targets/apple-m3-pro/README.md:722-726: 618.2 ms = 3.861 TFLOP/s and
    194.6 ms = 3.680 TFLOP/s on an M3 Pro).  Three weight sets in turn; TFLOP/s = 2*M*N*K over device time."""
    n, k = 14336, 5376
    weights = [ctx.synth_weight(200 + index, 0, n, k // 64) for index in range(3)]
    results = []
    for m in (4646, 15485):
        x = ctx.synth_x(m, 0, m, k)
        y = ctx.alloc(m * n * 2)

        def run():
            for weight in weights:
                ctx.matmul(weight, x.ptr, q4b.F16, m, y.ptr)
        run()
        ctx.sync()
        reps = 3
        ctx.timer_start()
        for _ in range(reps):
            run()
        ms = ctx.sync(timed=True) / (reps * len(weights))
        tflops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        results.append({"m_rows": m, "ms": ms, "tflops": tflops,
                        "frac_of_measured_bf16_burst": tflops / peaks["bf16_tflops"],
                        "reference_m3_pro_ms": 618.205 if m == 15485 else 194.602})
        x.free()
        y.free()
    for weight in weights:
        weight.free()
    return results


def sharded_prefill(q4b, sharded, orc, ctx, rank, world, dist, peaks, barrier, max_over_ranks, gather, parity,
                    layers=8, m=512):
    """The column-sharded layer at M = 512: every rank runs the tensor-core GEMM on its N-slices of the 27B layer
    set and the slices are gathered (stored into every rank by the epilogue, or NCCL on the context's stream);
    device time, max over ranks; every rank then checks its gathered outputs against the oracle."""
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
    parity[f"sharded_prefill_m{m}"] = stack_parity(orc, stack, q4b.LAYER_27B, (0, layers - 1))
    tflops = q4b.layer_flops(q4b.LAYER_27B, m) / (ms * 1e-3) / 1e12
    barrier()
    stack.free()
    return [{"m_rows": m, "ms_per_layer": ms, "tflops": tflops,
             "gather": ("nccl all-gather per projection" if gather != "push" else
                        "slices stored into every rank's output by the GEMM epilogue + rank barrier" if world <= 2 else
                        "slices copied into every rank's output by a copy kernel after the GEMM + rank barrier"),
             "frac_of_measured_bf16_burst_per_gpu": tflops / world / peaks["bf16_tflops"]}]


# ----------------------------------------------------------------------------
# small self-ending cases of one kernel, for a profiler capture
# ----------------------------------------------------------------------------
CASE_SHAPES = {"q": (5120, 6144, False), "o": (6144, 5120, False), "gate_up": (5120, 17408, True),
               "down": (17408, 5120, False),
               # MiniMax-H3 block projections (compiler/minimax-h3/apple-m3-pro/minimax_h3_q4_layer.c:15-20)
               "h3_qkv": (5376, 21504, False), "h3_fc1": (5376, 28672, False), "h3_fc2": (14336, 5376, False)}


def run_case(spec: str):
    """decode:<shape>:<M>   the decode kernel on one projection (M <= 16), one launch per weight set
    gemm:<shape>:<M>[:bf16] the tcgen05 kernel (M > 16)
    sequence:<layers>:<M>   whole 27B layers as one persistent launch per pass, three passes
    Shapes: q, o, gate_up, down, h3_qkv, h3_fc1, h3_fc2.  A few sets of distinct weights (about 0.4 GB on the
    device, more than L2, so DRAM counters mean something), two passes, a handful of launches in all."""
    q4b = importlib.import_module("cpu-llms-in-c_b200")
    parts = spec.split(":")
    kind = parts[0]
    ctx = q4b.Q4Context(0)
    if kind == "sequence":
        sharded = importlib.import_module("cpu-llms-in-c_b200.sharded")
        layers, m = int(parts[1]), int(parts[2])
        stack = sharded.ShardedLayerStack(ctx, q4b.LAYER_27B, layers, m, mode="sequence")
        for _ in range(3):
            stack.step()
        ctx.sync()
        print(f"sequence of {layers} layers, M={m}: 3 launches")
        stack.free()
        ctx.close()
        return
    which, m = parts[1], int(parts[2])
    if kind == "decode" and m > 16 or kind == "gemm" and m <= 16 or kind not in ("decode", "gemm"):
        raise SystemExit("decode takes M <= 16, gemm M > 16")
    k, n, fused = CASE_SHAPES[which]
    dtype = q4b.BF16 if len(parts) > 3 and parts[3] == "bf16" else q4b.F16
    if dtype == q4b.BF16 and kind != "gemm":
        raise SystemExit("bf16 activations run on the tcgen05 kernel: use gemm")
    sets = max(2, int(0.4e9 // (k * n * (1.0 if fused else 0.5) * 1.125)))
    weights = [(ctx.synth_weight(index, 0, n, k // 64), ctx.synth_weight(index, 1, n, k // 64) if fused else None)
               for index in range(sets)]
    x = ctx.synth_x(0, 0, m, k)
    y = ctx.alloc(m * n * 2)
    for _ in range(2):
        for gate, up in weights:
            if fused:
                ctx.gate_up_silu(gate, up, x.ptr, dtype, m, y.ptr, dtype)
            else:
                ctx.matmul(gate, x.ptr, dtype, m, y.ptr, dtype)
    ctx.sync()
    print(f"{kind} {which} M={m}: {2 * sets} launches over {sets} weight sets")
    ctx.close()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--m", type=int, default=1, help="activation rows (1 decode, 4 verify)")
    parser.add_argument("--cpu-seconds", type=float, default=12.0)
    parser.add_argument("--no-prefill", action="store_true", help="skip the prefill GEMM sections")
    parser.add_argument("--no-extras", action="store_true", help="skip the M = 4, small-layer and single-GEMV sections")
    parser.add_argument("--gather", default="push", choices=["push", "nccl"],
                        help="N > 1: slices stored into every rank's y by the kernel, or NCCL all-gather per projection")
    parser.add_argument("--mode", default="auto", choices=["auto", "graph", "sequence"],
                        help="N = 1: one launch per projection group replayed from a graph, one persistent launch "
                             "for the whole pass, or whichever is faster")
    parser.add_argument("--case", default=None, help="run one small case of one kernel and exit (see run_case)")
    args = parser.parse_args()
    if args.case is not None:
        run_case(args.case)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
