"""Headline benchmark: Q4_0 x Q8_0 decode GEMV over the Llama-7B-shaped layers.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one decode pass over the four layer shapes (4096x4096, 11008x4096,
4096x11008, 32000x4096), batch 1: four GEMV launches.  Weights rotate over distinct copies
whose total size is several times the 126 MB L2, so every launch streams from HBM.  The
metric is algorithmic bytes (weights once + activations + outputs) per second.  The GEMV
does not shard: with N > 1 every rank runs an independent replica (weak scaling) and
`value` is the sum over ranks divided by the slowest rank's time.

`--impl reference` times the CPU oracle (the restatement of the reference's scalar
semantics; the reference's own generated code needs an RVV toolchain) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]  # (N rows, K)
METRIC = "q4_0_q8_0_decode_gemv_hbm_gbs"
UNIT = "GB/s"
WORKLOAD = "q4_0_q8_0_gemv_llama7b_layers_batch1"
ROTATION_SETS = 8       # distinct copies of every weight matrix; 8 x 134 MB, far beyond the 126 MB L2
GRAPH_STEPS = 32        # most steps per CUDA graph of the timed region (measured: 8..32 steps 4.51-4.53 TB/s,
                        # 64: 4.46, 128: 4.32, 256: 4.16 -- long graphs dispatch their nodes more slowly)
MIN_REGIONS = 30        # the K-step region is timed this many times at least; the median is reported
MIN_TIMED_MS = 20.0     # ... and often enough that the timed regions add up to this much device time
MIN_WARM_SECONDS = 1.5  # warm-up runs at least this long so that the clock sampler sees load


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of the
# 32000x4096 and 4096x4096 launches; the other two shapes are scaled from the larger one by
# their weight bytes (traffic grows in proportion to the rows streamed).
NCU_TRAFFIC = {"32000x4096": 74_489_856, "4096x4096": 9_463_040}
NCU_TRAFFIC_RATIO = 74_489_856 / 73_860_352  # traffic / algorithmic bytes of the measured launch


def gemv_bytes(nr: int, k: int, batch: int) -> int:
    nb = k // 32
    return nr * nb * 18 + batch * nb * 34 + 4 * batch * nr


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self, first_line: int = 0):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines[first_line:]:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------- CPU arm


def cpu_sample(threads: int, target_seconds: float = 5.0):
    """Times the oracle's Q4_0 x Q8_0 GEMV on a bounded sample: the first `rows` rows of each
    layer shape, batch 1, all `threads` host threads.  Returns (GB/s, description)."""
    O = entry.load_oracle()
    rows = 2048
    total_bytes, total_time = 0, 0.0
    while True:
        total_bytes, total_time = 0, 0.0
        for nr, k in SHAPES:
            r = min(rows, nr)
            w = O.quantize_q4_0(O.fill_normal(r * k, 900 + k, 0.0, 0.02).reshape(r, k))
            x = O.quantize_q8_0(O.fill_normal(k, 901 + k).reshape(1, k))
            O.gemm(w[:64], x, threads=threads)  # warm caches / page in
            t0 = time.perf_counter()
            O.gemm(w, x, threads=threads)
            total_time += time.perf_counter() - t0
            total_bytes += gemv_bytes(r, k, 1)
        if total_time >= target_seconds / 4 or rows >= 32000:
            break
        rows *= 4
    return total_bytes / total_time / 1e9, f"first {rows} rows (or all) of each of the 4 layer shapes, batch 1, one pass"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    O = entry.load_oracle()
    O.build()
    for _ in range(args.warmup):
        cpu_sample(threads, 0.5)
    t_total, b_total = 0.0, 0.0
    desc = ""
    for _ in range(args.steps):
        gbs, desc = cpu_sample(threads, 2.0)
        b_total += gbs
        t_total += 1
    value = b_total / max(t_total, 1)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 products, int32 block sums, fp32 fold",
        "data": "synthetic", "config": bench_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU oracle (restatement of the reference's scalar kernel); the reference's generated RVV C "
                "cannot be built on this host",
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------- GPU arm


def run_ours(args):
    import torch

    pkg = entry.load_package()
    pkg.lib()  # fails loudly when the CUDA library is missing
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    if args.gemm_only:
        # the prefill-GEMM section alone (N-sharded over the ranks): a short run for tuning and
        # profiling; prints its own object, not the benchmark line
        gemm = measure_gemm(pkg, torch, dist, rank, world)
        if rank == 0:
            print(json.dumps({"gemm_only": True, "n_gpus": world, "gemm": gemm}))
        if dist is not None:
            dist.destroy_process_group()
        return

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- inputs: fp32 weights ~ N(0, 0.02) quantised on the GPU, x ~ N(0, 1) -> Q8_0
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    layers = []
    for nr, k in SHAPES:
        wf = torch.randn((nr, k), generator=gen, device="cuda") * 0.02
        w = pkg.quantize_q4_0(wf)
        del wf
        copies = [w] + [w.clone() for _ in range(ROTATION_SETS - 1)]
        x = pkg.quantize_q8_0(torch.randn((1, k), generator=gen, device="cuda"))
        y = torch.empty((nr, 1), dtype=torch.float32, device="cuda")
        layers.append({"nr": nr, "k": k, "w": copies, "x": x, "y": y, "bytes": gemv_bytes(nr, k, 1)})
    step_bytes = sum(l["bytes"] for l in layers)
    launches_per_step = len(layers)

    def launch_set(r: int):
        for l in layers:
            pkg.gemv(l["w"][r], l["x"], out=l["y"], flags=pkg.FLAG_STATIC_WEIGHTS)

    # First launches outside capture (function attributes, lazy loading).
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for r in range(ROTATION_SETS):
            launch_set(r)
    torch.cuda.synchronize()
    pkg.check_device_errors()
    # Warm-up replays one graph per rotation set (one decode pass, 4 GEMV kernels).
    graphs = []
    for r in range(ROTATION_SETS):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            launch_set(r)
        graphs.append(g)

    # The timed region is K consecutive steps (step i uses weight copy i mod 8) captured in CUDA
    # graphs, the way a decoder captures all the layers of a token, so that Python's per-call cost
    # does not sit between kernels: ONE graph when K <= --graph-steps, otherwise graphs of
    # --graph-steps steps plus one for the remainder, each starting at the rotation offset where
    # its predecessor stopped.
    def steps_graph(first: int, count: int):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(first, first + count):
                launch_set(i % ROTATION_SETS)
        return g

    region, done = [], 0
    while done < args.steps:
        count = min(args.graph_steps, args.steps - done)
        region.append(steps_graph(done, count))
        done += count

    def run_steps():
        for g in region:
            g.replay()

    def step(i: int):
        graphs[i % ROTATION_SETS].replay()

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    t_warm = time.perf_counter()
    warm_mark = len(sampler.lines)
    i = 0
    while i < args.warmup or time.perf_counter() - t_warm < args.min_warm_seconds:
        step(i)
        i += 1
        if i % 64 == 0:
            torch.cuda.synchronize()
    pkg.check_device_errors()
    run_steps()  # the region's graphs once, untimed (first replay uploads them)
    sync_all()

    # The K-step region is timed `regions` times (events on the replay stream, a barrier and a
    # synchronize on both sides of each) and the median is reported: K steps alone last well under
    # a millisecond.  One untimed pass is queued directly before the start event so that the
    # region's first kernel follows a predecessor, as every other one does.
    def time_region():
        sync_all()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        step(ROTATION_SETS - 1)
        start.record()
        run_steps()
        stop.record()
        sync_all()
        return start.elapsed_time(stop)

    times = [time_region() for _ in range(max(1, args.regions))]
    # more regions until they add up to --min-timed-ms; every rank must run the same number
    more = 0
    if sum(times) < args.min_timed_ms:
        more = min(2000, int((args.min_timed_ms - sum(times)) / (sum(times) / len(times))) + 1)
    if dist is not None:
        t = torch.tensor([more], dtype=torch.int64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        more = int(t.item())
    times += [time_region() for _ in range(more)]
    times.sort()
    elapsed_ms = times[len(times) // 2]
    elapsed_best = times[0]
    launches = launches_per_step * args.steps
    clocks = sampler.stop(warm_mark) if rank == 0 else None
    pkg.check_device_errors()
    if dist is not None:
        t = torch.tensor([elapsed_ms, elapsed_best], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, elapsed_best = float(t[0].item()), float(t[1].item())

    # ---- per-shape timing (explains the aggregate): one graph per shape holding one launch
    # per rotation copy, timed with events on the replay stream
    per_shape = []
    for l in layers:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for r in range(ROTATION_SETS):
                pkg.gemv(l["w"][r], l["x"], out=l["y"], flags=pkg.FLAG_STATIC_WEIGHTS)
        reps = max(5, args.steps // ROTATION_SETS)
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (reps * ROTATION_SETS)
        per_shape.append({"shape": f"{l['nr']}x{l['k']}", "us": round(us, 3), "gbs": round(l["bytes"] / us / 1e3, 1)})

    batch8 = measure_batch8(pkg, torch, layers, side, gen)
    grouped = measure_grouped(pkg, torch, layers, side)
    e2e = measure_e2e(pkg, torch, layers, max(10, min(args.steps, 50)), dist)
    try:
        others = measure_other_kernels(pkg, torch) if (rank == 0 and not args.skip_gemm) else None
    except Exception as exc:
        others = {"error": f"{type(exc).__name__}: {exc}"}
    try:
        gemm = None if args.skip_gemm else measure_gemm(pkg, torch, dist, rank, world)
    except Exception as exc:  # the headline line must still be printed
        gemm = {"error": f"{type(exc).__name__}: {exc}"}

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1:
        threads = os.cpu_count() or 1
        gbs, desc = cpu_sample(threads, 8.0)
        cpu = {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "sample": desc}

    peaks, peak_kind = measured_peaks()
    step_traffic = sum(NCU_TRAFFIC.get(f"{l['nr']}x{l['k']}", l["bytes"] * NCU_TRAFFIC_RATIO) for l in layers)
    value = step_bytes * args.steps * world / (elapsed_ms * 1e-3) / 1e9
    per_gpu = value / world
    big = per_shape[-1]
    b8_bytes = sum(gemv_bytes(l["nr"], l["k"], 8) for l in layers)
    roofline = {
        "bound": "hbm", "achieved": round(per_gpu, 2), "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": round(per_gpu / peaks["hbm_gbs"], 4), "traffic": round(step_traffic / launches_per_step),
        "algorithmic_bytes_per_launch": round(step_bytes / launches_per_step),
        "traffic_source": "from profile: ncu dram bytes per launch (32000x4096 and 4096x4096 captured, the other "
                          "two shapes scaled by weight bytes), averaged over the step's 4 launches",
        "peak_kind": f"of {peak_kind}", "kernel": "gemv_stream_kernel<q4_0, 1 column>", "largest_shape": big,
        "per_shape_sum_us": round(sum(p["us"] for p in per_shape), 3),
        # batch 8 (tensor-core decode kernel): the same four-shape pass and its largest launch
        "batch8": {"kernel": "gemv_mma_rows_kernel<q4_0> (K = 4096), gemv_mma_kernel<q4_0> (K = 11008), 8 columns", "pass_us": batch8["pass_us"],
                   "pass_gbs": round(b8_bytes / batch8["pass_us"] / 1e3, 1),
                   "frac": round(b8_bytes / batch8["pass_us"] / 1e3 / peaks["hbm_gbs"], 4),
                   "per_shape": batch8["per_shape"],
                   "largest_shape_frac": round(batch8["per_shape"][-1]["gbs"] / peaks["hbm_gbs"], 4)},
        "grouped_step": {"kernel": "gemv_stream_group_kernel<q4_0>: the step's four GEMVs as one launch "
                                   "(tcrv_cuda_gemv_group_q4_0_q8_0), batch 1",
                         "note": "not the headline: valid where the GEMVs do not depend on one another "
                                 "(shared-input projections, experts, the queued host calls of a replayed step)",
                         "us": grouped["own_order"], "gbs": round(step_bytes / grouped["own_order"] / 1e3, 1),
                         "frac": round(step_bytes / grouped["own_order"] / 1e3 / peaks["hbm_gbs"], 4),
                         "reference_order_us": grouped["reference_order"],
                         "reference_order_frac": round(step_bytes / grouped["reference_order"] / 1e3 / peaks["hbm_gbs"], 4)},
        # prefill GEMM (the metric's second half): int8 TOP/s of the N-sharded GEMM on this many GPUs
        "gemm": gemm_summary(gemm),
    }
    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(elapsed_ms / args.steps, 6), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8 products, int32 block sums, fp32 fold",
        "data": "synthetic",
        "config": bench_config(args, world),
        "roofline": roofline,
        "e2e": e2e,
        "cpu_baseline": cpu,
        "gpu_launches": launches,
        "clocks": clocks,
        "timing": {"regions": len(times), "region_ms_median": round(elapsed_ms, 5), "region_ms_best": round(elapsed_best, 5),
                   "note": "the K-step region is replayed `regions` times; value and ms_per_step use the median"},
        "per_shape": per_shape,
        "other_kernels": others,
        "gemm": gemm,
    }
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def bench_config(args, world):
    """The `config` object; both arms print the same workload, shapes and batch."""
    return {"workload": WORKLOAD, "shapes": [f"{n}x{k}" for n, k in SHAPES], "batch": 1,
            "l2": f"weights rotate over {ROTATION_SETS} distinct copies per shape ({ROTATION_SETS} x 134 MB in all, L2 is 126 MB)",
            "launch": f"CUDA graphs of up to {args.graph_steps} consecutive steps (4 GEMV kernels each)",
            "parallelism": "replicas only" if world > 1 else "single GPU"}


def gemm_summary(gemm):
    """The figures of measure_gemm() a reader needs first, one short object per shape."""
    if not isinstance(gemm, list):
        return gemm
    keys = ("shape", "rows_per_gpu", "compute_ms", "compute_tops", "with_allgather_ms", "with_allgather_tops",
            "fused_allgather_ms", "fused_allgather_tops", "fused_equals_nccl", "fused_link_gbs_per_gpu")
    out = []
    for g in gemm:
        e = {k: g[k] for k in keys if k in g}
        r = g.get("roofline", {})
        e.update({"bound": "tensor", "frac": r.get("frac"), "peak_tops": r.get("peak"),
                  "library_int8_gemm_tops": r.get("library_int8_gemm_tops"),
                  "frac_of_library_int8": r.get("frac_of_library_int8_gemm")})
        out.append(e)
    return out


def measure_batch8(pkg, torch, layers, side, gen):
    """The four-shape decode pass with 8 activation columns (tensor-core decode kernel) over the
    same rotating weight copies: one graph of 8 passes, events on the replay stream."""
    xs = [pkg.quantize_q8_0(torch.randn((8, l["k"]), generator=gen, device="cuda")) for l in layers]
    ys = [torch.empty((l["nr"], 8), dtype=torch.float32, device="cuda") for l in layers]

    def timed(fn, launches):
        with torch.cuda.stream(side):
            fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        reps = 10
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) * 1e3 / (reps * launches)

    def whole():
        for r in range(ROTATION_SETS):
            for l, x, y in zip(layers, xs, ys):
                pkg.gemv(l["w"][r], x, out=y, flags=pkg.FLAG_STATIC_WEIGHTS)

    pass_us = timed(whole, ROTATION_SETS)
    per_shape = []
    for l, x, y in zip(layers, xs, ys):
        def one(l=l, x=x, y=y):
            for r in range(ROTATION_SETS):
                pkg.gemv(l["w"][r], x, out=y, flags=pkg.FLAG_STATIC_WEIGHTS)
        us = timed(one, ROTATION_SETS)
        per_shape.append({"shape": f"{l['nr']}x{l['k']}", "us": round(us, 3),
                          "gbs": round(gemv_bytes(l["nr"], l["k"], 8) / us / 1e3, 1)})
    pkg.check_device_errors()
    return {"pass_us": round(pass_us, 3), "per_shape": per_shape}


def measure_grouped(pkg, torch, layers, side):
    """The four layer shapes (batch 1) as ONE grouped launch per step (`tcrv_cuda_gemv_group_q4_0_q8_0`:
    the SMs dealt out among the four problems, all streaming at once) over the same rotating weight
    copies, in the kernel's own order and in the reference's.  Not the headline: the layers of a
    model depend on one another; this is what callers with independent GEMVs (projections that
    share an input, experts, the queued host calls of a replayed step) get."""
    out = {}
    for name, flags in (("own_order", pkg.FLAG_STATIC_WEIGHTS), ("reference_order", pkg.FLAG_STATIC_WEIGHTS | pkg.FLAG_STRICT_ORDER)):
        groups = [pkg.gemv_group_calls([(l["w"][r], l["x"], l["y"]) for l in layers]) for r in range(ROTATION_SETS)]

        def whole():
            for calls in groups:
                pkg.gemv_group(calls, flags=flags)

        with torch.cuda.stream(side):
            whole()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            whole()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        reps = 10
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        out[name] = round(a.elapsed_time(b) * 1e3 / (reps * ROTATION_SETS), 3)
    pkg.check_device_errors()
    return out


def measure_e2e(pkg, torch, layers, steps, dist):
    """The same decode pass through the host-pointer entry point a reference harness would
    call (`tcrv_cuda_host_gemm_q4_0_q8_0`, the int-returning twin of
    `tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm`): activations start in pinned
    host memory and every step's outputs land in pinned host memory.  Weights are registered
    once (resident, like model parameters) and are not re-uploaded per step.  The timed loops run
    in a C++ caller of the entries (examples/gpu/decode_loop.cpp) when its library has been built."""
    import ctypes

    L = pkg.lib()
    # the entry's default is the reference's strict block order (timed below as `reference_order`); a
    # decoder that accepts rel 1e-5 opts in to the streaming kernels' own summation orders, as the
    # device-timed arm does
    previous_order = L.tcrv_cuda_host_set_fold_order(1)
    host = []
    for l in layers:
        w_host = l["w"][0].cpu().numpy()  # pageable host copy of the block_q4_0 rows
        x_host = l["x"].cpu().pin_memory()
        y_host = torch.empty((l["nr"], 1), dtype=torch.float32).pin_memory()
        st = L.tcrv_cuda_host_register_weights(w_host.ctypes.data, w_host.nbytes)
        if st != 0:
            raise RuntimeError(f"register_weights failed: {st}")
        host.append((l, w_host, x_host, y_host))
    # the argument lists are fixed: build them once so that the timed loop is the C call itself
    calls = [(l["k"], y_host.data_ptr(), w_host.ctypes.data, x_host.data_ptr(), x_host.stride(0), l["nr"], 1,
              w_host.strides[0], 1) for l, w_host, x_host, y_host in host]

    def one_pass_blocking():
        # one synchronous call per layer: every call returns with its result in host memory
        for args in calls:
            st = L.tcrv_cuda_host_gemm_q4_0_q8_0(*args)
            if st != 0:
                raise RuntimeError(f"host gemv failed: {st}")

    def one_pass_queued():
        # the four layers of a step queued one after the other, one wait at the end of the step
        for args in calls:
            st = L.tcrv_cuda_host_gemm_q4_0_q8_0_async(*args)
            if st != 0:
                raise RuntimeError(f"host gemv failed: {st}")
        st = L.tcrv_cuda_host_sync()
        if st != 0:
            raise RuntimeError(f"host sync failed: {st}")

    # The timed loops run in a C++ caller of the same entries (examples/gpu/decode_loop.cpp, a
    # shared library built beside the C-ABI library): what is timed is then the entries, not this
    # interpreter's foreign-call overhead of five calls per step.  Without that library the loops
    # below run here and the line says so.
    loop = None
    loop_path = os.path.join(os.path.dirname(pkg.LIB_PATH), "libtcrv_decode_loop.so")
    if os.path.exists(loop_path):
        class DecodeCall(ctypes.Structure):
            _fields_ = [("n", ctypes.c_size_t), ("s", ctypes.c_void_p), ("vx", ctypes.c_void_p), ("vy", ctypes.c_void_p),
                        ("by", ctypes.c_size_t), ("nr", ctypes.c_size_t), ("nc", ctypes.c_size_t),
                        ("bx", ctypes.c_size_t), ("bs", ctypes.c_size_t)]

        loop = ctypes.CDLL(loop_path)
        loop.tcrv_decode_loop_run.argtypes = [ctypes.POINTER(DecodeCall), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.POINTER(ctypes.c_double)]
        loop.tcrv_decode_loop_run.restype = ctypes.c_int
        call_array = (DecodeCall * len(calls))(*[DecodeCall(*args) for args in calls])

    def run_steps(one_pass, count):
        """`count` decode steps; returns the elapsed wall time in seconds."""
        if loop is not None:
            seconds = ctypes.c_double(0.0)
            st = loop.tcrv_decode_loop_run(call_array, len(calls), count, 1 if one_pass is one_pass_queued else 0,
                                           ctypes.byref(seconds))
            if st != 0:
                raise RuntimeError(f"host gemv failed: {st}")
            return seconds.value
        t0 = time.perf_counter()
        for _ in range(count):
            one_pass()
        return time.perf_counter() - t0

    device_flags = [0]

    def check():
        # the resident path must agree with the device-pointer path
        for l, w_host, x_host, y_host in host:
            pkg.gemv(l["w"][0], l["x"], out=l["y"], flags=device_flags[0])
            torch.cuda.synchronize()
            if not torch.equal(l["y"].cpu(), y_host):
                raise RuntimeError("host-pointer path disagrees with the device-pointer path")
            y_host.fill_(float("nan"))

    def timed(one_pass):
        for _ in range(3):
            one_pass()
        check()
        one_pass()
        run_steps(one_pass, 3)
        if dist is not None:
            dist.barrier()
        dt = run_steps(one_pass, steps)
        if dist is not None:
            t = torch.tensor([dt], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt

    dt_blocking = timed(one_pass_blocking)
    dt = timed(one_pass_queued)
    one_pass_queued()
    check()
    # the same queued step called from this interpreter (five foreign calls per step)
    dt_interp = None
    if loop is not None:
        for _ in range(3):
            one_pass_queued()
        t0 = time.perf_counter()
        for _ in range(steps):
            one_pass_queued()
        dt_interp = time.perf_counter() - t0
    # the same queued step in the entries' default, the reference's strict block order (every
    # output byte-identical with the generated kernel's): the strict streaming kernel
    L.tcrv_cuda_host_set_fold_order(0)
    device_flags[0] = pkg.FLAG_STRICT_ORDER
    dt_strict = timed(one_pass_queued)
    one_pass_queued()
    check()
    world = dist.get_world_size() if dist is not None else 1
    for l, w_host, x_host, y_host in host:
        L.tcrv_cuda_host_unregister_weights(w_host.ctypes.data)
    L.tcrv_cuda_host_release()
    L.tcrv_cuda_host_set_fold_order(previous_order)
    step_bytes = sum(l["bytes"] for l in layers)
    return {"value": round(step_bytes * steps * world / dt / 1e9, 2), "unit": UNIT,
            "h2d_bytes_per_step": sum(int(x.numel()) for _, _, x, _ in host),
            "d2h_bytes_per_step": sum(int(y.numel()) * 4 for _, _, _, y in host),
            "ms_per_step": round(dt / steps * 1e3, 4), "steps": steps,
            "call": "tcrv_cuda_host_gemm_q4_0_q8_0_async per layer + tcrv_cuda_host_sync per step (one host round trip "
                    "per step; the library replays a repeated step as one graph: one fetch of the four layers' "
                    "activations, then one grouped launch in which the four independent GEMVs stream at once)",
            "caller": ("a C++ loop over the entries (examples/gpu/decode_loop.cpp), wall clock around all steps"
                       if loop is not None else "this interpreter (ctypes), wall clock around all steps"),
            "interpreter_caller": (None if dt_interp is None else
                                   {"value": round(step_bytes * steps / dt_interp / 1e9, 2),
                                    "ms_per_step": round(dt_interp / steps * 1e3, 4),
                                    "call": "the same queued step with the five calls made through ctypes (this rank)"}),
            "blocking_calls": {"value": round(step_bytes * steps * world / dt_blocking / 1e9, 2),
                               "ms_per_step": round(dt_blocking / steps * 1e3, 4),
                               "call": "tcrv_cuda_host_gemm_q4_0_q8_0 per layer (each call waits for its result)"},
            "fold_order": "TCRV_CUDA_HOST_FOLD_FAST (lane pairs), selected with tcrv_cuda_host_set_fold_order",
            "reference_order": {"value": round(step_bytes * steps * world / dt_strict / 1e9, 2),
                                "ms_per_step": round(dt_strict / steps * 1e3, 4),
                                "call": "the same queued step with the entries' default TCRV_CUDA_HOST_FOLD_STRICT: "
                                        "every output has the bits of the reference's ascending block order"},
            "weights": "registered once (resident); activations and outputs cross PCIe every step "
                       "(inputs by a copy from the pinned buffer, results stored by the kernel into the pinned "
                       "output through its device mapping)"}


def measure_other_kernels(pkg, torch):
    """The remaining kernels of the path at their benchmark sizes, device-resident, timed with
    events over CUDA-graph replays on rotating buffers (> L2 in total): algorithmic GB/s."""
    side = torch.cuda.Stream()
    gen = torch.Generator(device="cuda").manual_seed(5)
    out = []

    def timed(name, fn_for_copy, ncopies, nbytes, note):
        with torch.cuda.stream(side):
            for c in range(ncopies):
                fn_for_copy(c)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for c in range(ncopies):
                fn_for_copy(c)
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 10
        a.record()
        for _ in range(reps):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / (reps * ncopies)
        out.append({"kernel": name, "us": round(us, 3), "gbs": round(nbytes / us / 1e3, 1), "bytes": nbytes, "case": note})

    # add f32, n = 1,048,576 (12.6 MB per launch; 24 buffer sets = 302 MB)
    n = 1 << 20
    sets = [(torch.rand(n, generator=gen, device="cuda") * 2 - 1, torch.rand(n, generator=gen, device="cuda") * 2 - 1,
             torch.empty(n, device="cuda")) for _ in range(24)]
    timed("add_f32", lambda c: pkg.add(sets[c][0], sets[c][1], out=sets[c][2]), 24, 12 * n, "n = 1,048,576")
    del sets
    # the same kernel on 64 Mi elements (805 MB per launch; 2 buffer sets): long enough that launch
    # latency no longer hides the kernel's own bandwidth
    nbig = 64 << 20
    big = [(torch.rand(nbig, generator=gen, device="cuda"), torch.rand(nbig, generator=gen, device="cuda"),
            torch.empty(nbig, device="cuda")) for _ in range(2)]
    timed("add_f32_64Mi", lambda c: pkg.add(big[c][0], big[c][1], out=big[c][2]), 2, 12 * nbig, "n = 67,108,864")
    del big
    # Q8_0 dequant 4096 x 4096 (84.9 MB per launch; 4 sets)
    wf = torch.randn((4096, 4096), generator=gen, device="cuda") * 0.02
    q8 = [pkg.quantize_q8_0(wf) for _ in range(4)]
    q4 = [pkg.quantize_q4_0(wf) for _ in range(4)]
    outs = [torch.empty((4096, 4096), device="cuda") for _ in range(4)]
    nb = 4096 * 4096 // 32
    timed("dequantize_row_q8_0", lambda c: pkg.dequantize_q8_0(q8[c], out=outs[c]), 4, nb * (34 + 128), "4096 x 4096")
    timed("dequantize_row_q4_0", lambda c: pkg.dequantize_q4_0(q4[c], out=outs[c]), 4, nb * (18 + 128), "4096 x 4096")
    timed("quantize_row_q8_0", lambda c: pkg.quantize_q8_0(outs[c], out=q8[c]), 4, nb * (34 + 128), "4096 x 4096")
    del q4, outs, wf
    # Q8_0 x Q8_0 GEMV 11008 x 4096 and Q4_0 x Q8_0 GEMV with 8 activation columns
    w8 = [pkg.quantize_q8_0(torch.randn((11008, 4096), generator=gen, device="cuda") * 0.02) for _ in range(6)]
    x1 = pkg.quantize_q8_0(torch.randn((1, 4096), generator=gen, device="cuda"))
    y1 = torch.empty((11008, 1), device="cuda")
    timed("gemv_q8_0_q8_0", lambda c: pkg.gemv(w8[c], x1, q8_weights=True, out=y1, flags=pkg.FLAG_STATIC_WEIGHTS), 6,
          11008 * 128 * 34 + 128 * 34 + 4 * 11008, "11008 x 4096, batch 1")
    del w8
    w4 = [pkg.quantize_q4_0(torch.randn((32000, 4096), generator=gen, device="cuda") * 0.02) for _ in range(5)]
    x8 = pkg.quantize_q8_0(torch.randn((8, 4096), generator=gen, device="cuda"))
    y8 = torch.empty((32000, 8), device="cuda")
    timed("gemv_q4_0_q8_0_batch8", lambda c: pkg.gemv(w4[c], x8, out=y8, flags=pkg.FLAG_STATIC_WEIGHTS), 5,
          gemv_bytes(32000, 4096, 8), "32000 x 4096, batch 8")
    # the strict-order (reference order) GEMV on the same matrix, 1 and 8 columns
    for cols in (1, 8):
        xs_ = pkg.quantize_q8_0(torch.randn((cols, 4096), generator=gen, device="cuda"))
        ys_ = torch.empty((32000, cols), device="cuda")
        timed(f"gemv_q4_0_q8_0_strict_order_b{cols}",
              lambda c, xs_=xs_, ys_=ys_: pkg.gemv(w4[c], xs_, out=ys_, flags=pkg.FLAG_STRICT_ORDER), 5,
              32000 * 128 * 18 + cols * 128 * 34 + 4 * cols * 32000, f"32000 x 4096, batch {cols}, strict ascending block order")
    del w4
    # consumers of the 16-row interleaved layouts: decode GEMV over block_q4_0x16 / block_q8_0x16
    # (random bytes stand in for the weights: the timing does not depend on the values), and the
    # prefill GEMM over block_q4_0x16 x block_q8_0x4 with resident weights
    x1r = x1.reshape(-1)
    for q8w, rows, block, copies in ((False, 32000, 288, 5), (True, 11008, 544, 6)):
        wx = [torch.randint(0, 256, (rows // 16 * 128 * block,), dtype=torch.uint8, device="cuda", generator=gen)
              for _ in range(copies)]
        yr = torch.empty(rows, device="cuda")
        timed("repack_gemv_q8_0x16" if q8w else "repack_gemv_q4_0x16",
              lambda c, wx=wx, yr=yr, rows=rows, q8w=q8w: pkg.repack_gemv(wx[c], x1r, rows, q8_weights=q8w, out=yr),
              copies, rows * 128 * (34 if q8w else 18) + 128 * 34 + 4 * rows, f"{rows} x 4096, batch 1")
        timed(("repack_gemv_q8_0x16" if q8w else "repack_gemv_q4_0x16") + "_strict_order",
              lambda c, wx=wx, yr=yr, rows=rows, q8w=q8w: pkg.repack_gemv(wx[c], x1r, rows, q8_weights=q8w, out=yr,
                                                                          flags=pkg.FLAG_STRICT_ORDER),
              copies, rows * 128 * (34 if q8w else 18) + 128 * 34 + 4 * rows,
              f"{rows} x 4096, batch 1, the reference's one chain per row")
        del wx
    wx = torch.randint(0, 256, (11008 // 16 * 128 * 288,), dtype=torch.uint8, device="cuda", generator=gen)
    xx = torch.randint(0, 256, (GEMM_TOKENS // 4 * 128 * 136,), dtype=torch.uint8, device="cuda", generator=gen)
    pw = pkg.PreparedX16Weights(wx, 4096, 11008)
    og = torch.empty((GEMM_TOKENS, 11008), device="cuda")
    wsg = torch.empty(int(pkg.lib().tcrv_cuda_gemm_acts_workspace_bytes(4096, GEMM_TOKENS)), dtype=torch.uint8,
                      device="cuda")
    timed("repack_gemm_q4_0x16_q8_0x4", lambda c: pw.gemm(xx, GEMM_TOKENS, out=og, workspace=wsg), 4,
          11008 * 128 * 18 + GEMM_TOKENS * 128 * 34 + 4 * GEMM_TOKENS * 11008,
          "M512 x N11008 x K4096, resident weights; tensor-bound: see tops")
    out[-1]["tops"] = round(2 * GEMM_TOKENS * 11008 * 4096 / out[-1]["us"] / 1e6, 1)
    del wx, xx, pw, og, wsg
    # sibling block formats, one column against 32000 x 4096 (strict ascending order): random quants,
    # fp16 scales in a sane range so that the arithmetic sees ordinary numbers
    def sibling_blocks(rows, nb, block, scale_fields):
        b = torch.randint(0, 256, (rows, nb, block), dtype=torch.uint8, device="cuda", generator=gen)
        for f in range(scale_fields):
            d = (torch.rand((rows, nb), generator=gen, device="cuda") * 0.05 + 0.01).to(torch.float16)
            b[:, :, 2 * f:2 * f + 2] = d.view(torch.uint8).reshape(rows, nb, 2)
        return b.reshape(rows, nb * block)

    for fmt, name, (wb, ab), (wf, af) in ((1, "q4_1_q8_1", (20, 36), (2, 2)), (2, "q5_0_q8_0", (22, 34), (1, 1)),
                                          (3, "q5_1_q8_1", (24, 36), (2, 2))):
        rows, copies = 32000, 3
        ws = [sibling_blocks(rows, 128, wb, wf) for _ in range(copies)]
        xs1 = sibling_blocks(1, 128, ab, af)
        ys = torch.empty((rows, 1), device="cuda")
        timed(f"sibling_dot_rows_{name}", lambda c, ws=ws, xs1=xs1, ys=ys, fmt=fmt: pkg.sibling_dot_rows(fmt, ws[c], xs1, out=ys),
              copies, rows * 128 * wb + 128 * ab + 4 * rows, f"{rows} x 4096, one column, strict block order")
        del ws
    # f32 forward-pass ops on a prefill-sized activation (512 tokens x 11008 = 22.5 MB; 8 sets)
    acts = [torch.randn((512, 11008), generator=gen, device="cuda") for _ in range(8)]
    outs = [torch.empty((512, 11008), device="cuda") for _ in range(8)]
    nbytes = 512 * 11008 * 4
    timed("vec_silu_f32", lambda c: pkg.vec_silu(acts[c], out=outs[c]), 8, 2 * nbytes, "512 x 11008")
    timed("rms_norm_f32", lambda c: pkg.rms_norm(acts[c], 1e-6, out=outs[c]), 8, 2 * nbytes,
          "512 rows x 11008 (each row read once, kept in registers)")
    timed("vec_scale_f32", lambda c: pkg.vec_scale_(outs[c], 0.5), 8, 2 * nbytes, "512 x 11008, in place")
    pkg.check_device_errors()
    return out


GEMM_SHAPES = [(11008, 4096), (32000, 4096)]
GEMM_TOKENS = 512


def measure_gemm(pkg, torch, dist, rank, world):
    """Prefill GEMM (M = 512 tokens): int8 TOPS with prepared weights; with N > 1 the weight
    rows are sharded across ranks and the fp32 output slabs are all-gathered over NCCL."""
    peaks, peak_kind = measured_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    gen = torch.Generator(device="cuda").manual_seed(99 + rank)
    results = []
    for nr, k in GEMM_SHAPES:
        ops = 2.0 * GEMM_TOKENS * nr * k
        first_row, rows = pkg.row_shard(nr, world, rank)
        wq = pkg.quantize_q4_0(torch.randn((rows, k), generator=gen, device="cuda") * 0.02)
        x = pkg.quantize_q8_0(torch.randn((GEMM_TOKENS, k), generator=gen, device="cuda"))
        pw = pkg.PreparedWeights(wq)
        full = torch.empty((nr, GEMM_TOKENS), dtype=torch.float32, device="cuda")
        slab = full[first_row:first_row + rows]
        ws = torch.empty(pkg.lib().tcrv_cuda_gemm_acts_workspace_bytes(k, GEMM_TOKENS), dtype=torch.uint8, device="cuda")
        ws_plain = torch.empty(pkg.lib().tcrv_cuda_gemm_workspace_bytes(k, rows, GEMM_TOKENS), dtype=torch.uint8,
                               device="cuda")

        def timed(fn, reps=20):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / reps
            if dist is not None:
                t = torch.tensor([ms], dtype=torch.float64, device="cuda")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            return ms

        def compute():
            pkg.gemm(pw, x, out=slab, workspace=ws)

        def compute_plain():
            pkg.gemm(wq, x, out=slab, workspace=ws_plain)

        def with_gather():
            pkg.gemm(pw, x, out=slab, workspace=ws)
            pkg.gather_row_slabs(full, dist, rank, world)

        ms_c = timed(compute)
        ms_p = timed(compute_plain)
        # the multi-destination kernel with two copies in THIS GPU's memory: what the staged bulk
        # stores cost without a link behind them
        import ctypes
        second = torch.empty((rows, GEMM_TOKENS), dtype=torch.float32, device="cuda")
        dst2 = (ctypes.c_void_p * 2)(slab.data_ptr(), second.data_ptr())

        def compute_two_local():
            st = pkg.lib().tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(k, dst2, 2, pw.buffer.data_ptr(), x.data_ptr(), x.stride(0),
                                                                    rows, GEMM_TOKENS, GEMM_TOKENS, ws.data_ptr(), ws.numel(), 0,
                                                                    torch.cuda.current_stream().cuda_stream)
            if st != 0:
                raise RuntimeError(f"prepared_multi failed: {st}")

        ms_2 = timed(compute_two_local)
        del second
        # calibration of the int8 tensor pipe on this GPU and this shape: the plain library
        # int8 GEMM (cuBLASLt through torch._int_mm, int32 out, no scales), this rank's rows
        cal_tops = None
        try:
            a8 = torch.randint(-127, 128, (GEMM_TOKENS, k), dtype=torch.int8, device="cuda", generator=gen)
            b8 = torch.randint(-8, 8, (rows, k), dtype=torch.int8, device="cuda", generator=gen).t()
            ms_cal = timed(lambda: torch._int_mm(a8, b8))
            cal_tops = 2.0 * GEMM_TOKENS * rows * k / ms_cal / 1e9
            del a8, b8
        except Exception as exc:  # noqa: BLE001 - the calibration is optional
            cal_note = f"{type(exc).__name__}: {exc}"[:120]
        entry_ = {"shape": f"M{GEMM_TOKENS}xN{nr}xK{k}", "rows_per_gpu": rows,
                  "compute_ms": round(ms_c, 4), "compute_tops": round(ops / ms_c / 1e9, 1),
                  "plain_format_ms": round(ms_p, 4), "plain_format_tops": round(ops / ms_p / 1e9, 1),
                  "two_local_copies_ms": round(ms_2, 4)}
        if dist is not None:
            ms_g = timed(with_gather)
            entry_.update({"with_allgather_ms": round(ms_g, 4), "with_allgather_tops": round(ops / ms_g / 1e9, 1),
                           "allgather_bytes": nr * GEMM_TOKENS * 4})
            # the all-gather fused into the epilogue: finished tiles are stored into every rank's
            # copy of the output (peer memory over NVLink) while later tiles compute
            # (SharedOutput agrees on success or failure across the ranks, so every rank takes
            # the same branch below)
            shared = pkg.SharedOutput(nr, GEMM_TOKENS, dist, rank, world,
                                      torch.device("cuda", torch.cuda.current_device()))
            if shared.error is not None:
                entry_["fused_allgather_error"] = f"{type(shared.error).__name__}: {shared.error}"
                shared.close()
            else:
                def fused():
                    shared.gemm_into(pw, x, workspace=ws)

                with_gather()
                fused()
                shared.wait()
                same = bool(torch.equal(shared.local(), full))
                ms_f = timed(fused)
                shared.wait()
                entry_.update({"fused_allgather_ms": round(ms_f, 4), "fused_allgather_tops": round(ops / ms_f / 1e9, 1),
                               "fused_equals_nccl": same,
                               "fused_link_gbs_per_gpu": round(rows * GEMM_TOKENS * 4 * (world - 1) / ms_f / 1e6, 1)})
                shared.close()
        entry_["roofline"] = {"bound": "tensor", "achieved": entry_["compute_tops"], "peak": int8_peak,
                              "unit": "TOP/s", "frac": round(entry_["compute_tops"] / world / int8_peak, 4),
                              "peak_kind": f"2 x bf16 burst peak ({peak_kind}); no int8 figure is measured on this pool"}
        if cal_tops is not None:
            # per-GPU figures on both sides: this rank's share of the work over the calibration
            entry_["roofline"]["library_int8_gemm_tops"] = round(cal_tops, 1)
            entry_["roofline"]["frac_of_library_int8_gemm"] = round(ops / world / ms_c / 1e9 / cal_tops, 4)
            entry_["roofline"]["library_int8_gemm"] = ("torch._int_mm (cuBLASLt), same M, K and rows per GPU, int32 "
                                                       "output, no block scales: what the tensor pipe sustains "
                                                       "without the per-block fp32 fold")
        else:
            entry_["roofline"]["library_int8_gemm"] = "unavailable: " + cal_note
        pkg.check_device_errors()
        results.append(entry_)
        del wq, pw, full, ws, ws_plain
    return results


PROFILE_CASES = ["gemv", "gemv_q8", "gemv_strict", "gemv_strict_cta", "gemv_group", "gemm", "dequant", "quantize", "silu", "rms_norm", "repack_gemv", "repack_gemv_q8",
                 "repack_gemm", "sibling_q4_1", "sibling_q5_0", "sibling_q5_1"]


def run_profile_case(args):
    """`--profile-case NAME`: a small, self-ending workload that launches ONE kernel family a
    handful of times (a few GB on the device at most, rotating weight copies larger than the L2
    so that DRAM counters mean something), for a profiler to capture.  Prints no metric."""
    args.case = args.profile_case
    args.rows = args.case_rows
    args.k = args.case_k
    args.cols = args.case_cols
    args.tokens = args.case_tokens
    args.launches = args.case_launches
    import torch

    pkg = entry.load_package()
    torch.cuda.set_device(0)
    gen = torch.Generator(device="cuda").manual_seed(7)
    if args.case in ("gemv", "gemv_q8", "gemv_strict", "gemv_strict_cta"):
        rows = args.rows or 32000
        q8w = args.case == "gemv_q8"
        # gemv_strict_cta: the strict order on the kernel with one term table per CTA (tuning
        # bit 13), which serves 2 columns and the sibling formats by default
        flags = {"gemv_strict": pkg.FLAG_STRICT_ORDER, "gemv_strict_cta": pkg.FLAG_STRICT_ORDER | 0x2000}.get(args.case, 0)
        wf = torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02
        w = pkg.quantize_q8_0(wf) if q8w else pkg.quantize_q4_0(wf)
        copies = [w] + [w.clone() for _ in range(max(2, (300 << 20) // w.numel()))]
        x = pkg.quantize_q8_0(torch.randn((args.cols, args.k), generator=gen, device="cuda"))
        y = torch.empty((rows, args.cols), dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.gemv(copies[i % len(copies)], x, q8_weights=q8w, out=y, flags=flags)
    elif args.case == "gemv_group":
        # the four layer shapes of the decode step as one grouped launch, 3 rotating copies of each
        problems = []
        for r in range(3):
            group = []
            for nr, k in SHAPES:
                w = pkg.quantize_q4_0(torch.randn((nr, k), generator=gen, device="cuda") * 0.02)
                x = pkg.quantize_q8_0(torch.randn((1, k), generator=gen, device="cuda"))
                group.append((w, x, torch.empty((nr, 1), dtype=torch.float32, device="cuda")))
            problems.append(group)
        calls = [pkg.gemv_group_calls(g) for g in problems]
        for i in range(args.launches):
            pkg.gemv_group(calls[i % len(calls)], flags=pkg.FLAG_STATIC_WEIGHTS)
    elif args.case in ("repack_gemv", "repack_gemv_q8"):
        # random bytes stand in for the interleaved weights (timing and traffic do not depend on them)
        rows = args.rows or 32000
        q8w = args.case == "repack_gemv_q8"
        nbytes = rows // 16 * (args.k // 32) * (544 if q8w else 288)
        copies = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda", generator=gen)
                  for _ in range(max(3, (300 << 20) // nbytes + 1))]
        x = pkg.quantize_q8_0(torch.randn((1, args.k), generator=gen, device="cuda")).reshape(-1)
        y = torch.empty(rows, dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.repack_gemv(copies[i % len(copies)], x, rows, q8_weights=q8w, out=y)
    elif args.case.startswith("sibling_"):
        # random quants, fp16 scales in a sane range; one column against `rows` rows
        fmt, wb, ab, wf, af = {"sibling_q4_1": (1, 20, 36, 2, 2), "sibling_q5_0": (2, 22, 34, 1, 1),
                               "sibling_q5_1": (3, 24, 36, 2, 2)}[args.case]
        rows, nb = args.rows or 32000, args.k // 32

        def blocks(r, block, fields):
            b = torch.randint(0, 256, (r, nb, block), dtype=torch.uint8, device="cuda", generator=gen)
            for f in range(fields):
                d = (torch.rand((r, nb), generator=gen, device="cuda") * 0.05 + 0.01).to(torch.float16)
                b[:, :, 2 * f:2 * f + 2] = d.view(torch.uint8).reshape(r, nb, 2)
            return b.reshape(r, nb * block)

        copies = [blocks(rows, wb, wf) for _ in range(4)]
        x = blocks(1, ab, af)
        y = torch.empty((rows, 1), dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.sibling_dot_rows(fmt, copies[i % len(copies)], x, out=y)
    elif args.case == "repack_gemm":
        rows = args.rows or 11008
        nb = args.k // 32
        wx = torch.randint(0, 256, (rows // 16 * nb * 288,), dtype=torch.uint8, device="cuda", generator=gen)
        xx = torch.randint(0, 256, (args.tokens // 4 * nb * 136,), dtype=torch.uint8, device="cuda", generator=gen)
        pw = pkg.PreparedX16Weights(wx, args.k, rows)
        out = torch.empty((args.tokens, rows), dtype=torch.float32, device="cuda")
        for _ in range(args.launches):
            pw.gemm(xx, args.tokens, out=out)
    elif args.case == "gemm":
        rows = args.rows or 11008
        w = pkg.quantize_q4_0(torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02)
        x = pkg.quantize_q8_0(torch.randn((args.tokens, args.k), generator=gen, device="cuda"))
        pw = pkg.PreparedWeights(w)
        out = torch.empty((rows, args.tokens), dtype=torch.float32, device="cuda")
        for _ in range(args.launches):
            pkg.gemm(pw, x, out=out)
    elif args.case in ("quantize", "silu", "rms_norm"):
        rows = args.rows or (4096 if args.case == "quantize" else 512)
        k = args.k if (args.case == "quantize" or args.k != 4096) else 11008
        xs = [torch.randn((rows, k), generator=gen, device="cuda") for _ in range(6)]
        out = torch.empty((rows, k), dtype=torch.float32, device="cuda")
        qout = torch.empty((rows, k // 32 * 34), dtype=torch.uint8, device="cuda")
        for i in range(args.launches):
            if args.case == "quantize":
                pkg.quantize_q8_0(xs[i % len(xs)], out=qout)
            elif args.case == "silu":
                pkg.vec_silu(xs[i % len(xs)], out=out)
            else:
                pkg.rms_norm(xs[i % len(xs)], 1e-6, out=out)
    else:
        rows = args.rows or 4096
        q = pkg.quantize_q8_0(torch.randn((rows, args.k), generator=gen, device="cuda") * 0.02)
        copies = [q] + [q.clone() for _ in range(8)]
        out = torch.empty((rows, args.k), dtype=torch.float32, device="cuda")
        for i in range(args.launches):
            pkg.dequantize_q8_0(copies[i % len(copies)], out=out)
    torch.cuda.synchronize()
    pkg.check_device_errors()
    print("profile case done")




def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--min-warm-seconds", type=float, default=MIN_WARM_SECONDS,
                    help="warm-up lasts at least this long (0 for a profiler's launch-list pass)")
    ap.add_argument("--skip-gemm", action="store_true", help="leave out the prefill-GEMM section")
    ap.add_argument("--gemm-only", action="store_true", help="run the prefill-GEMM section alone (not the benchmark line)")
    ap.add_argument("--graph-steps", type=int, default=GRAPH_STEPS, help="most steps captured per CUDA graph of the timed region")
    ap.add_argument("--regions", type=int, default=MIN_REGIONS, help="how often the K-step region is timed (median reported)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="more regions are timed until they add up to this much device time (0 for a profiler pass)")
    ap.add_argument("--profile-case", choices=PROFILE_CASES, default=None,
                    help="run a small self-ending workload of one kernel family for a profiler instead of the benchmark")
    ap.add_argument("--case-rows", type=int, default=None)
    ap.add_argument("--case-k", type=int, default=4096)
    ap.add_argument("--case-cols", type=int, default=1)
    ap.add_argument("--case-tokens", type=int, default=512)
    ap.add_argument("--case-launches", type=int, default=6)
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
