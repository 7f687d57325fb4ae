#!/usr/bin/env python
"""Benchmark of the direct 2-D cross-correlation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: the five
benchmark configurations (one-to-one 16x16 and 256x256, one-to-many 64x64 x512, n-to-m
32x32 32x64, n-to-mn 48x48 16x128), each as ONE library call.  Inputs are seeded
uniform[0,1) float32 -- the value distribution of the reference's own generator
(benchmark/input_generator.py:20-32) -- and are resident in HBM before the timed region.

With N > 1 (one process per GPU, launched by torch.distributed.run) every rank runs the
same pass on its own GPU: the independent result matrices of the many-matrix modes are the
sharding unit, so N ranks holding one configuration's worth each is the N-times larger
problem (N*512 right matrices, N*32 left matrices, N*16 left groups) sharded with the
other operand replicated -- weak scaling, no collective on the data path.  The fixed-size
split of each configuration over N GPUs ("strong") is reported per configuration as well.

Output: ONE JSON line on rank 0.  `value` is the whole-job GFLOP/s (algorithmic FLOP =
2 * pairs * rows^2 * cols^2) over all ranks; per-configuration GFLOP/s, output shifts/s and
fraction of FP32-FFMA peak are under `per_config`.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# name -> (mode, rows, cols, n_left, n_right)
CONFIGS = {
    "C1": ("one_to_one", 16, 16, 1, 1),
    "C2": ("one_to_one", 256, 256, 1, 1),
    "C3": ("one_to_many", 64, 64, 1, 512),
    "C4": ("n_to_m", 32, 32, 32, 64),
    "C5": ("n_to_mn", 48, 48, 16, 2048),
}
L2_BYTES = 126 * 1024 * 1024
NOMINAL_SM, NOMINAL_LANES = 148, 128


def pairs_of(mode, nl, nr):
    return {"one_to_one": 1, "one_to_many": nr, "n_to_mn": nr, "n_to_m": nl * nr}[mode]


def flop_of(k):
    mode, r, c, nl, nr = CONFIGS[k]
    return 2.0 * pairs_of(mode, nl, nr) * r * r * c * c


def shifts_of(k):
    mode, r, c, nl, nr = CONFIGS[k]
    return pairs_of(mode, nl, nr) * (2 * r - 1) * (2 * c - 1)


def bytes_of(k):
    """Compulsory bytes of one launch: every input matrix read once, every output written once."""
    mode, r, c, nl, nr = CONFIGS[k]
    return 4 * ((nl + nr) * r * c + shifts_of(k))


def config_inputs(k, rank=0):
    """Seeds 1000+k (left) and 2000+k (right); other ranks offset the seed (they hold other
    matrices of the N-times larger problem)."""
    mode, r, c, nl, nr = CONFIGS[k]
    idx = int(k[1])
    left = np.random.default_rng(1000 + idx).random((nl, r, c), dtype=np.float32)
    right = np.random.default_rng(2000 + idx + 100 * rank).random((nr, r, c), dtype=np.float32)
    return left, right


def strong_shard(xc, k, world, rank):
    """The part of configuration k that rank `rank` of `world` owns when the configuration
    itself is split (strong scaling): (units_first, units_count, n_left, n_right) where the
    units are right matrices for one_to_many and left matrices (with all / their own rights)
    for n_to_m / n_to_mn.  one_to_one does not shard: rank 0 owns it."""
    mode, r, c, nl, nr = CONFIGS[k]
    if mode == "one_to_one":
        return (0, 1, 1, 1) if rank == 0 else (0, 0, 0, 0)
    units = nr if mode == "one_to_many" else nl
    first, count = xc.shard_range(units, world, rank)
    if mode == "one_to_many":
        return first, count, 1, count
    if mode == "n_to_m":
        return first, count, count, nr
    return first, count, count, count * (nr // nl)


def max_over_ranks(values, dist=None, device="cpu"):
    """Element-wise maximum of a list of floats over all ranks (identity without a group)."""
    import torch
    vec = torch.tensor(values, dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(vec, op=dist.ReduceOp.MAX)
    return vec.cpu().tolist()


def load_package():
    name = "jpdc23_artifact_b200"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "jpdc23-artifact_b200", "__init__.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


# ---- clocks -------------------------------------------------------------------------------------
class ClockSampler:
    """nvidia-smi samples of one GPU every 100 ms while the timed region runs (read-only)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s, p in zip(sm, pw) if p >= 0.5 * max(pw)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "power_w_max": max(pw),
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU baseline (the reference's own CPU path) ------------------------------------------------
def cpu_baseline(target_seconds: float, threads: int):
    """Time the reference's CPU implementation (oracle/_ref, validate.hpp:94-298, compiled
    unmodified) -- or the C restatement when that library is absent -- on a bounded sample of
    each configuration: as many whole result matrices as fit the time budget, split over
    `threads` host threads.  Returns (GFLOP/s over the sample, description)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pyoracle
    if pyoracle.Reference.available():
        ref = pyoracle.Reference()
        kind = "reference"

        def run(mode, left, right):
            return ref.run_threaded(mode, left, right, threads)
    else:
        orc = pyoracle.Oracle()
        kind = "port"

        def run(mode, left, right):
            return orc.run(mode, left, right, threads=threads)

    est_rate = 2.2e9 * threads              # FLOP/s guess to size the sample; measured below
    budget = target_seconds / len(CONFIGS)
    total_flop, total_s, parts = 0.0, 0.0, []
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        left, right = config_inputs(k)
        per_pair = 2.0 * r * r * c * c
        want_pairs = max(1, int(budget * est_rate / per_pair))
        if mode == "one_to_one":
            l, rt, npairs = left, right, 1
        elif mode == "one_to_many":
            n = min(nr, max(threads, want_pairs))
            l, rt, npairs = left, right[:n], n
        elif mode == "n_to_m":
            nls = min(nl, max(1, want_pairs // nr)) if want_pairs >= nr else 1
            nrs = nr if want_pairs >= nr else min(nr, max(threads, want_pairs))
            l, rt, npairs = left[:nls], right[:nrs], nls * nrs
        else:  # n_to_mn, file order t*n + l: keep every left, cut the number of groups t
            m = nr // nl
            ms = min(m, max(1, want_pairs // nl))
            l, rt, npairs = left, right[:ms * nl], ms * nl
        t0 = time.perf_counter()
        run(mode, l, rt)
        dt = time.perf_counter() - t0
        total_flop += per_pair * npairs
        total_s += dt
        parts.append(f"{k}:{npairs}/{pairs_of(mode, nl, nr)} pairs {dt:.2f}s")
    return total_flop / total_s / 1e9, kind, "; ".join(parts)


def cpu_single_thread():
    """The reference's CPU path exactly as the reference runs it: one thread (validate.hpp:237 leaves
    the pair loop sequential).  A small sample of every configuration: the whole of the two single
    pairs, a few pairs of the three many-matrix ones.  Returns (GFLOP/s, description)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pyoracle
    if pyoracle.Reference.available():
        ref = pyoracle.Reference()
        run = lambda mode, l, r: ref.run_threaded(mode, l, r, 1)      # noqa: E731
    else:
        orc = pyoracle.Oracle()
        run = lambda mode, l, r: orc.run(mode, l, r, threads=1)       # noqa: E731
    sample = {"one_to_one": 1, "one_to_many": 4, "n_to_m": 16, "n_to_mn": 8}
    flop, secs, parts = 0.0, 0.0, []
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        left, right = config_inputs(k)
        n = sample[mode]
        if mode == "one_to_one":
            l, rt = left, right
        elif mode == "one_to_many":
            l, rt = left, right[:n]
        elif mode == "n_to_m":
            l, rt = left[:1], right[:n]
        else:                                   # file order t*n + l: n_left lefts, one right each
            n = nl
            l, rt = left, right[:nl]
        t0 = time.perf_counter()
        run(mode, l, rt)
        dt = time.perf_counter() - t0
        flop += 2.0 * r * r * c * c * n
        secs += dt
        parts.append(f"{k}:{n} pairs {dt:.2f}s")
    return flop / secs / 1e9, "; ".join(parts)


# ---- the reference arm -----------------------------------------------------------------------------
def graph_replay_us(call, launches=20, replays=10):
    """Device time per launch, in microseconds, of `call(stream_handle)`: `launches` calls
    recorded into one CUDA graph on a side stream, the graph replayed `replays` times between
    two events.  For kernels of a few microseconds, where back-to-back launches measure the
    host's launch rate instead."""
    import torch
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        call(side.cuda_stream)
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(launches):
                call(torch.cuda.current_stream().cuda_stream)
        g.replay()
        side.synchronize()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record(side)
        for _ in range(replays):
            g.replay()
        b.record(side)
        side.synchronize()
    return a.elapsed_time(b) * 1e3 / (launches * replays)


def reference_gpu_baseline(dev, launch, iters=20, launch_on=None):
    """The reference's own best CUDA kernels, recompiled unmodified for sm_100 (optional
    libraries under oracle/_ref/, see oracle/Makefile targets refcuda / refcuda_n2m), timed on
    this GPU on the same resident inputs with the best published arguments: a reported
    baseline next to `cpu_baseline`, nothing of the product runs through it.  Returns None
    when the library was not built."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pyoracle
    if not pyoracle.ReferenceCuda.available():
        return None
    rc = pyoracle.ReferenceCuda()
    wps = pyoracle.ReferenceWarpPerShift() if pyoracle.ReferenceWarpPerShift.available() else None
    side = [torch.cuda.Stream() for _ in range(8)]
    legacy = torch.cuda.default_stream()        # launchers without a stream argument use it
    out = {"kind": "reference CUDA kernels (warp-per-overlap for 16x16, grouped-overlap / multi-matrix families "
                   "for the rest) compiled for sm_100",
           "args": {"one_to_one 16x16": "warp_per_shift 16" if wps else "4_8_8 (warp_per_shift library not built)",
                    "one_to_one": "4_8_8", "one_to_many": "4_4_4_4", "n_to_mn": "4_4_4_4 on 8 streams",
                    "n_to_m": "4_4_4_4_4"}, "per_config": {}}
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        if mode == "n_to_m" and rc.n2m is None:
            out["per_config"][k] = {"unavailable": "n-to-m kernel library not built (hours of compile time)"}
            continue
        d = dev[k]
        res = torch.empty_like(d["out"])
        L, R, O = d["left"].data_ptr(), d["right"].data_ptr(), res.data_ptr()

        def run():
            if mode == "one_to_one" and wps is not None and r * c <= 32 * 32:
                wps.warp_per_shift(L, R, O, r, c, 16)      # the reference's published winner at 16 x 16
            elif mode == "one_to_one":
                rc.one_to_one(L, R, O, r, c)
            elif mode == "one_to_many":
                rc.one_to_many(L, R, O, r, c, nr)
            elif mode == "n_to_m":
                rc.n_to_m(L, R, O, r, c, nl, nr)
            else:
                start = torch.cuda.Event()
                start.record(legacy)
                for s_ in side:
                    s_.wait_event(start)
                rc.n_to_mn(L, R, O, r, c, nl, nr, streams=[s_.cuda_stream for s_ in side])
                for s_ in side:
                    e = torch.cuda.Event()
                    e.record(s_)
                    legacy.wait_event(e)
        torch.cuda.synchronize()
        for _ in range(3):
            run()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record(legacy)
        for _ in range(iters):
            run()
        b.record(legacy)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        diff = float((res - d["out"]).abs().max() / res.abs().max())
        # this library's call timed the same way: `iters` back-to-back calls between two events
        for _ in range(3):
            launch(k)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            launch(k)
        b.record()
        torch.cuda.synchronize()
        ours = a.elapsed_time(b) / iters
        out["per_config"][k] = {"ms": ms, "gflops": flop_of(k) / (ms * 1e-3) / 1e9,
                                "max_abs_diff_to_ours_over_max": diff, "ours_ms": ours, "speedup": ms / ours}
        if mode == "one_to_one" and wps is not None and r * c <= 32 * 32 and launch_on is not None:
            # a few microseconds each: back-to-back calls above time the host; these are graph replays
            ref_us = wps.graph_us(L, R, O, r, c, 16)
            ours_us = graph_replay_us(lambda s_: launch_on(k, s_))
            out["per_config"][k].update({"device_us": ref_us, "ours_device_us": ours_us,
                                         "device_speedup": ref_us / ours_us if ref_us > 0 else None,
                                         "device_timing": "20 launches in a CUDA graph, 10 replays between two events"})
    return out


def fft_path_timings(xc, dev, stream, hbm_peak, iters=20):
    """The cuFFT path (xcorr_fft_f32, normalized layout) on the same resident inputs: the
    algorithmic alternative the reference carries next to the direct kernels.  Reported beside
    the headline, not part of it.  `bytes` is the compulsory traffic of its five passes (pad,
    forward transform, product, inverse transform, unpack), each reading and writing its
    operands once."""
    import torch
    out = {}
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        d = dev[k]
        wsb = xc.fft_workspace_bytes(mode, r, c, nl, nr)
        ws = torch.empty(wsb + 256, dtype=torch.uint8, device="cuda")
        base = (ws.data_ptr() + 255) // 256 * 256
        res = torch.empty_like(d["out"])

        def run():
            xc.run_fft_device(mode, d["left"].data_ptr(), d["right"].data_ptr(), res.data_ptr(), r, c, nl, nr,
                              "normalized", base, wsb, stream)
        for _ in range(3):
            run()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            run()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        pairs = pairs_of(mode, nl, nr)
        real, cplx = 4 * r * c * 4, 2 * r * (c + 1) * 8          # bytes of one padded matrix / one spectrum
        n_in = nl + nr
        traffic = (n_in * (r * c * 4 + real)                      # pad
                   + n_in * (real + cplx)                         # forward
                   + pairs * 3 * cplx                             # product (left spectra re-read from L2)
                   + pairs * (cplx + real)                        # inverse
                   + pairs * (real + (2 * r - 1) * (2 * c - 1) * 4))   # unpack
        diff = float((res - d["out"]).abs().max() / d["out"].abs().max())
        out[k] = {"ms": ms, "equivalent_gflops": flop_of(k) / (ms * 1e-3) / 1e9, "bytes": traffic,
                  "hbm_gbs": traffic / (ms * 1e-3) / 1e9, "frac_hbm_measured": traffic / (ms * 1e-3) / 1e9 / hbm_peak,
                  "max_abs_diff_to_direct_over_max": diff}
        del ws, res
    return out


def f64_path_timings(xc, dev, stream, iters=5):
    """The double-precision entry point (xcorr_run_f64) on the same configurations, inputs widened
    to double: GFLOP/s, fraction of the FP64-FMA peak measured now, and the distance of the float
    result to it.  Reported beside the headline, not part of it."""
    import torch
    dfma_flops, _ = xc.dfma_peak_probe(stream)
    out = {"dfma_peak_measured_tflops": dfma_flops / 1e12}
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        d = dev[k]
        left, right = d["left"].double(), d["right"].double()
        res = torch.empty(d["out"].shape, dtype=torch.float64, device="cuda")

        def run():
            xc.run_device_f64(mode, left.data_ptr(), right.data_ptr(), res.data_ptr(), r, c, nl, nr, stream)
        for _ in range(2):
            run()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(iters):
            run()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / iters
        out[k] = {"ms": ms, "gflops": flop_of(k) / (ms * 1e-3) / 1e9,
                  "frac_dfma_measured": flop_of(k) / (ms * 1e-3) / dfma_flops,
                  "float_result_max_abs_diff_over_max": float((d["out"].double() - res).abs().max() / res.abs().max())}
        del left, right, res
    return out


# The reference's own benchmark grid (benchmark/benchmark.yml: groups one_to_one, one_to_many,
# n_to_mn, n_to_m and their "saturated" variants), as rows x cols x left x right.
GRID = {
    "one_to_one": ["16x16x1x1", "24x24x1x1", "32x32x1x1", "48x48x1x1", "64x64x1x1", "96x96x1x1", "128x128x1x1",
                   "192x192x1x1", "256x256x1x1"],
    "one_to_many": ["16x16x1x2", "16x16x1x8", "16x16x1x32", "32x32x1x2", "32x32x1x8", "32x32x1x32", "64x64x1x2",
                    "64x64x1x8", "64x64x1x32", "128x128x1x2", "128x128x1x8", "128x128x1x32", "256x256x1x2",
                    "256x256x1x8", "256x256x1x32", "16x16x1x4000", "32x32x1x4000", "64x64x1x4000",
                    "128x128x1x4000", "256x256x1x4000"],
    "n_to_mn": ["16x16x2x8", "16x16x4x16", "16x16x8x32", "32x32x2x8", "32x32x4x16", "32x32x8x32", "64x64x2x8",
                "64x64x4x16", "64x64x8x32", "128x128x2x8", "128x128x4x16", "128x128x8x32", "256x256x2x8",
                "256x256x4x16", "256x256x8x32", "16x16x100x4000", "32x32x100x4000", "64x64x100x4000",
                "128x128x100x4000", "256x256x100x4000"],
    "n_to_m": ["16x16x2x2", "16x16x8x8", "16x16x32x32", "32x32x2x2", "32x32x8x8", "32x32x32x32", "64x64x2x2",
               "64x64x8x8", "64x64x32x32", "128x128x2x2", "128x128x8x8", "128x128x32x32", "256x256x2x2",
               "256x256x8x8", "256x256x32x32", "16x16x128x128", "32x32x128x128", "64x64x128x128",
               "128x128x128x128"],
}


def run_grid(args):
    """`bench.py --grid`: every size of the reference's benchmark file on one GPU -- the direct
    kernels (automatic plan), the cuFFT path and, where oracle/_ref holds them, the reference's
    own best CUDA kernels -- resident inputs, CUDA events, one JSON line.  Sizes above
    --grid-max-tflop of arithmetic are skipped (the reference kernels above a fifth of that)."""
    import torch
    xc = load_package()
    xc.lib()
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import pyoracle
    rc = pyoracle.ReferenceCuda() if pyoracle.ReferenceCuda.available() else None
    wps = pyoracle.ReferenceWarpPerShift() if pyoracle.ReferenceWarpPerShift.available() else None
    side = [torch.cuda.Stream() for _ in range(8)]
    legacy = torch.cuda.default_stream()
    gen = torch.Generator(device="cuda").manual_seed(1234)

    def timed(fn, flop, on=None):
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(on)
        fn()
        b.record(on)
        torch.cuda.synchronize()
        once = max(a.elapsed_time(b), 1e-3)
        n = int(min(200, max(3, 30.0 / once)))
        a.record(on)
        for _ in range(n):
            fn()
        b.record(on)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / n

    rows_out = []
    for mode, sizes in GRID.items():
        for size in sizes:
            r, c, nl, nr = (int(v) for v in size.split("x"))
            pairs = pairs_of(mode, nl, nr)
            flop = 2.0 * pairs * r * r * c * c
            entry = {"mode": mode, "size": size, "gflop": flop / 1e9}
            if flop > args.grid_max_tflop * 1e12:
                entry["skipped"] = "above --grid-max-tflop"
                rows_out.append(entry)
                continue
            left = torch.rand((nl, r, c), device="cuda", generator=gen)
            right = torch.rand((nr, r, c), device="cuda", generator=gen)
            out = torch.empty(xc.out_shape(mode, r, c, nl, nr), dtype=torch.float32, device="cuda")
            L, R, O = left.data_ptr(), right.data_ptr(), out.data_ptr()
            wsb = xc.workspace_bytes(mode, r, c, nl, nr)
            ws = torch.empty(max(wsb, 16), dtype=torch.uint8, device="cuda")
            ms = timed(lambda: xc.run_device(mode, L, R, O, r, c, nl, nr, None, ws.data_ptr() if wsb else 0, wsb, stream), flop)
            entry.update(direct_ms=ms, direct_gflops=flop / ms / 1e6, plan=xc.last_launch().split(" plan{")[0])
            if ms < 0.03:       # back-to-back calls of a few microseconds time the host: also as graph replays
                entry["direct_graph_us"] = graph_replay_us(
                    lambda s_: xc.run_device(mode, L, R, O, r, c, nl, nr, None, ws.data_ptr() if wsb else 0, wsb, s_))
            direct = out.clone()
            fwsb = xc.fft_workspace_bytes(mode, r, c, nl, nr)
            fws = torch.empty(fwsb + 256, dtype=torch.uint8, device="cuda")
            fbase = (fws.data_ptr() + 255) // 256 * 256
            fms = timed(lambda: xc.run_fft_device(mode, L, R, O, r, c, nl, nr, "normalized", fbase, fwsb, stream), flop)
            entry.update(fft_ms=fms, fft_vs_direct=float((out - direct).abs().max() / direct.abs().max()))
            del fws
            if rc is not None and flop <= 0.2 * args.grid_max_tflop * 1e12 and not (mode == "n_to_m" and rc.n2m is None):
                def ref():
                    if mode == "one_to_one" and wps is not None and r * c <= 32 * 32:
                        wps.warp_per_shift(L, R, O, r, c, 16)
                    elif mode == "one_to_one":
                        rc.one_to_one(L, R, O, r, c)
                    elif mode == "one_to_many":
                        rc.one_to_many(L, R, O, r, c, nr)
                    elif mode == "n_to_m":
                        rc.n_to_m(L, R, O, r, c, nl, nr)
                    else:
                        start = torch.cuda.Event()
                        start.record(legacy)
                        for s_ in side:
                            s_.wait_event(start)
                        rc.n_to_mn(L, R, O, r, c, nl, nr, streams=[s_.cuda_stream for s_ in side])
                        for s_ in side:
                            e = torch.cuda.Event()
                            e.record(s_)
                            legacy.wait_event(e)
                torch.cuda.synchronize()
                rms = timed(ref, flop, legacy)
                entry.update(reference_ms=rms, speedup=rms / ms,
                             reference_vs_direct=float((out - direct).abs().max() / direct.abs().max()))
                if mode == "one_to_one" and wps is not None and r * c <= 32 * 32:
                    entry["reference_graph_us"] = wps.graph_us(L, R, O, r, c, 16)
                    if entry.get("direct_graph_us") and entry["reference_graph_us"] > 0:
                        entry["speedup_graph"] = entry["reference_graph_us"] / entry["direct_graph_us"]
            rows_out.append(entry)
            del left, right, out, direct, ws
            torch.cuda.empty_cache()
    xc.check_device()
    print(json.dumps({"grid": rows_out, "reference_args": {"one_to_one up to 32x32": "warp_per_shift 16" if wps else "4_8_8",
                                                            "one_to_one": "4_8_8", "one_to_many": "4_4_4_4",
                                                            "n_to_mn": "4_4_4_4", "n_to_m": "4_4_4_4_4"}}))
    return 0


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    vals = []
    desc = kind = ""
    # Each step is a bounded sample of the workload (about --cpu-seconds of CPU work; the one
    # 256x256 pair is indivisible for the reference code and takes ~2.5 s on one core).  The
    # whole run is kept within a few minutes by capping the number of steps actually timed;
    # the value is a rate (GFLOP/s over the samples), so fewer steps do not change its meaning.
    per_step = max(1.0, min(30.0, args.cpu_seconds))
    budget_s = 150.0
    steps_run = max(1, min(args.steps, int(budget_s / (per_step * 0.5 + 2.5))))
    warmups = min(args.warmup, 5)               # each costs >= 2.5 s: the one 256x256 pair cannot be cut
    for _ in range(warmups):
        cpu_baseline(min(per_step, 1.0), threads)
    t0 = time.perf_counter()
    for _ in range(steps_run):
        v, kind, desc = cpu_baseline(per_step, threads)
        vals.append(v)
    wall = time.perf_counter() - t0
    value = statistics.mean(vals)
    line = {
        "impl": "reference", "metric": "xcorr_gflops", "value": value, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": steps_run, "steps_requested": args.steps, "warmup": warmups,
        "warmup_requested": args.warmup,
        "ms_per_step": 1e3 * wall / steps_run, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "GFLOP/s", "cores": threads, "kind": kind,
                         "sample": desc + " (each step; result matrices split over host threads, "
                                          "each thread running the single-threaded reference loop)"},
        "e2e": {"value": value, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))
    return 0


def plan_signature(plan_text):
    """The part of a launch string that identifies the plan: kernel, grid, block, schedule, combine."""
    import re
    m = re.search(r"kernel=(\S+) grid=\((\d+),.*?block=\((\d+),", plan_text)
    sched = re.search(r"schedule=([a-z-]+)", plan_text)
    comb = re.search(r"combine=([a-z]+)", plan_text)
    if not m:
        return plan_text.split(" ")[0]
    return "%s/grid=%s/block=%s/%s/%s" % (m.group(1), m.group(2), m.group(3), sched.group(1) if sched else "-",
                                          comb.group(1) if comb else "-")


def workload_config(n_gpus):
    ws = sum(bytes_of(k) for k in CONFIGS)
    return {
        "workload": "one pass over the five BASELINE configurations per GPU: "
                    "C1 one_to_one 16x16; C2 one_to_one 256x256; C3 one_to_many 64x64 1x512; "
                    "C4 n_to_m 32x32 32x64; C5 n_to_mn 48x48 16x(128 each)",
        "sharding": "weak: every rank holds one configuration's worth of independent result matrices "
                    "(N*512 rights, N*32 lefts, N*16 left groups in total); no collective on the data path",
        "flop_per_step_per_gpu": sum(flop_of(k) for k in CONFIGS),
        "l2": f"no explicit flush: one pass reads and writes {ws / 1e6:.0f} MB, more than the 126 MB L2",
        "n_gpus": n_gpus,
    }


# ---- our arm -------------------------------------------------------------------------------------------
def bind_to_gpu_numa_node(device_index):
    """Pins this process to the CPUs of the NUMA node its GPU hangs off, before any page-locked
    buffer is allocated: with several ranks per host the device -> host copies of a rank then
    land in memory next to its GPU instead of crossing the socket link.  Returns what was done
    (for the JSON line); any missing piece (no NVML, no sysfs entry, one node) leaves the
    affinity as it is."""
    info = {"numa_node": None}
    try:
        import pynvml
        import torch
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
        bus = pynvml.nvmlDeviceGetPciInfo(handle).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        domain, rest = bus.lower().split(":", 1)
        path = f"/sys/bus/pci/devices/{domain[-4:]}:{rest}/numa_node"
        node = int(open(path).read().strip())
        info["numa_node"] = node
        if node >= 0:
            cpus = set()
            for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
            cpus &= os.sched_getaffinity(0)
            if cpus:
                os.sched_setaffinity(0, cpus)
                info["cpus"] = len(cpus)
    except Exception as e:                      # noqa: BLE001 -- best effort, never fatal
        info["note"] = f"{type(e).__name__}: {e}"[:120]
    return info


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the FFT-path and reference-GPU-kernel legs (short profiling runs)")
    ap.add_argument("--cpu-seconds", type=float, default=6.0)
    ap.add_argument("--grid", action="store_true",
                    help="run the sizes of the reference's benchmark file instead of the headline step")
    ap.add_argument("--grid-max-tflop", type=float, default=40.0)
    ap.add_argument("--only", default="", help="comma-separated subset of C1..C5 (profiling runs; "
                    "the default line always covers all five)")
    ap.add_argument("--hints", default="", help='JSON {"C3": {"overlap_rows": 4, ...}} or {"C1": {"kernel": "warp_per_overlap"}}: force plan hints of '
                    "a configuration (profiling and tuning runs; the default line uses automatic plans)")
    args = ap.parse_args()
    if args.only:
        keep = [k.strip() for k in args.only.split(",") if k.strip()]
        for k in list(CONFIGS):
            if k not in keep:
                del CONFIGS[k]
        if not CONFIGS:
            raise SystemExit("--only selected no configuration")
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.grid:
        return run_grid(args)

    import torch
    import torch.distributed as dist

    xc = load_package()
    xc.lib()                                   # raises if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU path")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    host_group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        host_group = dist.new_group(backend="gloo")     # barriers that keep waiting ranks off their GPUs
    warmup = max(3, args.warmup)
    stream = torch.cuda.current_stream().cuda_stream

    forced = {k: xc.make_hints(**{"kernel": "tile", **v}) for k, v in (json.loads(args.hints) if args.hints else {}).items()}

    # ---- resident inputs, outputs, workspaces
    dev = {}
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        left, right = config_inputs(k, rank)
        wsb = xc.workspace_bytes(mode, r, c, nl, nr, forced.get(k))
        dev[k] = dict(
            left=torch.from_numpy(left).cuda(), right=torch.from_numpy(right).cuda(),
            out=torch.empty(xc.out_shape(mode, r, c, nl, nr), dtype=torch.float32, device="cuda"),
            ws=torch.empty(max(wsb, 16), dtype=torch.uint8, device="cuda"), wsb=wsb)

    def launch(k):
        mode, r, c, nl, nr = CONFIGS[k]
        d = dev[k]
        xc.run_device(mode, d["left"].data_ptr(), d["right"].data_ptr(), d["out"].data_ptr(), r, c, nl, nr,
                      forced.get(k), d["ws"].data_ptr() if d["wsb"] else 0, d["wsb"], stream)

    def launch_on(k, stream_handle):
        mode, r, c, nl, nr = CONFIGS[k]
        d = dev[k]
        xc.run_device(mode, d["left"].data_ptr(), d["right"].data_ptr(), d["out"].data_ptr(), r, c, nl, nr,
                      forced.get(k), d["ws"].data_ptr() if d["wsb"] else 0, d["wsb"], stream_handle)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def host_barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=host_group)

    for _ in range(warmup):
        for k in CONFIGS:
            launch(k)
    plans = {}
    for k in CONFIGS:
        launch(k)
        plans[k] = xc.last_launch()
    torch.cuda.synchronize()

    # ---- timed region: K steps, one event pair around the region, one per launch
    ev = {k: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(args.steps)] for k in CONFIGS}
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    xc.reset_launch_count()
    e_start.record()
    for s in range(args.steps):
        for k in CONFIGS:
            a, b = ev[k][s]
            a.record()
            launch(k)
            b.record()
    e_stop.record()
    barrier()
    launches = xc.launch_count()
    region_ms = e_start.elapsed_time(e_stop)
    clocks = sampler.stop() if rank == 0 else None
    per_ms = {k: statistics.mean(a.elapsed_time(b) for a, b in ev[k]) for k in CONFIGS}
    per_min = {k: min(a.elapsed_time(b) for a, b in ev[k]) for k in CONFIGS}

    # ---- strong scaling of each shardable configuration: its own units split over the ranks
    strong_ms = {}
    if world > 1:
        for k, (mode, r, c, nl, nr) in CONFIGS.items():
            if mode == "one_to_one":
                continue
            first, count, a_nl, a_nr = strong_shard(xc, k, world, rank)
            if count == 0:
                strong_ms[k] = 0.0
                continue
            d = dev[k]

            def shard_launch():
                xc.run_device(mode, d["left"].data_ptr(), d["right"].data_ptr(), d["out"].data_ptr(),
                              r, c, a_nl, a_nr, None, 0, 0, stream)
            for _ in range(3):
                shard_launch()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(args.steps):
                shard_launch()
            b.record()
            barrier()
            strong_ms[k] = a.elapsed_time(b) / args.steps

    # ---- end to end through the host-buffer entry point (pinned host memory both ways)
    original_affinity = os.sched_getaffinity(0)
    host_affinity = bind_to_gpu_numa_node(local_rank)      # page-locked buffers next to this rank's GPU
    host = {}
    for k, (mode, r, c, nl, nr) in CONFIGS.items():
        left, right = config_inputs(k, rank)
        hl = torch.from_numpy(left).pin_memory()
        hr = torch.from_numpy(right).pin_memory()
        ho = torch.empty(xc.out_shape(mode, r, c, nl, nr), dtype=torch.float32).pin_memory()
        host[k] = (hl, hr, ho)
    lib = xc.lib()

    def e2e_pass():
        for k, (mode, r, c, nl, nr) in CONFIGS.items():
            hl, hr, ho = host[k]
            xc.check(lib.xcorr_run_host_f32(xc.MODES[mode], hl.data_ptr(), hr.data_ptr(), ho.data_ptr(),
                                            r, c, nl, nr, None, local_rank))
    # The same five problems as one batch call: the copies and kernels of a problem run under the
    # result copy of the one before.  Order: the problem whose first results are ready soonest
    # goes first, the two single pairs (tiny results) last, under the big result copies.
    batch_order = [k for k in ("C4", "C3", "C5", "C2", "C1") if k in CONFIGS]
    jobs = (xc.HostJob * len(batch_order))()
    for j, k in enumerate(batch_order):
        mode, r, c, nl, nr = CONFIGS[k]
        hl, hr, ho = host[k]
        jobs[j].mode, jobs[j].rows, jobs[j].cols, jobs[j].n_left, jobs[j].n_right = xc.MODES[mode], r, c, nl, nr
        jobs[j].h_left, jobs[j].h_right, jobs[j].h_out = hl.data_ptr(), hr.data_ptr(), ho.data_ptr()

    def e2e_batch_pass():
        xc.check(lib.xcorr_run_host_batch_f32(jobs, len(batch_order), local_rank))

    e2e_steps = max(3, min(args.steps, 10))

    def time_e2e(one_pass):
        for _ in range(2):
            one_pass()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            one_pass()
        return (time.perf_counter() - t0) * 1e3 / e2e_steps

    e2e_percall_ms = time_e2e(e2e_pass)
    for k in CONFIGS:
        host[k][2].zero_()
    e2e_ms = time_e2e(e2e_batch_pass)

    # ---- what the host links can carry: the same pinned bytes per step, copies only, all ranks at once
    copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()

    def copies_only():
        for k in CONFIGS:
            hl, hr, ho = host[k]
            with torch.cuda.stream(copy_in):
                dev[k]["left"].copy_(hl, non_blocking=True)
                dev[k]["right"].copy_(hr, non_blocking=True)
            with torch.cuda.stream(copy_out):
                ho.copy_(dev[k]["out"], non_blocking=True)
        copy_in.synchronize()
        copy_out.synchronize()
    link_ms = time_e2e(copies_only)

    # ---- the library's own multi-GPU call: rank 0 alone runs xcorr_run_host_sharded_f32 over all N
    #      devices on the fixed configurations; the other ranks wait on the host, off their GPUs
    sharded_api = {}
    if world > 1:
        host_barrier()
        if rank == 0:
            devs = (xc.C.c_int32 * world)(*range(world))
            for k, (mode, r, c, nl, nr) in CONFIGS.items():
                if mode == "one_to_one":
                    continue
                hl, hr, ho = host[k]

                def one_gpu():
                    xc.check(lib.xcorr_run_host_f32(xc.MODES[mode], hl.data_ptr(), hr.data_ptr(), ho.data_ptr(),
                                                    r, c, nl, nr, None, local_rank))

                def all_gpus():
                    xc.check(lib.xcorr_run_host_sharded_f32(xc.MODES[mode], hl.data_ptr(), hr.data_ptr(), ho.data_ptr(),
                                                            r, c, nl, nr, None, devs, world))
                res = {}
                for name, fn in (("ms_1gpu", one_gpu), ("ms_ngpu", all_gpus)):
                    for _ in range(2):
                        fn()
                    t0 = time.perf_counter()
                    for _ in range(e2e_steps):
                        fn()
                    res[name] = (time.perf_counter() - t0) * 1e3 / e2e_steps
                res["speedup"] = res["ms_1gpu"] / res["ms_ngpu"]
                res["gflops"] = flop_of(k) / (res["ms_ngpu"] * 1e-3) / 1e9
                sharded_api[k] = res
        host_barrier()
    last = list(CONFIGS)[-1]
    checksum = float(host[last][2].reshape(-1)[0])   # a device result read on the host
    barrier()

    os.sched_setaffinity(0, original_affinity)             # the CPU baseline uses every core again
    xc.check_device()          # no failed launch, no bounded device-side wait that gave up

    # ---- FFMA peak of this GPU, measured now
    ffma_flops, _ = xc.ffma_peak_probe(stream)

    # ---- max over ranks
    vec = max_over_ranks([region_ms, e2e_ms] + [per_ms[k] for k in CONFIGS] +
                         [strong_ms.get(k, 0.0) for k in CONFIGS] + [link_ms, e2e_percall_ms],
                         dist if world > 1 else None, "cuda")
    e2e_percall_ms = vec[-1]
    link_ms = vec[-2]
    region_ms, e2e_ms = vec[0], vec[1]
    per_ms_max = dict(zip(CONFIGS, vec[2:2 + len(CONFIGS)]))
    strong_max = dict(zip(CONFIGS, vec[2 + len(CONFIGS):2 + 2 * len(CONFIGS)]))

    if rank == 0:
        ms_per_step = region_ms / args.steps
        flop_step = sum(flop_of(k) for k in CONFIGS)
        value = world * flop_step / (ms_per_step * 1e-3) / 1e9
        peaks = {}
        mp = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(mp):
            peaks = json.load(open(mp))
        hbm_peak = peaks.get("hbm_gbs", 6650.0)
        sm_max = (clocks or {}).get("sm_max_mhz") or peaks.get("sm_max_mhz", 1965.0)
        nominal_peak = NOMINAL_SM * NOMINAL_LANES * 2 * sm_max * 1e6
        per_config = {}
        for k, (mode, r, c, nl, nr) in CONFIGS.items():
            t = per_ms_max[k] * 1e-3
            entry = {
                "mode": mode, "shape": f"{r}x{c} {nl}x{nr}", "ms": per_ms_max[k], "ms_min_rank0": per_min[k],
                "gflops": world * flop_of(k) / t / 1e9, "shifts_per_s": world * shifts_of(k) / t,
                "frac_ffma_measured": flop_of(k) / t / ffma_flops,
                "frac_ffma_nominal": flop_of(k) / t / nominal_peak,
                "hbm_gbs": bytes_of(k) / t / 1e9, "plan": plans[k],
            }
            if k in strong_ms:
                ts = strong_max[k] * 1e-3
                entry["strong"] = {"ms": strong_max[k], "gflops": flop_of(k) / ts / 1e9 if ts > 0 else None,
                                   "shifts_per_s": shifts_of(k) / ts if ts > 0 else None}
            per_config[k] = entry
        dom = max(CONFIGS, key=lambda k: per_ms_max[k])
        # DRAM bytes per launch of the dominant kernel: not measurable inside this run (it takes a
        # profiler); the committed capture's figure is given only when it was taken for the very plan
        # that ran now (profiles/dram_traffic.txt: configuration, bytes, plan signature)
        traffic, traffic_note = None, "no capture on file for this configuration"
        tp = os.path.join(ROOT, "profiles", "dram_traffic.txt")
        if os.path.exists(tp):
            for tl in open(tp):
                parts = tl.split(None, 2)
                if len(parts) == 3 and parts[0] == dom:
                    if parts[2].strip() == plan_signature(plans[dom]):
                        traffic = int(parts[1])
                        traffic_note = "ncu capture profiles/tile_kernel_%s.md, plan %s" % (dom, parts[2].strip())
                    else:
                        traffic_note = ("the capture on file is for plan %s, this run used %s: figure withheld"
                                        % (parts[2].strip(), plan_signature(plans[dom])))
        achieved = flop_of(dom) / (per_ms_max[dom] * 1e-3) / 1e12
        roofline = {
            "bound": "fp32_ffma", "kernel": plans[dom].split(" ")[0].replace("kernel=", "") + f" ({dom})",
            "achieved": achieved, "peak": ffma_flops / 1e12, "unit": "TFLOP/s",
            "frac": achieved / (ffma_flops / 1e12),
            "peak_source": "of measured: register-only FFMA probe on this GPU in this run "
                           f"(nominal 148 SM x 128 lanes x 2 x {sm_max:.0f} MHz = {nominal_peak / 1e12:.1f})",
            "traffic": traffic, "traffic_source": traffic_note,
            "hbm": {"achieved": bytes_of(dom) / (per_ms_max[dom] * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                    "frac": bytes_of(dom) / (per_ms_max[dom] * 1e-3) / 1e9 / hbm_peak,
                    "note": "compulsory bytes / time: far below the HBM roofline, the kernel is FFMA-bound"},
        }
        line = {
            "metric": "xcorr_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(world),
            "shifts_per_s": world * sum(shifts_of(k) for k in CONFIGS) / (ms_per_step * 1e-3),
            "frac_ffma_measured": flop_step / (ms_per_step * 1e-3) / ffma_flops,
            "ffma_peak_measured_tflops": ffma_flops / 1e12, "ffma_peak_nominal_tflops": nominal_peak / 1e12,
            "per_config": per_config, "roofline": roofline, "clocks": clocks,
            "e2e": {"value": world * flop_step / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": sum(4 * (CONFIGS[k][3] + CONFIGS[k][4]) * CONFIGS[k][1] * CONFIGS[k][2]
                                              for k in CONFIGS),
                    "d2h_bytes_per_step": sum(4 * shifts_of(k) for k in CONFIGS),
                    "api": "xcorr_run_host_batch_f32, the five configurations as one batch (order "
                           + ", ".join(batch_order) + "): pinned host in, H2D, kernels, D2H, pinned host out",
                    "per_call": {"value": world * flop_step / (e2e_percall_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                                 "ms_per_step": e2e_percall_ms,
                                 "api": "xcorr_run_host_f32, one call per configuration"},
                    "link_ceiling": {
                        "ms_per_step": link_ms,
                        "gbs": world * sum(bytes_of(k) for k in CONFIGS) / (link_ms * 1e-3) / 1e9,
                        "what": "the same pinned bytes per step, copies only (H2D and D2H on two streams), "
                                "all ranks at once, max over ranks"},
                    "frac_of_link_ceiling": link_ms / e2e_ms,
                    "host_affinity": host_affinity, "result_probe": checksum},
            "gpu_launches": int(launches),
        }
        if world == 1 and not args.no_extras:
            line["fft_path"] = fft_path_timings(xc, dev, stream, hbm_peak)
            line["f64_path"] = f64_path_timings(xc, dev, stream)
            for k, e in line["fft_path"].items():
                e["direct_ms"] = per_ms_max[k]
            ref_gpu = reference_gpu_baseline(dev, launch, launch_on=launch_on)
            if ref_gpu is not None:
                line["reference_gpu_kernels"] = ref_gpu
        if world == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            v, kind, desc = cpu_baseline(args.cpu_seconds, threads)
            v1, desc1 = cpu_single_thread()
            line["cpu_baseline"] = {"value": v, "unit": "GFLOP/s", "cores": threads, "kind": kind, "sample": desc,
                                    "single_thread": {"value": v1, "unit": "GFLOP/s", "threads": 1, "sample": desc1,
                                                      "note": "how the reference itself runs its CPU path"}}
        # last key of the line: the fixed-size (strong) figures in compact form
        summary = {"n_gpus": world, "e2e_ms": round(e2e_ms, 4), "link_ceiling_ms": round(link_ms, 4)}
        if world > 1:
            summary["strong"] = {
                k: {"ms_1gpu": round(per_ms_max[k], 4), "ms_ngpu": round(strong_max[k], 4),
                    "eff": round(per_ms_max[k] / (world * strong_max[k]), 3) if strong_max[k] > 0 else None}
                for k in strong_ms}
            summary["sharded_api"] = {k: {kk: round(vv, 4) for kk, vv in v.items()} for k, v in sharded_api.items()}
        line["scaling_summary"] = summary
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
