#!/usr/bin/env python
"""Benchmark of the INT4 linear GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload m8|c1..c5]
                    [--impl ours|reference|reference-gpu] [--scaling strong|weak]

One process per GPU (for N > 1 launch through torch.distributed.run); rank 0
prints ONE JSON line.  A step is one launch of the operator on seeded synthetic
operands (i.i.d. uniform [-8, 7], packed as the reference's utils/packer does).

Metric: INT4 GEMM TOPS = 2*M*N*K / t (the formula of the reference's
test/benchmark.cu:112-113), default workload M=N=K=8192.
  value     device-timed (CUDA events), operands resident in HBM, L2 flushed
            before every timed launch as test/benchmark.cu:93-96 does
  e2e       same metric through the host-buffer C-ABI entry point: pinned host
            operands up, launch, result down, every step
  roofline  achieved TOPS of the kernel against an 8-bit tensor rate MEASURED in
            this run (a library int8 GEMM and this library's own byte GEMM on
            resident operands, whichever is faster), or GB/s against the
            measured HBM copy rate for the decode shape
  configs   (1 GPU) a short event-timed figure for each of the five benchmark
            configurations and for the decode shape with 32, 64 and 128 rows,
            outside `value`
  cpu_baseline  the reference's own CPU GEMM on a bounded row sample

With N > 1 ranks the weight matrix is sharded along N: every rank holds the
full X and its own rows of W and produces its own columns of Y; no collective is
on the data path.  --scaling strong (default) splits the workload's own N across
the ranks, so the problem is the same at every N; --scaling weak gives every
rank the workload's N (the problem grows with N, and the metric string says so).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M, N, K, bound)
    "c1": (1024, 1024, 1024, "tensor"),
    "c2": (4096, 4096, 4096, "tensor"),
    "c3": (4096, 4096, 8192, "tensor"),
    "c4": (16, 14336, 4096, "hbm"),
    "c5": (8192, 28672, 8192, "tensor"),
    "m8": (8192, 8192, 8192, "tensor"),
    # the decode shape c4 with a batch of 32, 64 and 128 rows (not BASELINE configurations: the shapes
    # between the decode kernels and full 128-row tiles)
    "d32": (32, 14336, 4096, "hbm"),
    "d64": (64, 14336, 4096, "hbm"),
    "d128": (128, 14336, 4096, "hbm"),
}
NOMINAL_INT8_TOPS = 4500.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
L2_BYTES = 126e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return p, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def ncu_traffic(workload):
    """DRAM bytes per launch from the committed ncu capture, if one exists."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get(workload)
    return None


def describe_config(workload, world, scaling, variant="default"):
    """The `config` object of the JSON line -- the same for this library's arm and the reference
    arm, because it describes the WORK (shape, how it is sharded, how caches are treated), not the
    implementation."""
    m, n_work, k, bound = WORKLOADS[workload]
    n_total = n_work if scaling == "strong" else n_work * world
    n_local = n_total // world
    return {"workload": f"{workload}: M={m} N={n_total} K={k}",
            "shard": f"{world} x (M={m}, N={n_local}, K={k}), W and Y split along N, X replicated",
            "l2": ("256 MiB flush write before every timed launch" if bound == "tensor"
                   else "rotating copies of W, together larger than L2"),
            "variant": variant}


def metric_name(workload, world, scaling):
    m, n_work, k, bound = WORKLOADS[workload]
    n_total = n_work if scaling == "strong" else n_work * world
    return (f"INT4 GEMM TOPS at M={m} N={n_total} K={k}" if bound == "tensor"
            else f"INT4 GEMM achieved HBM GB/s at M={m} N={n_total} K={k}")


class ClockSampler:
    """Reads SM clock and clock-event (throttle) reasons through NVML every few milliseconds while
    the timed region runs.  Read-only: nothing about the GPU is changed."""

    REASONS = {
        "hw_slowdown": 0x0000000000000008,
        "sw_power_cap": 0x0000000000000004,
        "hw_thermal_slowdown": 0x0000000000000040,
        "sw_thermal_slowdown": 0x0000000000000020,
    }

    def __init__(self, index, period_s=0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.stop_flag = threading.Event()
        self.thread = None
        self.max_mhz = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for name, bit in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": []}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "samples": len(self.samples), "reasons": sorted(self.reasons)}


def cpu_reference_sample(m, n, k, seconds_target=15.0):
    """Times the reference's CPU GEMM (test/test_correctness.cu:12-19) on rows 0..R-1 of
    the workload, R sized for about `seconds_target` seconds.  Uses the reference's own
    compiled function when oracle/_ref is there (one call per thread on its own row
    block, all host cores), else the C restatement with OpenMP."""
    import ctypes
    from concurrent.futures import ThreadPoolExecutor
    from int4linear_b200 import uniform_s4
    from oracle import oracle as O

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    w = np.ascontiguousarray(uniform_s4(0xB008, n, k).astype(np.int32))
    ref = O.ref_lib()
    kind = "reference" if ref is not None else "port"

    def run(rows_per_thread):
        rows = rows_per_thread * cores
        x = np.ascontiguousarray(uniform_s4(0xA008, rows, k).astype(np.int32))
        y = np.empty((rows, n), dtype=np.int32)
        t0 = time.perf_counter()
        if ref is not None:
            ip = ctypes.POINTER(ctypes.c_int)

            def job(t):
                xs, ys = x[t * rows_per_thread:(t + 1) * rows_per_thread], y[t * rows_per_thread:(t + 1) * rows_per_thread]
                ref.ref_linear_ref(xs.ctypes.data_as(ip), w.ctypes.data_as(ip), ys.ctypes.data_as(ip),
                                   rows_per_thread, n, k)
            with ThreadPoolExecutor(cores) as ex:
                list(ex.map(job, range(cores)))
        else:
            y[:] = O.linear_ref(x, w)
        return rows, time.perf_counter() - t0

    rows, dt = run(1)
    per_row_block = dt
    reps = max(1, min(int(seconds_target / max(per_row_block, 1e-3)), max(1, m // cores)))
    if reps > 1:
        rows, dt = run(reps)
    tops = 2.0 * rows * n * k / dt / 1e12
    return {"value": tops, "unit": "TOPS", "cores": cores, "kind": kind,
            "sample": f"rows 0..{rows - 1} of M={m} (N={n}, K={k}), {rows // cores} rows per thread, {dt:.1f} s"}


def reference_gpu_kernel(m, n, k, steps, warmup):
    """The reference's own kernel (cp.async + ldmatrix + mma.sync m16n8k64 s4,
    kernels/linear_v21.h) built for sm_100a from its unmodified sources into oracle/_ref, timed
    with the method of test/benchmark.cu.  None when that build or a GPU is not there."""
    try:
        import torch
        from int4linear_b200 import uniform_s4_packed
        from oracle import oracle as O
        ref = O.ref_lib()
        if ref is None or not torch.cuda.is_available():
            return None
        torch.cuda.set_device(0)
        dev = torch.device("cuda:0")
        xd = torch.from_numpy(uniform_s4_packed(0xA008, m, k)).to(dev)
        wd = torch.from_numpy(uniform_s4_packed(0xB008, n, k)).to(dev)
        yd = torch.empty((m, n), dtype=torch.int32, device=dev)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for _ in range(max(3, warmup)):
            ref.ref_linear_v21_launch(xd.data_ptr(), wd.data_ptr(), yd.data_ptr(), m, n, k)
        times = []
        for _ in range(steps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            ref.ref_linear_v21_launch(xd.data_ptr(), wd.data_ptr(), yd.data_ptr(), m, n, k)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = sum(times) / len(times)
        return {"value": 2.0 * m * n * k / (ms * 1e-3) / 1e12, "unit": "TOPS", "ms_per_step": ms, "steps": steps,
                "kernel": "reference linear_v21 (mma.sync m16n8k64 s4) built unmodified for sm_100a"}
    except Exception as e:  # a comparison figure only: never let it take the line down
        return {"unavailable": repr(e)[:200]}


def measure_int8_peak(torch, L, dev, launches=10):
    """The 8-bit tensor rate this GPU delivers, measured here and now on resident operands
    (M=N=K=8192, best of `launches`, CUDA events): a library int8 GEMM (torch._int_mm) and this
    library's own byte GEMM (TMA -> tcgen05.mma kind::i8, no unpack stage).  Measurement only:
    neither is on the operator's path."""
    n = 8192
    out = {"shape": f"M=N=K={n}", "launches": launches,
           "data": "bytes = 16 x uniform s4, i.e. exactly what the operator's tensor-core stage multiplies "
                   "(a part at its power limit runs full-range random bytes slower; that figure is given too)"}
    g = torch.Generator(device=dev)
    g.manual_seed(0x18)
    a = (torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev, generator=g) * 16).contiguous()
    b = (torch.randint(-8, 8, (n, n), dtype=torch.int8, device=dev, generator=g) * 16).contiguous()
    ops = 2.0 * n * n * n

    def best(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(launches):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return ops / (min(ts) * 1e-3) / 1e12

    try:
        bt = b.t()  # column-major second operand, as the library call wants it
        out["library_int8_gemm_tops"] = best(lambda: torch._int_mm(a, bt))
    except Exception as e:
        out["library_int8_gemm_tops"] = None
        out["library_int8_gemm_error"] = repr(e)[:160]
    try:
        y = torch.empty((n, n), dtype=torch.int32, device=dev)
        au, bu = a.view(torch.uint8), b.view(torch.uint8)
        out["own_byte_gemm_tops"] = best(lambda: L.linear_expanded(au, bu, out=y))
    except Exception as e:
        out["own_byte_gemm_tops"] = None
        out["own_byte_gemm_error"] = repr(e)[:160]
    try:
        a2 = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev, generator=g)
        b2 = torch.randint(-128, 128, (n, n), dtype=torch.int8, device=dev, generator=g)
        b2t = b2.t()
        out["library_int8_gemm_tops_full_range_bytes"] = best(lambda: torch._int_mm(a2, b2t))
    except Exception:
        out["library_int8_gemm_tops_full_range_bytes"] = None
    cands = [v for v in (out["library_int8_gemm_tops"], out["own_byte_gemm_tops"],
                         out["library_int8_gemm_tops_full_range_bytes"]) if v]
    out["peak_tops"] = max(cands) if cands else None
    return out


def device_operands(torch, dev, rows, k, seed):
    """Packed operand made on the device: every byte uniform in 0..255 is two i.i.d. uniform
    signed nibbles in [-8, 7] (seeded)."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return torch.randint(0, 256, (rows, k // 2), dtype=torch.uint8, device=dev, generator=g)


def graph_replay_ms(torch, L, launch_fns, overlap=0):
    """Captures the given launches into one CUDA graph and times one replay (ms for all)."""
    L.set_overlap(overlap)
    try:
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for fn in launch_fns:
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)
    finally:
        L.set_overlap(0)


def quick_config(torch, L, dev, flush, name, int8_peak, hbm_peak, launches=5):
    """A short figure for one benchmark configuration: `launches` event-timed launches after an L2
    flush each (median); microsecond-scale shapes also as a CUDA-graph replay over rotating operand
    sets larger than L2; the decode shape with its launch-overlap modes and the read-only floor."""
    from int4linear_b200 import _lib
    m, n, k, bound = WORKLOADS[name]
    xd = device_operands(torch, dev, m, k, 0xA100 + m % 251)
    wd = device_operands(torch, dev, n, k, 0xB100 + n % 251)
    yd = torch.empty((m, n), dtype=torch.int32, device=dev)
    ops = 2.0 * m * n * k
    nbytes = m * k // 2 + n * k // 2 + 4 * m * n
    out = {"M": m, "N": n, "K": k, "bound": bound,
           "kernel_path": {1: "tcgen05", 2: "legacy", 3: "skinny"}[L.path_for(m, n, k)]}
    for _ in range(3):
        L.linear(xd, wd, out=yd)
    torch.cuda.synchronize()
    ts = []
    for _ in range(launches):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        L.linear(xd, wd, out=yd)
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ms = statistics.median(ts)
    out["event_timed"] = {"ms": ms, "tops": ops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9,
                          "note": f"median of {launches} launches, 256 MiB L2 flush before each"}
    best_ms = ms
    if nbytes < 64e6:
        sets = int(2 * L2_BYTES // nbytes) + 1
        xs = [xd] + [xd.clone() for _ in range(sets - 1)]
        ws = [wd] + [wd.clone() for _ in range(sets - 1)]
        ys = [yd] + [torch.empty_like(yd) for _ in range(sets - 1)]
        reps = 4 * sets
        fns = [(lambda i=i: L.linear(xs[i % sets], ws[i % sets], out=ys[i % sets])) for i in range(reps)]
        gms = graph_replay_ms(torch, L, fns) / reps
        out["graph_replay"] = {"ms": gms, "tops": ops / (gms * 1e-3) / 1e12, "gbs": nbytes / (gms * 1e-3) / 1e9,
                               "note": f"{reps} launches in one CUDA graph over {sets} rotating operand sets (> L2)"}
        best_ms = min(best_ms, gms)
        if bound == "hbm":
            for mode in (1, 2):
                oms = graph_replay_ms(torch, L, fns, overlap=mode) / reps
                out[f"overlap_{mode}"] = {"ms": oms, "gbs": nbytes / (oms * 1e-3) / 1e9,
                                          "frac_of_hbm_peak": nbytes / (oms * 1e-3) / 1e9 / hbm_peak}
            # floor for one launch: a read-only streaming pass over the same weight bytes
            sink = torch.zeros(1, dtype=torch.int32, device=dev)
            lib = _lib.load()
            fl = [(lambda i=i: lib.int4_linear_probe_stream_read(ws[i % sets].data_ptr(), ws[i % sets].numel(), sink.data_ptr(),
                                                                   torch.cuda.current_stream().cuda_stream)) for i in range(reps)]
            fms = graph_replay_ms(torch, L, fl) / reps
            out["read_only_floor"] = {"ms": fms, "gbs": (n * k // 2) / (fms * 1e-3) / 1e9,
                                      "note": "one launch of a read-only streaming kernel over the same W bytes"}
    if bound == "tensor":
        # for scale: a library int8 GEMM of the same shape on resident bytes (measurement only)
        try:
            g = torch.Generator(device=dev)
            g.manual_seed(0x19)
            a8 = (torch.randint(-8, 8, (m, k), dtype=torch.int8, device=dev, generator=g) * 16).contiguous()
            b8 = (torch.randint(-8, 8, (n, k), dtype=torch.int8, device=dev, generator=g) * 16).contiguous().t()
            for _ in range(2):
                torch._int_mm(a8, b8)
            ls = []
            for _ in range(launches):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                torch._int_mm(a8, b8)
                e1.record()
                torch.cuda.synchronize()
                ls.append(e0.elapsed_time(e1))
            out["library_int8_gemm_same_shape_tops"] = ops / (statistics.median(ls) * 1e-3) / 1e12
            del a8, b8
        except Exception as e:
            out["library_int8_gemm_same_shape_tops"] = None
        tops = ops / (best_ms * 1e-3) / 1e12
        out["tops"] = tops
        out["frac_of_measured_int8_peak"] = tops / int8_peak if int8_peak else None
        out["frac_of_nominal_int8_4500"] = tops / NOMINAL_INT8_TOPS
    else:
        gbs = nbytes / (best_ms * 1e-3) / 1e9
        out["gbs"] = gbs
        out["frac_of_hbm_peak"] = gbs / hbm_peak
        if "overlap_2" in out:
            out["frac_of_hbm_peak_overlapped"] = out["overlap_2"]["frac_of_hbm_peak"]
    return out


SWEEP_SHAPES = ["1024x1024x1024", "2048x2048x2048", "2048x2048x1024", "512x4096x4096", "256x8192x4096",
                "1024x4096x1024", "128x14336x4096", "64x14336x4096", "4096x4096x4096", "4096x1024x4096",
                "3072x3072x3072", "1536x6144x2048", "8192x1024x1024"]


def tile_sweep(shapes, launches=40):
    """Times the tile configurations of the tensor-memory GEMM (CTA pairs; single-CTA tiles 256, 128
    and 64 columns wide; the dispatcher's own choice) on the given MxNxK shapes, each as a CUDA graph of
    `launches` launches over rotating operand sets larger than L2.  The relative tile times are what
    the dispatcher's cost model (launch_tcgen05 in csrc/gemm_tcgen05.cu) is fitted to.  Prints one JSON
    line: {"tile_sweep_us": {shape: {config: microseconds per launch}}}."""
    import torch
    import int4linear_b200 as L
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    configs = {"auto": (0, -1), "pairs": (0, 1), "c256": (256, 0), "c128": (128, 0), "c64": (64, 0)}
    table = {}
    for shape in shapes:
        m, n, k = (int(v) for v in shape.lower().split("x"))
        nbytes = m * k // 2 + n * k // 2 + 4 * m * n
        sets = min(64, int(2 * L2_BYTES // nbytes) + 1)
        xs = [device_operands(torch, dev, m, k, 1 + i) for i in range(sets)]
        ws = [device_operands(torch, dev, n, k, 101 + i) for i in range(sets)]
        ys = [torch.empty((m, n), dtype=torch.int32, device=dev) for _ in range(sets)]
        row = {}
        try:
            for name, (tile, pairs) in configs.items():
                if name == "pairs" and m <= 128:
                    continue  # a lone row block would leave the second CTA of a pair idle
                L.set_tuning(tile, False, pairs)
                L.linear(xs[0], ws[0], out=ys[0])  # the library's first call must not happen inside a capture
                torch.cuda.synchronize()
                fns = [(lambda i=i: L.linear(xs[i % sets], ws[i % sets], out=ys[i % sets])) for i in range(launches)]
                row[name] = round(graph_replay_ms(torch, L, fns) / launches * 1e3, 2)
        finally:
            L.set_tuning(0, False, -1)
        best = min((v, name) for name, v in row.items() if name != "auto")
        row["best"] = best[1]
        row["auto_over_best"] = round(row["auto"] / best[0], 3)
        table[shape] = row
        del xs, ws, ys
        torch.cuda.empty_cache()
    print(json.dumps({"tile_sweep_us": table}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="m8", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"])
    ap.add_argument("--path", default="auto", choices=["auto", "tcgen05", "legacy", "skinny"],
                    help="force one kernel family of this library (default: shape dispatch)")
    ap.add_argument("--variant", default="default", choices=["default", "two-pass", "prepared"],
                    help="opt-in variants of the tensor-memory path: expand pre-pass + byte GEMM, weights "
                         "pre-expanded outside the timed region")
    ap.add_argument("--tail", default="auto", choices=["auto", "none", "half", "kcut"],
                    help="how a last, partial wave of tiles is run (int4_linear_set_tail)")
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration figures (1 GPU)")
    ap.add_argument("--no-peak", action="store_true", help="skip the int8 tensor-rate measurement")
    ap.add_argument("--gather", action="store_true", help="also time an NCCL all-gather of Y (N > 1)")
    ap.add_argument("--tile-sweep", nargs="*", metavar="MxNxK", default=None,
                    help="instead of the benchmark: time every tile configuration on these shapes (1 GPU)")
    args = ap.parse_args()
    if args.tile_sweep is not None:
        tile_sweep(args.tile_sweep or SWEEP_SHAPES)
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m, n_work, k, bound = WORKLOADS[args.workload]

    if args.impl == "reference":
        # The reference's own CPU implementation of the path on the host cores; one rank does it.
        if rank != 0:
            return
        gpus = max(1, args.gpus)
        n_ref = n_work if args.scaling == "strong" else n_work * gpus
        cb = cpu_reference_sample(m, n_ref, k, seconds_target=max(5.0, min(60.0, 4.0 * args.steps)))
        line = {"impl": "reference", "metric": metric_name(args.workload, gpus, args.scaling),
                "value": cb["value"], "unit": "TOPS",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": None, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "s4 x s4 -> s32 (int32 arithmetic on the CPU)",
                "data": "synthetic", "config": describe_config(args.workload, gpus, args.scaling),
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                # for scale: what the reference's GPU kernel itself does on this box (not this arm's value)
                "reference_gpu_kernel": reference_gpu_kernel(m, n_work, k, steps=3, warmup=3)}
        print(json.dumps(line))
        return

    if args.impl == "reference-gpu":
        # The north star's path (b): the reference's own kernel recompiled for sm_100a from its
        # unmodified sources, timed with the same method.  A comparison arm, not this library.
        if rank != 0:
            return
        r = reference_gpu_kernel(m, n_work, k, steps=args.steps, warmup=args.warmup)
        if r is None or "unavailable" in r:
            print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref was not built (needs the reference checkout)"
                              if r is None else r["unavailable"]}))
            return
        print(json.dumps({"impl": "reference-gpu", "metric": f"INT4 GEMM TOPS at M={m} N={n_work} K={k}", "value": r["value"],
                          "unit": "TOPS", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
                          "ms_per_step": r["ms_per_step"], "higher_is_better": True, "data": "synthetic",
                          "config": dict(describe_config(args.workload, 1, "strong"), kernel=r["kernel"])}))
        return

    import torch
    import torch.distributed as dist
    import int4linear_b200 as L
    from int4linear_b200 import numa

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    # Run on the CPUs next to this GPU before any host buffer is allocated and pinned (first touch).
    bus = numa.torch_pci_bus_id(local_rank)
    all_cpus = os.sched_getaffinity(0) if hasattr(os, "sched_getaffinity") else None
    numa_info = numa.bind_to_gpu_node(bus) if bus else {"node": None, "cpus": 0, "bound": False}
    L.set_path({"auto": L.PATH_AUTO, "tcgen05": L.PATH_TCGEN05, "legacy": L.PATH_LEGACY,
                "skinny": L.PATH_SKINNY}[args.path])
    L.set_tail({"auto": -1, "none": 0, "half": 1, "kcut": 2}[args.tail])
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    # ---- shard of the weight matrix this rank owns
    if args.scaling == "strong":
        n_total = n_work
        n_local = n_total // world
    else:
        n_local = n_work
        n_total = n_work * world
    row_start = rank * n_local
    xp = L.uniform_s4_packed(0xA008, m, k)
    wp = L.uniform_s4_packed(0xB008, n_local, k, row_start=row_start)
    xd = torch.from_numpy(xp).to(dev)
    wd = torch.from_numpy(wp).to(dev)
    yd = torch.empty((m, n_local), dtype=torch.int32, device=dev)

    # For the microsecond-scale decode shape each timed launch gets its own copy of W so that
    # it streams from HBM, not from L2.
    rotate = bound == "hbm"
    w_copies = [wd]
    if rotate:
        copies = max(2, int(2 * L2_BYTES // wp.nbytes) + 1)
        w_copies = [wd] + [wd.clone() for _ in range(copies - 1)]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    if args.variant == "two-pass":
        L.set_two_pass(1)
    w_prepared = L.prepare_weights(wd) if args.variant == "prepared" else None

    def step(i):
        if w_prepared is not None:
            L.linear_prepared(xd, w_prepared, out=yd)
        else:
            L.linear(xd, w_copies[i % len(w_copies)], out=yd)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    if L.last_status() != 0:
        raise SystemExit("device-side failure during warm-up")

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = L.launch_count()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    pipelined = None
    step_ms = None
    if rotate:
        # A single ~5 us launch is below what an event pair (or a Python call) resolves, so the K
        # steps are captured into one CUDA graph -- K launches, each on its own copy of W -- and
        # the replay is timed as a whole.  `value` is measured with ordinary launches (each waits
        # for the previous one); the same graph is then re-captured with the library's launch
        # overlap modes (programmatic dependent launch) and reported under "pipelined".
        fns = [(lambda i=i: step(i)) for i in range(args.steps)]
        flush.zero_()
        total_ms = graph_replay_ms(torch, L, fns)
        pipelined = {f"overlap_{mode}": graph_replay_ms(torch, L, fns, overlap=mode) / args.steps for mode in (1, 2)}
        launches = args.steps  # the timed replay ran the K captured launches
    else:
        # Three more untimed steps queued directly in front of the timed ones: the host work between
        # the warm-up and here (barrier, sampler thread) leaves the GPU idle long enough to drop its
        # clocks, and the first timed launch would otherwise pay for the ramp.
        for i in range(3):
            flush.zero_()
            step(i)
        launches0 = L.launch_count()
        for i in range(args.steps):
            flush.zero_()  # evict operands and result from L2 (test/benchmark.cu:93-96)
            starts[i].record()
            step(i)
            ends[i].record()
        barrier()
        step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
        total_ms = sum(step_ms)
        launches = L.launch_count() - launches0
    # Second figure for the tensor-bound shapes: the same K launches back to back, no flush between
    # them (meaningful only where operands + result exceed L2, as the layers of a model would run).
    back_to_back = None
    b2b_note = "same launches without the L2 flush between them; working set > 2 x L2"
    ws_bytes = m * k // 2 + n_local * k // 2 + 4 * m * n_local
    if not rotate and w_prepared is None:
        # Working sets that fit twice into L2 (the shards of a strong-scaled run) rotate over enough
        # copies of X, W and Y to exceed it, so that no launch finds its operands cached.
        sets = 1 if ws_bytes > 2 * L2_BYTES else int(2 * L2_BYTES // ws_bytes) + 1
        if sets > 1:
            b2b_note = f"launches back to back over {sets} rotating sets of X, W and Y ({sets * ws_bytes >> 20} MiB > L2), no flush"
        xs = [xd] + [xd.clone() for _ in range(sets - 1)]
        ws_ = [wd] + [wd.clone() for _ in range(sets - 1)]
        ys = [yd] + [torch.empty_like(yd) for _ in range(sets - 1)]
        reps = max(args.steps, 2 * sets)
        for i in range(sets):
            L.linear(xs[i], ws_[i], out=ys[i])
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.zero_()
        barrier()
        b0.record()
        for i in range(reps):
            L.linear(xs[i % sets], ws_[i % sets], out=ys[i % sets])
        b1.record()
        barrier()
        back_to_back = max_over_ranks(b0.elapsed_time(b1) / reps)
        del xs, ws_, ys
    # Microsecond-scale tensor shapes (c1): one launch is comparable with the launch overhead an
    # event pair sees, so the K launches are also timed as one CUDA-graph replay over rotating
    # copies of X, W and Y that together exceed L2.
    graph_replay = None
    if not rotate and ws_bytes < 32e6 and world == 1:
        sets = int(2 * L2_BYTES // ws_bytes) + 1
        xs = [xd] + [xd.clone() for _ in range(sets - 1)]
        ws_ = [wd] + [wd.clone() for _ in range(sets - 1)]
        ys = [yd] + [torch.empty_like(yd) for _ in range(sets - 1)]
        per = graph_replay_ms(torch, L, [(lambda i=i: L.linear(xs[i % sets], ws_[i % sets], out=ys[i % sets]))
                                         for i in range(args.steps)]) / args.steps
        graph_replay = {"ms_per_step": per, "value": 2.0 * m * n_local * k / (per * 1e-3) / 1e12, "unit": "TOPS",
                        "note": f"{args.steps} launches in one CUDA graph over {sets} rotating operand sets "
                                f"({sets * ws_bytes / 2**20:.0f} MiB > L2)"}
    clocks = sampler.stop() if rank == 0 else None
    if L.last_status() != 0:
        raise SystemExit("device-side failure during the timed region")

    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps
    ops = 2.0 * m * n_total * k
    tops = ops / (ms_per_step * 1e-3) / 1e12
    alg_bytes_local = m * k // 2 + n_local * k // 2 + 4 * m * n_local
    gbs = alg_bytes_local * world / (ms_per_step * 1e-3) / 1e9

    # ---- N > 1: the largest configuration (c5) strong-scaled the same way, as a second figure,
    # and a correctness check of the gathering GEMM against the NCCL all-gather on a small shape.
    strong_c5 = None
    gather_check = None
    if world > 1 and args.workload == "m8" and args.variant == "default":
        cm, cn, ck, _ = WORKLOADS["c5"]
        cn_local = cn // world
        cx = device_operands(torch, dev, cm, ck, 0xA5C5)
        cw = device_operands(torch, dev, cn_local, ck, 0xB5C5 + rank)
        cy = torch.empty((cm, cn_local), dtype=torch.int32, device=dev)
        for _ in range(3):
            L.linear(cx, cw, out=cy)
        barrier()
        cts = []
        for _ in range(5):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            L.linear(cx, cw, out=cy)
            e1.record()
            torch.cuda.synchronize()
            cts.append(e0.elapsed_time(e1))
        barrier()
        cms = max_over_ranks(sum(cts) / len(cts))
        strong_c5 = {"metric": f"INT4 GEMM TOPS at M={cm} N={cn} K={ck}", "scaling": "strong",
                     "shard": f"{world} x (M={cm}, N={cn_local}, K={ck})", "ms_per_step": cms, "steps": 5,
                     "value": 2.0 * cm * cn * ck / (cms * 1e-3) / 1e12, "unit": "TOPS",
                     "per_gpu_tops": 2.0 * cm * cn_local * ck / (cms * 1e-3) / 1e12,
                     "note": "max over ranks of the mean of 5 event-timed launches, L2 flushed before each"}
        del cx, cw, cy
        gm, gn, gk = 512, 256 * world, 512
        ok, err = 0.0, None
        try:
            from int4linear_b200.sharding import ShardedInt4Linear, shard_bounds
            sh = shard_bounds(gn, world, rank)
            gx = device_operands(torch, dev, gm, gk, 0xA6C6)
            gw = device_operands(torch, dev, gn, gk, 0xB6C6)[sh.row_start:sh.row_start + sh.rows].contiguous()
            layer = ShardedInt4Linear(gw, gn, gk)
            fused = layer.forward(gx, gather="fused").clone()
            torch.cuda.synchronize()
            plain = layer.forward(gx, gather=True)
            ok = 1.0 if torch.equal(fused, plain) else 0.0
        except Exception as e:  # every rank still takes part in the reduction below
            err = repr(e)[:200]
        same = torch.tensor([ok], dtype=torch.float64, device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        gather_check = {"shape": f"M={gm} N={gn} K={gk}", "fused_equals_all_gather": bool(same.item() == 1.0)}
        if err:
            gather_check["error"] = err

    # ---- optional: all-gather of the Y shards (reported separately, never in `value`)
    gather_ms = None
    gather_cmp = None
    if args.gather and world > 1:
        out = torch.empty((world, m, n_local), dtype=torch.int32, device=dev)
        for _ in range(2):
            dist.all_gather_into_tensor(out, yd)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            dist.all_gather_into_tensor(out, yd)
        e1.record()
        barrier()
        gather_ms = max_over_ranks(e0.elapsed_time(e1) / 5)

        # GEMM followed by the all-gather, against the GEMM whose epilogue stores straight into
        # every rank's full-width Y over NVLink (plus the device-side rank barriers around it).
        from int4linear_b200.sharding import FusedGatherBuffer, Shard

        def timed(fn, reps=5):
            for _ in range(2):
                fn()
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            barrier()
            return max_over_ranks(a.elapsed_time(b) / reps)

        def unfused():
            L.linear(xd, wd, out=yd)
            dist.all_gather_into_tensor(out, yd)

        fused_buf = FusedGatherBuffer(m, n_total, dev)
        shard = Shard(rank, world, row_start, n_local)
        unfused_ms = timed(unfused)
        fused_ms = timed(lambda: fused_buf.run(xd, wd, shard, k))
        same = torch.equal(fused_buf.y.view(m, world, n_local), out.permute(1, 0, 2))
        gather_cmp = {"gemm_then_all_gather_ms": unfused_ms, "fused_gather_ms": fused_ms,
                      "fused_equals_all_gather": bool(same)}

    # ---- end to end through the host-buffer entry point
    e2e = None
    if not args.no_e2e:
        xh = torch.from_numpy(xp).pin_memory()
        wh = torch.from_numpy(wp).pin_memory()
        yh = torch.empty((m, n_local), dtype=torch.int32).pin_memory()
        xn, wn, yn = xh.numpy(), wh.numpy(), yh.numpy()
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(2):
            L.linear_host(xn, wn, k, out=yn)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            L.linear_host(xn, wn, k, out=yn)
        torch.cuda.synchronize()
        dt = max_over_ranks(time.perf_counter() - t0) / e2e_steps
        # The legs by themselves, all ranks at once: what the host's links give N ranks together.
        xdev, ydev = torch.empty_like(xd), torch.empty_like(yd)
        legs = {}
        for name, fn in (("h2d_x", lambda: xdev.copy_(xh, non_blocking=True)), ("d2h_y", lambda: yh.copy_(ydev, non_blocking=True))):
            fn()
            barrier()
            l0 = time.perf_counter()
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            legs[name + "_ms"] = max_over_ranks(time.perf_counter() - l0) / 3 * 1e3
        legs["h2d_x_gbs_all_ranks"] = xp.nbytes * world / (legs["h2d_x_ms"] * 1e-3) / 1e9
        legs["d2h_y_gbs_all_ranks"] = yn.nbytes * world / (legs["d2h_y_ms"] * 1e-3) / 1e9
        del xdev, ydev
        e2e = {"value": (ops / dt / 1e12) if bound == "tensor" else (alg_bytes_local * world / dt / 1e9),
               "unit": "TOPS" if bound == "tensor" else "GB/s",
               "h2d_bytes_per_step": int(xp.nbytes + wp.nbytes), "d2h_bytes_per_step": int(yn.nbytes),
               "ms_per_step": dt * 1e3, "steps": e2e_steps,
               "host_numa": numa_info, "legs_alone": legs,
               "note": "per rank: X and this rank's rows of W uploaded from pinned host memory and this rank's "
                       "columns of Y downloaded, every step; max over ranks"}

    if all_cpus is not None and numa_info.get("bound"):
        os.sched_setaffinity(0, all_cpus)  # the CPU baseline below uses every core again
    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0: denominators, per-configuration figures, the JSON line
    peaks, peak_kind = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    int8 = None if args.no_peak else measure_int8_peak(torch, L, dev)
    int8_peak = int8["peak_tops"] if int8 and int8.get("peak_tops") else None
    if bound == "tensor":
        per_gpu = tops / world
        if int8_peak:
            peak = int8_peak
            lib_t, own_t = int8["library_int8_gemm_tops"], int8["own_byte_gemm_tops"]
            basis = ("8-bit tensor rate measured in this run on this GPU (M=N=K=8192, resident operands, best of "
                     f"{int8['launches']} launches): the faster of a library int8 GEMM ({lib_t and round(lib_t)} TOPS) "
                     f"and this library's byte GEMM without an unpack stage ({own_t and round(own_t)} TOPS)")
        else:
            peak = 2.0 * float(peaks["bf16_tflops"])
            basis = f"2 x dense bf16 burst of {peak_kind} ({peaks['bf16_tflops']} TFLOP/s): no int8 figure was measured in this run"
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TOPS",
                    "frac": per_gpu / peak, "peak_basis": basis,
                    "frac_of_nominal_int8_4500": per_gpu / NOMINAL_INT8_TOPS,
                    "frac_of_2x_measured_bf16_burst": per_gpu / (2.0 * float(peaks["bf16_tflops"])),
                    "traffic": ncu_traffic(args.workload)}
        value, unit = tops, "TOPS"
    else:
        per_gpu = gbs / world
        roofline = {"bound": "hbm", "achieved": per_gpu, "peak": hbm_peak, "unit": "GB/s", "frac": per_gpu / hbm_peak,
                    "peak_basis": f"{peak_kind} HBM copy bandwidth", "traffic": ncu_traffic(args.workload)}
        value, unit = gbs, "GB/s"

    line = {"metric": metric_name(args.workload, world, args.scaling), "value": value, "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "s4 operands, s8 x s8 -> s32 tensor-core arithmetic",
            "data": "synthetic", "config": describe_config(args.workload, world, args.scaling, args.variant),
            "kernel_path": args.path if args.path != "auto"
            else {1: "tcgen05", 2: "legacy", 3: "skinny"}[L.path_for(m, n_local, k)],
            "tail": args.tail,
            "tops": tops, "algorithmic_gbs": gbs,
            "clocks": clocks, "gpu_launches": int(launches), "roofline": roofline}
    if rotate:
        line["l2_detail"] = f"{len(w_copies)} rotating copies of W ({len(w_copies) * wp.nbytes >> 20} MiB > L2)"
    if int8 is not None:
        line["int8_peak_measurement"] = int8
    if pipelined is not None:
        line["pipelined"] = {
            name: {"ms_per_step": ms, "GB/s": alg_bytes_local * world / (ms * 1e-3) / 1e9,
                   "frac_of_hbm_peak": alg_bytes_local / (ms * 1e-3) / 1e9 / hbm_peak}
            for name, ms in pipelined.items()}
        line["pipelined"]["note"] = ("back-to-back launches with int4_linear_set_overlap: 1 = weights not written "
                                     "by preceding work, 2 = weights and X; `value` uses ordinary launches")
    if e2e is not None:
        line["e2e"] = e2e
    if step_ms is not None:
        line["step_ms"] = {"min": min(step_ms), "median": statistics.median(step_ms), "max": max(step_ms)}  # rank 0
    if graph_replay is not None:
        line["graph_replay"] = graph_replay
    if back_to_back is not None:
        line["back_to_back"] = {"ms_per_step": back_to_back, "value": ops / (back_to_back * 1e-3) / 1e12,
                                "unit": "TOPS", "note": b2b_note}
    if strong_c5 is not None:
        line["strong_c5"] = strong_c5
    if gather_check is not None:
        line["gather_check"] = gather_check
    if gather_ms is not None:
        line["all_gather_ms"] = gather_ms
        line["gather"] = gather_cmp
    if world == 1 and not args.no_configs:
        cfgs = {}
        for name in ("c1", "c2", "c3", "c4", "c5", "d32", "d64", "d128"):
            try:
                cfgs[name] = quick_config(torch, L, dev, flush, name, int8_peak, hbm_peak)
            except Exception as e:
                cfgs[name] = {"error": repr(e)[:200]}
            torch.cuda.empty_cache()
        cfgs["note"] = ("short figures outside `value`: seeded operands made on the device, 5 event-timed launches each; "
                        "the best of event-timed and graph-replay time gives tops / gbs and the fractions")
        line["configs"] = cfgs
        if L.last_status() != 0:
            raise SystemExit("device-side failure in the per-configuration runs")
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_reference_sample(m, n_total, k)
    print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
