#!/usr/bin/env python
"""Benchmark of the INT4 linear GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload m8|c1..c5]
                    [--impl ours|reference] [--scaling weak|strong]

One process per GPU (for N > 1 launch through torch.distributed.run); rank 0
prints ONE JSON line.  A step is one launch of the operator on seeded synthetic
operands (i.i.d. uniform [-8, 7], packed as the reference's utils/packer does).

Metric: INT4 GEMM TOPS = 2*M*N*K / t (the formula of the reference's
test/benchmark.cu:112-113), default workload M=N=K=8192.
  value     device-timed (CUDA events), operands resident in HBM, L2 flushed
            before every timed launch as test/benchmark.cu:93-96 does
  e2e       same metric through the host-buffer C-ABI entry point: pinned host
            operands up, launch, result down, every step
  roofline  achieved TOPS of the kernel against 2 x the measured dense bf16
            tensor rate (B200's int8 rate is twice its bf16 rate), or GB/s
            against the measured HBM copy rate for the decode shape
  cpu_baseline  the reference's own CPU GEMM on a bounded row sample

With N > 1 ranks the weight matrix is sharded along N: every rank holds the
full X and its own rows of W and produces its own columns of Y; no collective is
on the data path.  --scaling weak (default) keeps the per-GPU shard at the
workload's N, --scaling strong splits the workload's N across the ranks.
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
}
NOMINAL_INT8_TOPS = 4500.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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

    cores = os.cpu_count() or 1
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


def reference_gpu_arm(args, m, n, k):
    import torch
    from int4linear_b200 import uniform_s4_packed
    from oracle import oracle as O
    ref = O.ref_lib()
    if ref is None:
        print(json.dumps({"impl": "reference-gpu", "unavailable": "oracle/_ref was not built (needs the reference checkout)"}))
        return
    torch.cuda.set_device(0)
    dev = torch.device("cuda:0")
    xd = torch.from_numpy(uniform_s4_packed(0xA008, m, k)).to(dev)
    wd = torch.from_numpy(uniform_s4_packed(0xB008, n, k)).to(dev)
    yd = torch.empty((m, n), dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(max(3, args.warmup)):
        ref.ref_linear_v21_launch(xd.data_ptr(), wd.data_ptr(), yd.data_ptr(), m, n, k)
    times = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ref.ref_linear_v21_launch(xd.data_ptr(), wd.data_ptr(), yd.data_ptr(), m, n, k)
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = sum(times) / len(times)
    tops = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    print(json.dumps({"impl": "reference-gpu", "metric": f"INT4 GEMM TOPS at M={m} N={n} K={k}", "value": tops,
                      "unit": "TOPS", "n_gpus": 1, "steps": args.steps, "warmup": max(3, args.warmup),
                      "ms_per_step": ms, "higher_is_better": True, "data": "synthetic",
                      "config": {"workload": f"{args.workload}: M={m} N={n} K={k}",
                                 "kernel": "reference linear_v21 (mma.sync m16n8k64 s4) built for sm_100a"}}))


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
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--gather", action="store_true", help="also time an NCCL all-gather of Y (N > 1)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    m, n_work, k, bound = WORKLOADS[args.workload]
    metric = (f"INT4 GEMM TOPS at M={m} N={n_work} K={k}" if bound == "tensor"
              else f"INT4 GEMM achieved HBM GB/s at M={m} N={n_work} K={k}")

    if args.impl == "reference":
        if rank != 0:
            return
        cb = cpu_reference_sample(m, n_work, k, seconds_target=max(5.0, min(60.0, 4.0 * args.steps)))
        line = {"impl": "reference", "metric": f"INT4 GEMM TOPS at M={m} N={n_work} K={k}", "value": cb["value"], "unit": "TOPS",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": None, "higher_is_better": True, "scaling": args.scaling,
                "vs_baseline": None, "dtype": "s4 x s4 -> s32 (int32 arithmetic on the CPU)",
                "data": "synthetic", "config": {"workload": f"{args.workload}: M={m} N={n_work} K={k}"},
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if args.impl == "reference-gpu":
        # The north star's path (b): the reference's own kernel (cp.async + ldmatrix + mma.sync
        # m16n8k64 s4, kernels/linear_v21.h) recompiled for sm_100a from its unmodified sources
        # into oracle/_ref, timed with the same method.  A comparison arm, not this library.
        if rank != 0:
            return
        reference_gpu_arm(args, m, n_work, k)
        return

    import torch
    import torch.distributed as dist
    import int4linear_b200 as L

    L.set_path({"auto": L.PATH_AUTO, "tcgen05": L.PATH_TCGEN05, "legacy": L.PATH_LEGACY,
                "skinny": L.PATH_SKINNY}[args.path])
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
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
        copies = max(2, int(2 * 126e6 // wp.nbytes) + 1)
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
        def graph_ms(mode):
            L.set_overlap(mode)
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(args.steps):
                        step(i)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            barrier()
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            barrier()
            L.set_overlap(0)
            return e0.elapsed_time(e1)
        total_ms = graph_ms(0)
        pipelined = {f"overlap_{mode}": graph_ms(mode) / args.steps for mode in (1, 2)}
        launches0 = L.launch_count() - args.steps  # the timed replay ran the K captured launches
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
    ws_bytes = m * k // 2 + n_local * k // 2 + 4 * m * n_local
    if not rotate and ws_bytes > 2 * 126e6:
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        flush.zero_()
        b0.record()
        for i in range(args.steps):
            step(i)
        b1.record()
        barrier()
        bt = torch.tensor([b0.elapsed_time(b1) / args.steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)  # every rank takes part; max over ranks
        back_to_back = float(bt.item())
    # Microsecond-scale tensor shapes (c1): one launch is comparable with the launch overhead an
    # event pair sees, so the K launches are also timed as one CUDA-graph replay over rotating
    # copies of X, W and Y that together exceed L2.
    graph_replay = None
    if not rotate and ws_bytes < 32e6 and world == 1:
        sets = int(2 * 126e6 // ws_bytes) + 1
        xs = [xd] + [xd.clone() for _ in range(sets - 1)]
        ws_ = [wd] + [wd.clone() for _ in range(sets - 1)]
        ys = [yd] + [torch.empty_like(yd) for _ in range(sets - 1)]
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in range(args.steps):
                    L.linear(xs[i % sets], ws_[i % sets], out=ys[i % sets])
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        graph.replay()
        g1.record()
        barrier()
        per = g0.elapsed_time(g1) / args.steps
        graph_replay = {"ms_per_step": per, "value": 2.0 * m * n_local * k / (per * 1e-3) / 1e12, "unit": "TOPS",
                        "note": f"{args.steps} launches in one CUDA graph over {sets} rotating operand sets "
                                f"({sets * ws_bytes / 2**20:.0f} MiB > L2)"}
    clocks = sampler.stop() if rank == 0 else None
    if L.last_status() != 0:
        raise SystemExit("device-side failure during the timed region")

    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    ops = 2.0 * m * n_total * k
    tops = ops / (ms_per_step * 1e-3) / 1e12
    alg_bytes_local = m * k // 2 + n_local * k // 2 + 4 * m * n_local
    gbs = alg_bytes_local * world / (ms_per_step * 1e-3) / 1e9

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
        g = torch.tensor([e0.elapsed_time(e1) / 5], dtype=torch.float64, device=dev)
        dist.all_reduce(g, op=dist.ReduceOp.MAX)
        gather_ms = float(g.item())

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
            v = torch.tensor([a.elapsed_time(b) / reps], dtype=torch.float64, device=dev)
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
            return float(v.item())

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
        dt = time.perf_counter() - t0
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item()) / e2e_steps
        e2e = {"value": (ops / dt / 1e12) if bound == "tensor" else (alg_bytes_local * world / dt / 1e9),
               "unit": "TOPS" if bound == "tensor" else "GB/s",
               "h2d_bytes_per_step": int(xp.nbytes + wp.nbytes), "d2h_bytes_per_step": int(yn.nbytes),
               "ms_per_step": dt * 1e3, "steps": e2e_steps,
               "note": "X and W uploaded from pinned host memory and Y downloaded every step"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    if bound == "tensor":
        per_gpu = tops / world
        peak = 2.0 * float(peaks["bf16_tflops"])
        roofline = {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TOPS",
                    "frac": per_gpu / peak,
                    "peak_basis": f"2 x dense bf16 burst of {peak_kind} ({peaks['bf16_tflops']} TFLOP/s); "
                                  "int8 issues at twice the bf16 rate on B200",
                    "frac_of_nominal_int8_4500": per_gpu / NOMINAL_INT8_TOPS,
                    "traffic": ncu_traffic(args.workload)}
        value, unit = tops, "TOPS"
    else:
        per_gpu = gbs / world
        peak = float(peaks["hbm_gbs"])
        roofline = {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                    "peak_basis": f"{peak_kind} HBM copy bandwidth", "traffic": ncu_traffic(args.workload)}
        value, unit = gbs, "GB/s"

    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "s4 operands, s8 x s8 -> s32 tensor-core arithmetic",
            "data": "synthetic",
            "config": {"workload": f"{args.workload}: M={m} N={n_total} K={k}",
                       "shard": f"{world} x (M={m}, N={n_local}, K={k}), W and Y split along N, X replicated",
                       "l2": "256 MiB flush write before every timed launch" if not rotate
                             else f"{len(w_copies)} rotating copies of W ({len(w_copies) * wp.nbytes >> 20} MiB > L2)",
                       "variant": args.variant,
                       "kernel_path": args.path if args.path != "auto"
                       else {1: "tcgen05", 2: "legacy", 3: "skinny"}[L.path_for(m, n_local, k)]},
            "tops": tops, "algorithmic_gbs": gbs,
            "clocks": clocks, "gpu_launches": int(launches), "roofline": roofline}
    if pipelined is not None:
        line["pipelined"] = {
            name: {"ms_per_step": ms, "GB/s": alg_bytes_local * world / (ms * 1e-3) / 1e9,
                   "frac_of_hbm_peak": alg_bytes_local / (ms * 1e-3) / 1e9 / float(peaks["hbm_gbs"])}
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
                                "unit": "TOPS", "note": "same launches without the L2 flush between them; working set > 2 x L2"}
    if gather_ms is not None:
        line["all_gather_ms"] = gather_ms
        line["gather"] = gather_cmp
    if world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_reference_sample(m, n_total, k)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
