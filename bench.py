#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--variant auto|binned|merge] [--scale F]

One step = one y = alpha*A*x + beta*y (or Y = alpha*A*X + beta*Y) over the whole matrix.
Default workload: fp32 CSR SpMV on a 4,194,304-row matrix with Poisson(16) row lengths and
uniform random columns, alpha=1.5, beta=0.5 (per GPU; with N GPUs every rank owns such a
row shard of an N-times taller matrix, x is replicated, y stays sharded: weak scaling).
The metric is effective HBM GB/s on the algorithmic bytes
    nnz*(sizeof(val)+4) + (rows+1)*sizeof(offset) + cols*sizeof(val) + rows*sizeof(val)*(1+[beta!=0])
(SpMM: the A terms + cols*N*sizeof(B) + rows*N*sizeof(C)*(1+[beta!=0])).

Rank 0 prints one JSON line.  `--impl reference` times the reference's own CPU code
(oracle/_ref, or the C restatement when that library is absent) on the same configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, description)
    "spmv_poisson16_f32": "CSR SpMV fp32, 4,194,304 rows, row length ~ Poisson(16), uniform columns, alpha=1.5 beta=0.5",
    "spmv_rmat22_f32": "CSR SpMV fp32, R-MAT scale 22 edge factor 16 (0.57,0.19,0.19,0.05), alpha=1 beta=0",
    "spmv_lap2d256_f64": "CSR SpMV fp64, 5-point Laplacian 256x256, alpha=1 beta=0",
    "spmv_lap3d_f64_i64": "CSR SpMV fp64, 7-point Laplacian n^3 (n=512 at scale 1), int64 offsets, alpha=1 beta=0",
    "spmm_s27_128_f32_n8": "CSR SpMM fp32, 27-point stencil 128^3, N=8",
    "spmm_s27_128_f32_n32": "CSR SpMM fp32, 27-point stencil 128^3, N=32",
    "spmm_s27_128_f32_n128": "CSR SpMM fp32, 27-point stencil 128^3, N=128",
    "spmv_lap3d_f16_i64": "CSR SpMV fp16 A and x / fp32 y and arithmetic, 7-point Laplacian 512^3, int64 row offsets",
    "spmv_poisson16_bf16": "CSR SpMV bf16 A, x and y / fp32 arithmetic, Poisson(16) row lengths, 4,194,304 rows, alpha=1.5 beta=0.5",
    "spmm_s27_128_bf16_n64": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=64",
    "spmm_s27_128_bf16_n128": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=128",
    "spmm_s27_128_bf16_n256": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=256",
    "spmv_rmat26_f32_i64": "CSR SpMV fp32, R-MAT scale 26 edge factor 32, int64 offsets, alpha=1 beta=0",
}
# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel from the
# ncu captures summarised under profiles/, as a ratio to the algorithmic bytes of the captured case.
# The Laplacian was captured on a 256^3 grid (1/8 of the rows); its traffic grows with the rows, so the
# ratio is applied to the full launch.
TRAFFIC_RATIO = {
    "spmv_poisson16_f32": 605.7e6 / 603.9e6,
    "spmv_lap3d_f64_i64": 1804.2e6 / 1807.2e6,
    "spmv_rmat22_f32": 583.6e6 / 572.0e6,
    "spmm_s27_128_f32_n8": 580.7e6 / 588.5e6,
    "spmm_s27_128_f32_n32": 969.5e6 / 991.2e6,
    "spmm_s27_128_f32_n128": 2647.0e6 / 2601.8e6,
    "spmm_s27_128_bf16_n128": 1900.8e6 / 1946.0e6,
    "spmv_lap3d_f16_i64": 933.6e6 / 937.0e6,   # captured on the 256^3 grid, traffic grows with the units processed
}
DEFAULT_WORKLOAD = "spmv_poisson16_f32"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", choices=["auto", "binned", "merge"])
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the workload's row count by this factor (for profiler captures)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank owns a workload-sized row shard; strong: one matrix is "
                         "row-partitioned by balanced nnz across the ranks")
    ap.add_argument("--x-exchange", default="broadcast", choices=["broadcast", "window"],
                    help="N > 1: how x reaches the ranks.  broadcast: whole x from rank 0.  window (strong scaling, "
                         "SpMV): x is sharded like y and a rank receives only the column window of its rows")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def make_workload(name, device, rank, scale):
    """Returns dict(A=Csr, kind, n, alpha, beta, x_lo, dtype) for this rank's shard."""
    import torch
    from library_b200 import generators as G
    seed = 1000 * rank
    if name == "spmv_poisson16_f32":
        rows = max(1024, int(4194304 * scale))
        A = G.poisson_random(rows, rows, 16.0, dtype=torch.float32, device=device, seed=2 + seed)
        return dict(A=A, kind="spmv", n=1, alpha=1.5, beta=0.5, lo=-1.0, dtype=torch.float32)
    if name == "spmv_rmat22_f32":
        sc = 22 + int(round(__import__("math").log2(scale))) if scale != 1.0 else 22
        A = G.rmat(sc, 16, dtype=torch.float32, device=device, seed=3 + seed)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=0.0, dtype=torch.float32)
    if name == "spmv_rmat26_f32_i64":
        sc = 26 + int(round(__import__("math").log2(scale))) if scale != 1.0 else 26
        A = G.rmat(sc, 32, dtype=torch.float32, device=device, seed=5 + seed, index64=True)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=0.0, dtype=torch.float32)
    if name == "spmv_lap2d256_f64":
        A = G.laplacian_2d_5pt(256, dtype=torch.float64, device=device)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float64)
    if name == "spmv_lap3d_f64_i64":
        n = max(16, int(round(512 * scale ** (1.0 / 3.0))))
        A = G.laplacian_3d_7pt(n, dtype=torch.float64, device=device, index64=True)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float64)
    if name == "spmv_lap3d_f16_i64":
        n = max(16, int(round(512 * scale ** (1.0 / 3.0))))
        A = G.laplacian_3d_7pt(n, dtype=torch.float32, device=device, index64=True)
        A.val = A.val.to(torch.float16)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float16, ydtype=torch.float32)
    if name == "spmv_poisson16_bf16":
        rows = max(1024, int(4194304 * scale))
        A = G.poisson_random(rows, rows, 16.0, dtype=torch.float32, device=device, seed=2 + seed)
        A.val = A.val.to(torch.bfloat16)
        return dict(A=A, kind="spmv", n=1, alpha=1.5, beta=0.5, lo=-1.0, dtype=torch.bfloat16, ydtype=torch.bfloat16)
    if name.startswith("spmm_s27_128"):
        n = int(name.rsplit("_n", 1)[1])
        g = max(8, int(round(128 * scale ** (1.0 / 3.0))))
        bf16 = "bf16" in name
        A = G.stencil_3d_27pt(g, dtype=torch.float32, device=device, seed=4 + seed)
        if bf16:
            A.val = A.val.to(torch.bfloat16)
        return dict(A=A, kind="spmm", n=n, alpha=1.0, beta=0.0, lo=-1.0,
                    dtype=torch.bfloat16 if bf16 else torch.float32)
    raise KeyError(name)


def algorithmic_bytes(w):
    from library_b200 import generators as G
    A = w["A"]
    vb = A.val.element_size()
    ob = A.row_ptr.element_size()
    if w["kind"] == "spmv":
        if "ydtype" in w:  # 16-bit operands: x in the matrix type, y in its own
            yb = 4 if w["ydtype"] == __import__("torch").float32 else 2
            return A.nnz * (vb + 4) + (A.rows + 1) * ob + A.cols * vb + A.rows * yb * (2 if w["beta"] != 0 else 1)
        return G.spmv_bytes(A.rows, A.cols, A.nnz, vb, ob, w["beta"] != 0)
    yb = 4 if vb == 2 else vb
    return G.spmm_bytes(A.rows, A.cols, A.nnz, w["n"], vb, ob, vb, yb, w["beta"] != 0)


class ClockSampler:
    """Reads SM clock and clock-event (throttle) reasons through NVML while the timed region
    runs (read-only queries; nothing on the GPU is changed)."""

    def __init__(self, index):
        self.index, self.samples, self.stop = index, [], threading.Event()
        self.th = threading.Thread(target=self._run, daemon=True)
        self.nv = self.dev = None
        self.max_mhz = None
        try:
            import pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if vis:
                ids = [v for v in vis.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _once(self):
        if self.nv is None:
            return
        try:
            nv = self.nv
            mhz = float(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM))
            try:
                r = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.dev))
            except Exception:
                r = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev))
            self.samples.append((mhz, r))
        except Exception:
            pass

    def _run(self):
        while not self.stop.is_set():
            self._once()
            self.stop.wait(0.002)

    def __enter__(self):
        self._once()
        self.th.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.th.join(timeout=2)
        self._once()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"], "samples": 0}
        bits = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                0x4: "sw_power_cap"}
        seen = 0
        for _, r in self.samples:
            seen |= r
        return {"sm_mhz": statistics.median(m for m, _ in self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": [n for b, n in bits.items() if seen & b], "samples": len(self.samples)}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def cpu_sample_workload(args, w):
    """The workload the CPU arm times.  SpMV: the same matrix in full.  SpMM: the reference's CPU
    kernel allocates rows_per_thread x (cols / 256) offsets per call
    (hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:15-25, about 70 GB at 128^3), so it is timed on the
    same stencil on a 48^3 grid and its rate (GB/s on its own algorithmic bytes) is what is reported."""
    if w["kind"] != "spmm" or w["A"].rows <= 200_000:
        return w, "the same matrix in full"
    small = make_workload(args.workload, "cpu", 0, (48.0 / 128.0) ** 3)
    return small, "the same stencil on a 48^3 grid (110,592 rows): the reference's mm needs ~70 GB of offsets at 128^3"


def cpu_reference_time(w, repeats, threads):
    """Per-call seconds of the reference's CPU code (or the C restatement) on host arrays."""
    import numpy as np
    import oracle
    import torch
    from library_b200 import generators as G
    A = w["A"]
    rp, ci = A.row_ptr.cpu().numpy(), A.col_idx.cpu().numpy()
    ddt = torch.float32 if w["dtype"] in (torch.bfloat16, torch.float16) else w["dtype"]
    v = A.val.to(ddt).cpu().numpy()   # 16-bit operands are timed as the fp32 CPU kernel (the CPU path has no 16-bit types)
    kind = "reference" if (oracle.have_ref() and rp.dtype == np.int32) else "port"
    # the reference re-reads OMP_NUM_THREADS on every call (hygon/util/thread.cpp:32-42), and a
    # torchrun launch sets it to 1: give the CPU arm the cores it is entitled to
    os.environ["OMP_NUM_THREADS"] = str(threads)
    if w["kind"] == "spmv":
        x = G.uniform((A.cols,), w["lo"], 1.0, dtype=ddt, seed=11).numpy()
        y0 = G.uniform((A.rows,), -1.0, 1.0, dtype=ddt, seed=12).numpy()
        if kind == "reference":
            oracle.ref_set_threads(threads)
            _, t = oracle.ref_spmv(rp, ci, v, x, w["alpha"], w["beta"], y0, repeats=repeats + 1)
            return list(t[1:]), kind
        os.environ["OMP_NUM_THREADS"] = str(threads)
        ts = []
        for _ in range(repeats + 1):
            t0 = time.perf_counter()
            oracle.spmv(rp, ci, v, x, w["alpha"], w["beta"], y0)
            ts.append(time.perf_counter() - t0)
        return ts[1:], kind
    X = G.uniform((A.cols, w["n"]), w["lo"], 1.0, dtype=ddt, seed=11).numpy()
    if kind == "reference":
        oracle.ref_set_threads(threads)
        _, t = oracle.ref_spmm(rp, ci, v, X, w["alpha"], w["beta"], None, repeats=repeats + 1)
        return list(t[1:]), kind
    ts = []
    for _ in range(repeats + 1):
        t0 = time.perf_counter()
        oracle.spmm(rp, ci, v, X, w["alpha"], w["beta"])
        ts.append(time.perf_counter() - t0)
    return ts[1:], kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = make_workload(args.workload, "cpu", 0, args.scale)
    w, sample = cpu_sample_workload(args, w)
    nbytes = algorithmic_bytes(w)
    cores = host_cores()
    steps = max(1, min(args.steps, 20))
    ts, kind = cpu_reference_time(w, steps + min(args.warmup, 2), cores)
    ts = ts[min(args.warmup, 2):] or ts
    sec = statistics.median(ts)
    val = nbytes / sec / 1e9
    A = w["A"]
    flops = 2.0 * A.nnz * w["n"]
    line = {
        "impl": "reference", "metric": "effective HBM GB/s on algorithmic bytes (CSR SpMV/SpMM)",
        "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": len(ts), "warmup": min(args.warmup, 2),
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": {4: "f32", 8: "f64", 2: "f32"}[A.val.element_size()], "data": "synthetic",
        "gflops": flops / sec / 1e9,
        "config": {"workload": args.workload, "description": WORKLOADS[args.workload], "rows": A.rows,
                   "cols": A.cols, "nnz": A.nnz, "n": w["n"], "algorithmic_bytes": nbytes},
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{sample}, {len(ts)} calls, median"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from library_b200 import api
    from library_b200 import generators as G

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL's kernels on a high-priority stream: a halo exchange launched beside a product that fills the
        # GPU gets its few CTAs scheduled as soon as any slot frees, instead of after the product
        opts = None
        try:
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        except Exception:
            pass
        dist.init_process_group("nccl", device_id=dev, pg_options=opts)
    if args.variant != "auto":
        os.environ["ASP_SPMV_VARIANT"] = args.variant

    strong = args.scaling == "strong" and world > 1
    window = args.x_exchange == "window" and strong
    if args.x_exchange == "window" and not window:
        raise SystemExit("--x-exchange window needs --scaling strong and more than one rank")
    h = api.Handle()
    stream = torch.cuda.Stream()
    h.set_stream(stream.cuda_stream)
    if strong:
        # every rank builds the same matrix (same seed), takes its nnz-balanced row range and drops the rest
        from library_b200.generators import Csr
        from library_b200.sharding import shard_csr
        w = make_workload(args.workload, dev, 0, args.scale)
        full = w["A"]
        with torch.cuda.stream(stream):
            bounds = api.partition_rows_by_nnz(h, full.row_ptr, world)
            Aloc, (r0, r1) = shard_csr(h, full.rows, full.cols, full.row_ptr, full.col_idx, full.val, rank, world)
            w["A"] = Csr(r1 - r0, full.cols, Aloc.row_ptr, Aloc.col_idx.clone(), Aloc.val.clone())
        torch.cuda.synchronize()
        del Aloc, full
        torch.cuda.empty_cache()
    else:
        w = make_workload(args.workload, dev, rank, args.scale)
    A = w["A"]
    nbytes = algorithmic_bytes(w)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    ydt = w.get("ydtype", torch.float32 if w["dtype"] == torch.bfloat16 else w["dtype"])

    # x lives on rank 0 and is replicated over NVLink once: it is constant across the repeats
    if w["kind"] == "spmv":
        x = G.uniform((A.cols,), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = G.uniform((A.rows,), -1.0, 1.0, dtype=ydt, device=dev, seed=12 + rank)
    else:
        x = G.uniform((A.cols, w["n"]), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = torch.zeros((A.rows, w["n"]), dtype=ydt, device=dev)
    ex = x_own = None
    if window:
        if w["kind"] != "spmv":
            raise SystemExit("--x-exchange window covers SpMV")
        from library_b200.sharding import XWindowExchange
        # x is sharded like y: this rank keeps x[r0, r1) and receives the rest of its column window
        with torch.cuda.stream(stream):
            cmin, cmax = api.column_range(h, A.col_idx)
            ex = XWindowExchange(bounds, cmin, cmax, rank, world, w["dtype"], dev)
            x_own = x[r0:r1].clone()
            x_win = ex.run(x_own)
        torch.cuda.synchronize()
        del x
        x = x_own
        torch.cuda.empty_cache()
    elif world > 1:
        dist.broadcast(x, src=0)
    torch.cuda.synchronize()

    if w["kind"] == "spmv":
        xd, yd = (api.DnVecWindow(x_win, A.cols, ex.lo) if window else api.DnVec(x)), api.DnVec(y)
        buf = torch.empty(api.spmv_buffer_size(h, Am, xd, yd, w["alpha"], w["beta"]), dtype=torch.uint8, device=dev)
        with torch.cuda.stream(stream):
            Am.analyse(h)

        def step():
            api.spmv(h, Am, xd, yd, w["alpha"], w["beta"], buffer=buf)
    else:
        xd, yd = api.DnMat(x), api.DnMat(y)
        with torch.cuda.stream(stream):
            api.spmm_preprocess(h, Am, xd, yd)

        def step():
            api.spmm(h, Am, xd, yd, w["alpha"], w["beta"])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # beta != 0 makes y drift over repeats; keep it bounded by restoring between phases
    y_init = y.clone()
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    y.copy_(y_init)
    barrier()
    l0 = h.launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clk:
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = h.launches - l0
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    tot = torch.tensor([float(nbytes), 2.0 * A.nnz * w["n"], float(A.rows), float(A.nnz)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    ms = float(t.item())
    ms_step = ms / args.steps
    total_bytes, total_flops = float(tot[0]), float(tot[1])
    value = total_bytes / (ms_step * 1e-3) / 1e9

    # end to end through the public call with HOST buffers: H2D of the step's dense inputs from
    # pinned memory (on rank 0, then the NVLink broadcast), the call, D2H of the result
    e2e = None
    if not args.no_e2e:
        hx = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
        hx.copy_(x)
        hy_in = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
        hy_in.copy_(y_init)
        hy_out = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
        reads_y = w["beta"] != 0

        # Two sets of device buffers and three streams: the H2D copies of step i+1, the call of step i
        # and the D2H copy of step i-1 overlap (PCIe is full duplex), every step still moves its own
        # inputs in and its own result out.
        nbuf = 2
        xs, ys = [x, torch.empty_like(x)], [y, torch.empty_like(y)]
        hy_outs = [hy_out, torch.empty(y.shape, dtype=y.dtype, pin_memory=True)]
        if w["kind"] == "spmv":
            descs = [((xd if window else api.DnVec(xs[b])), api.DnVec(ys[b])) for b in range(nbuf)]
        else:
            descs = [(api.DnMat(xs[b]), api.DnMat(ys[b])) for b in range(nbuf)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        ev_cmp = [torch.cuda.Event() for _ in range(nbuf)]
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]

        def e2e_step(i):
            b = i % nbuf
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_out[b])      # the buffers' previous result has left the device
                if window or rank == 0 or world == 1:
                    xs[b].copy_(hx, non_blocking=True)
                if reads_y:
                    ys[b].copy_(hy_in, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(stream):
                stream.wait_event(ev_in[b])
                if window:
                    ex.run(xs[b])
                elif world > 1:
                    dist.broadcast(xs[b], src=0)
                if w["kind"] == "spmv":
                    api.spmv(h, Am, descs[b][0], descs[b][1], w["alpha"], w["beta"], buffer=buf)
                else:
                    api.spmm(h, Am, descs[b][0], descs[b][1], w["alpha"], w["beta"])
                ev_cmp[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_cmp[b])
                hy_outs[b].copy_(ys[b], non_blocking=True)
                ev_out[b].record(s_out)
        e_steps = max(3, min(args.steps, 20))
        for i in range(4):
            e2e_step(i)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_in)
        for i in range(e_steps):
            e2e_step(i)
        e1.record(s_out)
        barrier()
        et = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(et, op=dist.ReduceOp.MAX)
        e_ms = float(et.item()) / e_steps
        # the exchange step alone (whole-x broadcast, or the window exchange)
        x_ms = None
        if world > 1:
            def xchg():
                with torch.cuda.stream(stream):
                    ex.run(x) if window else dist.broadcast(x, src=0)
            for _ in range(3):
                xchg()
            barrier()
            x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            x0.record(stream)
            for _ in range(10):
                xchg()
            x1.record(stream)
            barrier()
            xt = torch.tensor([x0.elapsed_time(x1) / 10], dtype=torch.float64, device=dev)
            dist.all_reduce(xt, op=dist.ReduceOp.MAX)
            x_ms = float(xt.item())
        # a solver-like iteration with x resident on the devices: exchange + product, plain and with the
        # exchange hidden behind the rows that need no halo
        iter_ms = None
        if window:
            from library_b200.sharding import OverlappedShardSpMV
            ov = OverlappedShardSpMV(h, Am, ex, A.cols, stream)

            xv = ex.own_view()          # x kept inside the window: a step moves only the halo
            with torch.cuda.stream(stream):
                xv.copy_(x[max(ex.lo - r0, 0):max(ex.lo - r0, 0) + xv.numel()])

            def it_serial():
                with torch.cuda.stream(stream):
                    ex.run(xv)
                    api.spmv(h, Am, xd, yd, w["alpha"], w["beta"], buffer=buf)

            def it_overlap():
                ov.step(xv, y, w["alpha"], w["beta"])
            iter_ms = {}
            for name, fn in (("serial", it_serial), ("overlapped", it_overlap)):
                for _ in range(3):
                    fn()
                barrier()
                i0, i1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                i0.record(stream)
                for _ in range(20):
                    fn()
                i1.record(stream)
                barrier()
                it = torch.tensor([i0.elapsed_time(i1) / 20], dtype=torch.float64, device=dev)
                dist.all_reduce(it, op=dist.ReduceOp.MAX)
                iter_ms[name] = float(it.item())
            iter_ms["interior_rows"] = [ov.i0, ov.i1]
        h2d = x.numel() * x.element_size() + (y.numel() * y.element_size() if reads_y else 0)
        e2e = {"value": total_bytes / (e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": y.numel() * y.element_size(),
               "x_exchange": args.x_exchange if world > 1 else None, "x_exchange_ms": x_ms,
               "exchange_plus_spmv_ms": iter_ms,
               "x_bytes_received_per_rank": (ex.bytes_received if window else
                                             (x.numel() * x.element_size() if world > 1 else 0)),
               "note": "A resident in HBM (like the reference's created matrix handle); x (+y when beta!=0) from "
                       "pinned host memory each step, y back to the host each step; steps pipelined over two buffer sets "
                       "(copy-in, call and copy-out of neighbouring steps overlap)"}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            cores = host_cores()
            reps = 10 if A.nnz > 10_000_000 else 50
            wc, sample = cpu_sample_workload(args, w)
            ts, kind = cpu_reference_time(wc, reps, cores)
            sec = statistics.median(ts)
            cpu = {"value": algorithmic_bytes(wc) / sec / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
                   "ms_per_step": sec * 1e3, "sample": f"{sample}, {len(ts)} calls after 1 warm-up, median"}
        except Exception as ex:  # the baseline must not take the bench line down with it
            cpu = {"value": None, "unit": "GB/s", "cores": host_cores(), "kind": "port", "sample": f"failed: {ex}"}

    if rank == 0:
        peak, peak_src = measured_peak()
        per_launch_ms = ms_step  # one call = one dominant kernel (+ a <1% carry fix-up for merge-path)
        ach = nbytes / (per_launch_ms * 1e-3) / 1e9 if world == 1 else (total_bytes / world) / (per_launch_ms * 1e-3) / 1e9
        variant = Am.last_variant() if w["kind"] == "spmv" else ("tcgen05" if w["dtype"] == torch.bfloat16 else "simt row-block")
        line = {
            "metric": "effective HBM GB/s on algorithmic bytes (CSR SpMV/SpMM)",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak",
            "vs_baseline": None,
            "dtype": {torch.float32: "f32", torch.float64: "f64", torch.bfloat16: "bf16", torch.float16: "f16"}[w["dtype"]],
            "data": "synthetic", "gflops": total_flops / (ms_step * 1e-3) / 1e9,
            "frac_of_nominal_8TBs": value / world / 8000.0,
            "config": {"workload": args.workload, "description": WORKLOADS[args.workload],
                       "rows_per_gpu": A.rows, "cols": A.cols, "nnz_per_gpu": A.nnz, "n": w["n"],
                       "alpha": w["alpha"], "beta": w["beta"], "variant": variant,
                       "algorithmic_bytes_per_gpu": nbytes, "l2": "inputs larger than L2 (126 MB), no flush"
                       if nbytes > 126e6 else "L2-resident workload, no flush (the configuration is smaller than L2)",
                       "sharding": ("one matrix row-partitioned by balanced nnz" if strong else
                                    "every rank owns a workload-sized row shard")
                       + (", x sharded like y and exchanged by column window (point-to-point over NVLink), y sharded"
                          if window else ", x replicated by NCCL broadcast, y sharded")},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src,
                         "traffic": (TRAFFIC_RATIO[args.workload] * nbytes) if args.workload in TRAFFIC_RATIO else None,
                         "traffic_source": "ncu dram__bytes_read+write of the dominant kernel, see profiles/"},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clk.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        # before any OpenMP runtime is loaded: a torchrun launch exports OMP_NUM_THREADS=1, and the CPU arm
        # is meant to use every core it may run on
        os.environ["OMP_NUM_THREADS"] = str(host_cores())
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
