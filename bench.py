#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload NAME] [--variant auto|binned|merge] [--scale F]
                    [--exchange overlap|window|allgather|broadcast]

One step = one y = alpha*A*x + beta*y (or Y = alpha*A*X + beta*Y) over the WHOLE matrix.  With N
GPUs that one matrix is cut into N contiguous row ranges of near-equal nnz
(alphasparseCsrPartitionRowsByNnz), y stays sharded, x is sharded like y, and a step is what an
iterative solver pays per iteration: the exchange of x over NVLink (alphasparseMg*, NCCL) plus the
product, both inside the timed region ("scaling": "strong").  Default workload: fp64 SpMV on the
7-point Laplacian of a 512^3 grid with 64-bit row offsets (134,217,728 rows, 937,951,232 entries,
14.5 GB), the largest configuration that fits one GPU.

The metric is effective HBM GB/s on the algorithmic bytes of the whole matrix, every array once:
    nnz*(sizeof(val)+4) + (rows+1)*sizeof(offset) + cols*sizeof(val) + rows*sizeof(val)*(1+[beta!=0])
(SpMM: the A terms + cols*N*sizeof(B) + rows*N*sizeof(C)*(1+[beta!=0])).

Rank 0 prints one JSON line.  At N = 1 the line also carries `per_config`: the other benchmark
configurations timed the same way in the same process.  `--impl reference` times the reference's
own CPU code (oracle/_ref, or the C restatement when that library is absent) on the host cores.
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

METRIC = "effective HBM GB/s on algorithmic bytes (CSR SpMV/SpMM)"
WORKLOADS = {
    "spmv_lap3d_f64_i64": "CSR SpMV fp64, 7-point Laplacian n^3 (n=512 at scale 1), int64 offsets, alpha=1 beta=0",
    "spmv_poisson16_f32": "CSR SpMV fp32, 4,194,304 rows, row length ~ Poisson(16), uniform columns, alpha=1.5 beta=0.5",
    "spmv_rmat22_f32": "CSR SpMV fp32, R-MAT scale 22 edge factor 16 (0.57,0.19,0.19,0.05), alpha=1 beta=0",
    "spmv_lap2d256_f64": "CSR SpMV fp64, 5-point Laplacian 256x256, alpha=1 beta=0",
    "spmm_s27_128_f32_n8": "CSR SpMM fp32, 27-point stencil 128^3, N=8",
    "spmm_s27_128_f32_n32": "CSR SpMM fp32, 27-point stencil 128^3, N=32",
    "spmm_s27_128_f32_n128": "CSR SpMM fp32, 27-point stencil 128^3, N=128",
    "spmm_rmat20_f32_n32": "CSR SpMM fp32, R-MAT scale 20 edge factor 16 (power-law rows), N=32",
    "spmv_lap3d_f16_i64": "CSR SpMV fp16 A and x / fp32 y and arithmetic, 7-point Laplacian 512^3, int64 row offsets",
    "spmv_poisson16_bf16": "CSR SpMV bf16 A, x and y / fp32 arithmetic, Poisson(16) row lengths, 4,194,304 rows, alpha=1.5 beta=0.5",
    "spmm_s27_128_bf16_n64": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=64",
    "spmm_s27_128_bf16_n128": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=128",
    "spmm_s27_128_bf16_n256": "CSR SpMM bf16 operands / fp32 accumulate (tcgen05), 27-point stencil 128^3, N=256",
    "spmv_rmat26_f32_i64": "CSR SpMV fp32, R-MAT scale 26 edge factor 32, int64 offsets, alpha=1 beta=0",
}
DEFAULT_WORKLOAD = "spmv_lap3d_f64_i64"
# The other configurations, timed at N = 1 after the headline workload (`per_config`).
PER_CONFIG = ["spmv_lap2d256_f64", "spmv_poisson16_f32", "spmv_rmat22_f32", "spmm_s27_128_f32_n8",
              "spmm_s27_128_f32_n32", "spmm_s27_128_f32_n128", "spmm_s27_128_bf16_n128", "spmm_rmat20_f32_n32",
              "spmv_rmat26_f32_i64"]
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
    "spmm_s27_128_bf16_n128": 1895.3e6 / 1953.5e6,
    "spmv_lap3d_f16_i64": 933.6e6 / 937.0e6,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--variant", default="auto", choices=["auto", "binned", "merge"])
    ap.add_argument("--scale", type=float, default=1.0,
                    help="shrink the workload's row count by this factor (for profiler captures)")
    ap.add_argument("--exchange", default="overlap", choices=["overlap", "window", "allgather", "broadcast"],
                    help="N > 1, SpMV: how x reaches the ranks inside a step.  overlap: column window by "
                         "send/recv, hidden behind the rows that need no halo; window: the same, serial; "
                         "allgather: every rank collects the whole x; broadcast: whole x from rank 0")
    ap.add_argument("--cpu-kind", default="auto", choices=["auto", "reference", "port"],
                    help="--impl reference: the reference's own compiled CPU code (auto, when it was built) or "
                         "the plain-C restatement")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-per-config", action="store_true")
    return ap.parse_args()


def lap3d_n(scale):
    return max(16, int(round(512 * scale ** (1.0 / 3.0))))


def make_workload(name, device, scale, cpu_sample=False):
    """dict(A=Csr, kind, n, alpha, beta, lo, dtype[, ydtype]) of the whole matrix.  With
    ``cpu_sample`` the bounded sample the CPU arm times (see cpu_sample_note)."""
    import math
    import torch
    from library_b200 import generators as G
    if name == "spmv_poisson16_f32":
        rows = max(1024, int(4194304 * scale))
        A = G.poisson_random(rows, rows, 16.0, dtype=torch.float32, device=device, seed=2)
        return dict(A=A, kind="spmv", n=1, alpha=1.5, beta=0.5, lo=-1.0, dtype=torch.float32)
    if name == "spmv_rmat22_f32":
        sc = 22 + int(round(math.log2(scale))) if scale != 1.0 else 22
        A = G.rmat(sc, 16, dtype=torch.float32, device=device, seed=3)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=0.0, dtype=torch.float32)
    if name == "spmv_rmat26_f32_i64":
        sc = 26 + int(round(math.log2(scale))) if scale != 1.0 else 26
        if cpu_sample:
            sc = min(sc, 22)
        A = G.rmat(sc, 32, dtype=torch.float32, device=device, seed=5, index64=not cpu_sample)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=0.0, dtype=torch.float32)
    if name == "spmv_lap2d256_f64":
        A = G.laplacian_2d_5pt(256, dtype=torch.float64, device=device)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float64)
    if name in ("spmv_lap3d_f64_i64", "spmv_lap3d_f16_i64"):
        n = lap3d_n(scale)
        f16 = "f16" in name
        if cpu_sample:
            # a slab of n x n x nz grid planes: the same band structure and plane size as the full grid
            nz = max(4, min(n, (1 << 24) // (n * n)))
            offs = [(0, 0, 0), (-1, 0, 0), (1, 0, 0), (0, -1, 0), (0, 1, 0), (0, 0, -1), (0, 0, 1)]
            A = G.stencil((n, n, nz), offs, [6.0] + [-1.0] * 6, dtype=torch.float32 if f16 else torch.float64,
                          device=device, index64=False, chunk_rows=1 << 22)
        else:
            A = G.laplacian_3d_7pt(n, dtype=torch.float32 if f16 else torch.float64, device=device, index64=True)
        if f16:
            A.val = A.val.to(torch.float16)
            return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float16, ydtype=torch.float32)
        return dict(A=A, kind="spmv", n=1, alpha=1.0, beta=0.0, lo=-1.0, dtype=torch.float64)
    if name == "spmv_poisson16_bf16":
        rows = max(1024, int(4194304 * scale))
        A = G.poisson_random(rows, rows, 16.0, dtype=torch.float32, device=device, seed=2)
        A.val = A.val.to(torch.bfloat16)
        return dict(A=A, kind="spmv", n=1, alpha=1.5, beta=0.5, lo=-1.0, dtype=torch.bfloat16, ydtype=torch.bfloat16)
    if name.startswith("spmm_s27_128"):
        n = int(name.rsplit("_n", 1)[1])
        g = max(8, int(round(128 * scale ** (1.0 / 3.0))))
        if cpu_sample:
            g = min(g, 48)
        bf16 = "bf16" in name
        A = G.stencil_3d_27pt(g, dtype=torch.float32, device=device, seed=4)
        if bf16:
            A.val = A.val.to(torch.bfloat16)
        return dict(A=A, kind="spmm", n=n, alpha=1.0, beta=0.0, lo=-1.0,
                    dtype=torch.bfloat16 if bf16 else torch.float32)
    if name == "spmm_rmat20_f32_n32":
        sc = 20 + int(round(math.log2(scale))) if scale != 1.0 else 20
        if cpu_sample:
            sc = min(sc, 16)
        A = G.rmat(sc, 16, dtype=torch.float32, device=device, seed=6)
        return dict(A=A, kind="spmm", n=32, alpha=1.0, beta=0.0, lo=0.0, dtype=torch.float32)
    raise KeyError(name)


def cpu_sample_note(name):
    """What the CPU arm times for this workload (a bounded sample where the whole matrix would take the
    host minutes to build, or where the reference's CPU kernel cannot hold it)."""
    if name.startswith("spmv_lap3d"):
        return ("a slab of 64 grid planes of the same Laplacian (512 x 512 x 64 = 16,777,216 rows, 1/8 of the rows, "
                "32-bit row offsets as the reference's CPU code requires)")
    if name.startswith("spmm_s27_128"):
        return ("the same stencil on a 48^3 grid (110,592 rows): the reference's mm allocates rows_per_thread x "
                "(cols / 256) offsets per call, ~70 GB at 128^3")
    if name == "spmv_rmat26_f32_i64":
        return "R-MAT scale 22 with the same edge factor (the reference's CPU code is 32-bit)"
    if name == "spmm_rmat20_f32_n32":
        return "R-MAT scale 16 with the same edge factor"
    return "the same matrix in full"


def static_config(args):
    """Facts of the configuration that do not depend on the run (both arms print the same dict)."""
    name = args.workload
    cfg = {"workload": name, "description": WORKLOADS[name], "scale": args.scale}
    if name.startswith("spmv_lap3d"):
        n = lap3d_n(args.scale)
        vb = 2 if "f16" in name else 8
        yb = 4 if "f16" in name else 8
        rows, nnz = n ** 3, 7 * n ** 3 - 6 * n ** 2
        cfg.update(rows=rows, cols=rows, nnz=nnz, n=1, alpha=1.0, beta=0.0,
                   algorithmic_bytes=nnz * (vb + 4) + (rows + 1) * 8 + rows * vb + rows * yb)
    return cfg


def algorithmic_bytes(w):
    import torch
    from library_b200 import generators as G
    A = w["A"]
    vb = A.val.element_size()
    ob = A.row_ptr.element_size()
    if w["kind"] == "spmv":
        if "ydtype" in w:  # 16-bit operands: x in the matrix type, y in its own
            yb = 4 if w["ydtype"] == torch.float32 else 2
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


def dtype_name(dt):
    import torch
    return {torch.float32: "f32", torch.float64: "f64", torch.bfloat16: "bf16", torch.float16: "f16"}[dt]


# ------------------------------------------------------------------------------------------------
# the reference arm: the reference's own CPU code on the host cores
# ------------------------------------------------------------------------------------------------

def cpu_reference_time(w, calls, threads, want="auto"):
    """Per-call seconds (list of ``calls``) of the reference's CPU code, or of the C restatement
    where that library is absent or the offsets are 64-bit, on host arrays."""
    import numpy as np
    import oracle
    import torch
    from library_b200 import generators as G
    A = w["A"]
    rp, ci = A.row_ptr.cpu().numpy(), A.col_idx.cpu().numpy()
    ddt = torch.float32 if w["dtype"] in (torch.bfloat16, torch.float16) else w["dtype"]
    v = A.val.to(ddt).cpu().numpy()   # 16-bit operands are timed as the fp32 CPU kernel (the CPU path has no 16-bit types)
    kind = "reference" if (oracle.have_ref() and rp.dtype == np.int32 and want != "port") else "port"
    # the reference re-reads OMP_NUM_THREADS on every call (hygon/util/thread.cpp:32-42), and a
    # torchrun launch sets it to 1: give the CPU arm the cores it is entitled to
    os.environ["OMP_NUM_THREADS"] = str(threads)
    if w["kind"] == "spmv":
        x = G.uniform((A.cols,), w["lo"], 1.0, dtype=ddt, seed=11).numpy()
        y0 = G.uniform((A.rows,), -1.0, 1.0, dtype=ddt, seed=12).numpy()
        if kind == "reference":
            oracle.ref_set_threads(threads)
            _, t = oracle.ref_spmv(rp, ci, v, x, w["alpha"], w["beta"], y0, repeats=calls)
            return list(t), kind
        ts = []
        for _ in range(calls):
            t0 = time.perf_counter()
            oracle.spmv(rp, ci, v, x, w["alpha"], w["beta"], y0)
            ts.append(time.perf_counter() - t0)
        return ts, kind
    X = G.uniform((A.cols, w["n"]), w["lo"], 1.0, dtype=ddt, seed=11).numpy()
    if kind == "reference":
        oracle.ref_set_threads(threads)
        _, t = oracle.ref_spmm(rp, ci, v, X, w["alpha"], w["beta"], None, repeats=calls)
        return list(t), kind
    ts = []
    for _ in range(calls):
        t0 = time.perf_counter()
        oracle.spmm(rp, ci, v, X, w["alpha"], w["beta"])
        ts.append(time.perf_counter() - t0)
    return ts, kind


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = make_workload(args.workload, "cpu", args.scale, cpu_sample=True)
    nbytes = algorithmic_bytes(w)
    cores = host_cores()
    warm = max(1, args.warmup)
    steps = max(1, args.steps)
    ts, kind = cpu_reference_time(w, warm + steps, cores, args.cpu_kind)
    ts = ts[warm:]
    sec = sum(ts) / len(ts)
    val = nbytes / sec / 1e9
    A = w["A"]
    flops = 2.0 * A.nnz * w["n"]
    sample = cpu_sample_note(args.workload)
    line = {
        "impl": "reference", "metric": METRIC,
        "value": val, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": {4: "f32", 8: "f64", 2: "f32"}[A.val.element_size()], "data": "synthetic",
        "gflops": flops / sec / 1e9,
        "config": static_config(args),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{sample}; {A.rows} rows, {A.nnz} entries, {nbytes} algorithmic bytes per call; "
                                   f"mean of {steps} calls after {warm} warm-up; one host ({cores} cores), whatever N is"},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def cpu_baseline_subprocess(args):
    """The in-line CPU baseline, taken the way the reference arm takes it: a fresh process whose thread
    count is set before any OpenMP runtime loads (inside this process torch, CUDA and the clock sampler
    are already running, which halves the CPU kernel's rate).  The reference's compiled code first; the
    plain-C restatement, in a process of its own, goes beside it as `port` (the reference's fp64 row
    kernel, hygon/kernel/level2/mv/gemv/csrmv/gemv_csr_serial_fma_fp64_u4.S, mixes legacy-SSE moves with
    VEX FMAs, which costs it dearly per row on hosts that penalise that mix)."""
    def run(kind):
        cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--workload", args.workload,
               "--scale", str(args.scale), "--steps", str(min(args.steps, 10)), "--warmup", "2", "--cpu-kind", kind]
        env = dict(os.environ)
        for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "OMP_NUM_THREADS"):
            env.pop(k, None)
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
        for ln in reversed(r.stdout.strip().splitlines()):
            if ln.startswith("{"):
                d = json.loads(ln)
                cb = d["cpu_baseline"]
                cb["ms_per_step"] = d["ms_per_step"]
                return cb
        raise RuntimeError((r.stderr.strip().splitlines() or ["no output"])[-1][:200])
    try:
        cb = run("auto")
        if cb.get("kind") == "reference":
            try:
                p = run("port")
                cb["port"] = {"value": p["value"], "unit": "GB/s", "ms_per_step": p["ms_per_step"], "cores": p["cores"]}
            except Exception as ex:
                cb["port"] = {"value": None, "error": str(ex)[:200]}
        return cb
    except Exception as ex:  # the baseline must not take the bench line down with it
        return {"value": None, "unit": "GB/s", "cores": host_cores(), "kind": "port", "sample": f"failed: {ex}"}


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def align_ranks(stream):
    """A device-side meeting point on the timing stream: the ranks leave the host barrier up to milliseconds
    apart, and without this the first step's exchange would absorb that skew into the timed region."""
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        with torch.cuda.stream(stream):
            dist.all_reduce(torch.zeros(1, device="cuda"))


def time_steps(fn, stream, steps, warmup, barrier):
    import torch
    for _ in range(warmup):
        fn()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    align_ranks(stream)
    e0.record(stream)
    for _ in range(steps):
        fn()
    e1.record(stream)
    barrier()
    return e0.elapsed_time(e1) / steps


def one_config(name, h, stream, dev, steps, warmup):
    """One single-GPU configuration timed like the headline (events on the launching stream)."""
    import torch
    from library_b200 import api
    from library_b200 import generators as G
    t_gen = time.perf_counter()
    w = make_workload(name, dev, 1.0)
    torch.cuda.synchronize()
    t_gen = time.perf_counter() - t_gen
    A = w["A"]
    nbytes = algorithmic_bytes(w)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    ydt = w.get("ydtype", torch.float32 if w["dtype"] == torch.bfloat16 else w["dtype"])
    if w["kind"] == "spmv":
        x = G.uniform((A.cols,), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = G.uniform((A.rows,), -1.0, 1.0, dtype=ydt, device=dev, seed=12)
        xd, yd = api.DnVec(x), api.DnVec(y)
        with torch.cuda.stream(stream):
            Am.analyse(h)
        fn = lambda: api.spmv(h, Am, xd, yd, w["alpha"], w["beta"])
    else:
        x = G.uniform((A.cols, w["n"]), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = torch.zeros((A.rows, w["n"]), dtype=ydt, device=dev)
        xd, yd = api.DnMat(x), api.DnMat(y)
        with torch.cuda.stream(stream):
            api.spmm_preprocess(h, Am, xd, yd)
        fn = lambda: api.spmm(h, Am, xd, yd, w["alpha"], w["beta"])
    torch.cuda.synchronize()
    l0 = h.launches
    fn()
    per_call = h.launches - l0
    with ClockSampler(dev.index or 0) as clk:
        ms = time_steps(fn, stream, steps, max(3, warmup), torch.cuda.synchronize)
    peak, _ = measured_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    variant = (Am.last_variant() if w["kind"] == "spmv" else api.spmm_last_variant(Am))
    out = {"workload": name, "ms": ms, "GB/s": gbs, "frac": gbs / peak, "variant": variant,
           "gflops": 2.0 * A.nnz * w["n"] / (ms * 1e-3) / 1e9, "rows": A.rows, "nnz": A.nnz, "n": w["n"],
           "algorithmic_bytes": nbytes, "launches_per_call": per_call, "device_error": Am.plan(h)[0]["device_error"],
           "generate_s": round(t_gen, 2), "sm_mhz": clk.summary()["sm_mhz"], "reasons": clk.summary()["reasons"],
           "l2": "larger than L2" if nbytes > 126e6 else "L2-resident"}
    del Am, xd, yd, x, y, A, w
    torch.cuda.empty_cache()
    return out


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from library_b200 import api
    from library_b200 import generators as G
    from library_b200.generators import Csr
    from library_b200.sharding import shard_csr

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if args.variant != "auto":
        os.environ["ASP_SPMV_VARIANT"] = args.variant

    h = api.Handle()
    stream = torch.cuda.Stream()
    h.set_stream(stream.cuda_stream)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # every rank builds the same matrix (same seed), takes its nnz-balanced row range and drops the rest
    w = make_workload(args.workload, dev, args.scale)
    full = w["A"]
    g_rows, g_cols, g_nnz = full.rows, full.cols, full.nnz
    nbytes = algorithmic_bytes(w)           # of the whole matrix: x and y counted once, whatever N is
    flops = 2.0 * g_nnz * w["n"]
    spmv = w["kind"] == "spmv"
    ydt = w.get("ydtype", torch.float32 if w["dtype"] == torch.bfloat16 else w["dtype"])
    r0, r1 = 0, g_rows
    bounds = np.array([0, g_rows], dtype=np.int64)
    if world > 1:
        if spmv and g_rows != g_cols:
            raise SystemExit("x is sharded like y: the multi-GPU SpMV bench needs a square matrix")
        with torch.cuda.stream(stream):
            bounds = api.partition_rows_by_nnz(h, full.row_ptr, world)
            Aloc, (r0, r1) = shard_csr(h, full.rows, full.cols, full.row_ptr, full.col_idx, full.val, rank, world)
            A = Csr(r1 - r0, full.cols, Aloc.row_ptr, Aloc.col_idx.clone(), Aloc.val.clone())
        torch.cuda.synchronize()
        del Aloc
    else:
        A = full
    del full
    w["A"] = A
    torch.cuda.empty_cache()
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)

    mode = {"overlap": api.MG_X_WINDOW_OVERLAP, "window": api.MG_X_WINDOW, "allgather": api.MG_X_ALLGATHER,
            "broadcast": api.MG_X_BROADCAST}[args.exchange]
    mg = None
    extras = {}
    if spmv:
        # x is the same vector on every rank's generator; a rank keeps its own part
        x_full = G.uniform((g_cols,), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = G.uniform((g_rows,), -1.0, 1.0, dtype=ydt, device=dev, seed=12)[r0:r1].clone()
        with torch.cuda.stream(stream):
            Am.analyse(h)
        if world > 1:
            if w["dtype"] not in (torch.float32, torch.float64):
                raise SystemExit("the multi-GPU SpMV entry points take fp32 / fp64 matrices")
            mg = api.Mg(h, rank, world)
            with torch.cuda.stream(stream):
                mg.set_shard(Am, bounds, mode, root=0)
            torch.cuda.synchronize()
            if mode == api.MG_X_BROADCAST:
                x_in = x_full if rank == 0 else None
            else:
                try:
                    x_in = mg.own_view()      # a solver keeps its part of x inside the window: a step moves only the halo
                    x_in.copy_(x_full[r0:r1])
                except api.AlphaSparseError:
                    x_in = x_full[r0:r1].clone()
            torch.cuda.synchronize()

            def step():
                mg.spmv(x_in, y, w["alpha"], w["beta"])
        else:
            xd, yd = api.DnVec(x_full), api.DnVec(y)
            buf = torch.empty(api.spmv_buffer_size(h, Am, xd, yd, w["alpha"], w["beta"]), dtype=torch.uint8, device=dev)

            def step():
                api.spmv(h, Am, xd, yd, w["alpha"], w["beta"], buffer=buf)
    else:
        x_full = G.uniform((g_cols, w["n"]), w["lo"], 1.0, dtype=w["dtype"], device=dev, seed=11)
        y = torch.zeros((A.rows, w["n"]), dtype=ydt, device=dev)
        xd, yd = api.DnMat(x_full), api.DnMat(y)
        with torch.cuda.stream(stream):
            api.spmm_preprocess(h, Am, xd, yd)

        def step():
            if world > 1:
                with torch.cuda.stream(stream):
                    dist.broadcast(x_full, src=0)      # X replicated over NVLink inside the step
            api.spmm(h, Am, xd, yd, w["alpha"], w["beta"])
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
        align_ranks(stream)
        ev0.record(stream)
        t_host = time.perf_counter()
        for _ in range(args.steps):
            step()
        t_host = (time.perf_counter() - t_host) / args.steps * 1e3   # host time to enqueue a step (no synchronisation inside)
        ev1.record(stream)
        barrier()
    ms = ev0.elapsed_time(ev1)
    launches = h.launches - l0
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    value = nbytes / (ms_step * 1e-3) / 1e9

    def max_over_ranks(v):
        tt = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    # N > 1, SpMV: the parts of a step, each timed alone (max over ranks)
    if world > 1 and spmv:
        info = mg.info()
        extras["exchange_ms"] = max_over_ranks(time_steps(lambda: mg.exchange(x_in), stream, 20, 3, barrier))

        def bcast():
            with torch.cuda.stream(stream):
                dist.broadcast(x_full, src=0)
        extras["whole_x_broadcast_ms"] = max_over_ranks(time_steps(bcast, stream, 10, 3, barrier))
        # the product alone on this rank's shard with the whole x resident (what a step would cost with a free exchange)
        xd_loc, yd_loc = api.DnVec(x_full), api.DnVec(y)
        extras["spmv_only_ms"] = max_over_ranks(time_steps(
            lambda: api.spmv(h, Am, xd_loc, yd_loc, w["alpha"], w["beta"]), stream, 20, 3, barrier))
        # the exchanged x gives the same y as the whole x resident on the rank (max over ranks of the relative error)
        y_a = torch.zeros_like(y)
        y_b = torch.zeros_like(y)
        with torch.cuda.stream(stream):
            mg.spmv(x_in, y_a, w["alpha"], 0.0)
            api.spmv(h, Am, xd_loc, api.DnVec(y_b), w["alpha"], 0.0)
        torch.cuda.synchronize()
        den = float(y_b.double().norm())
        rel = float((y_a.double() - y_b.double()).norm()) / (den if den > 0 else 1.0)
        extras["exchange_check_rel_l2"] = max_over_ranks(rel)
        extras["exchange_check_ok"] = extras["exchange_check_rel_l2"] <= (1e-12 if w["dtype"] == torch.float64 else 1e-5)
        del y_a, y_b
        extras["x_bytes_received_per_rank"] = info["bytes_received"]
        extras["interior_rows"] = [info["interior_begin"], info["interior_end"]]
        extras["window"] = [info["window_lo"], info["window_hi"]]
        y.copy_(y_init)
        barrier()

    # end to end through the public call with HOST buffers: every step copies its x (this rank's part)
    # and, when beta != 0, its y from pinned host memory, runs the call, and copies y back
    e2e = None
    if not args.no_e2e:
        x_loc = x_full if (world == 1 or not spmv) else x_full[r0:r1]
        hx = torch.empty(x_loc.shape, dtype=x_loc.dtype, pin_memory=True)
        hx.copy_(x_loc)
        reads_y = w["beta"] != 0
        hy_in = None
        if reads_y:
            hy_in = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
            hy_in.copy_(y_init)
        # Two sets of device buffers and three streams: the H2D copies of step i+1, the call of step i
        # and the D2H copy of step i-1 overlap (PCIe is full duplex); every step still moves its own
        # inputs in and its own result out.
        nbuf = 2
        xs = [torch.empty_like(x_loc) for _ in range(nbuf)]
        ys = [y, torch.empty_like(y)]
        hy_outs = [torch.empty(y.shape, dtype=y.dtype, pin_memory=True) for _ in range(nbuf)]
        if spmv and world == 1:
            descs = [(api.DnVec(xs[b]), api.DnVec(ys[b])) for b in range(nbuf)]
        elif not spmv:
            descs = [(api.DnMat(xs[b]), api.DnMat(ys[b])) for b in range(nbuf)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(nbuf)]
        ev_cmp = [torch.cuda.Event() for _ in range(nbuf)]
        ev_out = [torch.cuda.Event() for _ in range(nbuf)]
        sends_x = not (spmv and world > 1 and mode == api.MG_X_BROADCAST and rank != 0)

        def e2e_step(i):
            b = i % nbuf
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_out[b])      # the buffers' previous result has left the device
                if sends_x:
                    xs[b].copy_(hx, non_blocking=True)
                if reads_y:
                    ys[b].copy_(hy_in, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(stream):
                stream.wait_event(ev_in[b])
                if spmv and world > 1:
                    mg.spmv(xs[b] if sends_x else None, ys[b], w["alpha"], w["beta"])
                elif spmv:
                    api.spmv(h, Am, descs[b][0], descs[b][1], w["alpha"], w["beta"], buffer=buf)
                else:
                    if world > 1:
                        dist.broadcast(xs[b], src=0)
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
        align_ranks(s_in)
        e0.record(s_in)
        for i in range(e_steps):
            e2e_step(i)
        e1.record(s_out)
        barrier()
        e_ms = max_over_ranks(e0.elapsed_time(e1)) / e_steps
        h2d = x_loc.numel() * x_loc.element_size() * (1 if sends_x else 0) + (y.numel() * y.element_size() if reads_y else 0)
        d2h = y.numel() * y.element_size()
        tot = torch.tensor([float(h2d), float(d2h)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        e2e = {"value": nbytes / (e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": float(tot[0]), "d2h_bytes_per_step": float(tot[1]),
               "note": "A resident in HBM (like the reference's created matrix handle); every step copies x (each rank its "
                       "own part; + y when beta != 0) from pinned host memory, runs the public call (with the NVLink "
                       "exchange when N > 1) and copies y back; copy-in, call and copy-out of neighbouring steps "
                       "overlap over two buffer sets; bytes are summed over the ranks"}
        del xs, hy_outs, hx
        torch.cuda.empty_cache()

    variant = Am.last_variant() if spmv else api.spmm_last_variant(Am)
    dev_err = Am.plan(h)[0]["device_error"]

    cpu = None
    per_config = None
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            cpu = cpu_baseline_subprocess(args)
        if not args.no_per_config and args.workload == DEFAULT_WORKLOAD and args.scale == 1.0:
            peak, _ = measured_peak()
            per_config = [{"workload": args.workload, "ms": ms_step, "GB/s": value, "frac": value / peak,
                           "variant": variant, "rows": g_rows, "nnz": g_nnz, "n": 1, "algorithmic_bytes": nbytes}]
            # free the headline matrix first: R-MAT 26 needs the memory
            del Am, A, y, y_init, x_full
            w.pop("A", None)
            if spmv:
                del xd, yd
            torch.cuda.empty_cache()
            for name in PER_CONFIG:
                try:
                    per_config.append(one_config(name, h, stream, dev, 20, 5))
                except Exception as ex:
                    per_config.append({"workload": name, "error": f"{type(ex).__name__}: {ex}"[:300]})
                    torch.cuda.empty_cache()

    if rank == 0:
        peak, peak_src = measured_peak()
        ach = (nbytes / world) / (ms_step * 1e-3) / 1e9     # per GPU: its share of the bytes over the step time
        cfg = static_config(args)
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtype_name(w["dtype"]), "data": "synthetic",
            "gflops": flops / (ms_step * 1e-3) / 1e9, "frac_of_nominal_8TBs": value / world / 8000.0,
            "config": cfg,
            "run": {"rows": g_rows, "cols": g_cols, "nnz": g_nnz, "n": w["n"], "alpha": w["alpha"], "beta": w["beta"],
                    "algorithmic_bytes": nbytes, "variant": variant, "device_error": dev_err,
                    "rows_rank0": r1 - r0, "nnz_rank0": (Am.nnz if "Am" in locals() else None),
                    "l2": "inputs larger than L2 (126 MB), no flush" if nbytes / world > 126e6
                          else "L2-resident workload, no flush (the configuration is smaller than L2)",
                    "sharding": ("one GPU, the whole matrix" if world == 1 else
                                 f"one matrix row-partitioned by balanced nnz over {world} GPUs; y sharded; x "
                                 + ({"overlap": "sharded like y, column-window exchange (NCCL send/recv) hidden behind the interior rows",
                                     "window": "sharded like y, column-window exchange (NCCL send/recv), then the product",
                                     "allgather": "sharded like y, all-gathered before the product",
                                     "broadcast": "whole on rank 0, broadcast before the product"}[args.exchange]
                                    if spmv else "replicated by NCCL broadcast inside the step")
                                 + "; the exchange is inside the timed region"),
                    "step_parts_ms": extras or None,
                    "timing": "CUDA events on the launching stream around the K steps, max over ranks"
                              + ("; the ranks meet in a device-side all-reduce on that stream right before the first event "
                                 "(they leave the host barrier up to milliseconds apart)" if world > 1 else "")},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_source": peak_src,
                         "traffic": (TRAFFIC_RATIO[args.workload] * nbytes / world) if args.workload in TRAFFIC_RATIO else None,
                         "traffic_source": "ncu dram__bytes_read+write of the dominant kernel, see profiles/",
                         "note": "achieved = this GPU's share of the algorithmic bytes (x counted once over all GPUs) / "
                                 "time of a whole step" + (", exchange included" if world > 1 else "")},
            "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clk.summary(),
            "host_enqueue_ms_per_step": t_host,
        }
        if per_config is not None:
            line["per_config"] = per_config
        if world > 1:
            line["reference_arm_note"] = "the reference arm is the CPU code on ONE host, not N"
        print(json.dumps(line), flush=True)
    if mg is not None:
        torch.cuda.synchronize()
        mg.close()
    if world > 1:
        dist.barrier()
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
