#!/usr/bin/env python
"""Benchmark of the MACKO SpMV hot path on B200.

Workload (own arm, every N): the Llama-2-7B linear-layer sweep -- 4 shapes x 9 densities =
36 magnitude-pruned fp16 matrices, seeded synthetic stand-ins for the pruned checkpoints the
reference measured. One step = one SpMV on each of the 36 compressed matrices (at N > 1 every
matrix is row-sharded over the ranks, every product delivers its rows of y to all ranks, and the
step ends when every rank holds every full y). Metric = device time of one step in microseconds
(the sum of the 36 SpMV times), lower is better. The step touches ~2.7 GB of distinct compressed
data, far more than the 126 MB L2, so every SpMV streams its matrix from HBM.

Printed JSON line (rank 0, the last line of stdout): the contract keys plus
  y_check       every product of the step (and of the large matrices) compared, outside the timed
                region, with a dense fp32 product of this rank's rows and, at N > 1, bit for bit with
                the NCCL all-gather path; the run exits non-zero if it fails
  roofline      algorithmic bytes of a step / device time, against the measured HBM copy peak
  cpu_baseline  the reference's CPU path (compiled reference compressor + dense torch.mv of the
                decompressed matrix) on a bounded sample, and the reference's own CUDA kernel
                (compiled for sm_100a) on the same 36 matrices
  e2e           the same step through the public Python API with x coming from pinned host
                memory and y copied back to the host inside the timed region
  per_case / sharded_large / skewed / single_4096 / batched / decode   the other configurations
`--impl reference` times the reference's CPU path alone on all 36 matrices (rank 0 only).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "spmv_us_sum_llama7b_sweep"
UNIT = "us"
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per algorithmic byte of one step, from the profiler's launch list of this program
# (profiles/spmv_sweep_launches.md: dram__bytes_read.sum + dram__bytes_write.sum of the 36 launches of a step
# over the step's algorithmic bytes; 24 steps of the capture agree within 0.1 %). A single 32000x4096 product
# at 50 % reads 1.04 (profiles/spmv_kernel_32000x4096_d50.md).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.012
WORKLOAD = ("llama2-7b linear-layer sweep: shapes 4096x4096, 11008x4096, 4096x11008, 32000x4096 x densities "
            "0.1..0.9, per-row magnitude pruning; one step = one SpMV per matrix (36)")


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def load_workloads():
    """The workload generators, loaded from their file: importing the package would also load its native
    libraries, which the reference arm must not have in its process."""
    spec = importlib.util.spec_from_file_location("_macko_workloads", os.path.join(ROOT, "macko_spmv_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        if not out.strip():
            # the loop never got to print (a very short run): one query now, right behind the load
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=10).stdout
            except Exception:
                out = ""
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # the sampler runs over the timed regions and the idle gaps between them: the clock under load is the
        # upper half of the samples
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- helpers

def event_pair():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def time_rotating(launchers, reps):
    """Mean device microseconds of one launch, cycling through `launchers` (distinct buffers,
    together larger than L2) so that every launch streams from HBM."""
    for f in launchers[: min(8, len(launchers))]:
        f()
    torch.cuda.synchronize()
    e0, e1 = event_pair()
    n = len(launchers)
    e0.record()
    for i in range(reps):
        launchers[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / reps


def capture(fn, warm=True):
    """`fn` captured as a CUDA graph, after one eager run on a side stream unless `warm` is False."""
    if warm:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def check_against_dense(y_rows, block, x):
    """True when y (this rank's rows) is within 1e-3 * L1 per row and 5e-3 relative L2 of the dense fp32 product."""
    ref = block.float() @ x.float()
    l1 = block.float().abs() @ x.float().abs()
    err = (y_rows.float() - ref).abs()
    ok_abs = bool((err <= 1e-3 * l1 + 1e-6).all())
    nrm = float(ref.norm())
    ok_l2 = float((y_rows.float() - ref).norm()) <= 5e-3 * nrm + 1e-12
    return ok_abs and ok_l2


def capture_step_graphs(fn, two_halves: bool):
    """The step as one CUDA graph, or, when it goes through the exchange buffers, as two graphs that use the
    two halves of those buffers in turn (every call of `fn` switches to the other half)."""
    graphs = [capture(fn)]
    if two_halves:
        graphs.append(capture(fn, warm=False))
    return graphs


# --------------------------------------------------------------------------- workload

def build_sweep(device, rank: int, world: int):
    """The 36 compressed matrices of the sweep (this rank's row block of each), their x, and the dense
    block (kept for the checks and, at N == 1, for the cuBLAS comparison)."""
    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import sharded, workloads

    cases = []
    t_compress = 0.0
    dense_in_bytes = 0
    for si, (rows, cols) in enumerate(workloads.LLAMA7B_SHAPES):
        for di, d in enumerate(workloads.SWEEP_DENSITIES):
            seed = workloads.sweep_seed(si, di)
            M = workloads.magnitude_pruned_matrix(rows, cols, d, seed, device=device)
            lo, hi = sharded.row_block(rows, rank, world)
            block = M[lo:hi].contiguous()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            comp = macko_spmv.compress(block)
            torch.cuda.synchronize()
            t_compress += time.perf_counter() - t0
            dense_in_bytes += block.numel() * 2
            x = workloads.dense_vector(cols, seed + 500, device)
            cases.append({
                "rows": rows, "cols": cols, "density": d, "comp": comp, "x": x,
                "lo": lo, "hi": hi, "dense": block,
                "bytes": workloads.algorithmic_bytes(comp[0].numel(), hi - lo, cols),
                "dense_bytes": workloads.dense_bytes(hi - lo, cols),
            })
            del M
    return cases, t_compress, dense_in_bytes


def per_case_numbers(cases, lib, peak_gbs):
    """Cold-cache microseconds of our SpMV and of cuBLAS fp16 GEMV for every matrix."""
    from macko_spmv_b200 import cabi

    stream = torch.cuda.current_stream().cuda_stream
    out = []
    for c in cases:
        comp, x = c["comp"], c["x"]
        rows_l = c["hi"] - c["lo"]
        n_copy = max(2, min(48, int(300e6 / c["bytes"]) + 1))
        copies = [comp] + [(comp[0].clone(), comp[1].clone(), comp[2].clone(), comp[3], comp[4]) for _ in range(n_copy - 1)]
        xs = [x] + [x.clone() for _ in range(n_copy - 1)]
        ys = [torch.empty(rows_l, dtype=torch.float16, device=x.device) for _ in range(n_copy)]

        def mk(cc, xx, yy):
            args = (cc[0].data_ptr(), cc[1].data_ptr(), cc[2].data_ptr(), rows_l, c["cols"], cc[0].numel(),
                    xx.data_ptr(), yy.data_ptr(), 1.0, 0.0, cabi.SPMV_MATRIX_IMMUTABLE, stream)
            return lambda: cabi.check(lib, lib.macko_spmv_fp16_ex(*args))

        reps = max(30, min(300, int(1.5e9 / c["bytes"])))
        us = time_rotating([mk(a, b, y) for a, b, y in zip(copies, xs, ys)], reps)
        n_dense = max(2, min(n_copy, int(300e6 / c["dense_bytes"]) + 1))
        dense = [c["dense"]] + [c["dense"].clone() for _ in range(n_dense - 1)]
        us_dense = time_rotating([(lambda m=m, v=v: torch.mv(m, v)) for m, v in zip(dense, xs)],
                                 max(30, min(200, int(1.5e9 / c["dense_bytes"]))))
        out.append({
            "shape": [c["rows"], c["cols"]], "density": c["density"], "us": round(us, 2),
            "roofline_frac": round(c["bytes"] / (us * 1e-6) / 1e9 / peak_gbs, 4),
            "cublas_gemv_us": round(us_dense, 2), "speedup_vs_cublas": round(us_dense / us, 3),
            "target_speedup": round(0.8 / c["density"], 2),
        })
        del copies, xs, ys, dense
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- large row-sharded matrices

def sharded_large_leg(device, rank, world, lib, peer, peak_gbs, reps=40):
    """The two large shapes (12288x49152, 49152x12288; Bernoulli masks at densities 0.1 and 0.5), each rank
    holding a contiguous row block, the full y delivered to every rank. The four products run back to back
    (together they stream more than L2 holds on every rank up to 8 GPUs) as one CUDA graph, max over ranks;
    per-product times come from eager launches between events. Every full y is checked first. At one GPU the
    cuBLAS fp16 GEMV on the dense matrix is timed beside each product, and the planned launch as well."""
    import torch.distributed as dist

    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi, sharded, workloads

    cases = []
    for si, (rows, cols) in enumerate(workloads.SHARDED_SHAPES):
        for d in (0.1, 0.5):
            seed = 7000 + 10 * si + int(round(d * 10))
            M = workloads.bernoulli_matrix(rows, cols, d, seed, device=device, scale=0.02)
            lo, hi = sharded.row_block(rows, rank, world)
            block = M[lo:hi].contiguous()
            del M
            comp = macko_spmv.compress(block)
            x = workloads.dense_vector(cols, seed + 500, device)
            blocks = [sharded.row_block(rows, r, world) for r in range(world)]
            gemv_us = None
            if world == 1:
                for _ in range(3):
                    torch.mv(block, x)
                e0, e1 = event_pair()
                e0.record()
                for _ in range(10):
                    torch.mv(block, x)
                e1.record()
                torch.cuda.synchronize()
                gemv_us = e0.elapsed_time(e1) * 100.0
            cases.append({"rows": rows, "cols": cols, "density": d, "x": x, "gemv_us": gemv_us, "lo": lo, "hi": hi,
                          "shard": sharded.RowShard(comp, lo, hi, rows, blocks), "block": block,
                          "frozen": macko_spmv.freeze(comp, plan=True) if world == 1 else None,
                          "y": torch.empty(rows, dtype=torch.float16, device=device) if world == 1 else None,
                          "bytes": workloads.algorithmic_bytes(comp[0].numel(), hi - lo, cols)})
    torch.cuda.empty_cache()
    flag = cabi.SPMV_MATRIX_IMMUTABLE

    def step(planned=False):
        if peer is not None:
            peer.begin_step()
            ys = [peer.multiply_deferred(c["shard"], c["x"], immutable=True) for c in cases]
            peer.wait()
            return ys
        stream = torch.cuda.current_stream().cuda_stream   # read at call time: differs under graph capture
        for c in cases:
            if planned:
                macko_spmv.multiply(c["frozen"], c["x"])
            else:
                comp = c["shard"].compressed
                cabi.check(lib, lib.macko_spmv_fp16_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4],
                                                       comp[0].numel(), c["x"].data_ptr(), c["y"].data_ptr(), 1.0, 0.0, flag, stream))
        return [c["y"] for c in cases]

    # ---- check every full y (outside any timed region)
    ys = step()
    torch.cuda.synchronize()
    ok = True
    for c, y in zip(cases, ys):
        ok = ok and check_against_dense(y[c["lo"]:c["hi"]], c["block"], c["x"])
        if world > 1:
            ok = ok and torch.equal(y, sharded.multiply_sharded(c["shard"], c["x"]))
        if world == 1:
            ok = ok and check_against_dense(macko_spmv.multiply(c["frozen"], c["x"]), c["block"], c["x"])
    for c in cases:
        c["block"] = None
    torch.cuda.empty_cache()

    def time_graphs(graphs):
        for i in range(4):
            graphs[i % len(graphs)].replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = event_pair()
        e0.record()
        for i in range(reps):
            graphs[i % len(graphs)].replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / reps], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    graphs = capture_step_graphs(step, peer is not None)
    graph_us = time_graphs(graphs)
    planned_us = None
    if world == 1:
        planned_us = time_graphs([capture(lambda: step(planned=True))])
    if world > 1:
        dist.barrier()
    # per-product times: eager launches between events (they include host launch gaps for short products)
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(cases) + 1)] for _ in range(reps)]
    for r in range(reps):
        if peer is not None:
            peer.begin_step()
        marks[r][0].record()
        for i, c in enumerate(cases):
            if peer is not None:
                peer.multiply_deferred(c["shard"], c["x"], immutable=True)
            else:
                comp = c["shard"].compressed
                cabi.check(lib, lib.macko_spmv_fp16_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4],
                                                       comp[0].numel(), c["x"].data_ptr(), c["y"].data_ptr(), 1.0, 0.0, flag,
                                                       torch.cuda.current_stream().cuda_stream))
            marks[r][i + 1].record()
        if peer is not None:
            peer.wait()
    torch.cuda.synchronize()
    us = torch.tensor([[marks[r][i].elapsed_time(marks[r][i + 1]) * 1000.0 for i in range(len(cases))] for r in range(reps)],
                      device=device).mean(dim=0)
    if world > 1:
        dist.all_reduce(us, op=dist.ReduceOp.MAX)
    out = []
    for c, t in zip(cases, us.tolist()):
        row = {"shape": [c["rows"], c["cols"]], "density": c["density"], "us": round(t, 2),
               "per_gpu_roofline_frac": round(c["bytes"] / (t * 1e-6) / 1e9 / peak_gbs, 4)}
        if world == 1:
            row["cublas_gemv_us"] = round(c["gemv_us"], 2)
            row["speedup_vs_cublas"] = round(c["gemv_us"] / t, 3)
            row["plan_recommended"] = bool(c["frozen"].plan_meta[4])
        out.append(row)
    total_bytes = sum(c["bytes"] for c in cases)
    return {"cases": out, "us_sum_eager": round(sum(r["us"] for r in out), 2), "us_sum_graph": round(graph_us, 2),
            "us_sum_graph_planned_launch": None if planned_us is None else round(planned_us, 2),
            "per_gpu_roofline_frac_graph": round(total_bytes / (graph_us * 1e-6) / 1e9 / peak_gbs, 4),
            "y_ok": ok}


# --------------------------------------------------------------------------- skewed rows, single product

def time_one_matrix(launch, comp, x, reps=None):
    """Cold microseconds of `launch(comp_copy, x, y)` over rotating copies of the matrix (together > 2 x L2)."""
    from macko_spmv_b200 import workloads

    rows, cols = comp[3], comp[4]
    nbytes = workloads.algorithmic_bytes(comp[0].numel(), rows, cols)
    n_copy = max(2, min(48, int(300e6 / nbytes) + 1))
    copies = [comp] + [(comp[0].clone(), comp[1].clone(), comp[2].clone(), rows, cols) for _ in range(n_copy - 1)]
    ys = [torch.empty(rows, dtype=torch.float16, device=x.device) for _ in range(n_copy)]
    fns = [launch(c, x, y) for c, y in zip(copies, ys)]
    return time_rotating(fns, reps or max(30, min(300, int(1.5e9 / nbytes)))), nbytes, ys[0]


def skewed_leg(device, lib, peak_gbs):
    """The two skewed-density shapes: rows from empty to fully dense, clustered non-zeros. Default launch,
    planned launch (what `freeze` picks for such a matrix) and cuBLAS fp16 GEMV on the dense matrix."""
    import ctypes

    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi, workloads

    stream = torch.cuda.current_stream().cuda_stream
    out = []
    for si, (rows, cols) in enumerate(workloads.SKEWED_SHAPES):
        M = workloads.skewed_matrix(rows, cols, seed=5000 + si, device=device)
        x = workloads.dense_vector(cols, 5500 + si, device)
        comp = macko_spmv.compress(M)

        def plain(c, xx, y):
            args = (c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr(), rows, cols, c[0].numel(), xx.data_ptr(), y.data_ptr(),
                    1.0, 0.0, cabi.SPMV_MATRIX_IMMUTABLE, stream)
            return lambda: cabi.check(lib, lib.macko_spmv_fp16_ex(*args))

        keep = []

        def planned(c, xx, y):
            nb = lib.macko_spmv_plan_bytes(rows, cols, c[0].numel(), 0)
            plan = torch.empty(nb, dtype=torch.uint8, device=device)
            info = cabi.PlanInfo()
            cabi.check(lib, lib.macko_spmv_plan(c[1].data_ptr(), c[2].data_ptr(), rows, cols, c[0].numel(), 0, plan.data_ptr(), nb,
                                                ctypes.byref(info), stream))
            keep.append((plan, info))
            args = (c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr(), rows, cols, c[0].numel(), plan.data_ptr(),
                    ctypes.byref(info), xx.data_ptr(), y.data_ptr(), 1.0, 0.0, cabi.SPMV_MATRIX_IMMUTABLE, stream)
            return lambda: cabi.check(lib, lib.macko_spmv_fp16_planned(*args))

        us_plain, nbytes, y_plain = time_one_matrix(plain, comp, x)
        ok = check_against_dense(y_plain, M, x)
        us_planned, _, y_planned = time_one_matrix(planned, comp, x)
        ok = ok and check_against_dense(y_planned, M, x)
        info = keep[0][1]
        dense = [M, M.clone()]
        us_dense = time_rotating([(lambda m=m: torch.mv(m, x)) for m in dense], 40)
        out.append({"shape": [rows, cols], "stored_elements": comp[0].numel(), "longest_row": info.longest_row,
                    "virtual_rows": info.virtual_rows, "plan_recommended": bool(info.recommended),
                    "default_launch_us": round(us_plain, 2), "planned_launch_us": round(us_planned, 2),
                    "roofline_frac_default": round(nbytes / (us_plain * 1e-6) / 1e9 / peak_gbs, 4),
                    "roofline_frac_planned": round(nbytes / (us_planned * 1e-6) / 1e9 / peak_gbs, 4),
                    "cublas_gemv_us": round(us_dense, 2), "y_ok": ok})
        del M, dense, keep
        torch.cuda.empty_cache()
    return out


def single_4096_leg(device, lib, peak_gbs):
    """One 4096x4096 product: values N(0,1), Bernoulli(0.5) mask, x N(0,1), seed 1001 (CPU generator);
    compress then multiply, checked against the dense fp32 product computed on the CPU."""
    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi

    g = torch.Generator().manual_seed(1001)
    W = torch.randn(4096, 4096, generator=g).half()
    mask = torch.rand(4096, 4096, generator=g) < 0.5
    M_cpu = W * mask
    x_cpu = torch.randn(4096, generator=g).half()
    M, x = M_cpu.to(device), x_cpu.to(device)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    comp = macko_spmv.compress(M)
    torch.cuda.synchronize()
    t_comp = time.perf_counter() - t0
    stream = torch.cuda.current_stream().cuda_stream

    def plain(c, xx, y):
        args = (c[0].data_ptr(), c[1].data_ptr(), c[2].data_ptr(), 4096, 4096, c[0].numel(), xx.data_ptr(), y.data_ptr(),
                1.0, 0.0, cabi.SPMV_MATRIX_IMMUTABLE, stream)
        return lambda: cabi.check(lib, lib.macko_spmv_fp16_ex(*args))

    us, nbytes, y = time_one_matrix(plain, comp, x)
    ref = M_cpu.float() @ x_cpu.float()
    err = float((y.float().cpu() - ref).norm() / ref.norm())
    return {"shape": [4096, 4096], "density": 0.5, "mask": "Bernoulli", "us_cold": round(us, 2),
            "roofline_frac": round(nbytes / (us * 1e-6) / 1e9 / peak_gbs, 4), "compress_ms": round(t_comp * 1e3, 3),
            "rel_l2_vs_cpu_fp32": err, "y_ok": err <= 5e-3}


# --------------------------------------------------------------------------- several right-hand sides

def batched_leg(device):
    """The 11008x4096 layer at density 0.5 with several right-hand sides: one pass over the compressed
    matrix per 8 vectors (`multiply_batched`) against a loop of single-vector products, and the dense-copy
    route for a prefill-sized batch. Microseconds per call, same matrix every call (warm L2 where it fits)."""
    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import workloads

    rows, cols = 11008, 4096
    comp = macko_spmv.compress(workloads.magnitude_pruned_matrix(rows, cols, 0.5, 2913, device=device))

    def timed(fn, reps=40):
        for _ in range(3):
            fn()
        e0, e1 = event_pair()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) * 1000.0 / reps, 2)

    out = {"shape": [rows, cols], "density": 0.5}
    V = torch.randn(128, cols, device=device).half()
    out["single_us"] = timed(lambda: macko_spmv.multiply(comp, V[0]))
    for b in (2, 4, 8, 16):
        Vb = V[:b].contiguous()
        out[f"batched_{b}_us"] = timed(lambda: macko_spmv.multiply_batched(comp, Vb))   # the API's own routing
    V16 = V[:16].contiguous()
    out["two_passes_16_us"] = timed(lambda: torch.ops.macko_spmv.multiply_batched.default(*comp[:5], V16))
    out["dense_route_16_us"] = timed(lambda: V16 @ macko_spmv.decompress(comp).t())
    V8 = V[:8].contiguous()
    out["loop_of_8_us"] = timed(lambda: [macko_spmv.multiply(comp, V8[i]) for i in range(8)])
    out["prefill_128_dense_route_us"] = timed(lambda: macko_spmv.multiply_batched(comp, V))
    return out



# --------------------------------------------------------------------------- value types

def value_types_leg(device, peak_gbs):
    """The 11008x4096 layer at density 0.5 in the three value types of the format: fp16 (the reference's),
    bfloat16 (values, x and y) and int8 values with fp16 vectors (the reference's int8 variant). Cold (rotating
    copies larger than L2), matrices declared immutable, graph replay; microseconds per product and fraction
    of the measured peak on each type's own algorithmic bytes; y checked against a dense fp32 product."""
    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import workloads

    rows, cols = 11008, 4096
    W = workloads.magnitude_pruned_matrix(rows, cols, 0.5, 2914, device=device)
    x16 = workloads.dense_vector(cols, 2915, device)
    out = {"shape": [rows, cols], "density": 0.5}
    variants = {
        "fp16": (W, x16),
        "bf16": (W.to(torch.bfloat16), x16.to(torch.bfloat16)),
        "int8": (torch.clamp((W.float() * 2000.0).round(), -127, 127).to(torch.int8), x16),
    }
    for name, (M, x) in variants.items():
        comp = macko_spmv.compress(M.contiguous())
        stored = comp[0].numel()
        value_bytes = 1 if name == "int8" else 2
        nbytes = (value_bytes + 0.5) * stored + 4 * (rows + 1) + 2 * cols + 2 * rows
        ncopy = max(2, int(300e6 / nbytes) + 1)
        copies = [macko_spmv.freeze(comp, plan=False)] + [
            macko_spmv.freeze((comp[0].clone(), comp[1].clone(), comp[2].clone(), rows, cols), plan=False) for _ in range(ncopy - 1)]
        ys = [torch.empty(rows, dtype=x.dtype, device=device) for _ in range(ncopy)]

        def step():
            for c, y in zip(copies, ys):
                macko_spmv.multiply(c, x, out=y)
        g = capture(step)
        for _ in range(3):
            g.replay()
        e0, e1 = event_pair()
        e0.record()
        for _ in range(20):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1000.0 / (20 * ncopy)
        ref = M.float() @ x.float()
        rel = float((ys[0].float() - ref).norm() / ref.norm())
        out[name] = {"us": round(us, 2), "algorithmic_bytes": int(nbytes), "roofline_frac": round(nbytes / us / 1e3 / peak_gbs, 4),
                     "rel_l2_vs_dense_fp32": rel, "y_ok": rel < (2e-2 if name == "bf16" else 5e-3)}
        del g, copies, ys, comp
        torch.cuda.empty_cache()
    return out

# --------------------------------------------------------------------------- decode

def decode_leg(device, world, peer_factory, densities, layers, prompt, new_tokens):
    """Batch-1 decode of the Llama-2-7B architecture (random weights, every linear layer pruned per row and
    run through `multiply`): tokens per second for each density; 1.0 = dense nn.Linear (cuBLAS), one GPU only."""
    import torch.distributed as dist

    from macko_spmv_b200 import llama_decode

    out = {"layers": layers, "prompt_tokens": prompt, "new_tokens": new_tokens, "tensor_parallel": world, "tokens_per_s": {}}
    for d in densities:
        if d >= 1.0 and world > 1:
            continue
        peer = peer_factory() if world > 1 else None
        with torch.no_grad():
            model = llama_decode.LlamaDecoder(d, layers=layers, device=device, max_len=prompt + new_tokens, peer=peer)
            g = torch.Generator(device=device).manual_seed(4001)
            tokens = torch.randint(0, model.cfg["vocab"], (prompt,), generator=g, device=device)
            if world > 1:
                dist.barrier()
            _, gen_s, _ = llama_decode.generate(model, tokens, new_tokens)
        if world > 1:
            t = torch.tensor([gen_s], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            gen_s = float(t.item())
        out["tokens_per_s"]["dense" if d >= 1.0 else f"d{d}"] = round(new_tokens / gen_s, 1)
        del model
        if peer is not None:
            peer.close()
        torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- CPU reference path

def cpu_reference_cases(limit_shapes=None):
    """The reference's CPU path for the sweep: the matrices of the own arm (same seeds; generated on the GPU
    when one is visible, like the own arm does, else on the CPU), compressed by the reference's own host
    compressor (compiled, unmodified; else the oracle port), decompressed, and held as dense fp32 for torch.mv."""
    import numpy as np

    import oracle

    workloads = load_workloads()
    kind = "reference" if oracle.have_reference() else "port"
    compress = oracle.ref_compress if kind == "reference" else oracle.compress
    gen_device = "cuda" if torch.cuda.is_available() else "cpu"
    sample = []
    t_comp = 0.0
    shapes = list(enumerate(workloads.LLAMA7B_SHAPES))
    if limit_shapes is not None:
        shapes = shapes[:limit_shapes]
    for si, (rows, cols) in shapes:
        for di, d in enumerate(workloads.SWEEP_DENSITIES):
            seed = workloads.sweep_seed(si, di)
            M = workloads.magnitude_pruned_matrix(rows, cols, d, seed, device=gen_device).cpu()
            x = workloads.dense_vector(cols, seed + 500, gen_device).cpu().float()
            dense_bits = M.numpy().view(np.uint16)
            t0 = time.perf_counter()
            comp = compress(dense_bits)
            t_comp += time.perf_counter() - t0
            dec = torch.from_numpy(oracle.decompress(comp).view(np.float16).copy()).float()
            sample.append((dec, x))
            del M, dense_bits, comp
    return sample, t_comp, kind, gen_device


def cpu_reference_path(steps: int, warmup: int, limit_shapes=None):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)   # a launcher may have set OMP_NUM_THREADS=1 for its ranks; this arm is the only one computing
    sample, t_comp, kind, gen_device = cpu_reference_cases(limit_shapes)

    def one_step():
        for dec, x in sample:
            torch.mv(dec, x)

    for _ in range(max(warmup, 1)):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    t_mv = (time.perf_counter() - t0) / steps
    full = limit_shapes is None
    return {
        "value": t_mv * 1e6, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
        "sample": (f"all {len(sample)} matrices of the sweep" if full else f"{len(sample)} of the 36 matrices (the first {limit_shapes} shapes)")
                  + ": torch.mv fp32 of the matrix decompressed from the reference compressor's output, every step; "
                  f"matrices generated on {gen_device} with the own arm's seeds",
        "complete_workload": full,
        "compress_us": t_comp * 1e6, "compress_threads": 1,
        "spmv_plus_compress_us": (t_mv + t_comp) * 1e6,
    }


def reference_gpu_kernel_times(gpu_cases):
    """Baseline only: the reference's own CUDA kernel (compiled unmodified for sm_100a into oracle/_ref)
    on compressed matrices that already sit on the device, timed like the per-case numbers (rotating
    cold copies). `gpu_cases`: dicts with "comp" (device 5-tuple), "x", "rows", "cols", "density"."""
    import oracle

    stream = torch.cuda.current_stream().cuda_stream
    out = []
    for c in gpu_cases:
        comp, x = c["comp"], c["x"]
        rows, cols = comp[3], comp[4]
        if rows % 32 != 0:
            continue   # the reference kernel reads past row_indices for such shapes
        nbytes = 2.5 * comp[0].numel()
        n_copy = max(2, min(48, int(300e6 / max(nbytes, 1)) + 1))
        copies = [comp[:3]] + [tuple(t.clone() for t in comp[:3]) for _ in range(n_copy - 1)]
        ys = [torch.empty(rows, dtype=torch.float16, device=x.device) for _ in range(n_copy)]
        fns = [(lambda k=k, y=y: oracle.ref_spmv_gpu(k[0].data_ptr(), k[1].data_ptr(), k[2].data_ptr(), x.data_ptr(),
                                                    y.data_ptr(), rows, cols, stream)) for k, y in zip(copies, ys)]
        reps = max(30, min(200, int(1.5e9 / max(nbytes, 1))))
        out.append({"shape": [rows, cols], "density": c["density"], "us": round(time_rotating(fns, reps), 2)})
        del copies, ys
    torch.cuda.empty_cache()
    return {"kernel": "macko_spmv<false> of the reference, nvcc -arch sm_100a, reference launch shape",
            "sum_us": round(sum(o["us"] for o in out), 1), "cases": out}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpu_reference_path(max(args.steps, 1), max(args.warmup, 1))
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["value"] / 1000.0,
        "higher_is_better": False, "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32",
        "data": "synthetic",
        "config": {"workload": WORKLOAD},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- own arm

def run_own_arm(args):
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path is a CUDA kernel and has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi, sharded, workloads

    lib = cabi.load()
    peak_gbs, peak_kind = measured_hbm_peak()
    cases, t_compress, dense_in_bytes = build_sweep(device, rank, world)
    n_cases = len(cases)
    step_bytes = sum(c["bytes"] for c in cases)
    shards = [sharded.RowShard(c["comp"], c["lo"], c["hi"], c["rows"],
                               [sharded.row_block(c["rows"], r, world) for r in range(world)]) for c in cases]
    rows8 = lambda r: (r + 7) // 8 * 8
    step_rows = max(sum(rows8(c["rows"]) for c in cases), sum(rows8(r) for r, _ in workloads.SHARDED_SHAPES) * 2)
    peer = None
    if world > 1 and args.exchange in ("peer", "peer-fused"):
        peer = sharded.PeerGather(max(c["rows"] for c in cases), device, step_rows=step_rows,
                                  overlap_forward=(args.exchange == "peer"))
    ys_local = [torch.empty(c["hi"] - c["lo"], dtype=torch.float16, device=device) for c in cases]
    ys_full = [torch.empty(c["rows"], dtype=torch.float16, device=device) for c in cases] if world > 1 else ys_local
    flag = cabi.SPMV_MATRIX_IMMUTABLE   # the matrices are weights: compressed at set-up, never written again

    def step_device():
        """One step on the device: N == 1 the C ABI product per matrix; N > 1 the product with the exchange fused
        into it (every rank's slice stored into all ranks' y, arrival published, no wait) and one bounded wait
        for all 36 at the end, or (--exchange nccl) product + all-gather per matrix."""
        if peer is not None:
            peer.begin_step()
            out = [peer.multiply_deferred(sh, c["x"], immutable=True) for sh, c in zip(shards, cases)]
            peer.wait()
            return out
        stream = torch.cuda.current_stream().cuda_stream
        for c, yl, yf in zip(cases, ys_local, ys_full):
            comp = c["comp"]
            cabi.check(lib, lib.macko_spmv_fp16_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(),
                                                   c["hi"] - c["lo"], c["cols"], comp[0].numel(),
                                                   c["x"].data_ptr(), yl.data_ptr(), 1.0, 0.0, flag, stream))
            if world > 1:
                dist.all_gather_into_tensor(yf, yl)
        return ys_full

    # ---- every y of the step checked before anything is timed --------------------------------------
    ys = step_device()
    torch.cuda.synchronize()
    ok = True
    for c, sh, y in zip(cases, shards, ys):
        ok = ok and check_against_dense(y[c["lo"]:c["hi"]], c["dense"], c["x"])
        if world > 1 and peer is not None:
            ok = ok and torch.equal(y, sharded.multiply_sharded(sh, c["x"]))
    y_cases = n_cases

    # ---- the step as CUDA graph(s): at N > 1 two graphs, one per half of the exchange buffers ------
    graphs = None
    try:
        graphs = capture_step_graphs(step_device, peer is not None)
        run_step = lambda i: graphs[i % len(graphs)].replay()
    except Exception:  # a collective that cannot be captured: time eager launches instead
        graphs = None
        run_step = lambda i: step_device()
    used_graph = graphs is not None
    # the sampler starts in front of the warm-up steps (the same load): nvidia-smi needs some tens of
    # milliseconds before its first line, more than the timed region lasts
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        run_step(i)
    torch.cuda.synchronize()

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = event_pair()
    e0.record()
    for i in range(args.steps):
        run_step(i)
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms_total = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_total], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps

    # the same step without the immutable-matrix flag (N == 1), for comparison
    plain_us = None
    if world == 1:
        def step_plain():
            stream = torch.cuda.current_stream().cuda_stream
            for c, yl in zip(cases, ys_local):
                comp = c["comp"]
                cabi.check(lib, lib.macko_spmv_fp16(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), c["rows"], c["cols"],
                                                    comp[0].numel(), c["x"].data_ptr(), yl.data_ptr(), 1.0, 0.0, stream))
        gp = capture(step_plain)
        for _ in range(3):
            gp.replay()
        e0.record()
        for _ in range(args.steps):
            gp.replay()
        e1.record()
        torch.cuda.synchronize()
        plain_us = e0.elapsed_time(e1) * 1000.0 / args.steps
        del gp

    # ---- end to end through the public API with host buffers ------------------------------------
    # Every step: x of all 36 products from pinned host memory (one arena, one copy), the products through
    # macko_spmv_b200.multiply on views of the device arena, every y back to pinned host memory (one copy).
    x_off, y_off = [0], [0]
    for c in cases:
        x_off.append(x_off[-1] + rows8(c["cols"]))
        y_off.append(y_off[-1] + rows8(c["rows"]))
    x_host = torch.zeros(x_off[-1], dtype=torch.float16).pin_memory()
    for c, o in zip(cases, x_off):
        x_host[o:o + c["cols"]] = c["x"].cpu()
    x_dev = torch.empty(x_off[-1], dtype=torch.float16, device=device)
    y_dev = torch.zeros(y_off[-1], dtype=torch.float16, device=device)
    y_host = torch.zeros(max(y_off[-1], step_rows), dtype=torch.float16).pin_memory()
    frozen = [macko_spmv.freeze(c["comp"], plan=False) for c in cases]

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        if peer is not None:
            peer.begin_step()
            for c, sh, o in zip(cases, shards, x_off):
                peer.multiply_deferred(sh, x_dev[o:o + c["cols"]], immutable=True)
            peer.wait()
            half = peer.buf[peer._half]
            y_host[: half.numel()].copy_(half, non_blocking=True)
        elif world > 1:
            for c, sh, o, yo in zip(cases, shards, x_off, y_off):
                sharded.multiply_sharded(sh, x_dev[o:o + c["cols"]], out=y_dev[yo:yo + c["rows"]])
            y_host[: y_dev.numel()].copy_(y_dev, non_blocking=True)
        else:
            for c, fz, o, yo in zip(cases, frozen, x_off, y_off):
                macko_spmv.multiply(fz, x_dev[o:o + c["cols"]], out=y_dev[yo:yo + c["rows"]])
            y_host[: y_dev.numel()].copy_(y_dev, non_blocking=True)

    # The same step with the copies beside the products (one GPU): the matrices in four groups (the shapes, the
    # one with the longest y first), every group's x on one copy stream as soon as the step starts, its products
    # on the main stream once its x is there, its y back on a second copy stream while the next group multiplies.
    h2d_stream = torch.cuda.Stream(device=device)
    d2h_stream = torch.cuda.Stream(device=device)
    group_size = len(workloads.SWEEP_DENSITIES)
    groups = [list(range(g, min(g + group_size, n_cases))) for g in range(0, n_cases, group_size)][::-1]

    def step_e2e_pipelined():
        main = torch.cuda.current_stream()
        h2d_stream.wait_stream(main)
        d2h_stream.wait_stream(main)
        arrived = []
        with torch.cuda.stream(h2d_stream):
            for g in groups:
                lo, hi = x_off[g[0]], x_off[g[-1] + 1]
                x_dev[lo:hi].copy_(x_host[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(h2d_stream)
                arrived.append(ev)
        for g, ev in zip(groups, arrived):
            main.wait_event(ev)
            for k in g:
                c = cases[k]
                macko_spmv.multiply(frozen[k], x_dev[x_off[k]:x_off[k] + c["cols"]], out=y_dev[y_off[k]:y_off[k] + c["rows"]])
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(d2h_stream):
                d2h_stream.wait_event(done)
                lo, hi = y_off[g[0]], y_off[g[-1] + 1]
                y_host[lo:hi].copy_(y_dev[lo:hi], non_blocking=True)
        main.wait_stream(h2d_stream)
        main.wait_stream(d2h_stream)

    xs_host = [c["x"].cpu().pin_memory() for c in cases]
    ys_host = [torch.empty(c["rows"], dtype=torch.float16).pin_memory() for c in cases]

    def step_e2e_per_product_copies():
        for c, xh, yh in zip(cases, xs_host, ys_host):
            xd = xh.to(device, non_blocking=True)
            yh.copy_(macko_spmv.multiply(c["comp"], xd), non_blocking=True)

    def time_e2e(run):
        for i in range(4):
            run(i)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        n = max(4, min(args.steps, 20))
        e0.record()
        for i in range(n):
            run(i)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    e2e_eager_ms = time_e2e(lambda i: step_e2e())
    e2e_graph_ms = None
    try:
        ge = capture_step_graphs(step_e2e, peer is not None)
        y_host.zero_()
        e2e_graph_ms = time_e2e(lambda i: ge[i % len(ge)].replay())
        del ge
    except Exception:   # a capture the runtime refuses: the eager figure stands
        e2e_graph_ms = None
    # what arrived on the host is the step's y (product 4 and the last one, this rank's rows)
    torch.cuda.synchronize()
    for k in (4, n_cases - 1):
        c = cases[k]
        if peer is not None:
            o = sum(rows8(cc["rows"]) for cc in cases[:k])
        else:
            o = y_off[k]
        got = y_host[o:o + c["rows"]].to(device)
        ok = ok and check_against_dense(got[c["lo"]:c["hi"]], c["dense"], c["x"])
    e2e_ms = e2e_eager_ms if e2e_graph_ms is None else min(e2e_eager_ms, e2e_graph_ms)
    e2e_pipelined_ms = None
    if world == 1:
        y_host.zero_()
        e2e_pipelined_ms = time_e2e(lambda i: step_e2e_pipelined())
        try:
            gp2 = capture(step_e2e_pipelined)
            e2e_pipelined_ms = min(e2e_pipelined_ms, time_e2e(lambda i: gp2.replay()))
            del gp2
        except Exception:   # a capture the runtime refuses: the eager figure stands
            pass
        torch.cuda.synchronize()
        for k in (4, n_cases - 1):
            c = cases[k]
            got = y_host[y_off[k]:y_off[k] + c["rows"]].to(device)
            ok = ok and check_against_dense(got[c["lo"]:c["hi"]], c["dense"], c["x"])
        e2e_ms = min(e2e_ms, e2e_pipelined_ms)
    e2e_per_product_ms = time_e2e(lambda i: step_e2e_per_product_copies()) if world == 1 else None
    clocks = sampler.stop() if rank == 0 else None

    per_case = per_case_numbers(cases, lib, peak_gbs) if (world == 1 and not args.no_per_case) else None
    ref_gpu = None
    if world == 1 and not args.no_cpu_baseline:
        import oracle
        if oracle.have_reference_kernel():
            ref_gpu = reference_gpu_kernel_times(cases)
    for c in cases:
        c["dense"] = None
    torch.cuda.empty_cache()

    large = None
    if not args.no_sharded_large and (world == 1 or peer is not None):
        large = sharded_large_leg(device, rank, world, lib, peer, peak_gbs)
        ok = ok and large.pop("y_ok")
        y_cases += len(large["cases"])
    skewed = skewed_leg(device, lib, peak_gbs) if (world == 1 and not args.no_skewed) else None
    single = single_4096_leg(device, lib, peak_gbs) if world == 1 else None
    if skewed is not None:
        ok = ok and all(s["y_ok"] for s in skewed)
    if single is not None:
        ok = ok and single["y_ok"]
    batched = batched_leg(device) if (world == 1 and not args.no_batched) else None
    value_types = value_types_leg(device, peak_gbs) if (world == 1 and not args.no_batched) else None
    if value_types is not None:
        ok = ok and all(value_types[k]["y_ok"] for k in ("fp16", "bf16", "int8"))

    # ---- peer error flag and verdict of the checks, over all ranks ------------------------------
    peer_flag = peer.error_flag() if peer is not None else 0
    verdict = torch.tensor([1 if ok else 0, -peer_flag], device=device, dtype=torch.int64)
    if world > 1:
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN)
    ok_all, peer_flag_all = bool(verdict[0].item()), int(-verdict[1].item())

    decode = None
    if not args.no_decode:
        del graphs
        graphs = None
        dens = (0.5, 0.1, 1.0) if world == 1 else (0.5, 0.1)
        cfg_rows = max(world * 4096, 32000)   # N partial hidden vectors of a column-sharded layer, or the logits
        decode = decode_leg(device, world, lambda: sharded.PeerGather(cfg_rows, device), dens, args.decode_layers,
                            args.decode_prompt, args.decode_tokens)

    cpu_base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu_base = cpu_reference_path(3, 1, limit_shapes=1)   # bounded: the 4096x4096 layer at the 9 densities
        scale = sum(r * c for r, c in workloads.LLAMA7B_SHAPES) / float(4096 * 4096)
        cpu_base["value_sample_us"] = cpu_base["value"]
        cpu_base["value"] = cpu_base["value"] * scale
        cpu_base["sample"] += f"; value = the sample's time x {scale:.2f} (dense elements of the whole sweep over the sample's)"
        if ref_gpu is not None:
            cpu_base["reference_gpu_kernel_sum_us"] = ref_gpu["sum_us"]
            cpu_base["reference_gpu_kernel"] = ref_gpu

    line = None
    if rank == 0:
        achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
        launches_per_step = n_cases + (0 if peer is None else (n_cases + 1 if peer.overlap_forward else 1))
        large_fracs = [c["per_gpu_roofline_frac"] for c in large["cases"]] if large else []
        if per_case:
            large_fracs += [p["roofline_frac"] for p in per_case if p["shape"][0] * p["shape"][1] >= 8192 * 8192]
        line = {
            "metric": METRIC, "value": ms_per_step * 1000.0, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
            "config": {
                "workload": WORKLOAD,
                "parallelism": "single GPU" if world == 1 else (f"rows of every matrix split over {world} GPUs; " + (("every SpMV writes its rows into this rank's y; a forward kernel on a graph branch copies them into all ranks' y over NVLink and publishes the arrival beside the next products; one bounded wait per step for all 36 (no collective)" if peer.overlap_forward else "every SpMV kernel stores its y slice into all ranks' y over NVLink and publishes its arrival; one bounded wait per step for all 36 (no collective)") if peer is not None else "NCCL all-gather of y after each SpMV")),
                "l2": "inputs larger than L2: a step streams %.2f GB of distinct compressed data per GPU, each matrix once" % (step_bytes / 1e9),
                "launch": ("one CUDA graph per step" if used_graph else "eager launches")
                          + "; matrices declared immutable (weights compressed at set-up): first matrix loads may precede the end of the previous kernel",
            },
            "y_check": {"cases": y_cases, "ok": ok_all, "peer_error_flag": peer_flag_all,
                        "what": "every product of the step and of the large matrices: this rank's rows against a dense fp32 product "
                                "(1e-3*L1 per row, 5e-3 relative L2)" + ("; full y bit-equal to the NCCL all-gather path" if peer is not None else "")},
            "roofline": {
                "bound": "hbm", "achieved": round(achieved, 1), "peak": peak_gbs, "unit": "GB/s",
                "frac": round(achieved / peak_gbs, 4),
                "traffic": int(step_bytes * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE) if world == 1 else None,
                "traffic_source": "dram bytes per algorithmic byte (1.012) of the 36 launches of a step in the profiler's launch "
                                  "list of this program (profiles/spmv_sweep_launches.md), times the step's algorithmic bytes; "
                                  "not measured in this run",
                "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_step_per_gpu": step_bytes,
                "large_matrix_frac_min": round(min(large_fracs), 4) if large_fracs else None,
                "large_matrix_frac_max": round(max(large_fracs), 4) if large_fracs else None,
                "step_us_without_immutable_flag": None if plain_us is None else round(plain_us, 2),
                "note": "bytes = 2.5*P + 4*(rows+1) + 2*cols + 2*rows per SpMV, summed over the step, over the step's device time",
            },
            "e2e": {
                "value": e2e_ms * 1000.0, "unit": UNIT,
                "eager_us": e2e_eager_ms * 1000.0, "graph_replay_us": None if e2e_graph_ms is None else e2e_graph_ms * 1000.0,
                "per_product_copies_us": None if e2e_per_product_ms is None else e2e_per_product_ms * 1000.0,
                "copies_beside_products_us": None if e2e_pipelined_ms is None else e2e_pipelined_ms * 1000.0,
                "h2d_bytes_per_step": int(x_host.numel() * 2),
                "d2h_bytes_per_step": int((peer.buf[0].numel() if peer is not None else y_dev.numel()) * 2),
                "api": "every step: one copy of the step's 36 x vectors from a pinned host arena, macko_spmv_b200.multiply(frozen, x_view, out=y_view) "
                       "per matrix (N > 1: PeerGather.multiply_deferred + wait), one copy of all y to a pinned host arena; compressed matrices resident "
                       "on the device as the API requires; value = the fastest of eager calls, a CUDA-graph replay of the same calls and "
                       "(one GPU) copies_beside_products_us: the same calls in four groups of nine matrices, a group's x arriving on a copy "
                       "stream, its y leaving on another while the next group multiplies, the step ending when the last y is on the host; "
                       "per_product_copies_us = the same step with one H2D and one D2H copy per product",
            },
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks,
            "compress": {
                "seconds_for_sweep": round(t_compress, 4),
                "dense_input_GB_per_s": round(dense_in_bytes / t_compress / 1e9, 1),
                "note": "GPU compressor, wall clock including the 4-byte size read-back, per-rank blocks",
            },
        }
        if decode is not None:
            line["decode"] = decode
            for k, v in decode["tokens_per_s"].items():
                line["e2e"][f"decode_tokens_per_s_{k}"] = v
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        if large is not None:
            line["sharded_large"] = {
                "workload": "12288x49152 and 49152x12288, Bernoulli mask at densities 0.1 and 0.5, contiguous row block per GPU, "
                            "full y on every rank; microseconds per product, max over ranks, products back to back",
                "note": "per-case figures are eager launches between CUDA events (they include host launch gaps when a product is "
                        "shorter than the host's launch path); us_sum_graph replays the four products as one CUDA graph",
                **large}
        if skewed is not None:
            line["skewed"] = skewed
            line["roofline"]["skewed_frac_planned_min"] = min(s["roofline_frac_planned"] for s in skewed)
        if single is not None:
            line["single_4096"] = single
        if batched is not None:
            line["batched"] = batched
        if value_types is not None:
            line["value_types"] = value_types
        if per_case is not None:
            line["per_case"] = per_case
            sp = [p["speedup_vs_cublas"] for p in per_case]
            line["geomean_speedup_vs_cublas"] = round(float(torch.tensor(sp).log().mean().exp()), 3)

    # ---- tear down in order: graphs, exchange buffers, process group; the result line comes last ----
    graphs = None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        if peer is not None:
            peer.close()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if not ok_all or peer_flag_all != 0:
        raise SystemExit(f"y_check failed (ok={ok_all}, peer_error_flag={peer_flag_all})")


def run_single_case(args):
    """A few SpMVs on one synthetic matrix: the small workload profiler captures are taken on.
    `--single-kind`: plain (default launch), frozen (immutable matrix: early loads), planned, batched8, scatter (world of
    one), decompress, compress."""
    import ctypes

    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi, workloads

    rows, cols, density = args.single.split(",")
    rows, cols, density = int(rows), int(cols), float(density)
    torch.cuda.set_device(0)
    if args.single_kind == "planned":
        M = workloads.skewed_matrix(rows, cols, seed=2999, device="cuda", mean_density=density)
    else:
        M = workloads.magnitude_pruned_matrix(rows, cols, density, seed=2999, device="cuda")
    x = workloads.dense_vector(cols, 3001, "cuda")
    comp = macko_spmv.compress(M)
    lib = cabi.load()
    stream = torch.cuda.current_stream().cuda_stream
    kind = args.single_kind
    if kind == "plain":
        run = lambda: macko_spmv.multiply(comp, x)
    elif kind == "frozen":
        fz0 = macko_spmv.freeze(comp, plan=False)
        run = lambda: macko_spmv.multiply(fz0, x)
    elif kind == "planned":
        fz = macko_spmv.freeze(comp, plan=True)
        run = lambda: macko_spmv.multiply(fz, x)
    elif kind == "batched8":
        V = torch.stack([x] * 8).contiguous()
        run = lambda: macko_spmv.multiply_batched(comp, V)[0]
    elif kind == "scatter":
        ybuf = torch.zeros(rows, dtype=torch.float16, device="cuda")
        flags = torch.zeros(16, dtype=torch.int32, device="cuda")
        ptrs = ctypes.c_void_p * 1
        yt, ft = ptrs(ybuf.data_ptr()), ptrs(flags.data_ptr())

        def run():
            cabi.check(lib, lib.macko_spmv_fp16_scatter_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                                           comp[0].numel(), x.data_ptr(), yt, 0, ft, 0, 1, 0, 0, stream))
            return ybuf
    elif kind == "decompress":
        run = lambda: macko_spmv.decompress(comp)[:, 0].contiguous()
    elif kind == "compress":
        run = lambda: macko_spmv.compress(M)[0][:rows]
    else:
        raise SystemExit(f"unknown --single-kind {kind}")
    for _ in range(max(args.warmup, 1)):
        run()
    torch.cuda.synchronize()
    e0, e1 = event_pair()
    e0.record()
    for _ in range(args.steps):
        y = run()
    e1.record()
    torch.cuda.synchronize()
    nbytes = workloads.algorithmic_bytes(comp[0].numel(), rows, cols)
    res = {"single": [rows, cols, density], "kind": kind, "us_warm_l2": e0.elapsed_time(e1) * 1000 / args.steps,
           "algorithmic_bytes": nbytes}
    if kind in ("plain", "frozen", "planned", "batched8", "scatter"):
        ref = M.float() @ x.float()
        res["rel_l2_vs_dense_fp32"] = float((y.float() - ref).norm() / ref.norm())
    print(json.dumps(res), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-per-case", action="store_true", help="skip the per-matrix cuBLAS comparison")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-batched", action="store_true", help="skip the multi-vector product figures")
    ap.add_argument("--no-sharded-large", action="store_true", help="skip the large row-sharded matrices")
    ap.add_argument("--no-skewed", action="store_true", help="skip the skewed-density matrices")
    ap.add_argument("--no-decode", action="store_true", help="skip the Llama-architecture decode figures")
    ap.add_argument("--decode-layers", type=int, default=32)
    ap.add_argument("--decode-prompt", type=int, default=128)
    ap.add_argument("--decode-tokens", type=int, default=256)
    ap.add_argument("--exchange", choices=["peer", "peer-fused", "nccl"], default="peer",
                    help="N > 1: how the y slices are exchanged: peer stores by a forward kernel beside the next products, "
                         "peer stores from the tail of the product kernel, or NCCL all-gather")
    ap.add_argument("--single", default=None, metavar="ROWS,COLS,DENSITY",
                    help="run only a few products on one matrix (small case for profiler captures)")
    ap.add_argument("--single-kind", default="plain",
                    choices=["plain", "frozen", "planned", "batched8", "scatter", "decompress", "compress"])
    args = ap.parse_args()
    if args.single:
        run_single_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
