#!/usr/bin/env python
"""Benchmark of the MACKO SpMV hot path on B200.

Workload (own arm, every N): the Llama-2-7B linear-layer sweep -- 4 shapes x 9 densities =
36 magnitude-pruned fp16 matrices, seeded synthetic stand-ins for the pruned checkpoints the
reference measured. One step = one SpMV on each of the 36 compressed matrices (at N > 1 every
matrix is row-sharded over the ranks and each SpMV is followed by the all-gather of y).
Metric = device time of one step in microseconds (the sum of the 36 SpMV times), lower is
better. The step touches ~2.7 GB of distinct compressed data, far more than the 126 MB L2,
so every SpMV streams its matrix from HBM.

Printed JSON line (rank 0): the contract keys plus
  roofline      algorithmic bytes of a step / device time, against the measured HBM copy peak
  cpu_baseline  the reference's CPU path (compiled reference compressor + dense torch.mv of
                the decompressed matrix) on a bounded sample, scaled to one step
  e2e           the same step through the public Python API with x coming from pinned host
                memory and y copied back to the host, every SpMV
  per_case      per-matrix microseconds, roofline fraction and speed-up over cuBLAS fp16 GEMV
`--impl reference` times the reference's CPU path alone (rank 0 only).
"""
from __future__ import annotations

import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum over the 36 spmv launches of one step, from the
# ncu capture summarised in profiles/spmv_sweep_launches.md (None until captured).
NCU_STEP_TRAFFIC_BYTES = 2730896128


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


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
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- workload

def build_sweep(device, rank: int, world: int):
    """The 36 compressed matrices of the sweep (this rank's row block of each), their x, and
    the dense matrices at N == 1 (cuBLAS comparator)."""
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
                "lo": lo, "hi": hi, "dense": block if world == 1 else None,
                "bytes": workloads.algorithmic_bytes(comp[0].numel(), hi - lo, cols),
                "dense_bytes": workloads.dense_bytes(hi - lo, cols),
            })
            del M
    return cases, t_compress, dense_in_bytes


def time_rotating(launchers, reps):
    """Mean device microseconds of one launch, cycling through `launchers` (distinct buffers,
    together larger than L2) so that every launch streams from HBM."""
    for f in launchers[: min(8, len(launchers))]:
        f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = len(launchers)
    e0.record()
    for i in range(reps):
        launchers[i % n]()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1000.0 / reps


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
                    xx.data_ptr(), yy.data_ptr(), 1.0, 0.0, stream)
            return lambda: cabi.check(lib, lib.macko_spmv_fp16(*args))

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
    """The two large shapes (12288x49152, 49152x12288; Bernoulli masks at densities 0.1 and 0.5),
    each rank holding a contiguous row block, the full y delivered to every rank. The four products
    run back to back (together they stream more than L2 holds on every rank up to 8 GPUs), timed per
    product with CUDA events, max over ranks. At one GPU the cuBLAS fp16 GEMV on the dense matrix is
    timed beside each."""
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
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(10):
                    torch.mv(block, x)
                e1.record()
                torch.cuda.synchronize()
                gemv_us = e0.elapsed_time(e1) * 100.0
                ref = block.float() @ x.float()
            cases.append({"rows": rows, "cols": cols, "density": d, "x": x, "gemv_us": gemv_us,
                          "shard": sharded.RowShard(comp, lo, hi, rows, blocks),
                          "y": torch.empty(rows, dtype=torch.float16, device=device) if world == 1 else None,
                          "ref": ref if world == 1 else None,
                          "bytes": workloads.algorithmic_bytes(comp[0].numel(), hi - lo, cols)})
            del block
    torch.cuda.empty_cache()

    def product(c):
        sh = c["shard"]
        if peer is not None:
            return peer.multiply(sh, c["x"])
        comp = sh.compressed
        stream = torch.cuda.current_stream().cuda_stream   # read at call time: differs under graph capture
        cabi.check(lib, lib.macko_spmv_fp16(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4],
                                            comp[0].numel(), c["x"].data_ptr(), c["y"].data_ptr(), 1.0, 0.0, stream))
        if world > 1:
            raise RuntimeError("sharded leg needs the peer exchange")
        return c["y"]

    for _ in range(3):
        for c in cases:
            product(c)
    torch.cuda.synchronize()
    # the four products as one CUDA graph: device time of a cycle without host launch overhead
    graph_us = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for c in cases:
                product(c)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1000.0 / reps], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        graph_us = float(t.item())
    except Exception:   # capture refused: the eager figures below still stand
        graph_us = None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(cases) + 1)] for _ in range(reps)]
    for r in range(reps):
        marks[r][0].record()
        for i, c in enumerate(cases):
            product(c)
            marks[r][i + 1].record()
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
            err = float((c["y"].float() - c["ref"]).norm() / c["ref"].norm())
            assert err < 5e-3, f"large-matrix product is wrong (rel L2 {err})"
            row["cublas_gemv_us"] = round(c["gemv_us"], 2)
            row["speedup_vs_cublas"] = round(c["gemv_us"] / t, 3)
        out.append(row)
    total_bytes = sum(c["bytes"] for c in cases)
    return {"cases": out, "us_sum_eager": round(sum(r["us"] for r in out), 2),
            "us_sum_graph": None if graph_us is None else round(graph_us, 2),
            "per_gpu_roofline_frac_graph": None if graph_us is None else round(total_bytes / (graph_us * 1e-6) / 1e9 / peak_gbs, 4)}


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
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
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
        out[f"batched_{b}_us"] = timed(lambda: macko_spmv.multiply_batched(comp, Vb))
    V8 = V[:8].contiguous()
    out["loop_of_8_us"] = timed(lambda: [macko_spmv.multiply(comp, V8[i]) for i in range(8)])
    out["prefill_128_dense_route_us"] = timed(lambda: macko_spmv.multiply_batched(comp, V))
    return out


# --------------------------------------------------------------------------- CPU reference path

def cpu_reference_path(steps: int, warmup: int, gpu_cases=None):
    """The reference's CPU path on a bounded sample of the sweep: the reference compressor
    (compiled, unmodified; else the oracle port) followed by a dense fp32 torch.mv of the
    decompressed matrix, on the 4096x4096 layer at the 9 densities. Returns microseconds
    scaled to a whole step (the sweep has 14.27x the dense elements of the sample)."""
    import numpy as np
    import oracle
    from macko_spmv_b200 import workloads

    kind = "reference" if oracle.have_reference() else "port"
    compress = oracle.ref_compress if kind == "reference" else oracle.compress
    rows, cols = workloads.LLAMA7B_SHAPES[0]
    sample = []
    t_comp = 0.0
    for di, d in enumerate(workloads.SWEEP_DENSITIES):
        M = workloads.magnitude_pruned_matrix(rows, cols, d, workloads.sweep_seed(0, di), device="cpu")
        dense_bits = M.numpy().view(np.uint16)
        t0 = time.perf_counter()
        comp = compress(dense_bits)
        t_comp += time.perf_counter() - t0
        dec = torch.from_numpy(oracle.decompress(comp).view(np.float16).copy()).float()
        x = workloads.dense_vector(cols, 77 + di, "cpu").float()
        sample.append((dec, x))
    scale = sum(r * c for r, c in workloads.LLAMA7B_SHAPES) / float(rows * cols)
    ref_gpu = None
    if gpu_cases is not None and oracle.have_reference_kernel():
        ref_gpu = reference_gpu_kernel_times(gpu_cases)

    def one_step():
        for dec, x in sample:
            torch.mv(dec, x)

    for _ in range(max(warmup, 1)):
        one_step()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_step()
    t_mv = (time.perf_counter() - t0) / steps
    return {
        "value": t_mv * 1e6 * scale, "unit": UNIT, "cores": torch.get_num_threads(), "kind": kind,
        "sample": f"4096x4096 layer at densities 0.1..0.9 ({len(sample)} of 36 matrices), torch.mv fp32 of the "
                  f"decompressed matrix, scaled x{scale:.2f} by dense elements to the whole sweep",
        "compress_us": t_comp * 1e6 * scale, "compress_threads": 1,
        "spmv_plus_compress_us": (t_mv + t_comp) * 1e6 * scale,
        "reference_gpu_kernel": ref_gpu,
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
        "config": {"workload": "llama2-7b linear-layer sweep: 4 shapes x 9 densities, per-row magnitude pruning "
                               "(bounded sample, see cpu_baseline.sample)"},
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
        os.environ.pop("NCCL_DEBUG", None)  # keep NCCL banners off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)

    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import cabi

    lib = cabi.load()
    peak_gbs, peak_kind = measured_hbm_peak()
    cases, t_compress, dense_in_bytes = build_sweep(device, rank, world)
    n_cases = len(cases)
    step_bytes = sum(c["bytes"] for c in cases)

    # ---- one step, captured as a CUDA graph: 36 x (SpMV [+ all-gather of y]) -----------------
    ys_local = [torch.empty(c["hi"] - c["lo"], dtype=torch.float16, device=device) for c in cases]
    ys_full = [torch.empty(c["rows"], dtype=torch.float16, device=device) for c in cases] if world > 1 else ys_local
    from macko_spmv_b200 import sharded

    shards = [sharded.RowShard(c["comp"], c["lo"], c["hi"], c["rows"],
                               [sharded.row_block(c["rows"], r, world) for r in range(world)]) for c in cases]
    peer = None
    if world > 1 and args.exchange == "peer":
        from macko_spmv_b200 import workloads
        peer = sharded.PeerGather(max([c["rows"] for c in cases] + [r for r, _ in workloads.SHARDED_SHAPES]), device)

    def step_eager():
        stream = torch.cuda.current_stream().cuda_stream
        if peer is not None:   # SpMV with the exchange fused into its epilogue, then the flag wait
            for sh, c in zip(shards, cases):
                peer.multiply(sh, c["x"])
            return
        for c, yl, yf in zip(cases, ys_local, ys_full):
            comp = c["comp"]
            cabi.check(lib, lib.macko_spmv_fp16(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(),
                                                c["hi"] - c["lo"], c["cols"], comp[0].numel(),
                                                c["x"].data_ptr(), yl.data_ptr(), 1.0, 0.0, stream))
            if world > 1 and peer is None:
                dist.all_gather_into_tensor(yf, yl)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step_eager()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step_eager()
        run_step = graph.replay
    except Exception:  # a collective that cannot be captured: time eager launches instead
        graph = None
        run_step = step_eager
    for _ in range(max(args.warmup, 3)):
        run_step()
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
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

    # ---- end to end through the public API with host buffers ------------------------------------
    xs_host = [c["x"].cpu().pin_memory() for c in cases]
    ys_host = [torch.empty(c["rows"], dtype=torch.float16).pin_memory() for c in cases]
    def step_e2e():
        for c, sh, xh, yh in zip(cases, shards, xs_host, ys_host):
            xd = xh.to(device, non_blocking=True)
            if world == 1:
                y = macko_spmv.multiply(c["comp"], xd)
            elif peer is not None:
                y = peer.multiply(sh, xd)
            else:
                y = sharded.multiply_sharded(sh, xd)
            yh.copy_(y, non_blocking=True)

    e2e_branches = [torch.cuda.Stream(device=device) for _ in range(4)]

    def step_e2e_branches():
        """The same calls, the 36 independent chains spread over four streams forked from and joined back
        into the current one: captured as a graph, copies of one chain run under the kernels of the others."""
        main = torch.cuda.current_stream()
        for st in e2e_branches:
            st.wait_stream(main)
        for i, (c, xh, yh) in enumerate(zip(cases, xs_host, ys_host)):
            with torch.cuda.stream(e2e_branches[i % len(e2e_branches)]):
                xd = xh.to(device, non_blocking=True)
                y = macko_spmv.multiply(c["comp"], xd)
                yh.copy_(y, non_blocking=True)
        for st in e2e_branches:
            main.wait_stream(st)

    def time_e2e(run):
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        n = max(3, min(args.steps, 20))
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    e2e_eager_ms = time_e2e(step_e2e)
    # The same 36 chains of public-API calls captured once as a CUDA graph (the pinned host buffers are read
    # and written by every replay), which is how a caller with a fixed set of layers removes the host cost of
    # 108 asynchronous calls per step.
    def capture_and_time(step):
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        for yh in ys_host:
            yh.zero_()
        ms = time_e2e(g.replay)
        c = cases[4]   # the replay really delivers y to the host buffers
        ref = c["dense"].float() @ c["x"].float()
        err = float((ys_host[4].to(device).float() - ref).norm() / ref.norm())
        assert err < 5e-3, f"graph replay of the end-to-end step produced a wrong result (rel L2 {err})"
        return ms, g

    e2e_graph_ms = e2e_forked_ms = None
    if world == 1:   # ranks must not disagree on whether a capture worked: the row-sharded runs stay eager
        try:
            e2e_graph_ms, _g1 = capture_and_time(step_e2e)
            e2e_forked_ms, _g2 = capture_and_time(step_e2e_branches)
        except AssertionError:
            raise
        except Exception:   # a capture the runtime refuses: the eager figure stands
            pass
    e2e_ms = e2e_eager_ms if e2e_graph_ms is None else min(e2e_eager_ms, e2e_graph_ms)
    clocks = sampler.stop() if rank == 0 else None

    # correctness spot check of what was timed (dense fp32 product, N == 1)
    if world == 1:
        c = cases[4]
        ref = c["dense"].float() @ c["x"].float()
        err = float((ys_local[4].float() - ref).norm() / ref.norm())
        assert err < 5e-3, f"timed kernel produced a wrong result (rel L2 {err})"

    per_case = per_case_numbers(cases, lib, peak_gbs) if (world == 1 and not args.no_per_case) else None
    large = None
    if not args.no_sharded_large and (world == 1 or peer is not None):
        large = sharded_large_leg(device, rank, world, lib, peer, peak_gbs)
    batched = batched_leg(device) if (world == 1 and not args.no_batched) else None
    cpu_base = cpu_reference_path(3, 1, gpu_cases=cases) if (rank == 0 and world == 1 and not args.no_cpu_baseline) else None

    if rank == 0:
        achieved = step_bytes * world / (ms_per_step * 1e-3) / 1e9 if world == 1 else step_bytes / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": ms_per_step * 1000.0, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16xf16->f32", "data": "synthetic",
            "config": {
                "workload": "llama2-7b linear-layer sweep: shapes 4096x4096, 11008x4096, 4096x11008, 32000x4096 x "
                            "densities 0.1..0.9, per-row magnitude pruning; one step = one SpMV per matrix (36)",
                "parallelism": "single GPU" if world == 1 else (f"rows of every matrix split over {world} GPUs; " + ("every SpMV kernel stores its y slice into all ranks' y over NVLink and ends when all slices have arrived (no collective)" if peer is not None else "NCCL all-gather of y after each SpMV")),
                "l2": "inputs larger than L2: a step streams %.2f GB of distinct compressed data per GPU, each matrix once" % (step_bytes / 1e9),
                "launch": "one CUDA graph per step" if graph is not None else "eager launches",
            },
            "roofline": {
                "bound": "hbm", "achieved": round(achieved, 1), "peak": peak_gbs, "unit": "GB/s",
                "frac": round(achieved / peak_gbs, 4), "traffic": NCU_STEP_TRAFFIC_BYTES if world == 1 else None,
                "peak_source": f"of {peak_kind}", "algorithmic_bytes_per_step_per_gpu": step_bytes,
                "note": "bytes = 2.5*P + 4*(rows+1) + 2*cols + 2*rows per SpMV, summed over the step, over the step's device time",
            },
            "e2e": {
                "value": e2e_ms * 1000.0, "unit": UNIT,
                "eager_us": e2e_eager_ms * 1000.0, "graph_replay_us": None if e2e_graph_ms is None else e2e_graph_ms * 1000.0,
                "graph_replay_four_streams_us": None if e2e_forked_ms is None else e2e_forked_ms * 1000.0,
                "h2d_bytes_per_step": sum(2 * c["cols"] for c in cases),
                "d2h_bytes_per_step": sum(2 * c["rows"] for c in cases),
                "api": "macko_spmv_b200.multiply(compressed, x) per matrix; x from pinned host memory, y copied to pinned host memory; compressed matrix resident on the device as the API requires; value = the faster of eager calls and a CUDA-graph replay of the same calls, both on one stream like the device-only figure; graph_replay_four_streams_us spreads the 36 independent chains over four forked streams, where copies and kernels of different chains overlap",
            },
            "gpu_launches": args.steps * n_cases,
            "clocks": clocks,
            "compress": {
                "seconds_for_sweep": round(t_compress, 4),
                "dense_input_GB_per_s": round(dense_in_bytes / t_compress / 1e9, 1),
                "note": "GPU compressor, wall clock including the 4-byte size read-back, per-rank blocks",
            },
        }
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        if large is not None:
            line["sharded_large"] = {
                "workload": "12288x49152 and 49152x12288, Bernoulli mask at densities 0.1 and 0.5, contiguous row block per GPU, "
                            "full y on every rank; microseconds per product, max over ranks, products back to back",
                "note": "per-case figures are eager launches between CUDA events (they include host launch gaps when a product is "
                        "shorter than the host's launch path); us_sum_graph replays the four products as one CUDA graph",
                **large}
        if batched is not None:
            line["batched"] = batched
        if per_case is not None:
            line["per_case"] = per_case
            sp = [p["speedup_vs_cublas"] for p in per_case]
            line["geomean_speedup_vs_cublas"] = round(float(torch.tensor(sp).log().mean().exp()), 3)
        print(json.dumps(line), flush=True)
    if world > 1:
        # Leave without tearing NCCL down: destroying a communicator that a live CUDA graph still
        # references can block forever, and every result has been printed by now.
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_single_case(args):
    """A few SpMVs on one synthetic matrix: the small workload profiler captures are taken on."""
    import macko_spmv_b200 as macko_spmv
    from macko_spmv_b200 import workloads

    rows, cols, density = args.single.split(",")
    rows, cols, density = int(rows), int(cols), float(density)
    torch.cuda.set_device(0)
    M = workloads.magnitude_pruned_matrix(rows, cols, density, seed=2999, device="cuda")
    x = workloads.dense_vector(cols, 3001, "cuda")
    comp = macko_spmv.compress(M)
    for _ in range(max(args.warmup, 1)):
        macko_spmv.multiply(comp, x)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        y = macko_spmv.multiply(comp, x)
    e1.record()
    torch.cuda.synchronize()
    ref = M.float() @ x.float()
    err = float((y.float() - ref).norm() / ref.norm())
    nbytes = workloads.algorithmic_bytes(comp[0].numel(), rows, cols)
    print(json.dumps({"single": [rows, cols, density], "us_warm_l2": e0.elapsed_time(e1) * 1000 / args.steps,
                      "algorithmic_bytes": nbytes, "rel_l2_vs_dense_fp32": err}), flush=True)


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
    ap.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                    help="N > 1: how the y slices are exchanged (fused peer stores, or NCCL all-gather)")
    ap.add_argument("--single", default=None, metavar="ROWS,COLS,DENSITY",
                    help="run only a few SpMVs on one matrix (small case for profiler captures)")
    args = ap.parse_args()
    if args.single:
        run_single_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_own_arm(args)


if __name__ == "__main__":
    main()
