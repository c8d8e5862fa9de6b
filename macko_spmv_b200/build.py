"""In-tree build of the two native libraries of this package.

``libmacko_b200.so``  CUDA kernels + C ABI (nvcc, sm_100a only, no torch dependency)
``_torch_ops.so``     the `macko_spmv::*` torch operators, linked against the C ABI
``macko_bench``       command-line benchmark with the reference CLI's arguments (C ABI + cuBLAS)

Run ``python macko_spmv_b200/build.py`` (or call :func:`build`). Nothing is compiled at
import time; importing the package without the built libraries raises.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")
LIB_CORE = os.path.join(PKG_DIR, "libmacko_b200.so")
LIB_TORCH = os.path.join(PKG_DIR, "_torch_ops.so")
BENCH_CLI = os.path.join(PKG_DIR, "macko_bench")

CUDA_SOURCES = ["common.cu", "spmv.cu", "compress.cu", "decompress.cu", "plan.cu", "decode_glue.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, flush=True)


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def build_core(force: bool = False, verbose: bool = False) -> str:
    headers = [os.path.join(CSRC, "common.cuh"), os.path.join(CSRC, "plan.cuh"), os.path.join(INCLUDE, "macko_b200.h")]
    sources = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    if not force and _newer(LIB_CORE, sources + headers + [__file__]):
        return LIB_CORE
    objs = []
    build_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in sources:
        obj = os.path.join(build_dir, os.path.basename(src) + ".o")
        objs.append(obj)
        cmd = [_nvcc(), *NVCC_FLAGS, "-I", INCLUDE, "-I", CSRC, "-c", src, "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0:
            raise RuntimeError(f"nvcc failed: {' '.join(cmd)}\n{out}")
        if verbose and out:
            print(out, flush=True)
    _run([_nvcc(), "-shared", "-Wno-deprecated-gpu-targets", "-o", LIB_CORE, *objs], verbose)  # static cudart: self-contained
    return LIB_CORE


def build_torch_ops(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_binding.cpp")
    if not force and _newer(LIB_TORCH, [src, LIB_CORE, os.path.join(INCLUDE, "macko_b200.h"), __file__]):
        return LIB_TORCH
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths("cuda"):
        inc += ["-isystem", p]
    lib_dirs = ce.library_paths("cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
        "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", INCLUDE, *inc, src, "-o", LIB_TORCH,
        *[f"-L{d}" for d in lib_dirs], "-L", PKG_DIR,
        "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-l:libmacko_b200.so",
        "-Wl,-rpath,$ORIGIN", *[f"-Wl,-rpath,{d}" for d in lib_dirs],
    ]
    _run(cmd, verbose)
    return LIB_TORCH


def build_cli(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "bench_cli.cu")
    if not force and _newer(BENCH_CLI, [src, LIB_CORE, os.path.join(INCLUDE, "macko_b200.h"), __file__]):
        return BENCH_CLI
    _run([_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-I", INCLUDE, src, "-o", BENCH_CLI,
          "-L", PKG_DIR, "-l:libmacko_b200.so", "-lcublas", "-lcusparse", "-Xlinker", "-rpath=$ORIGIN"], verbose)
    return BENCH_CLI


def build(force: bool = False, verbose: bool = False) -> None:
    build_core(force, verbose)
    build_torch_ops(force, verbose)
    build_cli(force, verbose)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv or "--verbose" in sys.argv)
    print("built", LIB_CORE, LIB_TORCH, BENCH_CLI)
