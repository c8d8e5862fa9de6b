"""The command-line benchmark that takes the reference CLI's ten positional arguments
(c_benchmarking/utils.cuh:63-101) and ends with its tab-separated `Final results:` line
(c_benchmarking/benchmark.cu:229-233)."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "macko_spmv_b200", "macko_bench")


def _run(*args):
    return subprocess.run([CLI, *map(str, args)], capture_output=True, text=True, timeout=600)


def test_cli_is_built_and_rejects_bad_usage():
    assert os.path.exists(CLI), "run `python macko_spmv_b200/build.py`"
    p = _run(16, 64)
    assert p.returncode == 1 and "<bits_per_value> <rows> <cols> <warmup> <timing> <flush> <debug> <kernel_id> <seed> <density>" in p.stderr
    p = _run(4, 64, 64, 1, 1, 0, 0, 7, 0, 0.5)          # 16 and 8 bits per value exist: said so, before any CUDA call
    assert p.returncode == 1 and "16 and 8 bits" in p.stderr
    p = _run(16, 64, "x", 1, 1, 0, 0, 7, 0, 0.5)
    assert p.returncode == 1 and "Invalid arguments" in p.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("kernel_id", [7, 2, 1, 3])
def test_cli_result_line(kernel_id):
    p = _run(16, 4096, 4096, 5, 20, 1, 0, kernel_id, 47, 0.5)
    assert p.returncode == 0, p.stderr
    lines = p.stdout.splitlines()
    diff = [l for l in lines if l.startswith("Max diff:")]
    assert diff and float(diff[0].split(":")[1]) < 0.1 and "LOOKS BIG" not in p.stdout
    final = [l for l in lines if l.startswith("Final results:")]
    assert len(final) == 1
    f = final[0].split("\t")
    assert f[0] == "Final results:" and len(f) == 9
    assert f[1:5] == ["16", "4096", "4096", str(kernel_id)] and float(f[5]) == 0.5
    mean_us, dense_gflops, sparse_gflops = int(f[6]), int(f[7]), int(f[8])
    assert 0 < mean_us < 1000 and dense_gflops > 0 and abs(sparse_gflops - dense_gflops * 0.5) <= 1
    if kernel_id == 7:
        eff = [l for l in lines if l.startswith("Effective density:")][0].split()
        assert 0.6 < float(eff[2]) < 0.7          # 2.5 bytes per stored element at 50 % density, plus pads


@pytest.mark.gpu
def test_cli_int8_kernel():
    # bits_per_value 8, kernel id 8 (c_benchmarking/benchmark.cu:106-119): integer values in [-50, 50]
    p = _run(8, 4096, 4096, 5, 20, 1, 0, 8, 47, 0.5)
    assert p.returncode == 0, p.stderr
    lines = p.stdout.splitlines()
    diff = [l for l in lines if l.startswith("Max diff:")]
    assert diff and float(diff[0].split(":")[1]) < 1.0 and "NO KERNEL" not in p.stderr   # row sums reach the hundreds: fp16 y
    final = [l for l in lines if l.startswith("Final results:")][0].split("\t")
    assert final[1:5] == ["8", "4096", "4096", "8"] and 0 < int(final[6]) < 1000
    eff = [l for l in lines if l.startswith("Effective density:")][0].split()
    assert 0.7 < float(eff[2]) < 0.85          # 1.5 bytes per stored element against 1 byte dense, plus pads


@pytest.mark.gpu
def test_cli_refuses_unknown_kernel():
    p = _run(16, 256, 256, 1, 1, 0, 0, 9, 0, 0.5)
    assert p.returncode == 1 and "NO KERNEL" in p.stderr
    p = _run(16, 256, 256, 1, 1, 0, 0, 8, 0, 0.5)       # the int8 kernel needs bits_per_value 8
    assert p.returncode == 1 and "NO KERNEL" in p.stderr
