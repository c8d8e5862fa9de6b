"""GPU parity (`-m gpu`) on the benchmark configurations themselves, at full size: every matrix of the
Llama-2-7B layer sweep (4 shapes x 9 densities, the seeds bench.py uses), the single 4096x4096 Bernoulli-0.5
product, the two large row-sharded shapes at both densities, and the two skewed shapes. For each one the GPU
compressor must reproduce the oracle's buffers bit for bit and the product (default launch, and the planned
launch where it applies) must stay within
    |y - y_ref| <= 1e-3 * sum_k |val_k * x[col_k]|   per row,   ||y - y_ref||_2 <= 5e-3 * ||y_ref||_2
of the oracle's float64 product of the compressed buffers (the reference's own check is allclose against the
dense product, tests/test_macko_spmv.py:115-135, and a max-abs difference, c_benchmarking/benchmark.cu:160-172)."""
import numpy as np
import pytest
import torch

import oracle
import macko_spmv_b200 as macko_spmv
from macko_spmv_b200 import workloads

pytestmark = pytest.mark.gpu

MAX_ABS_FACTOR = 1e-3
REL_L2 = 5e-3


def _u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _check(M, x, what, planned=False):
    rows, cols = M.shape
    comp = macko_spmv.compress(M)
    exp = oracle.compress(_u16(M).reshape(rows, cols))
    assert np.array_equal(_u16(comp[0]), exp[0]), f"{what}: values differ"
    assert np.array_equal(comp[1].cpu().numpy(), exp[1]), f"{what}: deltas differ"
    assert np.array_equal(comp[2].cpu().numpy(), exp[2]), f"{what}: row_indices differ"
    y64, _, l1 = oracle.spmv(exp, _u16(x))
    nrm = np.linalg.norm(y64)
    variants = [("default", macko_spmv.multiply(comp, x))]
    variants.append(("immutable", macko_spmv.multiply(macko_spmv.freeze(comp, plan=False), x)))
    if planned:
        variants.append(("planned", macko_spmv.multiply(macko_spmv.freeze(comp, plan=True), x)))
    for name, y in variants:
        got = y.float().cpu().numpy().astype(np.float64)
        err = np.abs(got - y64)
        assert np.all(err <= MAX_ABS_FACTOR * l1 + 1e-12), f"{what} {name}: worst {float((err / (l1 + 1e-30)).max()):.3e} of L1"
        assert np.linalg.norm(got - y64) <= REL_L2 * nrm, f"{what} {name}: relative L2 {np.linalg.norm(got - y64) / nrm:.3e}"
    assert torch.equal(variants[0][1].view(torch.int16), variants[1][1].view(torch.int16)), f"{what}: the flag changed the result"


@pytest.mark.parametrize("shape_idx", range(len(workloads.LLAMA7B_SHAPES)))
def test_every_matrix_of_the_layer_sweep(shape_idx):
    rows, cols = workloads.LLAMA7B_SHAPES[shape_idx]
    for di, d in enumerate(workloads.SWEEP_DENSITIES):
        seed = workloads.sweep_seed(shape_idx, di)
        M = workloads.magnitude_pruned_matrix(rows, cols, d, seed, device="cuda")
        x = workloads.dense_vector(cols, seed + 500, "cuda")
        _check(M, x, f"{rows}x{cols} d={d}")
        del M
    torch.cuda.empty_cache()


def test_single_product_4096_bernoulli_half():
    # values N(0,1), Bernoulli(0.5) mask, x N(0,1), seed 1001 on the CPU generator
    g = torch.Generator().manual_seed(1001)
    W = torch.randn(4096, 4096, generator=g).half()
    mask = torch.rand(4096, 4096, generator=g) < 0.5
    M = (W * mask).cuda()
    x = torch.randn(4096, generator=g).half().cuda()
    _check(M, x, "4096x4096 Bernoulli 0.5 seed 1001", planned=True)
    ref = M.float().cpu() @ x.float().cpu()          # the configuration's own oracle: dense fp32 product on the CPU
    y = macko_spmv.multiply(macko_spmv.compress(M), x).float().cpu()
    assert float((y - ref).norm() / ref.norm()) <= REL_L2


@pytest.mark.parametrize("case", [(0, 0.1), (0, 0.5), (1, 0.1), (1, 0.5)])
def test_large_row_sharded_shapes_on_one_gpu(case):
    si, d = case
    rows, cols = workloads.SHARDED_SHAPES[si]
    seed = 7000 + 10 * si + int(round(d * 10))
    M = workloads.bernoulli_matrix(rows, cols, d, seed, device="cuda", scale=0.02)
    x = workloads.dense_vector(cols, seed + 500, "cuda")
    _check(M, x, f"{rows}x{cols} d={d}", planned=True)
    # and as row blocks (first and last of eight): every block is a compressed matrix of its own
    for r in (0, 7):
        lo, hi = rows * r // 8, rows * (r + 1) // 8
        _check(M[lo:hi].contiguous(), x, f"{rows}x{cols} d={d} rows [{lo}, {hi})")
    del M
    torch.cuda.empty_cache()


@pytest.mark.parametrize("si", range(len(workloads.SKEWED_SHAPES)))
def test_skewed_shapes(si):
    rows, cols = workloads.SKEWED_SHAPES[si]
    M = workloads.skewed_matrix(rows, cols, seed=5000 + si, device="cuda")
    x = workloads.dense_vector(cols, 5500 + si, "cuda")
    _check(M, x, f"skewed {rows}x{cols}", planned=True)
    lens = (M != 0).sum(dim=1)
    assert int(lens.min()) == 0 and int(lens.max()) == cols, "the stress matrix holds empty and fully dense rows"
