"""Seeded synthetic matrices shaped like the workloads the MACKO kernel is measured on.

They stand in for the pruned Llama-2-7B weights behind the reference's published numbers
(no checkpoint is available offline): same shapes, same value scale, same sparsity
patterns. All generators are deterministic for a given (seed, device type).
"""
from __future__ import annotations

import math

import torch

# (rows, cols) of the Llama-2-7B linear layers: attention projections, FFN up/gate,
# FFN down, LM head.
LLAMA7B_SHAPES = [(4096, 4096), (11008, 4096), (4096, 11008), (32000, 4096)]
SWEEP_DENSITIES = [0.1, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9]
SHARDED_SHAPES = [(12288, 49152), (49152, 12288)]
SKEWED_SHAPES = [(32000, 8192), (8192, 28672)]


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def bernoulli_matrix(rows: int, cols: int, density: float, seed: int, device="cpu", scale: float = 1.0):
    """fp16 N(0, scale^2) values under an iid Bernoulli(density) mask."""
    g = _gen(seed, device)
    w = torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32).mul_(scale).to(torch.float16)
    keep = torch.rand(rows, cols, generator=g, device=device) < density
    return w * keep


def magnitude_pruned_matrix(rows: int, cols: int, density: float, seed: int, device="cpu", scale: float = 0.02):
    """fp16 N(0, scale^2) weights; every row keeps exactly round(density*cols) largest-|w| entries."""
    g = _gen(seed, device)
    w = torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32).mul_(scale).to(torch.float16)
    k = int(round(density * cols))
    if k <= 0:
        return torch.zeros_like(w)
    if k >= cols:
        return w
    # k-th largest magnitude per row as threshold; ties (rare in fp16 but possible) are
    # broken by column order so that exactly k entries survive.
    mag = w.abs().float()
    order = torch.argsort(mag, dim=1, descending=True, stable=True)
    keep = torch.zeros(rows, cols, dtype=torch.bool, device=w.device)
    keep.scatter_(1, order[:, :k], True)
    return w * keep


def skewed_matrix(rows: int, cols: int, seed: int, device="cpu", mean_density: float = 0.2):
    """Rows of very uneven length with clustered non-zeros.

    Row density ~ Beta(0.5, 2) rescaled to `mean_density`; 5 % of the rows are forced fully
    dense and a disjoint 5 % empty; inside a row non-zeros come in runs of length
    Geometric(0.3) separated by geometric gaps sized to hit the row's density.
    """
    g = _gen(seed, "cpu")
    beta = torch.distributions.Beta(torch.tensor(0.5), torch.tensor(2.0))
    with torch.random.fork_rng(devices=[]):
        torch.manual_seed(seed)
        rho = beta.sample((rows,))
    rho = (rho * (mean_density / rho.mean())).clamp_(0.0, 1.0)
    perm = torch.randperm(rows, generator=g)
    n5 = max(1, rows // 20)
    rho[perm[:n5]] = 1.0
    rho[perm[n5 : 2 * n5]] = 0.0

    # The row densities above are drawn on the CPU (small); the run / gap lengths and the values, which are
    # rows x cols sized, are drawn on `device` with that device's generator.
    dev = torch.device(device)
    gd = _gen(seed + 1, dev)
    rho = rho.to(dev)
    p_run = 0.3
    mean_run = 1.0 / p_run
    # Alternating run / gap lengths, drawn for all rows at once: enough segments to cover
    # `cols` with margin, then a cumulative sum gives the segment boundaries.
    rho_c = rho.clamp(min=1e-4)
    mean_gap = (mean_run * (1.0 - rho_c) / rho_c).clamp(min=1e-3)
    n_seg = int(min(cols, max(64, 4 * cols / (mean_run + float(mean_gap.median())))))
    u_run = torch.rand(rows, n_seg, generator=gd, device=dev).clamp_(min=1e-12)
    runs = torch.floor(torch.log(u_run) / math.log(1.0 - p_run)).to(torch.int32) + 1
    del u_run
    u_gap = torch.rand(rows, n_seg, generator=gd, device=dev).clamp_(min=1e-12)
    p_gap = (1.0 / (mean_gap + 1.0)).unsqueeze(1)  # support >= 0, mean = mean_gap
    gaps = torch.floor(torch.log(u_gap) / torch.log1p(-p_gap.clamp(max=1 - 1e-9))).clamp_(max=cols).to(torch.int32)
    del u_gap
    seg = torch.stack([gaps, runs], dim=2).reshape(rows, 2 * n_seg)
    del gaps, runs
    edges = torch.cumsum(seg, dim=1, dtype=torch.int64).clamp_(max=cols)
    del seg
    # +1 at run starts, -1 at run ends, prefix-sum to a mask
    marks = torch.zeros(rows, cols + 1, dtype=torch.int32, device=dev)
    starts = edges[:, 0::2]
    ends = edges[:, 1::2]
    marks.scatter_add_(1, starts, torch.ones_like(starts, dtype=torch.int32))
    marks.scatter_add_(1, ends, -torch.ones_like(ends, dtype=torch.int32))
    del edges, starts, ends
    mask = torch.cumsum(marks[:, :cols], dim=1) > 0
    del marks
    # rows whose segments ran out before the row end stay sparse at the tail; fine for a stress test
    mask[rho >= 1.0] = True
    mask[rho <= 0.0] = False
    w = torch.randn(rows, cols, generator=gd, device=dev, dtype=torch.float32).to(torch.float16)
    w[w == 0] = 1.0
    return w * mask


def dense_vector(cols: int, seed: int, device="cpu"):
    g = _gen(seed, device)
    return torch.randn(cols, generator=g, device=device, dtype=torch.float32).to(torch.float16)


def sweep_seed(shape_idx: int, density_idx: int) -> int:
    return 2000 + 10 * shape_idx + density_idx


def algorithmic_bytes(padded_count: int, rows: int, cols: int) -> int:
    """Bytes one SpMV must move: values + deltas + row_indices + x + y."""
    return 2 * padded_count + padded_count // 2 + 4 * (rows + 1) + 2 * cols + 2 * rows


def dense_bytes(rows: int, cols: int) -> int:
    """Bytes a dense fp16 GEMV must move."""
    return 2 * rows * cols + 2 * cols + 2 * rows
