"""Row-partitioned SpMV over several GPUs (one process per GPU, torch.distributed).

y[r] depends only on row r and on the whole x, so a matrix splits into contiguous row
blocks with no exchange on the way in; the one exchange step is the all-gather of the
y slices (NCCL over NVLink on GPUs, gloo in the CPU tests of the host logic). Every rank
compresses its own block, so its `row_indices` start at 0 and its buffers are exactly what
`compress` returns for that sub-matrix.

The reference is single-GPU; this module has no counterpart there.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


def row_block(rows: int, rank: int, world: int) -> tuple[int, int]:
    """Rows [lo, hi) owned by `rank`: contiguous blocks whose sizes differ by at most one."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    return rows * rank // world, rows * (rank + 1) // world


def balanced_row_blocks(row_indices: torch.Tensor, world: int) -> list[tuple[int, int]]:
    """Contiguous row blocks holding about the same number of stored elements each.

    `row_indices` is the int32 prefix array of the whole matrix. Useful when row lengths are
    very uneven and equal row counts would leave some GPUs with most of the bytes.
    """
    ri = row_indices.detach().to("cpu", torch.int64)
    rows = ri.numel() - 1
    total = int(ri[-1])
    cuts = [0]
    for k in range(1, world):
        target = total * k // world
        r = int(torch.searchsorted(ri, torch.tensor(target), right=False))
        cuts.append(min(max(r, cuts[-1]), rows))
    cuts.append(rows)
    return [(cuts[i], cuts[i + 1]) for i in range(world)]


@dataclass
class RowShard:
    """One rank's block of a row-partitioned compressed matrix."""

    compressed: tuple          # the 5-tuple of this block (rows of the block, all columns)
    row_lo: int
    row_hi: int
    total_rows: int
    blocks: list               # [(lo, hi)] of every rank, in rank order
    group: object = None

    @property
    def cols(self) -> int:
        return self.compressed[4]

    @property
    def even(self) -> bool:
        sizes = {hi - lo for lo, hi in self.blocks}
        return len(sizes) == 1


def shard_rows(M_block_or_full: torch.Tensor, total_rows: int | None = None, group=None,
               blocks: list | None = None, compress_fn=None) -> RowShard:
    """Compress this rank's row block.

    Pass either the full matrix (every rank slices its own block) or, with `total_rows`, the
    block itself. `compress_fn` defaults to this package's GPU `compress`.
    """
    if compress_fn is None:
        from . import compress as compress_fn  # late import: keeps this module importable on its own
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rows_full = M_block_or_full.size(0) if total_rows is None else total_rows
    if blocks is None:
        blocks = [row_block(rows_full, r, world) for r in range(world)]
    lo, hi = blocks[rank]
    block = M_block_or_full[lo:hi] if total_rows is None else M_block_or_full
    if block.size(0) != hi - lo:
        raise ValueError(f"rank {rank}: block has {block.size(0)} rows, expected {hi - lo}")
    return RowShard(compress_fn(block.contiguous()), lo, hi, rows_full, blocks, group)


def gather_rows(y_local: torch.Tensor, shard: RowShard, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gather the y slices into the full y (same on every rank).

    Equal blocks use one `all_gather_into_tensor` straight into `out`; uneven blocks are
    padded to the largest block for the collective and trimmed afterwards.
    """
    world = len(shard.blocks)
    if out is None:
        out = torch.empty(shard.total_rows, dtype=y_local.dtype, device=y_local.device)
    if world == 1:
        out.copy_(y_local)
        return out
    if shard.even:
        dist.all_gather_into_tensor(out, y_local.contiguous(), group=shard.group)
        return out
    width = max(hi - lo for lo, hi in shard.blocks)
    padded = torch.zeros(width, dtype=y_local.dtype, device=y_local.device)
    padded[: y_local.numel()] = y_local
    stage = torch.empty(world * width, dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(stage, padded, group=shard.group)
    for r, (lo, hi) in enumerate(shard.blocks):
        out[lo:hi] = stage[r * width : r * width + (hi - lo)]
    return out


def multiply_sharded(shard: RowShard, x: torch.Tensor, out: torch.Tensor | None = None,
                     multiply_fn=None) -> torch.Tensor:
    """Full y = M @ x on every rank: local SpMV on the block, then all-gather."""
    if multiply_fn is None:
        from . import multiply as multiply_fn
    y_local = multiply_fn(shard.compressed, x)
    return gather_rows(y_local, shard, out)
