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


class PeerGather:
    """Row-sharded SpMV whose kernel stores y straight into every rank's full y over NVLink.

    Replaces `multiply_sharded`'s NCCL all-gather by the fused epilogue of
    `macko_spmv_fp16_scatter`: no collective call and no extra kernel (the last CTA of the grid waits
    for the other ranks' flags before the kernel ends).
    The full-y buffers and the flag words live in torch symmetric memory (peer-mapped on every rank).
    Two y slots are used alternately, so the result of a call stays valid until the call after next.
    """

    def __init__(self, max_rows: int, device, group=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import cabi

        self._ctypes = ctypes
        self.lib = cabi.load()
        self.check = cabi.check
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerGather supports at most 8 ranks (one NVLink domain)")
        self.max_rows = int(max_rows)
        self.buf = symm_mem.empty((2, self.max_rows), dtype=torch.float16, device=device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        pad = self.handle.get_signal_pad(self.rank)
        pad.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        ptr_array = ctypes.c_void_p * self.world
        base = [int(p) for p in self.handle.buffer_ptrs]
        self._y_tables = [ptr_array(*[b + slot * self.max_rows * 2 for b in base]) for slot in (0, 1)]
        # the flag words sit 1 KiB into each rank's signal pad, clear of the slots torch's own barriers use
        self._flag_table = ptr_array(*[int(p) + 1024 for p in self.handle.signal_pad_ptrs])
        self._local_flags = int(self.handle.signal_pad_ptrs[self.rank]) + 1024
        self._slot = 0

    def multiply(self, shard: RowShard, x: torch.Tensor) -> torch.Tensor:
        """Full y (a view of the current slot, length shard.total_rows) after all ranks delivered."""
        if shard.total_rows > self.max_rows:
            raise ValueError(f"matrix has {shard.total_rows} rows, the exchange buffers hold {self.max_rows}")
        comp = shard.compressed
        stream = torch.cuda.current_stream().cuda_stream
        slot = self._slot
        self._slot ^= 1
        self.check(self.lib, self.lib.macko_spmv_fp16_scatter(
            comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(),
            x.data_ptr(), self._y_tables[slot], shard.row_lo, self._flag_table, self.rank, self.world, stream))
        # the kernel itself returns only after the slices of all ranks have landed (its last CTA waits)
        return self.buf[slot, : shard.total_rows]

    def error_flag(self) -> int:
        """0, or 1 + the rank whose slice never arrived in some earlier wait (reads device memory)."""
        pad = self.handle.get_signal_pad(self.rank).view(torch.int32)
        return int(pad[256 + self.world + 2].item())
