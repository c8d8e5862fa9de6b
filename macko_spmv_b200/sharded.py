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

    Replaces `multiply_sharded`'s NCCL all-gather by the fused epilogue of `macko_spmv_fp16_scatter_ex`:
    no collective call. The full-y buffers and the flag words live in torch symmetric memory (peer-mapped on
    every rank; plain peer stores and flags, no NVLink multicast: binding to a multicast object is switched
    off before the first allocation unless the environment already says otherwise).

    Two ways to use it:

    * `multiply(shard, x)`: the kernel ends only when the slices of all ranks have landed (its last CTA
      waits, bounded). Two y slots alternate, so a result stays valid until the call after next. Two
      consecutive calls must never use the same slot (a faster rank writes its slice of the next product while
      a slower one may still read the previous y): a fixed sequence with an odd number of calls that is
      replayed again and again (a captured decode step) gives one of its calls `slot=2`, the spare slot.
    * `begin_step()`, then any number of `multiply_deferred(shard, x)`, then `wait()`: every product writes
      its rows into this rank's own buffer with the ordinary kernel; a small forward kernel on a side stream
      (a branch of the graph when captured) copies them to the other ranks and publishes the arrival, beside
      the next products (`overlap_forward=False`: the scatter kernel does both, without waiting). Each product
      gets its own region of the step's half of the buffer, and one bounded wait kernel at the end makes all
      of them complete. The two halves alternate from step to step: a rank that is already in
      step s + 1 writes into the half nobody reads any more, because it passed `wait()` of step s only
      after every rank had delivered step s, i.e. had already consumed step s - 1 in stream order.
    """

    def __init__(self, max_rows: int, device, group=None, step_rows: int = 0, overlap_forward: bool = True):
        import ctypes
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        from . import cabi

        self._ctypes = ctypes
        self.lib = cabi.load()
        self.check = cabi.check
        self._cabi = cabi
        group = group if group is not None else dist.group.WORLD
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("PeerGather supports at most 8 ranks (one NVLink domain)")
        self.max_rows = int(max_rows)
        # rows of one deferred step (sum over its products, each rounded up to 8), at least one product
        self.step_rows = max(int(step_rows), (self.max_rows + 7) // 8 * 8)
        self.buf = symm_mem.empty((3, self.step_rows), dtype=torch.float16, device=device)   # two alternating slots / halves + a spare
        self.handle = symm_mem.rendezvous(self.buf, group)
        pad = self.handle.get_signal_pad(self.rank)
        pad.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        self._ptr_array = ctypes.c_void_p * self.world
        self._base = [int(p) for p in self.handle.buffer_ptrs]
        self._tables = {}
        # the flag words sit 1 KiB into each rank's signal pad, clear of the slots torch's own barriers use
        self._flag_table = self._ptr_array(*[int(p) + 1024 for p in self.handle.signal_pad_ptrs])
        self._local_flags = int(self.handle.signal_pad_ptrs[self.rank]) + 1024
        self._slot = 0
        self._half = 1
        self._cursor = 0
        self.spin_limit = 0   # 0 = library default (2^23 polls)
        self.overlap_forward = bool(overlap_forward)
        self._side = torch.cuda.Stream(device=device)
        self._side_busy = False

    def _table(self, half: int, offset: int):
        key = (half, offset)
        t = self._tables.get(key)
        if t is None:
            t = self._ptr_array(*[b + (half * self.step_rows + offset) * 2 for b in self._base])
            self._tables[key] = t
        return t

    def _launch(self, shard: RowShard, x: torch.Tensor, table, flags: int):
        comp = shard.compressed
        stream = torch.cuda.current_stream().cuda_stream
        self.check(self.lib, self.lib.macko_spmv_fp16_scatter_ex(
            comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(),
            x.data_ptr(), table, shard.row_lo, self._flag_table, self.rank, self.world, flags, self.spin_limit, stream))

    def multiply(self, shard: RowShard, x: torch.Tensor, immutable: bool = False, slot: int | None = None,
                 defer_wait: bool = False) -> torch.Tensor:
        """Full y (a view of the current slot, length shard.total_rows) after all ranks delivered.
        `immutable`: the shard's buffers are final (weights), see MACKO_SPMV_MATRIX_IMMUTABLE.
        `defer_wait`: the kernel publishes this rank's slice and returns; the reader of the view waits for the
        other ranks itself (`wait()`, or a kernel that takes `flags_address`, like `add_rmsnorm_peer`).
        `slot`: None = the two alternating slots; 2 = the spare slot (see the class description)."""
        if shard.total_rows > self.max_rows:
            raise ValueError(f"matrix has {shard.total_rows} rows, the exchange buffers hold {self.max_rows}")
        if slot is None:
            slot = self._slot
            self._slot ^= 1
        elif slot not in (0, 1, 2):
            raise ValueError("slot must be 0, 1 or 2")
        self._launch(shard, x, self._table(slot, 0), (self._cabi.SPMV_MATRIX_IMMUTABLE if immutable else 0) |
                     (self._cabi.SCATTER_DEFERRED_WAIT if defer_wait else 0))
        # the kernel itself returns only after the slices of all ranks have landed (its last CTA waits)
        return self.buf[slot, : shard.total_rows]

    def begin_step(self) -> None:
        """Start a new deferred step: switch to the other half of the buffer."""
        self._half ^= 1
        self._cursor = 0

    def multiply_deferred(self, shard: RowShard, x: torch.Tensor, immutable: bool = False) -> torch.Tensor:
        """Enqueue the product; the returned view of the step's buffer is complete only after `wait()`."""
        rows8 = (shard.total_rows + 7) // 8 * 8
        if self._cursor + rows8 > self.step_rows:
            raise ValueError(f"the step's products need more than the {self.step_rows} rows the buffers hold")
        off = self._cursor
        self._cursor += rows8
        table = self._table(self._half, off)
        if not self.overlap_forward:
            flags = self._cabi.SCATTER_DEFERRED_WAIT | (self._cabi.SPMV_MATRIX_IMMUTABLE if immutable else 0)
            self._launch(shard, x, table, flags)
            return self.buf[self._half, off : off + shard.total_rows]
        comp = shard.compressed
        main = torch.cuda.current_stream()
        y_own = int(table[self.rank]) + 2 * shard.row_lo
        self.check(self.lib, self.lib.macko_spmv_fp16_ex(
            comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(),
            x.data_ptr(), y_own, 1.0, 0.0, self._cabi.SPMV_MATRIX_IMMUTABLE if immutable else 0, main.cuda_stream))
        done = torch.cuda.Event()
        done.record(main)
        self._side.wait_event(done)
        self.check(self.lib, self.lib.macko_peer_forward(table, shard.row_lo, comp[3], self._flag_table, self.rank,
                                                         self.world, self._side.cuda_stream))
        self._side_busy = True
        return self.buf[self._half, off : off + shard.total_rows]

    def wait(self) -> None:
        """Enqueue the bounded wait for the slices of all ranks of every product issued so far."""
        main = torch.cuda.current_stream()
        if self._side_busy:
            main.wait_stream(self._side)   # the forwards of this step (joins the side branch when captured)
            self._side_busy = False
        self.check(self.lib, self.lib.macko_peer_wait_limited(self._local_flags, self.world, self.spin_limit, main.cuda_stream))

    @property
    def flags_address(self) -> int:
        """Device address of this rank's flag words, for kernels that wait for the exchange themselves."""
        return self._local_flags

    def error_flag(self) -> int:
        """0, or 1 + the rank whose slice never arrived in some earlier wait (reads device memory)."""
        pad = self.handle.get_signal_pad(self.rank).view(torch.int32)
        return int(pad[256 + self.world + 2].item())

    def close(self) -> None:
        """Drop the symmetric buffers (after a device synchronisation): call before the process group is torn down."""
        torch.cuda.synchronize()
        self._tables.clear()
        self.handle = None
        self.buf = None
