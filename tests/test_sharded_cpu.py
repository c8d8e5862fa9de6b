"""Host logic of the row-partitioned path on CPU: world_size-2 gloo processes partition a
matrix, multiply their blocks (the oracle stands in for the GPU kernel, as the checker it is)
and all-gather y; the result must equal the unsharded product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from macko_spmv_b200 import sharded


def _oracle_compress(M):
    v, d, ri, r, c = oracle.compress(M.numpy().view(np.uint16))
    return (torch.from_numpy(v.view(np.float16).copy()), torch.from_numpy(d.copy()), torch.from_numpy(ri.copy()), r, c)


def _oracle_multiply(comp, x):
    c = (comp[0].numpy().view(np.uint16), comp[1].numpy(), comp[2].numpy(), comp[3], comp[4])
    _, yh, _ = oracle.spmv(c, x.numpy().view(np.uint16))
    return torch.from_numpy(yh.view(np.float16).copy())


def _worker(rank, world, port, rows, cols, balanced, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(123)
        M = torch.randn(rows, cols, generator=g).half()
        dens = torch.rand(rows, 1, generator=g)  # uneven row lengths
        M[torch.rand(rows, cols, generator=g) > dens] = 0
        x = torch.randn(cols, generator=g).half()
        full = _oracle_compress(M)
        blocks = sharded.balanced_row_blocks(full[2], world) if balanced else None
        shard = sharded.shard_rows(M, blocks=blocks, compress_fn=_oracle_compress)
        lo, hi = shard.row_lo, shard.row_hi
        # a shard is exactly what compress returns for the sub-matrix
        sub = _oracle_compress(M[lo:hi].contiguous())
        assert all(torch.equal(a, b) for a, b in zip(shard.compressed[:3], sub[:3]))
        assert int(shard.compressed[2][0]) == 0 and shard.compressed[3] == hi - lo
        y = sharded.multiply_sharded(shard, x, multiply_fn=_oracle_multiply)
        ref = _oracle_multiply(full, x)
        ok = torch.equal(y.view(torch.int16), ref.view(torch.int16))
        q.put((rank, ok, (lo, hi)))
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("rows,balanced", [(64, False), (37, False), (50, True)])
def test_two_rank_row_sharding_gloo(rows, balanced):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, rows, 300, balanced, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(world))
    assert all(ok for _, ok, _ in results)
    blocks = [b for _, _, b in results]
    assert blocks[0][0] == 0 and blocks[0][1] == blocks[1][0] and blocks[1][1] == rows


def test_row_block_partition_properties():
    for rows in (0, 1, 7, 4096, 32000, 49152):
        for world in (1, 2, 3, 4, 8):
            blocks = [sharded.row_block(rows, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == rows
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in blocks]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharded.row_block(10, 2, 2)
    ri = torch.tensor([0, 100, 100, 110, 400, 401, 800], dtype=torch.int32)
    blocks = sharded.balanced_row_blocks(ri, 2)
    assert blocks[0][0] == 0 and blocks[-1][1] == 6 and blocks[0][1] == blocks[1][0]
    left = int(ri[blocks[0][1]] - ri[0])
    assert abs(left - 400) <= 300
