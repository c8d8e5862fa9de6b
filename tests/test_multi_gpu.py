"""Row-sharded product with the exchange fused into the kernel (`sharded.PeerGather`), run as child
processes, one per GPU: on a single GPU with world size 1 (the kernel's scatter epilogue, flags and
bounded wait run against its own buffers) and, when the box has two GPUs, with world size 2 against the
NCCL all-gather path and a dense fp32 product."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, ""
    try:
        from macko_spmv_b200 import sharded, workloads

        pg = sharded.PeerGather(12000, dev)
        for i, (rows, cols, d) in enumerate([(4096, 4096, 0.5), (11008, 2048, 0.1), (37 * world, 515, 0.5), (world, 64, 1.0)]):
            M = workloads.bernoulli_matrix(rows, cols, d, seed=10 + i, device=dev, scale=0.02)
            x = workloads.dense_vector(cols, 50 + i, dev)
            sh = sharded.shard_rows(M)
            ref = M.float() @ x.float()
            y_nccl = sharded.multiply_sharded(sh, x)
            for rep in range(3):   # consecutive calls alternate the two y slots and advance the counters
                y = pg.multiply(sh, x).clone()
                torch.cuda.synchronize()
                rel = float((y.float() - ref).norm() / ref.norm())
                if not torch.equal(y, y_nccl) or rel > 5e-3:
                    ok, msg = False, f"rank {rank}: {rows}x{cols} rep {rep} rel {rel}"
        if pg.error_flag() != 0:
            ok, msg = False, f"rank {rank}: wait gave up on rank {pg.error_flag() - 1}"
    except Exception as e:  # noqa: BLE001
        ok, msg = False, f"rank {rank}: {type(e).__name__}: {e}"
    q.put((rank, ok, msg))
    torch.cuda.synchronize()
    dist.barrier()
    os._exit(0)   # skip NCCL teardown, as bench.py does


def _run(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok, _ in results), [m for _, ok, m in results if not ok]


def test_fused_exchange_world_1():
    _run(1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_exchange_world_2():
    _run(2)
