"""Row-sharded product with the exchange fused into the kernel (`sharded.PeerGather`), run as child
processes, one per GPU: on a single GPU with world size 1 (the kernel's scatter epilogue, flags and
bounded wait run against its own buffers) and, when the box has two GPUs, with world size 2 against the
NCCL all-gather path and a dense fp32 product. NVLS is off in NCCL and the symmetric buffers are not bound
to an NVLink multicast object (`PeerGather` switches that off); every rank leaves between steps, after
dropping its buffers and the process group."""
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
        # deferred steps: several products publish without waiting, one wait at the end; two steps in a row use
        # the two halves of the buffers; the second pair of steps is replayed from CUDA graphs
        mats = []
        for i, (rows, cols, d) in enumerate([(4096, 1024, 0.5), (515, 2048, 0.2), (37 * world, 515, 0.5)]):
            M = workloads.bernoulli_matrix(rows, cols, d, seed=30 + i, device=dev, scale=0.02)
            x = workloads.dense_vector(cols, 70 + i, dev)
            sh = sharded.shard_rows(M)
            mats.append((sh, x, sharded.multiply_sharded(sh, x)))
        for overlap in (True, False):   # exchange by a forward kernel on a side stream / at the tail of the product kernel
            pd = sharded.PeerGather(4096, dev, step_rows=3 * 4096 + 64, overlap_forward=overlap)

            def step():
                pd.begin_step()
                ys = [pd.multiply_deferred(sh, x, immutable=True) for sh, x, _ in mats]
                pd.wait()
                return ys

            for rep in range(3):
                ys = step()
                torch.cuda.synchronize()
                for (sh, x, ref), y in zip(mats, ys):
                    if not torch.equal(y, ref):
                        ok, msg = False, f"rank {rank}: deferred step {rep}, {sh.total_rows} rows differ from the all-gather path"
            graphs, outs = [], []
            for _ in range(2):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    outs.append(step())
                graphs.append(g)
            for rep in range(4):
                for y in outs[rep % 2]:
                    y.zero_()
                torch.cuda.synchronize()
                dist.barrier()
                graphs[rep % 2].replay()
                torch.cuda.synchronize()
                for (sh, x, ref), y in zip(mats, outs[rep % 2]):
                    if not torch.equal(y, ref):
                        ok, msg = False, f"rank {rank}: graph replay {rep}, {sh.total_rows} rows differ"
            if pd.error_flag() != 0:
                ok, msg = False, f"rank {rank}: deferred wait gave up on rank {pd.error_flag() - 1}"
            del graphs, outs
            pd.close()
        pg.close()
    except Exception as e:  # noqa: BLE001
        ok, msg = False, f"rank {rank}: {type(e).__name__}: {e}"
    q.put((rank, ok, msg))
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def _decode_worker(rank, world, port, q):
    """A small Llama-architecture decoder, tensor parallel over `world` ranks, against the same model on
    one GPU: logits within tolerance of each other and bit-identical on every rank."""
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    ok, msg = True, ""
    try:
        from macko_spmv_b200 import llama_decode, sharded

        cfg = dict(hidden=256, heads=4, ffn=688, vocab=1000, layers=2, eps=1e-5, rope_theta=10000.0)
        pg = sharded.PeerGather(max(world * 256, 1000), dev)
        with torch.no_grad():
            tp = llama_decode.LlamaDecoder(0.5, cfg=cfg, device=dev, max_len=16, seed=123, peer=pg)
            one = llama_decode.LlamaDecoder(0.5, cfg=cfg, device=dev, max_len=16, seed=123)
            for i, tok in enumerate([5, 999, 0, 421]):
                token = torch.tensor([tok], device=dev)
                pos = torch.tensor([i], device=dev)
                a = tp.logits(token, pos).clone()
                b = one.logits(token, pos)
                rel = float((a.float() - b.float()).norm() / b.float().norm())
                ref = a.clone()
                dist.broadcast(ref, 0)
                if rel > 1e-2 or not torch.equal(ref, a):
                    ok, msg = False, f"rank {rank}: token {i} rel {rel} same_on_ranks {torch.equal(ref, a)}"
        if pg.error_flag() != 0:
            ok, msg = False, f"rank {rank}: wait gave up on rank {pg.error_flag() - 1}"
        del tp, one
        pg.close()
    except Exception as e:  # noqa: BLE001
        ok, msg = False, f"rank {rank}: {type(e).__name__}: {e}"
    q.put((rank, ok, msg))
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()


def _run(world, target=None):
    target = target or _worker
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=target, args=(r, world, port, q)) for r in range(world)]
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


def test_tensor_parallel_decode_world_1():
    _run(1, _decode_worker)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_decode_world_2():
    _run(2, _decode_worker)
