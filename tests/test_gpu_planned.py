"""GPU tests (`-m gpu`) of what sits around the plain product: the immutable-matrix flag, the planned
launch for long and uneven rows (plan against its definition, product against the oracle), bfloat16
values, the device-side bounds of the compressor, and the bounded waits of the row-sharded exchange.
Everything is called through the C ABI or the Python API, as in test_gpu_parity.py."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
import macko_spmv_b200 as macko_spmv
from macko_spmv_b200 import cabi, sharded, workloads

pytestmark = pytest.mark.gpu

MAX_ABS_FACTOR = 1e-3
REL_L2 = 5e-3


def _u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _check_y(y, comp_np, x_np, what=""):
    y64, _, l1 = oracle.spmv(comp_np, x_np)
    got = y.float().cpu().numpy().astype(np.float64)
    err = np.abs(got - y64)
    bad = err > MAX_ABS_FACTOR * l1 + 1e-12
    assert not bad.any(), f"{what}: {int(bad.sum())} rows beyond 1e-3*L1, worst {float((err / (l1 + 1e-30)).max()):.3e}"
    nrm = np.linalg.norm(y64)
    if nrm > 0:
        assert np.linalg.norm(got - y64) <= REL_L2 * nrm, f"{what}: relative L2 {np.linalg.norm(got - y64) / nrm:.3e}"
    else:
        assert np.all(got == 0)


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _build_plan(lib, comp, seg=0):
    rows, cols, P = comp[3], comp[4], comp[0].numel()
    nbytes = lib.macko_spmv_plan_bytes(rows, cols, P, seg)
    assert nbytes > 0
    plan = torch.empty(nbytes, dtype=torch.uint8, device=comp[0].device)
    info = cabi.PlanInfo()
    cabi.check(lib, lib.macko_spmv_plan(comp[1].data_ptr(), comp[2].data_ptr(), rows, cols, P, seg, plan.data_ptr(), nbytes,
                                        ctypes.byref(info), _stream()))
    return plan, info


def _planned(lib, comp, plan, info, x, y=None, alpha=1.0, beta=0.0, flags=0):
    rows, cols = comp[3], comp[4]
    if y is None:
        y = torch.full((rows,), float("nan"), dtype=torch.float16, device=x.device)
    cabi.check(lib, lib.macko_spmv_fp16_planned(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                                comp[0].numel(), plan.data_ptr(), ctypes.byref(info), x.data_ptr(),
                                                y.data_ptr(), alpha, beta, flags, _stream()))
    return y


def _long_and_short_rows(rows, cols, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    M = workloads.bernoulli_matrix(rows, cols, 0.03, seed=seed + 1, device="cuda")
    dense_rows = torch.randperm(rows, generator=g, device="cuda")[: max(2, rows // 12)]
    M[dense_rows] = (torch.randn(dense_rows.numel(), cols, generator=g, device="cuda") * 0.5).half()
    M[dense_rows[0], :3] = 0
    M[dense_rows[1], cols - 5:] = 0
    half_rows = torch.randperm(rows, generator=g, device="cuda")[: max(1, rows // 20)]
    M[half_rows, : cols // 2] = 1.0
    M[1] = 0
    return M


# ---------------------------------------------------------------- immutable-matrix flag

def test_immutable_flag_gives_the_same_bits():
    lib = cabi.load()
    for (rows, cols, d) in [(4096, 4096, 0.5), (333, 1001, 0.2), (11008, 4096, 0.1), (7, 30000, 0.5), (64, 120000, 0.05)]:
        M = workloads.bernoulli_matrix(rows, cols, d, seed=rows + cols, device="cuda", scale=0.02)
        comp = macko_spmv.compress(M)
        x = workloads.dense_vector(cols, 3, "cuda")
        plain = macko_spmv.multiply(comp, x)
        torch.cuda.synchronize()
        y = torch.full((rows,), float("nan"), dtype=torch.float16, device="cuda")
        for _ in range(3):   # back to back: the second and third launch overlap the one in front
            cabi.check(lib, lib.macko_spmv_fp16_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                                   comp[0].numel(), x.data_ptr(), y.data_ptr(), 1.0, 0.0,
                                                   cabi.SPMV_MATRIX_IMMUTABLE, _stream()))
        assert torch.equal(y.view(torch.int16), plain.view(torch.int16)), (rows, cols, d)
        frozen = macko_spmv.freeze(comp, plan=False)
        assert isinstance(frozen, tuple) and len(frozen) == 5 and frozen.plan is None
        assert torch.equal(macko_spmv.multiply(frozen, x).view(torch.int16), plain.view(torch.int16))
    with pytest.raises(cabi.MackoError):
        cabi.check(lib, lib.macko_spmv_fp16_ex(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                               comp[0].numel(), x.data_ptr(), y.data_ptr(), 1.0, 0.0, 64, _stream()))


def test_x_written_by_the_kernel_in_front_is_seen():
    # x is produced by the previous kernel of the stream and y feeds the next product: with the matrix loads
    # moved in front of the wait for that kernel, x and y still have to be read behind it
    rows = cols = 2048
    M = workloads.bernoulli_matrix(rows, cols, 0.3, seed=77, device="cuda", scale=0.05)
    frozen = macko_spmv.freeze(macko_spmv.compress(M))
    x0 = workloads.dense_vector(cols, 5, "cuda")
    ref = x0
    for _ in range(6):
        ref = (M.float() @ ref.float()).half()
    got = x0
    for _ in range(6):
        got = macko_spmv.multiply(frozen, got)
    assert float((got.float() - ref.float()).norm() / ref.float().norm()) < 2e-2
    # the same chain as one CUDA graph
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        macko_spmv.multiply(frozen, x0)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = x0
        for _ in range(6):
            out = macko_spmv.multiply(frozen, out)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), got.view(torch.int16))


# ---------------------------------------------------------------- plan

@pytest.mark.parametrize("seg", [256, 1024])
def test_plan_matches_its_definition(seg):
    lib = cabi.load()
    rows, cols = 700, 9000
    M = _long_and_short_rows(rows, cols, 9)
    comp = macko_spmv.compress(M)
    plan, info = _build_plan(lib, comp, seg)
    d0, d1, out, seg_first = oracle.plan_model(comp[1].cpu().numpy(), comp[2].cpu().numpy(), seg)
    V = int(seg_first[-1])
    assert info.virtual_rows == V and info.segment_elements == seg and info.rows == rows
    assert info.longest_row == int(np.diff(comp[2].cpu().numpy().astype(np.int64)).max())
    assert info.split_rows == int((np.diff(seg_first) > 1).sum())
    # sections of the plan buffer (offsets of macko_spmv_b200/csrc/plan.cuh: 256-byte aligned, in this order)
    raw = plan.cpu().numpy()
    up = lambda b: (b + 255) & ~255
    v_max = rows + (comp[0].numel() + 8 * rows) // seg + 1
    at = up(64)
    got_seg_first = raw[at: at + 4 * (rows + 1)].view(np.int32); at = up(at + 4 * (rows + 1))
    split_list = raw[at: at + 4 * info.split_rows].view(np.uint32); at = up(at + 4 * (rows + 1))
    desc = raw[at: at + 8 * V].view(np.uint32).reshape(V, 2); at = up(at + 8 * v_max)
    got_out = raw[at: at + 4 * V].view(np.uint32); at = up(at + 4 * v_max)
    assert np.array_equal(got_seg_first.astype(np.int64), seg_first)
    assert sorted(split_list.tolist()) == np.nonzero(np.diff(seg_first) > 1)[0].tolist(), "rows cut into several segments"
    assert np.array_equal(desc[:, 0].astype(np.int64), d0), "first elements / order"
    assert np.array_equal(desc[:, 1].astype(np.int64), d1), "lengths and column sums"
    assert np.array_equal(got_out.astype(np.int64), out), "destinations"


@pytest.mark.parametrize("shape", [(3000, 8192), (700, 28672), (40, 4096), (1, 9000), (5, 33), (64, 100000)])
def test_planned_product_long_rows_among_short_ones(shape):
    rows, cols = shape
    lib = cabi.load()
    M = _long_and_short_rows(rows, cols, rows) if rows >= 40 else workloads.bernoulli_matrix(rows, cols, 0.6, seed=rows, device="cuda")
    comp = macko_spmv.compress(M)
    comp_np = oracle.compress(_u16(M).reshape(rows, cols))
    x = workloads.dense_vector(cols, 9, "cuda")
    xn = _u16(x)
    for seg in (0, 256, 3840):
        plan, info = _build_plan(lib, comp, seg)
        y = _planned(lib, comp, plan, info, x)
        _check_y(y, comp_np, xn, f"{shape} seg={seg}")
        again = _planned(lib, comp, plan, info, x, flags=cabi.SPMV_MATRIX_IMMUTABLE)
        assert torch.equal(y.view(torch.int16), again.view(torch.int16)), "segments must be summed in a fixed order"
    # alpha / beta through the plan (cut rows read y once, when their last segment arrives)
    y0 = torch.ones(rows, dtype=torch.float16, device="cuda")
    _planned(lib, comp, plan, info, x, y=y0, alpha=0.5, beta=2.0)
    ref = macko_spmv.multiply(comp, x).float() * 0.5 + 2.0
    assert torch.allclose(y0.float(), ref, rtol=2e-3, atol=2e-3 * float(ref.abs().max()) + 1e-3)


def test_planned_product_edge_matrices():
    lib = cabi.load()
    g = torch.Generator().manual_seed(5)
    for (rows, cols) in [(1, 1), (3, 32), (33, 257), (1000, 1), (257, 1000)]:
        for dens in (0.0, 0.01, 0.5, 1.0):
            M = torch.randn(rows, cols, generator=g).half()
            M[torch.rand(rows, cols, generator=g) > dens] = 0
            comp_np = oracle.compress(_u16(M).reshape(rows, cols))
            comp = macko_spmv.compress(M.cuda())
            x = torch.randn(cols, generator=g).half().cuda()
            plan, info = _build_plan(lib, comp, 256)
            _check_y(_planned(lib, comp, plan, info, x), comp_np, _u16(x), f"{rows}x{cols} d={dens}")


def test_freeze_picks_the_plan_for_skewed_rows_only():
    skew = workloads.skewed_matrix(4000, 8192, seed=5000, device="cuda")
    comp = macko_spmv.compress(skew)
    fz = macko_spmv.freeze(comp)
    assert fz.plan is not None and fz.plan_meta[4] == 1
    x = workloads.dense_vector(8192, 5, "cuda")
    _check_y(macko_spmv.multiply(fz, x), oracle.compress(_u16(skew).reshape(4000, 8192)), _u16(x), "skewed, planned")
    even = macko_spmv.compress(workloads.magnitude_pruned_matrix(4096, 4096, 0.5, seed=1, device="cuda"))
    assert macko_spmv.freeze(even).plan is None
    from macko_spmv_b200.linear import MackoLinear

    layer = MackoLinear(comp).freeze()
    out = layer(x)
    assert torch.equal(out.view(torch.int16), macko_spmv.multiply(fz, x).view(torch.int16))


# ---------------------------------------------------------------- bfloat16

def test_bf16_compress_and_multiply():
    g = torch.Generator().manual_seed(11)
    for (rows, cols, d) in [(257, 1000, 0.3), (4096, 4096, 0.5), (33, 20000, 0.05)]:
        M = (torch.randn(rows, cols, generator=g) * 0.05).bfloat16()
        M[torch.rand(rows, cols, generator=g) > d] = 0
        bits = M.view(torch.int16)
        bits[(torch.rand(rows, cols, generator=g) < 0.02) & (bits == 0)] = -32768        # -0.0
        bits[0, 0] = 0x7F00          # a large finite bf16: an fp16 NaN test would destroy it
        bits[0, 1 % cols] = 0x7FA5   # a bf16 NaN: stored as 0x7fff
        exp = oracle.compress(_u16(M).reshape(rows, cols), bf16=True)
        comp = macko_spmv.compress(M.cuda())
        assert comp[0].dtype == torch.bfloat16
        assert np.array_equal(_u16(comp[0]), exp[0]) and np.array_equal(comp[1].cpu().numpy(), exp[1])
        assert np.array_equal(comp[2].cpu().numpy(), exp[2])
        # multiply on a NaN-free copy
        bits[0, 1 % cols] = 0
        bits[0, 0] = 0x3F80
        exp = oracle.compress(_u16(M).reshape(rows, cols), bf16=True)
        comp = macko_spmv.compress(M.cuda())
        x = torch.randn(cols, generator=g).bfloat16().cuda()
        y = macko_spmv.multiply(comp, x)
        assert y.dtype == torch.bfloat16
        y64, l1 = oracle.spmv_bf16(exp, _u16(x))
        got = y.float().cpu().numpy().astype(np.float64)
        # the result itself is rounded to bf16 (8 significant bits): half an ulp of y on top of the accumulation bound
        assert np.all(np.abs(got - y64) <= MAX_ABS_FACTOR * l1 + np.abs(y64) * 2.0 ** -8 + 1e-12), (rows, cols, d)
        assert np.linalg.norm(got - y64) <= REL_L2 * np.linalg.norm(y64)
        frozen = macko_spmv.freeze(comp)
        assert torch.equal(macko_spmv.multiply(frozen, x).view(torch.int16), y.view(torch.int16))
    with pytest.raises(RuntimeError, match="torch.half"):
        macko_spmv.multiply(comp, x.half())


# ---------------------------------------------------------------- compressor: device-side bounds

def test_emit_refuses_stores_beyond_padded_count():
    lib = cabi.load()
    rows, cols = 300, 2000
    M = workloads.bernoulli_matrix(rows, cols, 0.4, seed=3, device="cuda")
    stream = _stream()
    ri = torch.empty(rows + 1, dtype=torch.int32, device="cuda")
    cabi.check(lib, lib.macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr(), stream))
    n = int(ri[rows].item())
    P_true = (n + 7) // 8 * 8
    P_small = P_true - 64            # a stale, too small P: 57..64 stored elements have no room
    margin = 1 << 16                  # guard bytes far larger than the excess
    count = ctypes.c_uint32(123)
    cabi.check(lib, lib.macko_compress_overflow(ctypes.byref(count), stream))   # clear what earlier tests left

    def run(entry):
        vbuf = torch.full((P_small + margin,), 0x5A5A, dtype=torch.int16, device="cuda")
        dbuf = torch.full((P_small // 2 + margin,), 0xA5, dtype=torch.uint8, device="cuda")
        wbuf = torch.full((P_small + margin,), 0xC3, dtype=torch.uint8, device="cuda")
        if entry == "workspace":
            st = lib.macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr(), P_small, vbuf.data_ptr(), dbuf.data_ptr(),
                                         wbuf.data_ptr(), P_small, stream)
        else:
            st = lib.macko_compress_emit_static(M.data_ptr(), rows, cols, ri.data_ptr(), P_small, vbuf.data_ptr(),
                                                dbuf.data_ptr(), stream)
        cabi.check(lib, st)
        torch.cuda.synchronize()
        assert bool((vbuf[P_small:] == 0x5A5A).all()), f"{entry}: values written beyond P"
        assert bool((dbuf[P_small // 2:] == 0xA5).all()), f"{entry}: deltas written beyond P/2"
        if entry == "workspace":
            assert bool((wbuf[P_small:] == 0xC3).all()), "workspace written beyond its size"
        c = ctypes.c_uint32(0)
        cabi.check(lib, lib.macko_compress_overflow(ctypes.byref(c), stream))
        assert c.value > 0, f"{entry}: the refused stores were not counted"
        cabi.check(lib, lib.macko_compress_overflow(ctypes.byref(c), stream))
        assert c.value == 0, "reading the counter clears it"

    run("workspace")
    run("static")
    # a consistent call afterwards is complete and leaves the counter at zero
    comp = macko_spmv.compress(M)
    exp = oracle.compress(_u16(M).reshape(rows, cols))
    assert np.array_equal(_u16(comp[0]), exp[0]) and np.array_equal(comp[1].cpu().numpy(), exp[1])
    cabi.check(lib, lib.macko_compress_overflow(ctypes.byref(count), stream))
    assert count.value == 0


# ---------------------------------------------------------------- row-sharded exchange without other GPUs

def _flags(world):
    return torch.zeros(world + 3 + 13, dtype=torch.int32, device="cuda")


def test_bounded_wait_runs_out_and_says_who_was_missing():
    lib = cabi.load()
    stream = _stream()
    # one rank whose own arrival counter is behind its call counter
    f = _flags(1)
    f[1] = 1
    cabi.check(lib, lib.macko_peer_wait_limited(f.data_ptr(), 1, 1000, stream))
    torch.cuda.synchronize()
    assert int(f[1 + 2]) == 1
    # three ranks, rank 2 never arrives
    f = _flags(3)
    f[0] = 1; f[1] = 1; f[3] = 1
    cabi.check(lib, lib.macko_peer_wait_limited(f.data_ptr(), 3, 1000, stream))
    torch.cuda.synchronize()
    assert int(f[3 + 2]) == 1 + 2
    # all arrived: no flag
    f = _flags(3)
    f[0] = 5; f[1] = 4; f[2] = 4; f[3] = 4
    cabi.check(lib, lib.macko_peer_wait_limited(f.data_ptr(), 3, 1000, stream))
    torch.cuda.synchronize()
    assert int(f[3 + 2]) == 0
    # the wait at the tail of the scatter kernel: rank 0 of a world of two whose peer (buffers in this GPU's
    # own memory, nothing behind them) never delivers; the kernel gives up after `spin_limit` polls, records
    # rank 1 as missing and returns with its own slice in place
    rows, cols = 512, 1024
    M = workloads.bernoulli_matrix(rows, cols, 0.5, seed=8, device="cuda", scale=0.02)
    comp = macko_spmv.compress(M[: rows // 2].contiguous())
    x = workloads.dense_vector(cols, 9, "cuda")
    ys = [torch.zeros(rows, dtype=torch.float16, device="cuda") for _ in range(2)]
    fl = [_flags(2) for _ in range(2)]
    ptrs = ctypes.c_void_p * 2
    cabi.check(lib, lib.macko_spmv_fp16_scatter_ex(
        comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(), x.data_ptr(),
        ptrs(ys[0].data_ptr(), ys[1].data_ptr()), 0, ptrs(fl[0].data_ptr(), fl[1].data_ptr()), 0, 2, 0, 1000, stream))
    torch.cuda.synchronize()
    assert int(fl[0][2 + 2]) == 1 + 1, "rank 1 should be reported missing"
    assert int(fl[0][0]) == 1 and int(fl[1][0]) == 1, "rank 0 published its arrival to both ranks"
    ref = macko_spmv.multiply(comp, x)
    assert torch.equal(ys[0][: rows // 2], ref) and torch.equal(ys[1][: rows // 2], ref)
    # and an ordinary product afterwards is unaffected
    assert torch.equal(macko_spmv.multiply(comp, x), ref)


@pytest.mark.parametrize("split", [False, True])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_deferred_exchange_all_ranks_on_one_gpu(world, split):
    """The N-rank data path of the fused exchange with every rank's buffers in this GPU's memory: each rank's
    product forwards its slice to all "peers" and publishes its counter without waiting (deferred), then
    every rank's wait kernel runs. No kernel waits for a later one, so one stream on one GPU is enough.
    `split`: the exchange as a kernel of its own (macko_peer_forward) behind an ordinary product."""
    lib = cabi.load()
    stream = _stream()
    ptrs = ctypes.c_void_p * world
    for (rows, cols, d) in [(4096, 4096, 0.5), (37 * world + 3, 515, 0.5), (world, 64, 1.0), (11008, 2048, 0.1)]:
        M = workloads.bernoulli_matrix(rows, cols, d, seed=rows, device="cuda", scale=0.02)
        x = workloads.dense_vector(cols, 4, "cuda")
        ys = [torch.full((rows + 8,), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
        fl = [_flags(world) for _ in range(world)]
        ytab = ptrs(*[y.data_ptr() for y in ys])
        ftab = ptrs(*[f.data_ptr() for f in fl])
        full = torch.empty(rows, dtype=torch.float16, device="cuda")
        for rep in range(2):
            for r in range(world):
                lo, hi = sharded.row_block(rows, r, world)
                comp = macko_spmv.compress(M[lo:hi].contiguous())
                full[lo:hi] = macko_spmv.multiply(comp, x)
                if split:   # the product into the rank's own buffer, then the forward kernel
                    cabi.check(lib, lib.macko_spmv_fp16_ex(
                        comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(),
                        x.data_ptr(), ys[r].data_ptr() + 2 * lo, 1.0, 0.0, cabi.SPMV_MATRIX_IMMUTABLE * (rep == 1), stream))
                    cabi.check(lib, lib.macko_peer_forward(ytab, lo, hi - lo, ftab, r, world, stream))
                    continue
                cabi.check(lib, lib.macko_spmv_fp16_scatter_ex(
                    comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), comp[3], comp[4], comp[0].numel(),
                    x.data_ptr(), ytab, lo, ftab, r, world,
                    cabi.SCATTER_DEFERRED_WAIT | cabi.SPMV_MATRIX_IMMUTABLE * (rep == 1), 1000, stream))
            for r in range(world):
                cabi.check(lib, lib.macko_peer_wait_limited(fl[r].data_ptr(), world, 1000, stream))
            torch.cuda.synchronize()
            for r in range(world):
                assert torch.equal(ys[r][:rows].view(torch.int16), full.view(torch.int16)), (rows, cols, r, rep)
                assert int(fl[r][world + 2]) == 0, "a wait gave up"
                assert all(int(fl[r][p]) == rep + 1 for p in range(world))


# ---------------------------------------------------------------- int8 values

def _assert_int8_buffers(comp, exp, what=""):
    assert comp[0].dtype == torch.int8 and comp[1].dtype == torch.uint8 and comp[2].dtype == torch.int32
    assert np.array_equal(comp[0].cpu().numpy(), exp[0]), f"values differ {what}"
    assert np.array_equal(comp[1].cpu().numpy(), exp[1]), f"deltas differ {what}"
    assert np.array_equal(comp[2].cpu().numpy(), exp[2]), f"row_indices differ {what}"


def test_int8_compress_fixtures_from_compiled_reference(reference_cases_int8):
    lib = cabi.load()
    stream = _stream()
    for c in reference_cases_int8:
        M = torch.from_numpy(c["dense"]).cuda()
        exp = (c["values"], c["deltas"], c["row_indices"])
        _assert_int8_buffers(macko_spmv.compress(M), exp, c["name"] + " (python api)")
        # the C ABI with raw pointers, at a 1-byte-aligned address as well (scalar load path)
        rows, cols = M.shape
        buf = torch.zeros(rows * cols + 1, dtype=torch.int8, device="cuda")
        Mo = buf[1:].view(rows, cols)
        Mo.copy_(M)
        ri = torch.empty(rows + 1, dtype=torch.int32, device="cuda")
        cabi.check(lib, lib.macko_compress_count_int8(Mo.data_ptr(), rows, cols, ri.data_ptr(), stream))
        P = (int(ri[rows].item()) + 7) // 8 * 8
        values = torch.empty(P, dtype=torch.int8, device="cuda")
        deltas = torch.empty(P // 2, dtype=torch.uint8, device="cuda")
        ws = torch.empty(max(P, 8), dtype=torch.uint8, device="cuda")
        cabi.check(lib, lib.macko_compress_emit_int8(Mo.data_ptr(), rows, cols, ri.data_ptr(), P, values.data_ptr(),
                                                     deltas.data_ptr(), ws.data_ptr(), ws.numel(), stream))
        _assert_int8_buffers((values, deltas, ri), exp, c["name"] + " (c abi, unaligned)")


@pytest.mark.parametrize("shape", [(1, 1), (5, 33), (33, 257), (257, 1000), (1000, 1), (7, 30000), (4096, 4096), (11008, 4096)])
def test_int8_compress_and_multiply_against_oracle(shape):
    rows, cols = shape
    g = torch.Generator().manual_seed(rows * 131 + cols)
    for dens in (0.0, 0.01, 0.1, 0.5, 1.0):
        M = torch.randint(-128, 128, (rows, cols), generator=g, dtype=torch.int8)
        M[torch.rand(rows, cols, generator=g) > dens] = 0
        exp = oracle.compress_int8(M.numpy())
        comp = macko_spmv.compress(M.cuda())
        _assert_int8_buffers(comp, exp, f"{shape} d={dens}")
        x = (torch.randn(cols, generator=g) * 0.1).half()
        y64, l1 = oracle.spmv_int8(exp, _u16(x))
        for name, cm in (("default", comp), ("frozen", macko_spmv.freeze(comp))):
            y = macko_spmv.multiply(cm, x.cuda())
            assert y.dtype == torch.float16 and y.shape == (rows,)
            got = y.float().cpu().numpy().astype(np.float64)
            err = np.abs(got - y64)
            assert np.all(err <= MAX_ABS_FACTOR * l1 + 1e-12), f"{shape} d={dens} {name}: worst {float((err / (l1 + 1e-30)).max()):.3e} of L1"
            nrm = np.linalg.norm(y64)
            assert np.linalg.norm(got - y64) <= REL_L2 * nrm + 1e-12, f"{shape} d={dens} {name}"
    # alpha / beta and the error behaviour of the other entry points
    y0 = torch.ones(rows, dtype=torch.float16, device="cuda")
    torch.ops.macko_spmv.multiply_out(comp[0], comp[1], comp[2], rows, cols, x.cuda(), y0, 0.5, 2.0)
    ref = macko_spmv.multiply(comp, x.cuda()).float() * 0.5 + 2.0
    assert torch.allclose(y0.float(), ref, rtol=2e-3, atol=2e-3 * float(ref.abs().max()) + 1e-3)
    with pytest.raises(RuntimeError, match="torch.half"):
        macko_spmv.multiply(comp, x.cuda().float())
    with pytest.raises(RuntimeError):
        macko_spmv.decompress(comp)
