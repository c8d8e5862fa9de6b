"""GPU parity tests (run with `-m gpu` on a B200): the CUDA compressor must be bit-exact
against the oracle / the reference fixtures, and the SpMV must match the oracle within
    |y - y_ref| <= 1e-3 * sum_k |val_k * x[col_k]|     (per row)
    ||y - y_ref||_2 <= 5e-3 * ||y_ref||_2               (whole vector)
Everything goes through the shipped boundary: the Python API, the torch operator, or the
C ABI called with raw device pointers."""
import numpy as np
import pytest
import torch

import oracle
import macko_spmv_b200 as macko_spmv
from macko_spmv_b200 import cabi, workloads

pytestmark = pytest.mark.gpu

MAX_ABS_FACTOR = 1e-3
REL_L2 = 5e-3


def _dev():
    return torch.device("cuda:0")


def _u16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def _assert_buffers_equal(comp, exp, what=""):
    assert len(comp) == 5
    assert comp[0].dtype == torch.float16 and comp[1].dtype == torch.uint8 and comp[2].dtype == torch.int32
    assert np.array_equal(_u16(comp[0]), np.asarray(exp[0]).view(np.uint16)), f"values differ {what}"
    assert np.array_equal(comp[1].cpu().numpy(), exp[1]), f"deltas differ {what}"
    assert np.array_equal(comp[2].cpu().numpy(), exp[2]), f"row_indices differ {what}"


def _check_y(y, comp_np, x_np, what=""):
    y64, _, l1 = oracle.spmv(comp_np, x_np)
    got = y.float().cpu().numpy().astype(np.float64)
    err = np.abs(got - y64)
    bound = MAX_ABS_FACTOR * l1 + 1e-12
    bad = err > bound
    assert not bad.any(), f"{what}: {int(bad.sum())} rows beyond 1e-3*L1, worst {float((err / (l1 + 1e-30)).max()):.3e}"
    nrm = np.linalg.norm(y64)
    if nrm > 0:
        assert np.linalg.norm(got - y64) <= REL_L2 * nrm, f"{what}: relative L2 {np.linalg.norm(got - y64) / nrm:.3e}"
    else:
        assert np.all(got == 0)


def _compress_via_cabi(lib, M):
    rows, cols = M.shape
    stream = torch.cuda.current_stream().cuda_stream
    ri = torch.empty(rows + 1, dtype=torch.int32, device=M.device)
    cabi.check(lib, lib.macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr(), stream))
    n = int(ri[rows].item())
    P = (n + 7) // 8 * 8
    values = torch.empty(P, dtype=torch.float16, device=M.device)
    deltas = torch.empty(P // 2, dtype=torch.uint8, device=M.device)
    ws = torch.empty(lib.macko_compress_workspace_bytes(P), dtype=torch.uint8, device=M.device)
    cabi.check(lib, lib.macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr(), P, values.data_ptr(),
                                            deltas.data_ptr(), ws.data_ptr(), ws.numel(), stream))
    return values, deltas, ri, rows, cols


# ---------------------------------------------------------------- compressor: bit-exact

def test_compress_reference_known_answer_vectors(reference_vectors):
    # the reference's own two compressor tests, on both device types (tests/test_macko_spmv.py:43-103)
    for c in reference_vectors:
        for device in ("cpu", "cuda"):
            M = torch.from_numpy(c["dense"]).to(device)
            comp = macko_spmv.compress(M)
            assert comp[0].device.type == device
            _assert_buffers_equal(comp, (c["values"], c["deltas"], c["row_indices"]), c["name"])
            assert comp[3] == c["rows"] and comp[4] == c["cols"]


def test_compress_fixtures_from_compiled_reference(reference_cases):
    lib = cabi.load()
    for c in reference_cases:
        M = torch.from_numpy(c["dense"].view(np.float16)).to(_dev())
        exp = (c["values"], c["deltas"], c["row_indices"])
        _assert_buffers_equal(macko_spmv.compress(M), exp, c["name"] + " (python api)")
        _assert_buffers_equal(_compress_via_cabi(lib, M), exp, c["name"] + " (c abi)")


@pytest.mark.parametrize("shape", [(1, 1), (1, 4097), (3, 32), (37, 515), (257, 1000), (1000, 1), (2, 100003), (512, 4096)])
def test_compress_random_against_oracle(shape):
    rows, cols = shape
    g = torch.Generator().manual_seed(rows * 7919 + cols)
    for dens in (0.0, 0.001, 0.02, 0.1, 0.5, 0.9, 1.0):
        M = torch.randn(rows, cols, generator=g).half()
        M[torch.rand(rows, cols, generator=g) > dens] = 0
        bits = M.view(torch.int16)
        bits[(torch.rand(rows, cols, generator=g) < 0.05) & (bits == 0)] = -32768       # -0.0
        nan_mask = torch.rand(rows, cols, generator=g) < 0.002
        bits[nan_mask] = torch.tensor(0x7E01, dtype=torch.int16)                        # NaN payload
        exp = oracle.compress(_u16(M).reshape(rows, cols))
        _assert_buffers_equal(macko_spmv.compress(M.to(_dev())), exp, f"{shape} d={dens}")
        # same matrix at a 2-byte-aligned address: the scalar load path
        buf = torch.zeros(rows * cols + 1, dtype=torch.float16, device=_dev())
        Mo = buf[1:].view(rows, cols)
        Mo.copy_(M)
        assert Mo.data_ptr() % 16 != 0 and Mo.is_contiguous()
        _assert_buffers_equal(macko_spmv.compress(Mo), exp, f"{shape} d={dens} unaligned")


def test_compress_emit_into_a_2_byte_aligned_values_buffer():
    """`values` needs 2-byte alignment only: at an address that is not a multiple of 16 the emit kernel stores the
    values of a group one by one instead of as one 16-byte store; same bits."""
    lib = cabi.load()
    rows, cols = 300, 1999
    g = torch.Generator().manual_seed(5)
    M = torch.randn(rows, cols, generator=g).half()
    M[torch.rand(rows, cols, generator=g) > 0.3] = 0
    M = M.to(_dev())
    stream = torch.cuda.current_stream().cuda_stream
    ri = torch.empty(rows + 1, dtype=torch.int32, device=M.device)
    cabi.check(lib, lib.macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr(), stream))
    P = (int(ri[rows].item()) + 7) // 8 * 8
    backing = torch.full((P + 8,), 0x5A5A, dtype=torch.int16, device=M.device)
    values = backing[1 : P + 1]
    assert values.data_ptr() % 16 == 2
    deltas = torch.full((P // 2,), 0xA5, dtype=torch.uint8, device=M.device)
    ws = torch.empty(lib.macko_compress_workspace_bytes(P), dtype=torch.uint8, device=M.device)
    cabi.check(lib, lib.macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr(), P, values.data_ptr(),
                                            deltas.data_ptr(), ws.data_ptr(), ws.numel(), stream))
    exp = oracle.compress(_u16(M).reshape(rows, cols))
    _assert_buffers_equal((values.view(torch.float16), deltas, ri, rows, cols), exp, "2-byte-aligned values")
    assert int(backing[0]) == 0x5A5A and bool((backing[P + 1:] == 0x5A5A).all())


def test_compress_full_size_checksum():
    # a full-size layer: bit-exact against the oracle, and the decode property M e_j = M[:, j]
    rows, cols = 11008, 4096
    M = workloads.magnitude_pruned_matrix(rows, cols, 0.3, seed=2011, device="cuda")
    comp = macko_spmv.compress(M)
    exp = oracle.compress(_u16(M).reshape(rows, cols))
    _assert_buffers_equal(comp, exp, "11008x4096 d=0.3")
    for j in (0, 1, 15, 16, 2047, 4095):
        e = torch.zeros(cols, dtype=torch.float16, device="cuda")
        e[j] = 1.0
        y = macko_spmv.multiply(comp, e)
        assert torch.equal(y.view(torch.int16), (M[:, j] + 0.0).view(torch.int16)), f"column {j}"


# ---------------------------------------------------------------- multiply: tolerance tiers

EDGE_SHAPES = [(1, 1), (1, 7), (5, 33), (31, 100), (33, 257), (64, 4096), (100, 8200), (1000, 1), (7, 30000), (2, 120000)]


@pytest.mark.parametrize("shape", EDGE_SHAPES)
def test_multiply_edge_shapes_all_kernel_shapes(shape):
    rows, cols = shape
    lib = cabi.load()
    g = torch.Generator().manual_seed(rows * 31 + cols)
    stream = torch.cuda.current_stream().cuda_stream
    for dens in (0.0, 0.01, 0.1, 0.5, 1.0):
        M = torch.randn(rows, cols, generator=g).half()
        M[torch.rand(rows, cols, generator=g) > dens] = 0
        x = torch.randn(cols, generator=g).half()
        comp_np = oracle.compress(_u16(M).reshape(rows, cols))
        comp = macko_spmv.compress(M.to(_dev()))
        xd = x.to(_dev())
        _check_y(macko_spmv.multiply(comp, xd), comp_np, _u16(x), f"{shape} d={dens} default")
        for L in (4, 8, 16, 32):
            for D in (2, 4, 6):
                for xs in (0, 1):
                    if xs and cols > 100000:
                        continue
                    y = torch.full((rows,), float("nan"), dtype=torch.float16, device=_dev())
                    cabi.check(lib, lib.macko_spmv_fp16_tuned(
                        comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols, comp[0].numel(),
                        xd.data_ptr(), y.data_ptr(), 1.0, 0.0, stream, L, D, xs, 0))
                    _check_y(y, comp_np, _u16(x), f"{shape} d={dens} L={L} D={D} xs={xs}")


def test_multiply_reference_suite_replica():
    # tests/test_macko_spmv.py:106-139: manual sample, random sweep 4096x8192, dense case
    for density in (1.0, 0.5, 0.1, 0.01, 0.001, 0):
        for seed in range(2):
            torch.manual_seed(seed)
            M_cpu = torch.rand((4096, 8192), dtype=torch.float16, device="cpu")
            M_cpu[torch.rand_like(M_cpu) > density] = 0
            M_cuda = M_cpu.cuda()
            V_cuda = torch.rand((8192,), device="cuda", dtype=torch.float16)
            comp = macko_spmv.compress(M_cuda)
            result = macko_spmv.multiply(comp, V_cuda)
            expected = M_cuda @ V_cuda
            assert torch.allclose(expected, result, rtol=0.001, atol=0.001), f"Fail at {seed} {density}"


def test_multiply_manual_sample(reference_vectors):
    c = reference_vectors[0]
    M = torch.from_numpy(c["dense"]).cuda()
    comp = macko_spmv.compress(M)
    V = torch.rand((c["cols"],), device="cuda", dtype=torch.float16)
    assert torch.allclose(M @ V, macko_spmv.multiply(comp, V))


def test_multiply_misaligned_x_and_views():
    rows, cols = 300, 1001
    M = workloads.bernoulli_matrix(rows, cols, 0.3, seed=5).cuda()
    comp = macko_spmv.compress(M)
    comp_np = oracle.compress(_u16(M).reshape(rows, cols))
    buf = torch.randn(cols + 3, device="cuda").half()
    for off in (0, 1, 2, 3):
        x = buf[off:off + cols]
        assert x.is_contiguous()
        _check_y(macko_spmv.multiply(comp, x), comp_np, _u16(x), f"x offset {off}")
    with pytest.raises(AssertionError):
        macko_spmv.multiply(comp, torch.randn(2 * cols, device="cuda").half()[::2])


def test_multiply_alpha_beta_epilogue():
    rows, cols = 513, 2048
    M = workloads.bernoulli_matrix(rows, cols, 0.4, seed=9).cuda()
    comp = macko_spmv.compress(M)
    x = workloads.dense_vector(cols, 10, "cuda")
    y0 = torch.randn(rows, device="cuda").half()
    y = y0.clone()
    torch.ops.macko_spmv.multiply_out(comp[0], comp[1], comp[2], rows, cols, x, y, 0.5, -2.0)
    ref = 0.5 * (M.float() @ x.float()) - 2.0 * y0.float()
    assert torch.allclose(y.float(), ref, rtol=2e-3, atol=2e-3)
    # beta == 0 must not read y (NaN in y stays out of the result)
    y = torch.full((rows,), float("nan"), dtype=torch.float16, device="cuda")
    torch.ops.macko_spmv.multiply_out(comp[0], comp[1], comp[2], rows, cols, x, y, 1.0, 0.0)
    assert torch.equal(y, macko_spmv.multiply(comp, x))


def test_multiply_error_behaviour():
    M = workloads.bernoulli_matrix(16, 64, 0.5, seed=1).cuda()
    comp = macko_spmv.compress(M)
    with pytest.raises(RuntimeError, match="torch.half"):
        macko_spmv.multiply(comp, torch.zeros(64, device="cuda"))
    with pytest.raises(RuntimeError):
        macko_spmv.multiply(comp, torch.zeros(65, device="cuda", dtype=torch.float16))
    with pytest.raises(RuntimeError, match="torch.half"):
        macko_spmv.compress(torch.zeros(4, 4, device="cuda"))
    with pytest.raises(AssertionError):
        macko_spmv.multiply(macko_spmv.move_to_device(comp, "cpu"), torch.zeros(64, device="cuda", dtype=torch.float16))


def test_operator_registration_and_compile():
    # tests/test_macko_spmv.py:142-178
    torch.manual_seed(0)
    M_cuda = torch.rand((1024, 2048), dtype=torch.float16, device="cuda")
    M_cuda[torch.rand_like(M_cuda) > 0.5] = 0
    V_cuda = torch.rand((2048,), device="cuda", dtype=torch.float16)
    comp = macko_spmv.compress(M_cuda)
    args = (comp[0], comp[1], comp[2], comp[3], comp[4], V_cuda)
    expected = M_cuda @ V_cuda
    torch.library.opcheck(torch.ops.macko_spmv.multiply, args)
    compiled = torch.compile(macko_spmv.multiply, mode="reduce-overhead", fullgraph=True)
    for _ in range(3):
        out = compiled(comp, V_cuda)
    assert torch.allclose(expected, out, rtol=0.001, atol=0.001)
    f_c = torch.compile(lambda x: macko_spmv.multiply(comp, x + 1) - 1, mode="reduce-overhead", fullgraph=True)
    for _ in range(3):
        out2 = f_c(V_cuda)
    assert torch.allclose((M_cuda @ (V_cuda + 1)) - 1, out2, rtol=0.002, atol=0.002)


def test_cuda_graph_capture_and_vmap():
    rows, cols = 4096, 4096
    M = workloads.magnitude_pruned_matrix(rows, cols, 0.5, seed=2004, device="cuda")
    comp = macko_spmv.compress(M)
    x = workloads.dense_vector(cols, 1, "cuda")
    eager = macko_spmv.multiply(comp, x)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        macko_spmv.multiply(comp, x)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = macko_spmv.multiply(comp, x)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, eager)
    # the reference's LLM layer wraps multiply in vmap (python_scripts/util_run_pruned_llm.py:112-115)
    xb = torch.stack([x, 2 * x, -x])
    yb = torch.vmap(lambda v: macko_spmv.multiply(comp, v), in_dims=-2, out_dims=-2)(xb)
    assert yb.shape == (3, rows)
    assert torch.equal(yb[0], eager)


# ---------------------------------------------------------------- full-size properties

@pytest.mark.parametrize("case", [(32000, 4096, 0.5), (4096, 11008, 0.1), (12288, 49152, 0.1)])
def test_full_size_properties(case):
    rows, cols, d = case
    if rows * cols > 3e8:
        M = workloads.bernoulli_matrix(rows, cols, d, seed=3000, device="cuda", scale=0.02)
    else:
        M = workloads.magnitude_pruned_matrix(rows, cols, d, seed=2030, device="cuda")
    comp = macko_spmv.compress(M)
    P = comp[0].numel()
    assert P % 8 == 0 and comp[1].numel() * 2 == P and comp[2].numel() == rows + 1
    ri = comp[2].long()
    assert int(ri[0]) == 0 and bool((ri[1:] >= ri[:-1]).all()) and 0 <= P - int(ri[-1]) < 8
    # stored count = non-zeros + pads; pads = sum over gaps of floor(gap/16), bounded by zeros/16
    nnz = int((M != 0).sum())
    assert nnz <= int(ri[-1]) <= nnz + (rows * cols - nnz) // 16
    x1 = workloads.dense_vector(cols, 11, "cuda")
    x2 = workloads.dense_vector(cols, 12, "cuda")
    y1 = macko_spmv.multiply(comp, x1).float()
    # dense fp32 tier
    ref = M.float() @ x1.float()
    l1 = M.float().abs() @ x1.float().abs()
    assert bool(((y1 - ref).abs() <= MAX_ABS_FACTOR * l1 + 1e-6).all())
    assert float((y1 - ref).norm() / ref.norm()) <= REL_L2
    # linearity in x (up to the fp16 rounding of the three outputs)
    y2 = macko_spmv.multiply(comp, x2).float()
    x12 = (x1.float() + x2.float()).half()
    y12 = macko_spmv.multiply(comp, x12).float()
    ref12 = M.float() @ x12.float()
    assert float((y12 - ref12).norm() / ref12.norm()) <= REL_L2
    assert float((y12 - y1 - y2).norm() / (y1 + y2).norm()) <= 2e-2  # x12 itself was rounded to fp16
    # exact decode: a unit vector extracts a column bit for bit
    for j in (0, cols // 2 + 1, cols - 1):
        e = torch.zeros(cols, dtype=torch.float16, device="cuda")
        e[j] = 1.0
        assert torch.equal(macko_spmv.multiply(comp, e).view(torch.int16), (M[:, j] + 0.0).view(torch.int16))


def test_skewed_rows():
    rows, cols = 4000, 8192
    M = workloads.skewed_matrix(rows, cols, seed=5000, device="cuda")
    comp = macko_spmv.compress(M)
    comp_np = oracle.compress(_u16(M).reshape(rows, cols))
    _assert_buffers_equal(comp, comp_np, "skewed")
    x = workloads.dense_vector(cols, 5, "cuda")
    _check_y(macko_spmv.multiply(comp, x), comp_np, _u16(x), "skewed")


@pytest.mark.parametrize("shape", [(3000, 8192), (700, 28672), (40, 4096)])
def test_long_rows_among_short_ones_every_kernel_shape(shape):
    """Rows far longer than the average next to short and empty ones: dense rows, rows that start and end
    inside an 8-element unit, medium rows, for every lanes-per-row / units-in-flight combination through the
    default entry point and the tuned one; a second run must give the same bits."""
    rows, cols = shape
    lib = cabi.load()
    g = torch.Generator(device="cuda").manual_seed(rows)
    M = workloads.bernoulli_matrix(rows, cols, 0.03, seed=rows + 1, device="cuda")
    dense_rows = torch.randperm(rows, generator=g, device="cuda")[: max(2, rows // 12)]
    M[dense_rows] = (torch.randn(dense_rows.numel(), cols, generator=g, device="cuda") * 0.5).half()
    M[dense_rows[0], :3] = 0          # a long row that starts late ...
    M[dense_rows[1], cols - 5 :] = 0   # ... and one that ends early
    half_rows = torch.randperm(rows, generator=g, device="cuda")[: max(1, rows // 20)]
    M[half_rows, : cols // 2] = 1.0    # medium rows: longer than twice the average, shorter than dense
    M[1] = 0
    comp = macko_spmv.compress(M)
    comp_np = oracle.compress(_u16(M).reshape(rows, cols))
    _assert_buffers_equal(comp, comp_np, "long rows")
    x = workloads.dense_vector(cols, 9, "cuda")
    xn = _u16(x)
    _check_y(macko_spmv.multiply(comp, x), comp_np, xn, "default entry")
    stream = torch.cuda.current_stream().cuda_stream
    for L in (4, 8, 16, 32):
        for D in (2, 4, 6):
            y = torch.full((rows,), float("nan"), dtype=torch.float16, device="cuda")
            cabi.check(lib, lib.macko_spmv_fp16_tuned(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                                      comp[0].numel(), x.data_ptr(), y.data_ptr(), 1.0, 0.0, stream, L, D, 1, 0))
            _check_y(y, comp_np, xn, f"L={L} D={D}")
            again = torch.empty_like(y)
            cabi.check(lib, lib.macko_spmv_fp16_tuned(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), rows, cols,
                                                      comp[0].numel(), x.data_ptr(), again.data_ptr(), 1.0, 0.0, stream, L, D, 1, 0))
            assert torch.equal(y.view(torch.int16), again.view(torch.int16)), "rows must sum in a fixed order"
    # alpha / beta on long rows
    y0 = torch.ones(rows, dtype=torch.float16, device="cuda")
    torch.ops.macko_spmv.multiply_out(comp[0], comp[1], comp[2], rows, cols, x, y0, 0.5, 2.0)
    ref = macko_spmv.multiply(comp, x).float() * 0.5 + 2.0
    assert torch.allclose(y0.float(), ref, rtol=2e-3, atol=2e-3 * float(ref.abs().max()))


def test_corrupt_row_indices_stay_in_bounds():
    # Offsets outside [0, P] are clamped inside the kernel: rows that use them give garbage, but no
    # load leaves the buffers and rows with intact offsets keep their exact result.
    rows, cols = 256, 1024
    M = workloads.bernoulli_matrix(rows, cols, 0.3, seed=21).cuda()
    comp = macko_spmv.compress(M)
    x = workloads.dense_vector(cols, 22, "cuda")
    good = macko_spmv.multiply(comp, x)
    ri = comp[2].clone()
    ri[100] = 2 ** 30
    ri[101] = -7
    bad = macko_spmv.multiply((comp[0], comp[1], ri, rows, cols), x)
    torch.cuda.synchronize()
    keep = torch.ones(rows, dtype=torch.bool, device="cuda")
    keep[99:102] = False
    assert torch.equal(bad[keep], good[keep])


@pytest.mark.skipif(not oracle.have_reference_kernel(), reason="compiled reference kernel not present")
def test_multiply_against_reference_gpu_kernel():
    # y of this library vs y of the reference's own kernel (compiled unmodified for sm_100a) on the same
    # compressed buffers; both round fp32 sums to fp16, in different summation orders.
    for (rows, cols, d) in [(4096, 4096, 0.5), (1024, 8192, 0.1), (32000, 4096, 0.9), (64, 100, 0.02)]:
        M = workloads.bernoulli_matrix(rows, cols, d, seed=rows + cols).cuda()
        comp = macko_spmv.compress(M)
        x = workloads.dense_vector(cols, 7, "cuda")
        ours = macko_spmv.multiply(comp, x)
        theirs = torch.full((rows,), float("nan"), dtype=torch.float16, device="cuda")
        oracle.ref_spmv_gpu(comp[0].data_ptr(), comp[1].data_ptr(), comp[2].data_ptr(), x.data_ptr(), theirs.data_ptr(),
                            rows, cols, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        l1 = M.float().abs() @ x.float().abs()
        assert bool(((ours.float() - theirs.float()).abs() <= 2 * MAX_ABS_FACTOR * l1 + 1e-6).all()), (rows, cols, d)
        ref = M.float() @ x.float()
        assert float((theirs.float() - ref).norm() / ref.norm()) <= REL_L2
        assert float((ours.float() - ref).norm() / ref.norm()) <= REL_L2


def test_compress_structured_patterns_against_oracle():
    """Rows built from runs of zeros and non-zeros of drawn lengths (long pad runs, gaps of exactly 15, 16 and 17
    zeros, dense stretches, empty rows, a non-zero in the last column), many row widths around the 8- and
    256-column steps of the walk: compressed buffers bit for bit against the oracle, then decompressed and
    multiplied."""
    rng = np.random.default_rng(2024)
    for case in range(40):
        rows = int(rng.integers(1, 40))
        cols = int(rng.choice([1, 7, 8, 9, 15, 16, 17, 31, 255, 256, 257, 511, 1000, 4097, 9000]))
        M = np.zeros((rows, cols), dtype=np.float16)
        for r in range(rows):
            c = 0
            kind = rng.integers(0, 5)
            while c < cols:
                gap = int(rng.choice([0, 1, 14, 15, 16, 17, 31, 32, 33, 255, 256, 300, 5000])) if kind != 0 else cols
                c += gap
                run = int(rng.choice([1, 1, 2, 7, 8, 9, 64, 300]))
                if c < cols:
                    n = min(run, cols - c)
                    M[r, c:c + n] = rng.standard_normal(n).astype(np.float16) + np.float16(3.0)
                    c += n
            if kind == 1:
                M[r, cols - 1] = 1.5
            if kind == 2:
                M[r, 0] = -2.0
        neg = rng.random(M.shape) < 0.1
        M[(M == 0) & neg] = np.float16(-0.0)           # pads take the sign of the zero they sit on
        exp = oracle.compress(M.view(np.uint16))
        got = macko_spmv.compress(torch.from_numpy(M).to(_dev()))
        _assert_buffers_equal(got, exp, f"case {case}: {rows}x{cols}")
        # the same buffers back through the decompressor (bit for bit) and the product (tolerance tiers)
        comp_np = (exp[0], exp[1], exp[2], rows, cols)
        assert np.array_equal(_u16(macko_spmv.decompress(got)), oracle.decompress(comp_np)), f"decompress, case {case}"
        x = (rng.standard_normal(cols) * 0.5).astype(np.float16)
        y = macko_spmv.multiply(got, torch.from_numpy(x).to(_dev()))
        _check_y(y, comp_np, x.view(np.uint16), f"multiply, case {case}: {rows}x{cols}")
