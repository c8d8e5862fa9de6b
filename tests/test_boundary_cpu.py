"""CPU tests of the drop-in boundary: the C-ABI library loads and exports what the header
declares, argument validation answers with status codes before touching a device, and the
Python surface mirrors the reference's functions, schema and error behaviour."""
import os
import re

import pytest
import torch

import macko_spmv_b200 as macko_spmv
from macko_spmv_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "macko_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(macko_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = cabi.load()
    names = _declared_functions()
    assert "macko_spmv_fp16" in names and "macko_compress_emit" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/macko_b200.h but not exported"
        assert n in cabi.SIGNATURES, f"{n} has no ctypes signature in cabi.py"
    assert lib.macko_version() == 200
    assert lib.macko_status_string(0) == b"ok"


def test_argument_validation_returns_status_codes():
    lib = cabi.load()
    a16 = 0x1000  # fake, well-aligned "device pointers": validation must reject before any use
    # negative sizes
    assert lib.macko_spmv_fp16(a16, a16, a16, -1, 8, 0, a16, a16, 1.0, 0.0, None) == cabi.ERR_INVALID_ARGUMENT
    assert b"negative" in lib.macko_last_error()
    # P not a multiple of 8
    assert lib.macko_spmv_fp16(a16, a16, a16, 4, 8, 12, a16, a16, 1.0, 0.0, None) == cabi.ERR_INVALID_ARGUMENT
    # misaligned values / deltas / x
    assert lib.macko_spmv_fp16(a16 + 8, a16, a16, 4, 8, 8, a16, a16, 1.0, 0.0, None) == cabi.ERR_MISALIGNED
    assert lib.macko_spmv_fp16(a16, a16 + 2, a16, 4, 8, 8, a16, a16, 1.0, 0.0, None) == cabi.ERR_MISALIGNED
    assert lib.macko_spmv_fp16(a16, a16, a16, 4, 8, 8, a16 + 1, a16, 1.0, 0.0, None) == cabi.ERR_MISALIGNED
    # null pointers
    assert lib.macko_spmv_fp16(a16, a16, None, 4, 8, 8, a16, a16, 1.0, 0.0, None) == cabi.ERR_INVALID_ARGUMENT
    # sizes beyond 31-bit indexing
    assert lib.macko_spmv_fp16(a16, a16, a16, 4, 8, 1 << 31, a16, a16, 1.0, 0.0, None) == cabi.ERR_SIZE_OVERFLOW
    assert lib.macko_compress_count(a16, 1 << 20, 1 << 20, a16, None) == cabi.ERR_SIZE_OVERFLOW
    assert lib.macko_compress_count(a16, 4, 4, None, None) == cabi.ERR_INVALID_ARGUMENT
    # emit: P shape, workspace size
    assert lib.macko_compress_emit(a16, 4, 4, a16, 12, a16, a16, a16, 12, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_compress_emit(a16, 4, 4, a16, 16, a16, a16, a16, 8, None) == cabi.ERR_WORKSPACE
    assert lib.macko_compress_workspace_bytes(4096) == 4096
    # tuned entry point: bad shape parameters are rejected (after validation, before launch)
    assert lib.macko_spmv_fp16_tuned(a16, a16, a16, 4, 8, 8, a16, a16, 1.0, 0.0, None, 8, 2, 1, -1) == cabi.ERR_INVALID_ARGUMENT
    # an empty matrix is a no-op
    assert lib.macko_spmv_fp16(None, None, None, 0, 8, 0, None, None, 1.0, 0.0, None) == cabi.OK
    with pytest.raises(cabi.MackoError):
        cabi.check(lib, lib.macko_spmv_fp16(a16, a16, a16, -1, 8, 0, a16, a16, 1.0, 0.0, None))


def test_python_surface_matches_reference():
    assert macko_spmv.LIB_NAME == "macko_spmv"
    for name in ("compress", "multiply", "move_to_device"):
        assert callable(getattr(macko_spmv, name))
    schema = str(torch.ops.macko_spmv.multiply.default._schema)
    assert schema == ("macko_spmv::multiply(Tensor M_values, Tensor M_deltas, Tensor M_row_indices, "
                      "int M_rows, int M_cols, Tensor V) -> Tensor")


def test_python_error_behaviour_without_gpu():
    M = torch.zeros(4, 8, dtype=torch.float16)
    with pytest.raises(AssertionError):
        macko_spmv.compress(M.t())  # not contiguous
    with pytest.raises(NotImplementedError):
        macko_spmv.compress(torch.zeros(4, 8, dtype=torch.float16, device="meta"))
    comp = (torch.zeros(8, dtype=torch.float16), torch.zeros(4, dtype=torch.uint8),
            torch.zeros(5, dtype=torch.int32), 4, 8)
    with pytest.raises(AssertionError):
        macko_spmv.multiply(comp, torch.zeros(8, dtype=torch.float16))  # CPU operands
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="CUDA"):
            macko_spmv.compress(M)  # no host encoder: fails loudly instead of falling back
    moved = macko_spmv.move_to_device(comp, "cpu")
    assert len(moved) == 5 and moved[3] == 4 and moved[4] == 8


def test_fake_tensor_tracing():
    from torch._subclasses.fake_tensor import FakeTensorMode

    with FakeTensorMode():
        v = torch.empty(64, dtype=torch.float16, device="cuda")
        d = torch.empty(32, dtype=torch.uint8, device="cuda")
        ri = torch.empty(11, dtype=torch.int32, device="cuda")
        x = torch.empty(40, dtype=torch.float16, device="cuda")
        y = torch.ops.macko_spmv.multiply.default(v, d, ri, 10, 40, x)
        assert y.shape == (10,) and y.dtype == torch.float16 and y.device.type == "cuda"


def test_launch_shape_heuristic_table():
    """The launch shape chosen per matrix (host arithmetic only): the decisions that were calibrated on B200
    (148 SMs) for the benchmark shapes, and the limits of the rule."""
    import ctypes

    from macko_spmv_b200 import cabi

    lib = cabi.load()

    def shape(rows, cols, density, pad=1.03):
        L, D = ctypes.c_int(0), ctypes.c_int(0)
        P = int(rows * cols * density * pad) // 8 * 8
        assert lib.macko_spmv_shape(rows, cols, P, 148, ctypes.byref(L), ctypes.byref(D)) == cabi.OK
        return L.value, D.value

    assert shape(4096, 4096, 0.5) == (32, 6)        # few rows: a warp per row
    assert shape(4096, 4096, 0.1) == (32, 4)
    assert shape(4096, 11008, 0.5) == (32, 6)
    assert shape(8192, 8192, 0.5) == (16, 6)
    assert shape(11008, 4096, 0.5) == (8, 6)        # enough rows to fill the GPU with 8 lanes per row
    assert shape(32000, 4096, 0.9) == (8, 6)
    assert shape(12288, 49152, 0.5) == (32, 6)      # very long rows of a very wide matrix: back to a warp per row
    assert shape(49152, 12288, 0.5) == (16, 6)
    assert shape(100000, 64, 0.3)[0] == 4           # rows of ~20 stored elements: the smallest group
    assert shape(0, 64, 0.5, pad=0) == (4, 2)
    L, D = ctypes.c_int(0), ctypes.c_int(0)
    assert lib.macko_spmv_shape(-1, 1, 0, 148, ctypes.byref(L), ctypes.byref(D)) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_spmv_shape(1, 1, 0, 0, ctypes.byref(L), ctypes.byref(D)) == cabi.ERR_INVALID_ARGUMENT


def test_new_entry_points_validate_before_touching_the_device():
    import ctypes

    lib = cabi.load()
    a16 = 0x1000
    # unknown flag bits
    assert lib.macko_spmv_fp16_ex(a16, a16, a16, 4, 8, 8, a16, a16, 1.0, 0.0, 4, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_spmv_bf16(a16, a16, a16, 4, 8, 8, a16, a16, 1.0, 0.0, 1 << 7, None) == cabi.ERR_INVALID_ARGUMENT
    # plan: segment length rules, sizes, null pointers
    assert lib.macko_spmv_plan_bytes(100, 100, 800, 100) == -1
    assert lib.macko_spmv_plan_bytes(100, 100, 800, 4096) == -1
    assert lib.macko_spmv_plan_bytes(100, 1 << 21, 800, 0) == -1
    nbytes = lib.macko_spmv_plan_bytes(100, 100, 800, 0)
    assert nbytes > 0 and nbytes % 256 == 0
    info = cabi.PlanInfo()
    assert lib.macko_spmv_plan(a16, a16, 100, 100, 800, 0, None, nbytes, ctypes.byref(info), None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_spmv_plan(a16, a16, 100, 100, 800, 0, a16, nbytes - 1, ctypes.byref(info), None) == cabi.ERR_WORKSPACE
    assert lib.macko_spmv_plan(a16, a16, 100, 100, 800, 0, a16 + 4, nbytes, ctypes.byref(info), None) == cabi.ERR_MISALIGNED
    # planned product: an info that belongs to another matrix is refused
    info.rows, info.padded_count, info.virtual_rows, info.segment_elements, info.plan_bytes = 100, 800, 100, 1024, nbytes
    assert lib.macko_spmv_fp16_planned(a16, a16, a16, 101, 100, 800, a16, ctypes.byref(info), a16, a16, 1.0, 0.0, 0, None) \
        == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_spmv_fp16_planned(a16, a16, a16, 100, 100, 800, None, ctypes.byref(info), a16, a16, 1.0, 0.0, 0, None) \
        == cabi.ERR_INVALID_ARGUMENT
    # scatter: flags and world checked first
    ptrs = (ctypes.c_void_p * 2)(a16, a16)
    assert lib.macko_spmv_fp16_scatter_ex(a16, a16, a16, 4, 8, 8, a16, ptrs, 0, ptrs, 0, 2, 8, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_spmv_fp16_scatter_ex(a16, a16, a16, 4, 8, 8, a16, ptrs, 0, ptrs, 2, 2, 0, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_peer_wait_limited(None, 2, 10, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_compress_overflow(None, None) == cabi.ERR_INVALID_ARGUMENT
    # decode helpers: sizes, null pointers, head sizes that are not built
    assert lib.macko_decode_add_rmsnorm(a16, None, 1, 64, a16, a16, 64, 1e-5, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_add_rmsnorm(a16, a16, 2, 32, a16, a16, 64, 1e-5, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_add_rmsnorm(a16, None, 0, 0, a16, a16, 0, 1e-5, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_add_rmsnorm_peer(a16, a16, 2, 64, a16, a16, 64, 1e-5, None, 2, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_add_rmsnorm_peer(a16, a16, 2, 64, a16, a16, 64, 1e-5, a16, 9, 0, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_silu_mul(a16, None, 64, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_argmax(a16, 0, a16, None) == cabi.ERR_INVALID_ARGUMENT
    assert lib.macko_decode_rope_attention(a16, a16, a16, a16, a16, a16, a16, 4, 96, 16, None) == cabi.ERR_INVALID_ARGUMENT
    assert b"head_dim" in lib.macko_last_error()
    assert lib.macko_decode_rope_attention(a16, a16, a16, None, a16, a16, a16, 4, 128, 16, None) == cabi.ERR_INVALID_ARGUMENT


def test_plan_model_of_the_oracle_on_the_reference_vector(reference_vectors):
    import oracle

    c = reference_vectors[0]     # 5 x 32, row_indices [0, 6, 10, 12, 13, 22]
    d0, d1, out, seg_first = oracle.plan_model(c["deltas"], c["row_indices"], 256)
    assert list(seg_first) == [0, 1, 2, 3, 4, 5]
    # one virtual row per row, all in length class 1 except none: natural order is kept (stable)
    assert sorted(d0.tolist()) == [0, 6, 10, 12, 13] and sorted((d1 & 4095).tolist()) == [1, 2, 4, 6, 9]
    assert not (d1 >> 12).any() and sorted(out.tolist()) == [0, 1, 2, 3, 4]
