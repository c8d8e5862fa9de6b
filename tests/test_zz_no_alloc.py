"""The workspace-free compressor entry point, `macko_compress_emit_static`.

Some hosts cannot give the library scratch memory: they run inside an application that has handed all
device memory to its own pool, or they sit on a path where a cudaMalloc is not allowed. For them phase 2
of the compressor can run on a scratch array that is part of the library itself. The test calls it
through the C ABI with raw device pointers, twice in a row on different matrices (the second, smaller
one runs over whatever the first left in the shared scratch), and requires the same bits as the regular
entry point, which takes a caller-provided workspace. Collected last so that a failure here cannot hide
other tests behind `-x`.
"""
import numpy as np
import pytest
import torch

from macko_spmv_b200 import cabi, workloads

pytestmark = pytest.mark.gpu


def _count(lib, M, stream):
    rows, cols = M.shape
    ri = torch.empty(rows + 1, dtype=torch.int32, device=M.device)
    cabi.check(lib, lib.macko_compress_count(M.data_ptr(), rows, cols, ri.data_ptr(), stream))
    n = int(ri[rows].item())
    return ri, (n + 7) // 8 * 8


def _emit_with_workspace(lib, M, ri, P, stream):
    rows, cols = M.shape
    values = torch.full((P,), float("nan"), dtype=torch.float16, device=M.device)
    deltas = torch.full((P // 2,), 0xAB, dtype=torch.uint8, device=M.device)
    ws = torch.empty(lib.macko_compress_workspace_bytes(P), dtype=torch.uint8, device=M.device)
    cabi.check(lib, lib.macko_compress_emit(M.data_ptr(), rows, cols, ri.data_ptr(), P, values.data_ptr(),
                                            deltas.data_ptr(), ws.data_ptr(), ws.numel(), stream))
    return values, deltas


def _emit_static(lib, M, ri, P, stream):
    rows, cols = M.shape
    values = torch.full((P,), float("nan"), dtype=torch.float16, device=M.device)
    deltas = torch.full((P // 2,), 0xCD, dtype=torch.uint8, device=M.device)
    cabi.check(lib, lib.macko_compress_emit_static(M.data_ptr(), rows, cols, ri.data_ptr(), P,
                                                   values.data_ptr(), deltas.data_ptr(), stream))
    return values, deltas


def test_static_scratch_entry_point_matches_workspace_entry_point():
    lib = cabi.load()
    assert lib.macko_compress_static_capacity() == 16 * 1024 * 1024
    stream = torch.cuda.current_stream().cuda_stream
    # first a large matrix that fills most of the built-in scratch, then a small ragged one
    for (rows, cols, density, seed) in [(4096, 4096, 0.9, 11), (37, 515, 0.3, 12)]:
        M = workloads.bernoulli_matrix(rows, cols, density, seed=seed, device="cuda")
        M.view(torch.int16)[::7, ::5] = -32768          # some -0.0: pads must keep the sign bit
        ri, P = _count(lib, M, stream)
        assert 0 < P <= lib.macko_compress_static_capacity()
        v_ref, d_ref = _emit_with_workspace(lib, M, ri, P, stream)
        v_new, d_new = _emit_static(lib, M, ri, P, stream)
        torch.cuda.synchronize()
        assert torch.equal(v_new.view(torch.int16), v_ref.view(torch.int16)), f"values differ for {rows}x{cols}"
        assert torch.equal(d_new, d_ref), f"deltas differ for {rows}x{cols}"
        assert not torch.isnan(v_new.float()).any()


def test_static_scratch_entry_point_rejects_oversize():
    lib = cabi.load()
    cap = lib.macko_compress_static_capacity()
    a = 0x1000  # never dereferenced: the size check comes first
    st = lib.macko_compress_emit_static(a, 8192, 8192, a, cap + 8, a, a, None)
    assert st == cabi.ERR_WORKSPACE
    assert b"exceeds the built-in scratch" in lib.macko_last_error()
    assert lib.macko_compress_emit_static(a, 4, 4, a, 12, a, a, None) == cabi.ERR_INVALID_ARGUMENT
