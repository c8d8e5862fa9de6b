"""B200-native MACKO SpMV: drop-in for the ``macko_spmv`` Python API.

``compress(M)`` -> ``(values fp16[P], deltas uint8[P/2], row_indices int32[R+1], R, C)``
``multiply(compressed, V)`` -> ``y`` fp16[R]
``move_to_device(compressed, device)``

Same functions, argument meaning and error behaviour as the reference
(src/macko_spmv/__init__.py:110-149); same `macko_spmv::multiply` operator schema
(src/macko_spmv/__init__.py:56-63). The kernels come from a prebuilt sm_100a library
behind a C ABI (``include/macko_b200.h``) instead of an import-time JIT build; there is
no CPU or PyTorch fallback: without the built libraries the import fails, and without a
CUDA device every call raises.

Use ``import macko_spmv_b200 as macko_spmv`` to switch an existing program over.
"""
from __future__ import annotations

import ctypes
import os

import torch

LIB_NAME = "macko_spmv"
__version__ = "0.1.0"

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_CORE_PATH = os.path.join(_PKG_DIR, "libmacko_b200.so")
_OPS_PATH = os.path.join(_PKG_DIR, "_torch_ops.so")

# The reference reads this variable to choose its JIT cache directory
# (src/macko_spmv/__init__.py:12). Nothing is compiled at import here; it is accepted and ignored.
BUILD_DIRECTORY = os.environ.get("MACKO_SPMV_BUILD_DIRECTORY", "")


def _load_native():
    for path in (_CORE_PATH, _OPS_PATH):
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build the native libraries first with "
                "`python macko_spmv_b200/build.py` (needs nvcc and g++)."
            )
    core = ctypes.CDLL(_CORE_PATH, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(_OPS_PATH)
    return core


_core = _load_native()
_core.macko_version.restype = ctypes.c_int
_core.macko_last_error.restype = ctypes.c_char_p
_core.macko_status_string.restype = ctypes.c_char_p
_core.macko_status_string.argtypes = [ctypes.c_int]


def native_library_paths() -> tuple[str, str]:
    """Paths of the C-ABI library and of the torch operator library that were loaded."""
    return _CORE_PATH, _OPS_PATH


def native_version() -> int:
    return int(_core.macko_version())


@torch.library.register_fake("macko_spmv::multiply")
def _multiply_fake(M_values, M_deltas, M_row_indices, M_rows, M_cols, V):
    # Same meta kernel as the reference (src/macko_spmv/__init__.py:105-107); int8 values give fp16 like V.
    return torch.empty((M_rows,), device=M_values.device, dtype=V.dtype)


@torch.library.register_fake("macko_spmv::compress_dense")
def _compress_fake(M):
    n = torch.library.get_ctx().new_dynamic_size()
    return (
        M.new_empty((n * 8,)),
        M.new_empty((n * 4,), dtype=torch.uint8),
        M.new_empty((M.shape[0] + 1,), dtype=torch.int32),
    )


@torch.library.register_fake("macko_spmv::multiply_batched")
def _multiply_batched_fake(M_values, M_deltas, M_row_indices, M_rows, M_cols, V):
    return torch.empty((V.shape[0], M_rows), device=M_values.device, dtype=M_values.dtype)


@torch.library.register_fake("macko_spmv::decompress")
def _decompress_fake(M_values, M_deltas, M_row_indices, M_rows, M_cols):
    return torch.empty((M_rows, M_cols), device=M_values.device, dtype=M_values.dtype)


@torch.library.register_fake("macko_spmv::multiply_frozen")
def _multiply_frozen_fake(M_values, M_deltas, M_row_indices, M_rows, M_cols, V):
    return torch.empty((M_rows,), device=M_values.device, dtype=V.dtype)


@torch.library.register_fake("macko_spmv::multiply_planned")
def _multiply_planned_fake(M_values, M_deltas, M_row_indices, M_rows, M_cols, plan, virtual_rows, segment_elements, split_rows, V, frozen):
    return torch.empty((M_rows,), device=M_values.device, dtype=M_values.dtype)


@torch.library.register_fake("macko_spmv::add_rmsnorm")
def _add_rmsnorm_fake(x, pending, weight, eps):
    return torch.empty_like(x)


@torch.library.register_fake("macko_spmv::add_rmsnorm_peer")
def _add_rmsnorm_peer_fake(x, pending, weight, eps, flags_address, world, spin_limit):
    return torch.empty_like(x)


@torch.library.register_fake("macko_spmv::rope_attention")
def _rope_attention_fake(qkv, cos_table, sin_table, position, k_cache, v_cache):
    return qkv.new_empty((qkv.numel() // 3,))


@torch.library.register_fake("macko_spmv::silu_mul")
def _silu_mul_fake(gate_up):
    return gate_up.new_empty((gate_up.shape[0] // 2,))


@torch.library.register_fake("macko_spmv::argmax")
def _argmax_fake(values):
    return values.new_empty((1,), dtype=torch.int64)


def move_to_device(compressed, device):
    """Move the three buffers of a compressed matrix (src/macko_spmv/__init__.py:110-117)."""
    return (
        compressed[0].to(device=device),
        compressed[1].to(device=device),
        compressed[2].to(device=device),
        compressed[3],
        compressed[4],
    )


def compress(M):
    """Compress a contiguous fp16 matrix into the MACKO 5-tuple, on the device of ``M``.

    Mirrors src/macko_spmv/__init__.py:120-131, except that the encoder runs on the GPU:
    a CUDA matrix never leaves the device, and a CPU matrix is copied to the current CUDA
    device, compressed there and copied back (there is no host encoder in this package).
    The buffers are bit-identical to the reference's.
    """
    assert M.is_contiguous()
    if M.device.type == "cuda":
        values, deltas, row_indices = torch.ops.macko_spmv.compress_dense.default(M)
        return (values, deltas, row_indices, M.size(0), M.size(1))
    elif M.device.type == "cpu":
        if not torch.cuda.is_available():
            raise RuntimeError("macko_spmv_b200.compress needs a CUDA device: the encoder is a GPU kernel")
        values, deltas, row_indices = torch.ops.macko_spmv.compress_dense.default(M.to("cuda"))
        return move_to_device((values, deltas, row_indices, M.size(0), M.size(1)), "cpu")
    else:
        raise NotImplementedError()


class FrozenMatrix(tuple):
    """The 5-tuple of `compress` for a matrix that will not be written any more (weights), as returned by
    `freeze`. `multiply` recognises it and lets the kernel fetch matrix data while the previous kernel of
    the stream is still finishing; with a plan (see `freeze`) it runs the planned launch. It is still a
    tuple of the same five items, so everything that takes the reference's compressed object takes it."""

    plan = None        # device buffer of the plan, or None
    plan_meta = None   # (virtual_rows, segment_elements, longest_row, split_rows, recommended)

    def __new__(cls, compressed, plan=None, plan_meta=None):
        self = super().__new__(cls, tuple(compressed[:5]))
        self.plan = plan
        self.plan_meta = plan_meta
        return self


def freeze(compressed_M, plan="auto", segment_elements=0):
    """Declare a compressed CUDA matrix immutable and, if it pays, build its launch plan.

    Waits once for the device work that produced the buffers (they must be complete before a kernel may read
    them ahead of stream order). `plan`: "auto" builds the plan and keeps it only if the row statistics
    recommend it (rows far longer than the average, e.g. skewed matrices), True keeps it always, False builds
    none. The reference has no counterpart (src/macko_spmv/__init__.py has only compress / multiply)."""
    assert compressed_M[0].is_cuda and compressed_M[1].is_cuda and compressed_M[2].is_cuda
    torch.cuda.synchronize(compressed_M[0].device)
    if plan is False or compressed_M[0].dtype != torch.float16:
        return FrozenMatrix(compressed_M)
    buf, meta = torch.ops.macko_spmv.plan_build.default(
        compressed_M[1], compressed_M[2], compressed_M[3], compressed_M[4], compressed_M[0].numel(), int(segment_elements))
    meta = [int(v) for v in meta.tolist()]
    info = (meta[3], meta[4], meta[5], meta[6], meta[7])
    if plan is True or info[4]:
        return FrozenMatrix(compressed_M, buf, info)
    return FrozenMatrix(compressed_M, None, info)


def multiply(compressed_M, V, out=None):
    """y = M @ V for a compressed matrix and an fp16 CUDA vector (src/macko_spmv/__init__.py:134-149).

    `out` (not in the reference): a contiguous CUDA vector of M_rows elements that receives y, for callers
    that keep their results in one buffer; without it a new tensor is returned, as in the reference."""
    assert compressed_M[0].is_cuda
    assert compressed_M[1].is_cuda
    assert compressed_M[2].is_cuda
    assert V.is_cuda
    assert V.is_contiguous()
    if out is not None:
        frozen = isinstance(compressed_M, FrozenMatrix)
        torch.ops.macko_spmv.multiply_ex.default(
            compressed_M[0], compressed_M[1], compressed_M[2], compressed_M[3], compressed_M[4], V, out, 1.0, 0.0,
            1 if frozen else 0)
        return out
    if isinstance(compressed_M, FrozenMatrix):
        if compressed_M.plan is not None:
            return torch.ops.macko_spmv.multiply_planned.default(
                compressed_M[0], compressed_M[1], compressed_M[2], compressed_M[3], compressed_M[4],
                compressed_M.plan, compressed_M.plan_meta[0], compressed_M.plan_meta[1], compressed_M.plan_meta[3], V, True)
        return torch.ops.macko_spmv.multiply_frozen.default(
            compressed_M[0], compressed_M[1], compressed_M[2], compressed_M[3], compressed_M[4], V)
    return torch.ops.macko_spmv.multiply.default(
        compressed_M[0],
        compressed_M[1],
        compressed_M[2],
        compressed_M[3],
        compressed_M[4],
        V,
    )


# Above this many right-hand sides a dense copy of the matrix plus one tensor-core GEMM is always cheaper than
# streaming the compressed matrix once per 8 vectors; from 9 vectors on (two passes) it depends on the density.
DENSE_BATCH_THRESHOLD = 16


def _dense_copy_pays(compressed_M, batch: int) -> bool:
    """9..DENSE_BATCH_THRESHOLD vectors of an fp16 matrix: passes of the multi-vector kernel (8 vectors each, measured
    at 1.3 TB/s of compressed bytes) against one decompression (3.0 TB/s of compressed + dense bytes) plus about
    19 us for the GEMM and the dense buffer. At 50 % density the dense copy wins from 9 vectors on (68 against
    85 us for 16 vectors on 11008x4096), at 30 % and below the two passes do."""
    if batch <= 8 or compressed_M[0].dtype != torch.float16:
        return False
    stored_bytes = 2.5 * compressed_M[0].numel()
    passes = (batch + 7) // 8
    multi_vector_us = passes * stored_bytes / 1.3e6
    dense_us = (stored_bytes + 2.0 * compressed_M[3] * compressed_M[4]) / 3.0e6 + 19.0
    return dense_us < multi_vector_us


def decompress(compressed_M):
    """Dense fp16 [rows, cols] of a compressed CUDA matrix (every zero, pads included, comes back as +0)."""
    assert compressed_M[0].is_cuda
    return torch.ops.macko_spmv.decompress.default(*compressed_M[:5])


def multiply_batched(compressed_M, V):
    """Y[batch, rows] = V[batch, cols] @ M^T for a compressed matrix and fp16 CUDA vectors.

    The reference runs batched inputs as a loop of `multiply` calls (torch.vmap fallback,
    python_scripts/util_run_pruned_llm.py:112-115). Here up to 8 vectors share one pass over the compressed
    matrix; 9..DENSE_BATCH_THRESHOLD take two passes or, where the matrix is dense enough for that to be cheaper,
    the route of the larger batches: decompress once and run a dense GEMM.
    """
    assert compressed_M[0].is_cuda
    assert V.is_cuda
    assert V.is_contiguous()
    if V.dim() != 2:
        raise RuntimeError("V must have shape [batch, cols]")
    if V.shape[0] > DENSE_BATCH_THRESHOLD or _dense_copy_pays(compressed_M, V.shape[0]):
        return V @ decompress(compressed_M).t()
    return torch.ops.macko_spmv.multiply_batched.default(*compressed_M[:5], V)


__all__ = ["compress", "multiply", "multiply_batched", "decompress", "move_to_device", "freeze", "FrozenMatrix",
           "native_library_paths", "native_version", "LIB_NAME"]
