"""ctypes declarations of every entry point of ``include/macko_b200.h``.

This is the binding a non-torch host would write: plain integers for device pointers
(e.g. ``tensor.data_ptr()``), a ``cudaStream_t`` as an integer, ``int`` status back.
``check(status)`` turns a non-zero status into ``MackoError`` carrying the library's message.
"""
from __future__ import annotations

import ctypes
import os

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libmacko_b200.so")

OK = 0
ERR_INVALID_ARGUMENT = 1
ERR_MISALIGNED = 2
ERR_SIZE_OVERFLOW = 3
ERR_CUDA = 4
ERR_WORKSPACE = 5

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_f = ctypes.c_float
_int = ctypes.c_int
_u32 = ctypes.c_uint32
_i32 = ctypes.c_int32

# flag bits (include/macko_b200.h)
SPMV_MATRIX_IMMUTABLE = 1
SCATTER_DEFERRED_WAIT = 2


class PlanInfo(ctypes.Structure):
    """``macko_spmv_plan_info``: what ``macko_spmv_plan`` reports and ``macko_spmv_fp16_planned`` takes back."""

    _fields_ = [
        ("plan_bytes", _i64), ("rows", _i64), ("padded_count", _i64),
        ("virtual_rows", _i32), ("segment_elements", _i32), ("longest_row", _i32), ("split_rows", _i32),
        ("recommended", _i32), ("reserved", _i32 * 3),
    ]


SIGNATURES = {
    "macko_version": (_int, []),
    "macko_status_string": (ctypes.c_char_p, [_int]),
    "macko_last_error": (ctypes.c_char_p, []),
    "macko_spmv_fp16": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f, _f, _vp]),
    "macko_spmv_fp16_ex": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f, _f, _u32, _vp]),
    "macko_spmv_bf16": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f, _f, _u32, _vp]),
    "macko_spmv_int8": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f, _f, _u32, _vp]),
    "macko_spmv_plan_bytes": (_i64, [_i64, _i64, _i64, _i32]),
    "macko_spmv_plan": (_int, [_vp, _vp, _i64, _i64, _i64, _i32, _vp, _i64, ctypes.POINTER(PlanInfo), _vp]),
    "macko_spmv_fp16_planned": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, ctypes.POINTER(PlanInfo), _vp, _vp, _f, _f, _u32, _vp]),
    "macko_spmv_fp16_tuned": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _f, _f, _vp, _int, _int, _int, _int]),
    "macko_spmv_shape": (_int, [_i64, _i64, _i64, _int, _vp, _vp]),
    "macko_spmm_fp16": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _f, _f, _vp]),
    "macko_decompress_fp16": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "macko_compress_count": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "macko_compress_workspace_bytes": (_i64, [_i64]),
    "macko_compress_emit": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp]),
    "macko_compress_emit_bf16": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp]),
    "macko_compress_count_int8": (_int, [_vp, _i64, _i64, _vp, _vp]),
    "macko_compress_emit_int8": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp]),
    "macko_compress_emit_static": (_int, [_vp, _i64, _i64, _vp, _i64, _vp, _vp, _vp]),
    "macko_compress_static_capacity": (_i64, []),
    "macko_compress_overflow": (_int, [ctypes.POINTER(_u32), _vp]),
    "macko_spmv_fp16_scatter": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _int, _int, _vp]),
    "macko_peer_wait": (_int, [_vp, _int, _vp]),
    "macko_spmv_fp16_scatter_ex": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i64, _vp, _int, _int, _u32, _u32, _vp]),
    "macko_peer_wait_limited": (_int, [_vp, _int, _u32, _vp]),
    "macko_peer_forward": (_int, [_vp, _i64, _i64, _vp, _int, _int, _vp]),
    "macko_decode_add_rmsnorm": (_int, [_vp, _vp, _int, _i64, _vp, _vp, _i64, _f, _vp]),
    "macko_decode_add_rmsnorm_peer": (_int, [_vp, _vp, _int, _i64, _vp, _vp, _i64, _f, _vp, _int, _u32, _vp]),
    "macko_decode_rope_attention": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _int, _int, _int, _vp]),
    "macko_decode_silu_mul": (_int, [_vp, _vp, _i64, _vp]),
    "macko_decode_argmax": (_int, [_vp, _i64, _vp, _vp]),
}


class MackoError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"macko status {status}: {message}")
        self.status = status


def load(path: str = LIB_PATH) -> ctypes.CDLL:
    """Load the C-ABI library and attach the signatures above."""
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python macko_spmv_b200/build.py`")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


def check(lib: ctypes.CDLL, status: int) -> None:
    if status != OK:
        raise MackoError(status, lib.macko_last_error().decode())
