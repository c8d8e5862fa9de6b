"""ctypes front-end of the CPU oracle (``liboracle.so``) and of the compiled
reference compressor (``_ref/libref_compress.so``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the
benchmark's CPU-baseline leg. The shipped package never imports this module.

All matrices and vectors cross this boundary as numpy arrays of fp16 *bit
patterns* (``uint16``) so that -0.0 and NaN payloads are compared as bits.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_compress.so")
_REF_KERNEL_PATH = os.path.join(_HERE, "_ref", "libref_kernel.so")

_u16p = ctypes.POINTER(ctypes.c_uint16)
_u8p = ctypes.POINTER(ctypes.c_uint8)
_i8p = ctypes.POINTER(ctypes.c_int8)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f64p = ctypes.POINTER(ctypes.c_double)
_i64 = ctypes.c_int64


def _make_env() -> dict:
    """Environment for make: the reference checkout comes from MACKO_REFERENCE_DIR, else from a directory
    named `reference` beside this repository, if there is one."""
    env = dict(os.environ)
    if not env.get("MACKO_REFERENCE_DIR"):
        cand = os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
        if os.path.isdir(cand):
            env["MACKO_REFERENCE_DIR"] = cand
    return env


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference compressor when its sources exist)."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "macko_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True, env=_make_env())
    elif not os.path.exists(_REF_PATH) or not os.path.exists(_REF_KERNEL_PATH):
        subprocess.run(["make", "-C", _HERE, "ref"], check=True, capture_output=True, env=_make_env())


_lib = None
_ref = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        lib = ctypes.CDLL(_LIB_PATH)
        lib.oracle_compress_bound.restype = _i64
        lib.oracle_compress_bound.argtypes = [_i64, _i64]
        lib.oracle_compress_fp16.restype = _i64
        lib.oracle_compress_fp16.argtypes = [_u16p, _i64, _i64, _u16p, _u8p, _i32p, ctypes.POINTER(_i64)]
        lib.oracle_compress_16.restype = _i64
        lib.oracle_compress_16.argtypes = [_u16p, _i64, _i64, _u16p, _u8p, _i32p, ctypes.POINTER(_i64), ctypes.c_uint16]
        lib.oracle_decompress_fp16.restype = None
        lib.oracle_decompress_fp16.argtypes = [_u16p, _u8p, _i32p, _i64, _i64, _u16p]
        lib.oracle_spmv_fp16.restype = None
        lib.oracle_spmv_fp16.argtypes = [_u16p, _u8p, _i32p, _i64, _i64, _u16p, _f64p, _u16p, _f64p]
        lib.oracle_dense_matvec_fp16.restype = None
        lib.oracle_dense_matvec_fp16.argtypes = [_u16p, _i64, _i64, _u16p, _f64p]
        lib.oracle_compress_int8.restype = _i64
        lib.oracle_compress_int8.argtypes = [_i8p, _i64, _i64, _i8p, _u8p, _i32p, ctypes.POINTER(_i64)]
        lib.oracle_spmv_int8.restype = None
        lib.oracle_spmv_int8.argtypes = [_i8p, _u8p, _i32p, _i64, _i64, _u16p, _f64p, _f64p]
        lib.oracle_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def have_reference() -> bool:
    """True when the compiled, unmodified reference compressor is available."""
    return os.path.exists(_REF_PATH)


def _load_ref():
    global _ref
    if _ref is None:
        ref = ctypes.CDLL(_REF_PATH)
        ref.ref_compress_fp16.restype = _i64
        ref.ref_compress_fp16.argtypes = [
            _u16p, ctypes.c_int, ctypes.c_int,
            ctypes.POINTER(_u16p), ctypes.POINTER(_u8p), ctypes.POINTER(_i32p), ctypes.POINTER(_i64),
        ]
        ref.ref_compress_int8.restype = _i64
        ref.ref_compress_int8.argtypes = [
            _i8p, ctypes.c_int, ctypes.c_int,
            ctypes.POINTER(_i8p), ctypes.POINTER(_u8p), ctypes.POINTER(_i32p), ctypes.POINTER(_i64),
        ]
        ref.ref_free.restype = None
        ref.ref_free.argtypes = [ctypes.c_void_p]
        _ref = ref
    return _ref


_ref_kernel = None


def have_reference_kernel() -> bool:
    """True when the reference's own SpMV kernel, compiled unmodified for sm_100a, is available."""
    return os.path.exists(_REF_KERNEL_PATH)


def ref_spmv_gpu(values_ptr: int, deltas_ptr: int, row_indices_ptr: int, x_ptr: int, y_ptr: int,
                 rows: int, cols: int, stream: int = 0) -> None:
    """Launch the reference kernel (kernels.cuh:34-124, reference launch shape) on device pointers.
    rows must be a positive multiple of 32 (the reference reads past row_indices otherwise)."""
    global _ref_kernel
    if _ref_kernel is None:
        lib = ctypes.CDLL(_REF_KERNEL_PATH)
        lib.ref_macko_spmv_fp16.restype = ctypes.c_int
        lib.ref_macko_spmv_fp16.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        _ref_kernel = lib
    st = _ref_kernel.ref_macko_spmv_fp16(values_ptr, deltas_ptr, row_indices_ptr, x_ptr, y_ptr, rows, cols, stream)
    if st != 0:
        raise RuntimeError(f"reference kernel launch refused or failed (status {st})")


def _as_u16(a) -> np.ndarray:
    a = np.asarray(a)
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    if a.dtype != np.uint16:
        raise TypeError(f"expected fp16 bit patterns (uint16/float16), got {a.dtype}")
    return np.ascontiguousarray(a)


def num_threads() -> int:
    return int(_load().oracle_num_threads())


def compress(dense, bf16: bool = False):
    """Oracle compress: (values u16[P], deltas u8[P/2], row_indices i32[R+1], R, C).
    `bf16`: the 16-bit patterns are bfloat16 (only the NaN test differs)."""
    lib = _load()
    dense = _as_u16(dense)
    assert dense.ndim == 2
    rows, cols = dense.shape
    bound = int(lib.oracle_compress_bound(rows, cols))
    values = np.empty(bound, dtype=np.uint16)
    deltas = np.empty(bound // 2, dtype=np.uint8)
    ri = np.empty(rows + 1, dtype=np.int32)
    n = _i64(0)
    padded = int(lib.oracle_compress_16(
        dense.ctypes.data_as(_u16p), rows, cols,
        values.ctypes.data_as(_u16p), deltas.ctypes.data_as(_u8p), ri.ctypes.data_as(_i32p),
        ctypes.byref(n), 0x7F80 if bf16 else 0x7C00))
    return values[:padded].copy(), deltas[: padded // 2].copy(), ri, rows, cols


def ref_compress(dense):
    """The reference's own ``compress_rows_cpu`` (cpu_compressor.cuh:6-73), same 5-tuple."""
    ref = _load_ref()
    dense = _as_u16(dense)
    assert dense.ndim == 2
    rows, cols = dense.shape
    v, d, r = _u16p(), _u8p(), _i32p()
    n = _i64(0)
    padded = int(ref.ref_compress_fp16(dense.ctypes.data_as(_u16p), rows, cols,
                                       ctypes.byref(v), ctypes.byref(d), ctypes.byref(r), ctypes.byref(n)))
    try:
        if padded > 0:
            values = np.ctypeslib.as_array(v, shape=(padded,)).copy()
            deltas = np.ctypeslib.as_array(d, shape=(padded // 2,)).copy()
        else:  # the reference realloc()s to size 0, which frees and yields NULL
            values = np.empty(0, dtype=np.uint16)
            deltas = np.empty(0, dtype=np.uint8)
        ri = np.ctypeslib.as_array(r, shape=(rows + 1,)).copy()
    finally:
        ref.ref_free(v)
        ref.ref_free(d)
        ref.ref_free(r)
    return values, deltas, ri, rows, cols


def decompress(compressed) -> np.ndarray:
    """Dense fp16 bit patterns [R, C] rebuilt from a compressed 5-tuple."""
    lib = _load()
    values, deltas, ri, rows, cols = compressed
    values = _as_u16(values)
    deltas = np.ascontiguousarray(deltas, dtype=np.uint8)
    ri = np.ascontiguousarray(ri, dtype=np.int32)
    dense = np.empty((rows, cols), dtype=np.uint16)
    lib.oracle_decompress_fp16(values.ctypes.data_as(_u16p), deltas.ctypes.data_as(_u8p),
                               ri.ctypes.data_as(_i32p), rows, cols, dense.ctypes.data_as(_u16p))
    return dense


def spmv(compressed, x):
    """(y float64[R], y fp16 bits u16[R], row L1 mass float64[R]) from compressed buffers."""
    lib = _load()
    values, deltas, ri, rows, cols = compressed
    values = _as_u16(values)
    deltas = np.ascontiguousarray(deltas, dtype=np.uint8)
    ri = np.ascontiguousarray(ri, dtype=np.int32)
    x = _as_u16(x)
    assert x.shape == (cols,)
    y64 = np.empty(rows, dtype=np.float64)
    yh = np.empty(rows, dtype=np.uint16)
    l1 = np.empty(rows, dtype=np.float64)
    lib.oracle_spmv_fp16(values.ctypes.data_as(_u16p), deltas.ctypes.data_as(_u8p),
                         ri.ctypes.data_as(_i32p), rows, cols, x.ctypes.data_as(_u16p),
                         y64.ctypes.data_as(_f64p), yh.ctypes.data_as(_u16p), l1.ctypes.data_as(_f64p))
    return y64, yh, l1


def compress_int8(dense):
    """Oracle compress of an int8 matrix: (values i8[P], deltas u8[P/2], row_indices i32[R+1], R, C)."""
    lib = _load()
    dense = np.ascontiguousarray(dense, dtype=np.int8)
    assert dense.ndim == 2
    rows, cols = dense.shape
    bound = ((rows * cols + 7) // 8) * 8 + 8
    values = np.empty(bound, dtype=np.int8)
    deltas = np.empty(bound // 2, dtype=np.uint8)
    ri = np.empty(rows + 1, dtype=np.int32)
    n = _i64(0)
    padded = int(lib.oracle_compress_int8(dense.ctypes.data_as(_i8p), rows, cols, values.ctypes.data_as(_i8p),
                                          deltas.ctypes.data_as(_u8p), ri.ctypes.data_as(_i32p), ctypes.byref(n)))
    return values[:padded].copy(), deltas[: padded // 2].copy(), ri, rows, cols


def ref_compress_int8(dense):
    """The reference's own ``compress_rows_int8_cpu`` (cpu_compressor.cuh:75-117), same 5-tuple."""
    ref = _load_ref()
    dense = np.ascontiguousarray(dense, dtype=np.int8)
    rows, cols = dense.shape
    v, d, r = _i8p(), _u8p(), _i32p()
    n = _i64(0)
    padded = int(ref.ref_compress_int8(dense.ctypes.data_as(_i8p), rows, cols,
                                       ctypes.byref(v), ctypes.byref(d), ctypes.byref(r), ctypes.byref(n)))
    try:
        if padded > 0:
            values = np.ctypeslib.as_array(v, shape=(padded,)).copy()
            deltas = np.ctypeslib.as_array(d, shape=(padded // 2,)).copy()
        else:
            values = np.empty(0, dtype=np.int8)
            deltas = np.empty(0, dtype=np.uint8)
        ri = np.ctypeslib.as_array(r, shape=(rows + 1,)).copy()
    finally:
        ref.ref_free(v)
        ref.ref_free(d)
        ref.ref_free(r)
    return values, deltas, ri, rows, cols


def spmv_int8(compressed, x):
    """(y float64[R], row L1 mass float64[R]) for int8 values and fp16 x (bit patterns)."""
    lib = _load()
    values, deltas, ri, rows, cols = compressed
    values = np.ascontiguousarray(values, dtype=np.int8)
    deltas = np.ascontiguousarray(deltas, dtype=np.uint8)
    ri = np.ascontiguousarray(ri, dtype=np.int32)
    x = _as_u16(x)
    y64 = np.empty(rows, dtype=np.float64)
    l1 = np.empty(rows, dtype=np.float64)
    lib.oracle_spmv_int8(values.ctypes.data_as(_i8p), deltas.ctypes.data_as(_u8p), ri.ctypes.data_as(_i32p),
                         rows, cols, x.ctypes.data_as(_u16p), y64.ctypes.data_as(_f64p), l1.ctypes.data_as(_f64p))
    return y64, l1


def bf16_bits_to_f64(bits) -> np.ndarray:
    """float64 values of bfloat16 bit patterns (a bf16 is the upper half of a float32)."""
    b = np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16
    return b.view(np.float32).astype(np.float64)


def spmv_bf16(compressed, x):
    """(y float64[R], row L1 mass float64[R]) for bfloat16 values and x: the decode of `decompress`
    (kernels.cuh:86-108 index rule) followed by a float64 product; pads and dropped zeros add nothing."""
    dense = bf16_bits_to_f64(decompress(compressed))
    xv = bf16_bits_to_f64(x)
    return dense @ xv, np.abs(dense) @ np.abs(xv)


def plan_model(deltas, row_indices, seg: int = 1024):
    """Restatement of the launch plan (macko_spmv_b200/csrc/plan.cuh) for the tests: rows cut into virtual
    rows of at most `seg` stored elements, each (begin, length, column sum in front, destination), stably
    sorted by length class, longest first. Returns (desc0 i64[V], desc1 i64[V], out i64[V], seg_first i64[R+1])
    in sorted order. The reference has no such structure; this checks the GPU builder against its definition."""
    ri = np.asarray(row_indices, dtype=np.int64)
    d8 = np.asarray(deltas, dtype=np.uint8)
    nib = np.empty(d8.size * 2, dtype=np.int64)
    nib[0::2] = d8 & 15
    nib[1::2] = d8 >> 4
    adv = np.concatenate([[0], np.cumsum(nib + 1)])   # adv[k] = sum of (delta + 1) over elements < k
    begin, length, colsum, out, seg_first = [], [], [], [], [0]
    for r in range(ri.size - 1):
        b, e = int(ri[r]), int(ri[r + 1])
        if e <= b:
            begin.append(b); length.append(0); colsum.append(0); out.append(r)
            seg_first.append(seg_first[-1] + 1)
            continue
        a0 = b & ~7
        n = -(-(e - a0) // seg)
        first = seg_first[-1]
        for j in range(n):
            sb, se = max(b, a0 + j * seg), min(e, a0 + (j + 1) * seg)
            begin.append(sb); length.append(se - sb); colsum.append(int(adv[sb] - adv[b]))
            out.append(r if n == 1 else (1 << 31) | (first + j))
        seg_first.append(first + n)
    begin = np.array(begin, dtype=np.int64); length = np.array(length, dtype=np.int64)
    colsum = np.array(colsum, dtype=np.int64); out = np.array(out, dtype=np.int64)
    cls = np.minimum(((begin & 7) + length + 63) >> 6, 63)
    order = np.argsort(-cls, kind="stable")
    return begin[order], (length | (colsum << 12))[order], out[order], np.array(seg_first, dtype=np.int64)


def dense_matvec(dense, x) -> np.ndarray:
    """float64 y = M x for a dense fp16 matrix (bit patterns)."""
    lib = _load()
    dense = _as_u16(dense)
    x = _as_u16(x)
    rows, cols = dense.shape
    y = np.empty(rows, dtype=np.float64)
    lib.oracle_dense_matvec_fp16(dense.ctypes.data_as(_u16p), rows, cols, x.ctypes.data_as(_u16p),
                                 y.ctypes.data_as(_f64p))
    return y
