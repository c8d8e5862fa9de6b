"""Regenerates tests/golden/reference_cases.npz from the UNMODIFIED reference compressor.

Runs only where the reference checkout is available (it is compiled into
oracle/_ref/libref_compress.so by oracle/Makefile): the fixtures travel, the reference
does not.  Usage:  python tests/golden/make_golden.py

Every case stores the dense input (fp16 bit patterns) and the three buffers the reference
produced for it, so the oracle and the CUDA compressor can be checked bit for bit without
the reference being present.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import oracle  # noqa: E402


def cases():
    rng = np.random.default_rng(20251125)
    specials = np.array([0x7e00, 0xfe00, 0x7c01, 0xfc01, 0x7c00, 0xfc00, 0x0001, 0x8001, 0x7bff, 0xfbff],
                        dtype=np.uint16)
    out = {}

    def add(name, dense_u16):
        out[name] = np.ascontiguousarray(dense_u16, dtype=np.uint16)

    # random matrices over a range of shapes (odd sizes, single row / column) and densities,
    # with -0.0 sprinkled over the zeros and NaN / Inf / subnormals over everything
    for (r, c) in [(1, 1), (1, 9), (9, 1), (3, 32), (5, 33), (17, 100), (12, 257), (7, 515), (40, 64)]:
        for d in (0.0, 0.02, 0.1, 0.5, 0.9, 1.0):
            m = rng.standard_normal((r, c)).astype(np.float16)
            m[rng.random((r, c)) > d] = 0
            u = m.view(np.uint16).copy()
            u[(rng.random((r, c)) < 0.08) & (u == 0)] = 0x8000
            sp = rng.random((r, c)) < 0.02
            u[sp] = rng.choice(specials, size=int(sp.sum()))
            add(f"rand_{r}x{c}_d{int(d * 100):03d}", u)

    # zero gaps of exact lengths around the 15/16 pad boundary, from the row start and between non-zeros
    one = np.float16(1.0).view(np.uint16)
    for gap in (14, 15, 16, 17, 30, 31, 32, 33, 47, 48, 49, 255, 256):
        row = np.zeros((2, gap + 40), dtype=np.uint16)
        row[0, gap] = one                      # leading gap
        row[1, 3] = one
        row[1, 3 + gap + 1] = one              # interior gap
        row[1, 3 + gap + 2] = one
        add(f"gap_{gap}", row)
        neg = row.copy()
        neg[neg == 0] = 0x8000                 # pads carry the sign of the zero they sit on
        add(f"gap_{gap}_negzero", neg)

    # stored-element totals covering every residue mod 8 (tail padding), nibble bytes shared by rows
    for n in range(0, 17):
        m = np.zeros((3, 16), dtype=np.uint16)
        flat = m.reshape(-1)
        flat[: n] = one
        add(f"tail_{n}", m)
    return out


def cases_int8():
    """Inputs for the reference's int8 encoder (cpu_compressor.cuh:75-117): random matrices, exact zero gaps
    around the pad boundary at the start, in the middle and at the END of a row (that encoder keeps trailing
    pads), and every tail residue mod 8."""
    rng = np.random.default_rng(20251126)
    out = {}
    for (r, c) in [(1, 1), (1, 15), (1, 16), (1, 33), (9, 1), (3, 32), (5, 33), (17, 100), (12, 257), (7, 515)]:
        for d in (0.0, 0.02, 0.1, 0.5, 1.0):
            m = rng.integers(-128, 128, size=(r, c)).astype(np.int8)
            m[rng.random((r, c)) > d] = 0
            out[f"i8_rand_{r}x{c}_d{int(d * 100):03d}"] = m
    for gap in (14, 15, 16, 17, 31, 32, 33, 48, 255, 256):
        row = np.zeros((3, gap + 40), dtype=np.int8)
        row[0, gap] = 5                         # leading gap, then trailing zeros
        row[1, 3] = -7
        row[1, 3 + gap + 1] = 9                 # interior gap
        row[2, 0] = 1                           # only trailing zeros: gap + 39 of them
        out[f"i8_gap_{gap}"] = row
    for n in range(0, 17):
        m = np.zeros((3, 16), dtype=np.int8)
        m.reshape(-1)[:n] = -3
        out[f"i8_tail_{n}"] = m
    return out


def main():
    assert oracle.have_reference(), "build oracle/_ref first (make -C oracle)"
    data8 = {}
    for name, dense in cases_int8().items():
        v, d, ri, r, c = oracle.ref_compress_int8(dense)
        data8[f"{name}/dense"] = dense
        data8[f"{name}/values"] = v
        data8[f"{name}/deltas"] = d
        data8[f"{name}/row_indices"] = ri
    path8 = os.path.join(HERE, "reference_cases_int8.npz")
    np.savez_compressed(path8, **data8)
    print(f"wrote {path8}: {len(data8) // 4} cases, {os.path.getsize(path8)} bytes")
    data = {}
    for name, dense in cases().items():
        v, d, ri, r, c = oracle.ref_compress(dense)
        data[f"{name}/dense"] = dense
        data[f"{name}/values"] = v
        data[f"{name}/deltas"] = d
        data[f"{name}/row_indices"] = ri
    path = os.path.join(HERE, "reference_cases.npz")
    np.savez_compressed(path, **data)
    print(f"wrote {path}: {len(data) // 4} cases, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
