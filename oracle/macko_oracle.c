/*
 * CPU oracle for the MACKO fp16 compress / multiply path.
 *
 * TEST INFRASTRUCTURE ONLY. This file is a plain-C restatement of the reference
 * algorithm used to check the CUDA library; nothing in the shipped package may
 * call it. Only the test-suite, the smoke check and the benchmark's CPU-baseline
 * leg link against it.
 *
 * Parity status: PINNED. The restatement is checked against
 *   - the two golden vectors of the reference test-suite
 *     (tests/test_macko_spmv.py:5-36,48-61 and :74-95), and
 *   - the reference compressor itself (src/macko_spmv/cuda/cpu_compressor.cuh,
 *     compiled unmodified into oracle/_ref/ by the Makefile beside this file)
 *     on seeded random and adversarial inputs.
 *
 * Format restated (reference: src/macko_spmv/cuda/cpu_compressor.cuh:6-73):
 *   values      fp16[P]    stored elements, row after row, P = n rounded up to 8
 *   deltas      u8[P/2]    4-bit zero-run length before each stored element,
 *                          element k in byte k/2, even k in the low nibble
 *   row_indices i32[R+1]   row r owns stored elements [ri[r], ri[r+1])
 * A stored element is a true non-zero, or a pad (value +-0, delta 15) inserted
 * when 15 zeros have been skipped and the 16th column is zero as well.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- fp16 helpers (IEEE binary16, no hardware dependency) ---------------- */

static inline int h_is_nan(uint16_t h) { return (h & 0x7fffu) > 0x7c00u; }
static inline int h_is_zero(uint16_t h) { return (h & 0x7fffu) == 0; }

static inline float h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* float -> half, round to nearest even; every NaN becomes 0x7fff, which is what
 * the host-side conversion used by the reference produces
 * (cpu_compressor.cuh:26,36 goes half -> float -> half through cuda_fp16.h). */
static inline uint16_t f2h(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax > 0x7f800000u) return 0x7fffu;
    if (ax >= 0x47800000u) { /* >= 65536: overflow or inf */
        if (ax == 0x7f800000u) return (uint16_t)(sign | 0x7c00u);
        /* values in [65520, 65536) round to inf as well, handled below */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) return (uint16_t)sign; /* below half of min subnormal */
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { /* subnormal result */
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    uint32_t r = base + q;
    if (rem > half || (rem == half && (r & 1u))) ++r; /* carries into exponent correctly */
    return (uint16_t)(sign | r);
}

/* Value bits written for a stored element whose source bits are h:
 * identical bits except that NaNs are canonicalised (see f2h). */
static inline uint16_t stored_bits(uint16_t h) { return h_is_nan(h) ? 0x7fffu : h; }
/* The same for a value type whose +infinity has the bits `nan_above` (0x7c00 fp16, 0x7f80 bfloat16). */
static inline uint16_t stored_bits_typed(uint16_t h, uint16_t nan_above)
{
    return ((h & 0x7fffu) > nan_above) ? 0x7fffu : h;
}

/* ---- compress ------------------------------------------------------------ */

/* Number of stored elements of one row: every true non-zero at column c whose
 * predecessor (previous non-zero, or -1) sits at c0 emits floor((c-c0-1)/16)
 * pads and itself; trailing zeros emit nothing
 * (closed form of cpu_compressor.cuh:19-64). */
static int64_t row_stored_count(const uint16_t *row, int64_t cols)
{
    int64_t n = 0, prev = -1;
    for (int64_t c = 0; c < cols; ++c) {
        if (!h_is_zero(row[c])) {
            n += ((c - prev - 1) >> 4) + 1;
            prev = c;
        }
    }
    return n;
}

/* Upper bound on P for a rows x cols matrix (every element stored, rounded to 8). */
int64_t oracle_compress_bound(int64_t rows, int64_t cols)
{
    return ((rows * cols + 7) / 8) * 8;
}

/*
 * Compress a row-major fp16 matrix (bit patterns in `dense`).
 * Outputs: row_indices[rows+1]; values / deltas must hold oracle_compress_bound()
 * elements / half that many bytes and are fully defined up to the returned
 * padded count P (tail is zero). Returns P; *n_out receives the unpadded count.
 */
int64_t oracle_compress_16(const uint16_t *dense, int64_t rows, int64_t cols,
                           uint16_t *values, uint8_t *deltas, int32_t *row_indices,
                           int64_t *n_out, uint16_t nan_above);

int64_t oracle_compress_fp16(const uint16_t *dense, int64_t rows, int64_t cols,
                             uint16_t *values, uint8_t *deltas, int32_t *row_indices,
                             int64_t *n_out)
{
    return oracle_compress_16(dense, rows, cols, values, deltas, row_indices, n_out, 0x7c00u);
}

/* The same layout for any 16-bit value type that shares fp16's +-0 encoding (bfloat16): the reference
 * format does not depend on the meaning of the value bits beyond "is it zero" and "is it a NaN"
 * (cpu_compressor.cuh:26-27,36). The reference has no bf16 encoder: this branch is unpinned against it
 * except through the fp16 path it shares every line with. */
int64_t oracle_compress_16(const uint16_t *dense, int64_t rows, int64_t cols,
                           uint16_t *values, uint8_t *deltas, int32_t *row_indices,
                           int64_t *n_out, uint16_t nan_above)
{
    /* pass 1: per-row counts (rows are independent) -> prefix */
    row_indices[0] = 0;
    int64_t *counts = (int64_t *)malloc((size_t)(rows > 0 ? rows : 1) * sizeof(int64_t));
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) counts[r] = row_stored_count(dense + r * cols, cols);
    int64_t total = 0;
    for (int64_t r = 0; r < rows; ++r) {
        total += counts[r];
        row_indices[r + 1] = (int32_t)total;
    }
    free(counts);
    int64_t padded = ((total + 7) / 8) * 8;
    memset(values, 0, (size_t)padded * sizeof(uint16_t));
    memset(deltas, 0, (size_t)(padded / 2));

    /* pass 2: emit. Rows write disjoint value slots; two rows can share a delta byte, so the 4-bit
     * deltas go to one byte per element first and are packed afterwards. */
    uint8_t *nib = (uint8_t *)calloc((size_t)(padded > 0 ? padded : 1), 1);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t *row = dense + r * cols;
        int64_t k = row_indices[r];
        int64_t prev = -1;
        for (int64_t c = 0; c < cols; ++c) {
            uint16_t h = row[c];
            if (h_is_zero(h)) continue;
            int64_t gap = c - prev - 1;
            /* pads sit on columns prev+16, prev+32, ...; they keep the sign bit of
             * the zero found there (cpu_compressor.cuh:36 stores the source value) */
            for (int64_t p = prev + 16; p < c; p += 16) {
                values[k] = row[p];
                nib[k] = 15;
                ++k;
            }
            values[k] = stored_bits_typed(h, nan_above);
            nib[k] = (uint8_t)(gap & 15);
            ++k;
            prev = c;
        }
    }
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < padded / 2; ++b) deltas[b] = (uint8_t)(nib[2 * b] | (nib[2 * b + 1] << 4));
    free(nib);
    if (n_out) *n_out = total;
    return padded;
}

/* ---- decompress / multiply (restating src/macko_spmv/cuda/kernels.cuh:86-108) */

/* Column of the k-th stored element of a row = (sum of deltas 0..k) + k. */
void oracle_decompress_fp16(const uint16_t *values, const uint8_t *deltas,
                            const int32_t *row_indices, int64_t rows, int64_t cols,
                            uint16_t *dense)
{
    memset(dense, 0, (size_t)(rows * cols) * sizeof(uint16_t));
    for (int64_t r = 0; r < rows; ++r) {
        int64_t col = -1;
        for (int64_t k = row_indices[r]; k < row_indices[r + 1]; ++k) {
            int d = (deltas[k >> 1] >> (4 * (k & 1))) & 15;
            col += d + 1;
            if (col >= cols) col = cols - 1; /* kernels.cuh:104 clamps */
            uint16_t v = values[k];
            if (!h_is_zero(v)) dense[r * cols + col] = v;
        }
    }
}

/*
 * y = M x straight from the compressed buffers.
 *   y_f64 (optional)  exact products accumulated in double,
 *   y_h   (optional)  fp32 sequential accumulation rounded to fp16 (the rounding
 *                     the reference kernel applies, kernels.cuh:115-122, alpha=1).
 *   l1    (optional)  sum_k |val_k * x[col_k]| per row, for error bounds.
 * Rows are independent; with OpenMP they are spread over the host threads.
 */
void oracle_spmv_fp16(const uint16_t *values, const uint8_t *deltas,
                      const int32_t *row_indices, int64_t rows, int64_t cols,
                      const uint16_t *x, double *y_f64, uint16_t *y_h, double *l1)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 64)
#endif
    for (int64_t r = 0; r < rows; ++r) {
        int64_t col = -1;
        double acc = 0.0, mag = 0.0;
        float acc32 = 0.0f;
        for (int64_t k = row_indices[r]; k < row_indices[r + 1]; ++k) {
            int d = (deltas[k >> 1] >> (4 * (k & 1))) & 15;
            col += d + 1;
            int64_t c = col >= cols ? cols - 1 : col;
            float v = h2f(values[k]), xv = h2f(x[c]);
            double p = (double)v * (double)xv;
            acc += p;
            mag += p < 0 ? -p : p;
            acc32 += v * xv;
        }
        if (y_f64) y_f64[r] = acc;
        if (y_h) y_h[r] = f2h(acc32);
        if (l1) l1[r] = mag;
    }
}

/* ---- int8 values (restating src/macko_spmv/cuda/cpu_compressor.cuh:75-117 and kernels.cuh:127-216) ----
 * Same delta packing and row offsets; values are one signed byte each. The int8 encoder of the reference
 * has no trailing clean-up: a run of zeros at the end of a row still leaves a pad (value 0, delta 15) for
 * every full 16 of them (cpu_compressor.cuh:88-111), and the leftover count is simply dropped. Parity is
 * pinned against the compiled reference encoder (oracle/_ref) and the fixtures generated from it; the
 * reference has no known-answer test for int8. */
int64_t oracle_compress_int8(const int8_t *dense, int64_t rows, int64_t cols,
                             int8_t *values, uint8_t *deltas, int32_t *row_indices, int64_t *n_out)
{
    row_indices[0] = 0;
    int64_t total = 0;
    for (int64_t r = 0; r < rows; ++r) {
        const int8_t *row = dense + r * cols;
        int64_t n = 0, prev = -1;
        for (int64_t c = 0; c < cols; ++c)
            if (row[c] != 0) { n += ((c - prev - 1) >> 4) + 1; prev = c; }
        n += (cols - 1 - prev) >> 4;   /* pads inside the trailing zeros stay */
        total += n;
        row_indices[r + 1] = (int32_t)total;
    }
    int64_t padded = ((total + 7) / 8) * 8;
    memset(values, 0, (size_t)padded);
    memset(deltas, 0, (size_t)(padded / 2));
    for (int64_t r = 0; r < rows; ++r) {
        const int8_t *row = dense + r * cols;
        int64_t k = row_indices[r];
        int64_t prev = -1;
        for (int64_t c = 0; c <= cols; ++c) {
            if (c < cols && row[c] == 0) continue;
            for (int64_t p = prev + 16; p < c; p += 16) {   /* pads on columns prev+16, prev+32, ... (value 0) */
                values[k] = 0;
                deltas[k >> 1] |= (uint8_t)(15u << (4 * (k & 1)));
                ++k;
            }
            if (c == cols) break;
            values[k] = row[c];
            deltas[k >> 1] |= (uint8_t)(((c - prev - 1) & 15) << (4 * (k & 1)));
            ++k;
            prev = c;
        }
    }
    if (n_out) *n_out = total;
    return padded;
}

/* y = M x for int8 values and fp16 x: exact products accumulated in double, and the row L1 mass. */
void oracle_spmv_int8(const int8_t *values, const uint8_t *deltas, const int32_t *row_indices,
                      int64_t rows, int64_t cols, const uint16_t *x, double *y_f64, double *l1)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 64)
#endif
    for (int64_t r = 0; r < rows; ++r) {
        int64_t col = -1;
        double acc = 0.0, mag = 0.0;
        for (int64_t k = row_indices[r]; k < row_indices[r + 1]; ++k) {
            int d = (deltas[k >> 1] >> (4 * (k & 1))) & 15;
            col += d + 1;
            int64_t c = col >= cols ? cols - 1 : col;   /* kernels.cuh:196-197 clamps */
            double p = (double)values[k] * (double)h2f(x[c]);
            acc += p;
            mag += p < 0 ? -p : p;
        }
        if (y_f64) y_f64[r] = acc;
        if (l1) l1[r] = mag;
    }
}

/* Dense fp32-accumulated matvec of an fp16 matrix (the "dense M@V" tier). */
void oracle_dense_matvec_fp16(const uint16_t *dense, int64_t rows, int64_t cols,
                              const uint16_t *x, double *y_f64)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (int64_t r = 0; r < rows; ++r) {
        double acc = 0.0;
        const uint16_t *row = dense + r * cols;
        for (int64_t c = 0; c < cols; ++c) {
            if (h_is_zero(row[c])) continue;
            acc += (double)h2f(row[c]) * (double)h2f(x[c]);
        }
        y_f64[r] = acc;
    }
}

uint16_t oracle_f2h(float f) { return f2h(f); }
float oracle_h2f(uint16_t h) { return h2f(h); }
int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
