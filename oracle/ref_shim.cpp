// Thin C entry point around the UNMODIFIED reference compressor
// (src/macko_spmv/cuda/cpu_compressor.cuh:6-73). The reference source is included
// from where it lies (include path given by the Makefile); nothing is copied.
// Test infrastructure only: used to pin the oracle and as the CPU baseline.
#include <cstdlib>
#include <cstring>
#include <cstdint>
#include "cpu_compressor.cuh"

extern "C" {

// Runs the reference compressor and hands its malloc'd buffers to the caller.
// Returns the padded element count P; free the buffers with ref_free().
int64_t ref_compress_fp16(const uint16_t *dense, int rows, int cols,
                          uint16_t **values, uint8_t **deltas, int32_t **row_indices,
                          int64_t *n_out)
{
    int *ri = nullptr;
    unsigned char *dl = nullptr;
    __half *vals = nullptr;
    int n = 0, padded = 0;
    compress_rows_cpu(reinterpret_cast<const __half *>(dense), rows, cols, &ri, &dl, &vals, &n, &padded);
    *values = reinterpret_cast<uint16_t *>(vals);
    *deltas = dl;
    *row_indices = ri;
    if (n_out) *n_out = n;
    return padded;
}

// The same for the reference's int8 encoder (src/macko_spmv/cuda/cpu_compressor.cuh:75-117).
int64_t ref_compress_int8(const int8_t *dense, int rows, int cols,
                          int8_t **values, uint8_t **deltas, int32_t **row_indices, int64_t *n_out)
{
    int *ri = nullptr;
    unsigned char *dl = nullptr;
    int8_t *vals = nullptr;
    int n = 0, padded = 0;
    compress_rows_int8_cpu(dense, rows, cols, &ri, &dl, &vals, &n, &padded);
    *values = vals;
    *deltas = dl;
    *row_indices = ri;
    if (n_out) *n_out = n;
    return padded;
}

void ref_free(void *p) { free(p); }
}
