/*
 * macko_b200 -- C ABI of the sm_100a MACKO SpMV library (libmacko_b200.so).
 *
 * Every entry point
 *   - is extern "C", takes plain pointers and sizes, returns an int status
 *     (MACKO_OK == 0) and never throws or aborts;
 *   - works on DEVICE pointers of the CUDA device that is current on the calling
 *     thread, enqueues its work on `stream` (a cudaStream_t passed as void*,
 *     NULL = legacy default stream) and returns without synchronising;
 *   - allocates no device memory: the caller owns every buffer (inputs, outputs,
 *     workspace), which keeps the calls legal inside CUDA-graph capture.
 *
 * MACKO compressed matrix (byte layout identical to the reference,
 * src/macko_spmv/cuda/cpu_compressor.cuh:6-73 and
 * src/macko_spmv/cuda/cpu_compressor_torch_launcher.cuh:34-38):
 *   values       fp16  [P]      stored elements row after row, P % 8 == 0
 *   deltas       uint8 [P/2]    4-bit zero-run before each stored element,
 *                               element k in byte k/2, even k = low nibble
 *   row_indices  int32 [rows+1] row r owns stored elements [ri[r], ri[r+1])
 * Alignment required by the kernels: values 16 bytes, deltas 4 bytes,
 * row_indices 4 bytes, x and y 2 bytes (16-byte aligned x is staged faster).
 */
#ifndef MACKO_B200_H_
#define MACKO_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MACKO_B200_VERSION 100 /* major*10000 + minor*100 + patch */

enum macko_status {
    MACKO_OK = 0,
    MACKO_ERR_INVALID_ARGUMENT = 1, /* null pointer, negative size, bad flag            */
    MACKO_ERR_MISALIGNED = 2,       /* a buffer violates the alignment listed above     */
    MACKO_ERR_SIZE_OVERFLOW = 3,    /* rows*cols or a count does not fit 31-bit indices */
    MACKO_ERR_CUDA = 4,             /* a CUDA runtime call or the launch failed         */
    MACKO_ERR_WORKSPACE = 5         /* workspace too small                              */
};

/* Library version (MACKO_B200_VERSION of the build). */
int macko_version(void);

/* Static text for a status code. */
const char *macko_status_string(int status);

/* Message describing the last non-OK status returned on the calling thread
 * (thread-local, never NULL). */
const char *macko_last_error(void);

/*
 * y = fp16( alpha * (M x) [+ beta * y] ),  fp32 accumulation.
 *
 * Replaces: kernel `macko_spmv<reuse_value_from_c>` (src/macko_spmv/cuda/kernels.cuh:34-124)
 * and its host launcher `macko_spmv_launcher`
 * (src/macko_spmv/cuda/kernels_torch_launchers.cuh:3-48, which fixes alpha=1, beta=0).
 *
 *   values, deltas, row_indices   compressed matrix on the device
 *   padded_count                  P = number of fp16 in `values` (used for launch
 *                                 heuristics and argument checks)
 *   x  fp16[cols], y  fp16[rows]  device vectors; y is read only when beta != 0
 * x must hold finite numbers for the result to be defined row by row (a non-finite
 * x entry can turn any row into NaN, as in the reference kernel).
 */
int macko_spmv_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, void *stream);

/*
 * Same product with the kernel shape chosen by the caller, for tuning sweeps:
 *   lanes_per_row in {4, 8, 16, 32}; steps_in_flight in {2, 4, 6};
 *   x_in_shared 0/1; ctas_per_sm >= 1 (0 = library default).
 * No counterpart in the reference (its launch shape is fixed,
 * kernels_torch_launchers.cuh:15-17).
 */
int macko_spmv_fp16_tuned(const void *values, const void *deltas, const int32_t *row_indices,
                          int64_t rows, int64_t cols, int64_t padded_count,
                          const void *x, void *y, float alpha, float beta, void *stream,
                          int lanes_per_row, int steps_in_flight, int x_in_shared, int ctas_per_sm);

/*
 * The launch shape macko_spmv_fp16 picks for a matrix on a GPU with `sm_count` SMs: lanes per row (4, 8, 16
 * or 32) and 8-element units in flight per lane (2, 4 or 6), the two arguments macko_spmv_fp16_tuned takes.
 * Pure host arithmetic (no CUDA call), for logging and for tests of the heuristic. No counterpart in the
 * reference, whose launch shape is fixed (32 x 32 threads, one warp per row, kernels_torch_launchers.cuh:15-16).
 */
int macko_spmv_shape(int64_t rows, int64_t cols, int64_t padded_count, int sm_count,
                     int *lanes_per_row, int *steps_in_flight);

/*
 * Y = alpha * M X + beta * Y for `batch` right-hand sides at once: x is [batch][cols] and y is
 * [batch][rows], both row-major fp16 (the layout of a [tokens, features] activation). Up to 8 vectors
 * share one pass over the compressed matrix (their values are interleaved in shared memory so that one
 * vector load gathers a column of all of them); larger batches run in chunks of 8, and fewer vectors per
 * pass are used when `cols` is too large for that many copies of x in shared memory. Every vector
 * gets the result of macko_spmv_fp16 up to the order of the fp32 additions.
 *
 * Replaces the loop of single-vector launches that the reference runs for batched inputs through
 * torch.vmap (python_scripts/util_run_pruned_llm.py:112-115; the reference kernel is built for
 * BATCH = 1, c_benchmarking/utils.cuh:299).
 */
int macko_spmm_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, int64_t batch, float alpha, float beta, void *stream);

/*
 * Dense row-major fp16 [rows][cols] from a compressed matrix: element k of a row goes to column
 * (sum of the deltas of elements 0..k) + k, as the reference kernel decodes it
 * (src/macko_spmv/cuda/kernels.cuh:86-108); stored non-zeros keep their bits, everything else
 * (pads included) is +0. `dense` (rows * cols * 2 bytes) is written exactly once, on `stream` (16-byte stores when it is 16-byte aligned). The reference has no
 * decompressor; this one serves products with many right-hand sides (dense copy + GEMM) and round-trip
 * checks of the compressor.
 */
int macko_decompress_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                          int64_t rows, int64_t cols, int64_t padded_count, void *dense, void *stream);

/*
 * GPU compressor, phase 1: per-row stored-element counts and their prefix sum.
 *
 * Replaces (together with macko_compress_emit): `compress_rows_cpu`
 * (src/macko_spmv/cuda/cpu_compressor.cuh:6-73) and its tensor wrapper `cpu_compress`
 * (src/macko_spmv/cuda/cpu_compressor_torch_launcher.cuh:6-39).
 *
 *   dense        fp16[rows*cols], row-major, contiguous, device memory
 *   row_indices  int32[rows+1] out: ri[0]=0, ri[r+1]-ri[r] = stored elements of row r
 * After the stream reaches this point, ri[rows] = n (unpadded stored count); the
 * caller reads it back (one 4-byte copy) to size values/deltas: P = ceil(n/8)*8.
 * rows*cols must be < 2^31 (the reference indexes with `int`).
 */
int macko_compress_count(const void *dense, int64_t rows, int64_t cols,
                         int32_t *row_indices, void *stream);

/* Bytes of scratch macko_compress_emit needs for a padded stored count P. */
int64_t macko_compress_workspace_bytes(int64_t padded_count);

/*
 * GPU compressor, phase 2: write values[P] and deltas[P/2], bit-identical to the
 * reference compressor on the same input (pads, nibble packing, NaN -> 0x7fff,
 * zero tail up to the multiple of 8).
 *   row_indices   output of macko_compress_count for the same `dense`
 *   padded_count  P = ceil(ri[rows]/8)*8
 *   workspace     device scratch of macko_compress_workspace_bytes(P) bytes,
 *                 8-byte aligned; contents undefined afterwards
 */
int macko_compress_emit(const void *dense, int64_t rows, int64_t cols,
                        const int32_t *row_indices, int64_t padded_count,
                        void *values, void *deltas,
                        void *workspace, int64_t workspace_bytes, void *stream);

/*
 * macko_compress_emit without a workspace argument, for hosts that cannot hand the library any
 * scratch memory: a plug-in running inside an application that has already given every byte of
 * device memory to its own pool, or a code path on which a cudaMalloc (which may stall the whole
 * device) is not acceptable. The one-delta-per-byte scratch of phase 2 lives in an array built into
 * the library instead (16 MiB of device memory per GPU that loads the library, held until the
 * process exits), so padded_count may not exceed macko_compress_static_capacity() = 16 777 216
 * stored elements (a dense 4096x4096 matrix just fits); larger counts are refused with
 * MACKO_ERR_WORKSPACE. Same inputs, outputs and bit-exact result as macko_compress_emit. The
 * function calls no cudaMalloc/cudaFree and no allocating library routine.
 *
 * The first call on each device looks up the device address of the built-in array; make that
 * first call outside any stream capture. All calls on a device share the array and it keeps what
 * the previous call left in it (nothing in it needs clearing between calls), so two calls whose
 * kernels can overlap on the GPU - different streams without an ordering between them - race:
 * order them, or use macko_compress_emit with separate workspaces.
 *
 * This entry point has no counterpart in the reference.
 */
int macko_compress_emit_static(const void *dense, int64_t rows, int64_t cols,
                               const int32_t *row_indices, int64_t padded_count,
                               void *values, void *deltas, void *stream);

/* Largest padded_count macko_compress_emit_static accepts. */
int64_t macko_compress_static_capacity(void);

/*
 * Row-sharded product with the exchange fused into the kernel (several GPUs, one process each).
 * Rank `rank` of `world` (<= 8) holds the compressed block of rows [row_offset, row_offset + rows)
 * and the whole x. Instead of writing a local slice and calling a collective, the kernel delivers
 * its rows of y into the full-y buffer of EVERY rank (`peer_y[p]`, device pointers that are valid on
 * this device: peer-mapped / symmetric memory): its CTAs write into `peer_y[rank]`, and the CTA that
 * finishes last copies the rank's slice from there into the buffers of the other ranks, advances this
 * rank's call counter and releases it into slot `rank` of every rank's flag array.
 * `peer_flags[p]` points to at least world + 3 zero-initialised uint32 of rank p:
 *   [0, world) arrival counters, [world] calls issued, [world+1] internal ticket, [world+2] error.
 * `peer_y` and `peer_flags` are HOST arrays of `world` pointers, read during the call.
 *
 * The CTA of the grid that finishes last then stays until the arrival counters of all ranks have
 * reached this rank's call counter, so the completion of the kernel means that this rank's full y
 * is complete: nothing else has to be enqueued. The wait is bounded: if a rank never arrives it gives
 * up after a few seconds of polling and sets flags[world + 2] to 1 + that rank; it never hangs the
 * device. macko_peer_wait(local_flags, world, stream) enqueues the same bounded wait as a kernel of
 * its own, for hosts that want to re-check arrival at a later point of the stream.
 *
 * Every rank must issue the same sequence of scatter calls. Alternate between two full-y
 * buffers from one call to the next: a rank may start the next product while another still reads
 * the previous y. cols must fit shared memory (as for the default kernel shape).
 * No counterpart in the reference (it is single-GPU).
 */
int macko_spmv_fp16_scatter(const void *values, const void *deltas, const int32_t *row_indices,
                            int64_t rows, int64_t cols, int64_t padded_count, const void *x,
                            void *const *peer_y, int64_t row_offset, uint32_t *const *peer_flags,
                            int rank, int world, void *stream);
int macko_peer_wait(uint32_t *local_flags, int world, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* MACKO_B200_H_ */
