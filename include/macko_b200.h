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

#define MACKO_B200_VERSION 200 /* major*10000 + minor*100 + patch */

/* Flag bits of the *_ex / planned / scatter_ex entry points. */
/* The caller guarantees that values, deltas and row_indices (and the plan, if any) are not written by
 * work still in flight on `stream` when the call is made: weights compressed at set-up, not the output of
 * the kernel in front. The kernel may then fetch its first matrix data while the previous kernel of the
 * stream is still finishing (programmatic dependent launch); x and y are never touched early. */
#define MACKO_SPMV_MATRIX_IMMUTABLE 1u
/* macko_spmv_fp16_scatter_ex only: publish this rank's slice and return without waiting for the other
 * ranks; the caller enqueues macko_peer_wait before the full y is read. */
#define MACKO_SCATTER_DEFERRED_WAIT 2u

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
 * macko_spmv_fp16 with flag bits (MACKO_SPMV_MATRIX_IMMUTABLE). Same kernel, same result bits; the flag
 * only moves the first matrix loads in front of the wait for the previous kernel of the stream.
 * Replaces the same reference launcher (kernels_torch_launchers.cuh:3-48), which has no such option.
 */
int macko_spmv_fp16_ex(const void *values, const void *deltas, const int32_t *row_indices,
                       int64_t rows, int64_t cols, int64_t padded_count,
                       const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream);

/*
 * The same product for bfloat16: values, x and y hold bf16 bits instead of fp16 bits (the MACKO layout does
 * not depend on what the 16 bits of a stored value mean: the compressor only tests them for +-0 and
 * canonicalises NaNs, see macko_compress_emit_bf16), products are exact, accumulation is fp32, y is rounded
 * to bf16. The reference lists further value types as wanted (README.md:167) and ships fp16 and int8 kernels
 * (src/macko_spmv/cuda/kernels.cuh:34-124,127-216); it has no bf16 kernel.
 */
int macko_spmv_bf16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream);

/*
 * The same product for int8 values: values int8[P] (8-byte aligned), x and y fp16, fp32 accumulation; the
 * bytes are converted exactly to fp16 in registers and go through the same fused multiply-add.
 * Replaces: kernel `macko_spmv_int8<reuse_value_from_c>` (src/macko_spmv/cuda/kernels.cuh:127-216), which the
 * reference launches from its C benchmark only (c_benchmarking/benchmark.cu:106-119, kernel id 8).
 * Matrices come from macko_compress_count_int8 / macko_compress_emit_int8.
 */
int macko_spmv_int8(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream);

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
 * Planned launch, for matrices whose rows are very long or very uneven. A plan is side metadata built once
 * per matrix on the GPU from row_indices and deltas; the three MACKO buffers are not modified and stay what
 * the reference format defines. It cuts every row into virtual rows of at most `segment_elements` stored
 * elements (0 = default 1536; a multiple of 256, at most 3840), records for each where the decode has to
 * resume (the column sum in front of the segment), sorts them by length and deals them to the warps longest
 * first, so that every warp gets about the same number of stored elements whatever the row lengths are. The
 * segments of a cut row leave fp32 partial sums inside the plan; a second, tiny kernel enqueued right behind
 * the product adds them up in segment order, so y is reproducible from call to call. Results match
 * macko_spmv_fp16 up to the order of the fp32 additions.
 *
 *   macko_spmv_plan_bytes  size of the plan buffer for a matrix (-1 for arguments a plan cannot index)
 *   macko_spmv_plan        builds the plan into `plan` (device memory, 16-byte aligned) and fills `info`
 *                          (host memory); SYNCHRONISES `stream` once to read the counts back
 *   macko_spmv_fp16_planned  the product; `info` is the structure macko_spmv_plan filled for this matrix.
 *                          cols must fit shared memory (about 116 000). Calls that use one plan must not
 *                          overlap on the GPU (they share the partial sums inside it).
 * info->recommended is 1 when the row statistics say that the planned launch should beat macko_spmv_fp16
 * (rows cut into several segments and much longer than the average row).
 * No counterpart in the reference: its kernel gives every row one warp (kernels_torch_launchers.cuh:15-16),
 * which is what makes uneven rows slow there.
 */
typedef struct macko_spmv_plan_info {
    int64_t plan_bytes;       /* bytes of the plan buffer this info belongs to */
    int64_t rows;
    int64_t padded_count;
    int32_t virtual_rows;
    int32_t segment_elements;
    int32_t longest_row;      /* stored elements of the longest row */
    int32_t split_rows;       /* rows cut into more than one segment */
    int32_t recommended;
    int32_t reserved[3];
} macko_spmv_plan_info;

int64_t macko_spmv_plan_bytes(int64_t rows, int64_t cols, int64_t padded_count, int32_t segment_elements);
int macko_spmv_plan(const void *deltas, const int32_t *row_indices, int64_t rows, int64_t cols,
                    int64_t padded_count, int32_t segment_elements, void *plan, int64_t plan_bytes,
                    macko_spmv_plan_info *info, void *stream);
int macko_spmv_fp16_planned(const void *values, const void *deltas, const int32_t *row_indices,
                            int64_t rows, int64_t cols, int64_t padded_count,
                            const void *plan, const macko_spmv_plan_info *info,
                            const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream);

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
 *                 8-byte aligned; contents undefined afterwards. The fp16 and
 *                 bf16 calls check it and leave it alone (they pack the deltas
 *                 in the same pass, after clearing `deltas` on `stream`); the
 *                 int8 call writes one delta per byte into it and packs after.
 */
int macko_compress_emit(const void *dense, int64_t rows, int64_t cols,
                        const int32_t *row_indices, int64_t padded_count,
                        void *values, void *deltas,
                        void *workspace, int64_t workspace_bytes, void *stream);

/*
 * macko_compress_emit for a matrix of bfloat16 values. The count phase is the same call for both types (it
 * only tests the 16 bits for +-0, which fp16 and bf16 share); this phase differs in what counts as a NaN
 * (bits above 0x7f80 instead of 0x7c00; every NaN is stored as 0x7fff, a quiet NaN in either type). The
 * reference has no bf16 path (README.md:167 lists more value types as wanted); the layout is its fp16 layout.
 */
int macko_compress_emit_bf16(const void *dense, int64_t rows, int64_t cols,
                             const int32_t *row_indices, int64_t padded_count,
                             void *values, void *deltas,
                             void *workspace, int64_t workspace_bytes, void *stream);

/*
 * The compressor for int8 matrices, both phases (dense: int8[rows*cols]; values: int8[P]; same deltas and
 * row_indices as above). Bit-identical to the reference's int8 encoder `compress_rows_int8_cpu`
 * (src/macko_spmv/cuda/cpu_compressor.cuh:75-117), which, unlike its fp16 encoder, keeps the pads inside the
 * zeros at the end of a row: a row that ends in t zeros (an empty row: t = cols) stores floor(t / 16) pads there.
 */
int macko_compress_count_int8(const void *dense, int64_t rows, int64_t cols,
                              int32_t *row_indices, void *stream);
int macko_compress_emit_int8(const void *dense, int64_t rows, int64_t cols,
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
 * Both emit entry points check every store on the device against padded_count: a call whose row_indices
 * do not belong to the padded_count it passes (a stale P, or a matrix that changed between count and
 * emit) writes nothing outside values[0, P) / the scratch, leaves the outputs incomplete and counts the
 * warps that had to drop a store in a per-device counter. This call copies that counter to *count
 * (0 = every emit since the last call was complete) and clears it; it synchronises `stream`.
 * The reference over-allocates rows*cols + 8 slots for the same purpose (cpu_compressor.cuh:13-14).
 */
int macko_compress_overflow(uint32_t *count, void *stream);

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

/*
 * The same two calls with their options spelled out.
 *   flags       MACKO_SPMV_MATRIX_IMMUTABLE, MACKO_SCATTER_DEFERRED_WAIT
 *   spin_limit  polls of an arrival counter before a wait gives up (0 = default, 2^23: a few seconds)
 * With MACKO_SCATTER_DEFERRED_WAIT the kernel forwards this rank's slice, publishes its arrival counter and
 * ends; it overlaps with the next kernel of the stream like an ordinary product. Nothing may read the full
 * y before a macko_peer_wait(_limited) enqueued after the last such product has run: it waits until every
 * rank's arrival counter has reached this rank's call counter. A y buffer may be reused for a later product
 * only after a wait that every rank has passed since its last use (e.g. alternate two sets of buffers from
 * one wait to the next), because a faster rank writes its slice as soon as its own product is done.
 * A wait that runs out sets flags[world + 2] = 1 + the missing rank and returns; the stream carries on.
 */
int macko_spmv_fp16_scatter_ex(const void *values, const void *deltas, const int32_t *row_indices,
                               int64_t rows, int64_t cols, int64_t padded_count, const void *x,
                               void *const *peer_y, int64_t row_offset, uint32_t *const *peer_flags,
                               int rank, int world, uint32_t flags, uint32_t spin_limit, void *stream);
int macko_peer_wait_limited(uint32_t *local_flags, int world, uint32_t spin_limit, void *stream);

/*
 * The exchange step alone, for hosts that overlap it with further products: rank `rank` has written rows
 * [row_offset, row_offset + rows) of y into its own full-y buffer `peer_y[rank]` with an ordinary product
 * (macko_spmv_fp16_ex with y = peer_y[rank] + row_offset); this call enqueues one small kernel that copies
 * those rows into `peer_y[p]` of every other rank, makes them visible system-wide and publishes the rank's
 * arrival counter in every rank's flag array, exactly like the tail of macko_spmv_fp16_scatter_ex with
 * MACKO_SCATTER_DEFERRED_WAIT. Enqueue it behind the product (same stream, or another stream / graph branch
 * that waits for the product), and macko_peer_wait behind all forwards before the full y is read. The
 * product kernel then has no epilogue at all and the NVLink round trip of the exchange runs beside the next
 * products. Same tables, same counters and same buffer-reuse rule as the scatter calls; calls of one rank must
 * not overlap each other (they share the rank's call counter). No counterpart in the reference.
 */
int macko_peer_forward(void *const *peer_y, int64_t row_offset, int64_t rows, uint32_t *const *peer_flags,
                       int rank, int world, void *stream);

/*
 * Decode helpers: the steps between the products of a batch-1 decode step of a Llama-architecture
 * transformer (fp16 everywhere, fp32 arithmetic inside). The reference has no such code of its own: its
 * tokens/s are measured on a Hugging Face model whose projections are swapped for MACKO layers
 * (python_scripts/util_run_pruned_llm.py:102-133, 159-207), and the model code around them is the
 * library's. All three launch with programmatic stream serialization, like the products.
 *
 * macko_decode_add_rmsnorm: x[i] += pending[0][i] + ... + pending[n_pending-1][i] (row p of `pending` starts at
 *   pending + p * pending_stride elements; fp32 sum in that order, rounded once; n_pending may be 0), then
 *   out[i] = x[i] * rsqrt(mean(x^2) + eps) * weight[i]. x is updated in place; out must not alias x. `weight`
 *   is read ahead of stream order (a parameter: it must not be written by work still in flight on `stream`).
 * macko_decode_add_rmsnorm_peer: the same with `pending` = the full-y buffer of a row-sharded product launched
 *   with MACKO_SCATTER_DEFERRED_WAIT (macko_spmv_fp16_scatter_ex): the kernel itself waits, bounded by
 *   `spin_limit` polls (0 = default), until the arrival counters of all `world` ranks in `local_flags` (this
 *   rank's flag words) have reached the rank's call counter, what macko_peer_wait does as a kernel of its own;
 *   a rank that never arrives is recorded in local_flags[world + 2] and the kernel carries on.
 * macko_decode_rope_attention: qkv = [3][heads][head_dim] (q, k, v of the new token); rotary embedding
 *   (rotate-half convention, tables [max_len][head_dim] with both halves equal) of q and k at *position
 *   (an int64 on the device, clamped into [0, max_len)), k and v stored into row *position of the caches
 *   ([heads][max_len][head_dim]), out[heads][head_dim] = softmax(q k^T / sqrt(head_dim)) v over cache rows
 *   0..*position. One CTA per head: built for the contexts of a benchmark (hundreds of positions), not for
 *   long ones. head_dim 64, 128 or 256.
 * macko_decode_silu_mul: out[i] = silu(gate_up[i]) * gate_up[n + i], i < n.
 * macko_decode_argmax: *index (an int64 on the device) = position of the largest of n fp16 values, the lowest
 *   position among equal ones; NaN never wins (greedy choice of the next token from the logits).
 */
int macko_decode_add_rmsnorm(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                             void *out, int64_t n, float eps, void *stream);
int macko_decode_add_rmsnorm_peer(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                                  void *out, int64_t n, float eps, uint32_t *local_flags, int world, uint32_t spin_limit,
                                  void *stream);
int macko_decode_rope_attention(const void *qkv, const void *cos_table, const void *sin_table, const int64_t *position,
                                void *k_cache, void *v_cache, void *out, int heads, int head_dim, int max_len, void *stream);
int macko_decode_silu_mul(const void *gate_up, void *out, int64_t n, void *stream);
int macko_decode_argmax(const void *values, int64_t n, int64_t *index, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* MACKO_B200_H_ */
