// MACKO -> dense fp16 on the GPU.
//
// The reference has no decompressor; a dense copy is what a product with many right-hand sides wants
// (a tensor-core GEMM on the dense matrix beats streaming the compressed matrix once per few vectors),
// and it is the inverse used to check the compressor. Semantics follow the format as the reference SpMV
// reads it (src/macko_spmv/cuda/kernels.cuh:86-108): element k of a row sits at column
// (sum of the deltas of elements 0..k) + k; stored non-zeros are written with their stored bits and
// everything else (pads included, whatever their sign bit) is +0.
#include "common.cuh"

namespace macko {
namespace {

constexpr int kWarps = 8;        // warps (rows in flight) per CTA
// A step decodes 256 stored elements; consecutive stored elements are at most 16 columns apart, so the
// columns a step covers (from the end of the previous step) fit 15 + 256 * 16 slots; 7 more for alignment.
constexpr int kStage = 4128;     // fp16 slots of a warp's staging buffer (a multiple of 8)

// dense[g0 .. g0 + n) = stage[off .. off + n) with 16-byte stores wherever source and destination allow.
// `stage` index 0 corresponds to global index g0 - off, which is a multiple of 8, so aligned 8-element
// chunks of the destination are aligned chunks of the buffer. src == nullptr writes zeros.
__device__ __forceinline__ void flush_span(unsigned short *__restrict__ dense, long long g0, int n, const unsigned short *src,
                                           int off, bool vec_ok, int lane)
{
    if (n <= 0) return;
    int head = vec_ok ? min(n, (8 - off) & 7) : n;   // elements before the first aligned chunk
    for (int i = lane; i < head; i += 32) dense[g0 + i] = src ? src[off + i] : (unsigned short)0;
    if (!vec_ok) return;
    const int chunks = (n - head) >> 3;
    uint4 *dst = reinterpret_cast<uint4 *>(dense + g0 + head);
    const uint4 *s4 = src ? reinterpret_cast<const uint4 *>(src + off + head) : nullptr;
    for (int c = lane; c < chunks; c += 32) dst[c] = s4 ? s4[c] : make_uint4(0u, 0u, 0u, 0u);
    const int done = head + (chunks << 3);
    for (int i = done + lane; i < n; i += 32) dense[g0 + i] = src ? src[off + i] : (unsigned short)0;
}

// One warp per row. Each step's columns are assembled in the warp's shared-memory buffer (zeros, then the
// stored elements scattered to their columns) and written out with coalesced 16-byte stores, so the dense
// matrix is written exactly once and no separate clearing pass is needed.
__global__ void __launch_bounds__(kWarps * 32)
decompress_rows_kernel(const uint4 *__restrict__ values, const unsigned *__restrict__ deltas,
                       const int *__restrict__ ri, int rows, int cols, int stored,
                       unsigned short *__restrict__ dense, bool vec_ok)
{
    extern __shared__ __align__(16) unsigned short stage_all[];
    const int lane = threadIdx.x & 31;
    unsigned short *stage = stage_all + (threadIdx.x >> 5) * kStage;
    const long long n_warps = (long long)gridDim.x * kWarps;
    for (long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5); row < rows; row += n_warps) {
        // offsets clamped into [0, stored]: a corrupt row_indices cannot send loads outside the buffers
        const int begin = min(max(__ldg(ri + row), 0), stored);
        const int end = min(__ldg(ri + row + 1), stored);
        const long long row0 = row * (long long)cols;
        int col_base = 0;   // (sum of deltas) + (number of elements) of the row before this step
        int written = 0;    // columns of the row already written
        for (int pos = begin & ~7; pos < end && written < cols; pos += 256) {
            const int first = pos + lane * 8;   // first element of the lane's unit
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            unsigned w = 0u;
            if (first < end) {
                v = __ldg(values + (first >> 3));
                w = __ldg(deltas + (first >> 3));
            }
            const unsigned short *vh = reinterpret_cast<const unsigned short *>(&v);
            // columns relative to the lane's start: inclusive delta prefix + index, for elements inside the row
            int rel[8];
            int sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const bool inside = first + j >= begin && first + j < end;
                if (inside) sum += (int)((w >> (4 * j)) & 15u) + 1;
                rel[j] = inside ? sum - 1 : -1;
            }
            int inc = sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int u = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += u;
            }
            const int lane_base = col_base + inc - sum;
            col_base += __shfl_sync(0xffffffffu, inc, 31);
            // this step delivers columns [written, step_end): the gap since the last step, then its elements
            const int step_end = min(col_base, cols);
            const int n = step_end - written;
            if (n <= 0 || n > kStage - 8) continue;   // nothing new, or deltas that no compressor can produce
            const long long g0 = row0 + written;
            const int off = (int)(g0 & 7);
            uint4 *z = reinterpret_cast<uint4 *>(stage);
            for (int c = lane; c < (off + n + 7) >> 3; c += 32) z[c] = make_uint4(0u, 0u, 0u, 0u);
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int col = lane_base + rel[j];
                if (rel[j] >= 0 && col >= written && col < step_end && (vh[j] & 0x7fffu) != 0u) stage[off + col - written] = vh[j];
            }
            __syncwarp();
            flush_span(dense, g0, n, stage, off, vec_ok, lane);
            __syncwarp();
            written = step_end;
        }
        flush_span(dense, row0 + written, cols - written, nullptr, (int)((row0 + written) & 7), vec_ok, lane);   // zeros behind the last stored element
    }
}

}  // namespace
}  // namespace macko

extern "C" int macko_decompress_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                                     int64_t rows, int64_t cols, int64_t padded_count, void *dense, void *stream)
{
    using namespace macko;
    if (rows < 0 || cols < 0 || padded_count < 0 || padded_count % 8 != 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "bad sizes (rows=%lld cols=%lld P=%lld)", (long long)rows,
                    (long long)cols, (long long)padded_count);
    if (rows >= (1LL << 31) - 64 || cols >= (1LL << 30) || padded_count >= (1LL << 31))
        return fail(MACKO_ERR_SIZE_OVERFLOW, "rows=%lld cols=%lld P=%lld exceed 31-bit indexing", (long long)rows,
                    (long long)cols, (long long)padded_count);
    if (rows == 0 || cols == 0) return MACKO_OK;
    if (!row_indices || !dense) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices or dense");
    if (padded_count > 0 && (!values || !deltas)) return fail(MACKO_ERR_INVALID_ARGUMENT, "null values or deltas");
    if (!aligned(values, 16) || !aligned(deltas, 4) || !aligned(row_indices, 4) || !aligned(dense, 2))
        return fail(MACKO_ERR_MISALIGNED, "values need 16-, deltas and row_indices 4-, dense 2-byte alignment");
    const DeviceInfo *dev = nullptr;
    int st = current_device_info(&dev);
    if (st != MACKO_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int smem = kWarps * kStage * (int)sizeof(unsigned short);
    cudaError_t e = cudaFuncSetAttribute(decompress_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    long long grid = (rows + kWarps - 1) / kWarps;
    const long long cap = (long long)dev->sm_count * 3;   // three CTAs per SM fit by shared memory
    if (grid > cap) grid = cap;
    decompress_rows_kernel<<<(unsigned)grid, kWarps * 32, smem, s>>>(
        static_cast<const uint4 *>(values), static_cast<const unsigned *>(deltas), row_indices, (int)rows, (int)cols,
        (int)padded_count, static_cast<unsigned short *>(dense), aligned(dense, 16));
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "decompress launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}
