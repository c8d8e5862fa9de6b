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


constexpr int kRowThreads = 256;   // threads of a CTA of the row kernel: 256 units (2048 stored elements) per pass

// One CTA per row; the whole dense row is assembled in shared memory (zeroed once, re-zeroed while it is
// flushed). A pass takes 256 consecutive 8-element units of the row, one per thread: the 8 column offsets of a
// unit come from byte-wise prefix sums of its deltas (as in the product kernel: byte j of `ce` / `co` is twice
// the column of element 2j / 2j+1 relative to the unit's base, and the top byte of `co` plus 2 is twice the
// columns the unit advances), the units' bases from a scan over the CTA. Stored non-zeros are written to their
// columns with 2-byte shared stores; pads and everything else stay +0. The row leaves with 16-byte stores.
// `off` = (row * cols) mod 8 slots of the buffer lie in front of the row so that aligned chunks of the buffer are
// aligned chunks of the dense matrix.
__global__ void __launch_bounds__(kRowThreads)
decompress_row_cta_kernel(const uint4 *__restrict__ values, const unsigned *__restrict__ deltas,
                          const int *__restrict__ ri, int rows, int cols, int stored,
                          unsigned short *__restrict__ dense, bool vec_ok)
{
    extern __shared__ __align__(16) unsigned short rowbuf[];   // cols + 16 slots
    __shared__ unsigned warp_total[2][kRowThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int buf_chunks = (cols + 16) >> 3;
    for (int c = tid; c < buf_chunks; c += kRowThreads) reinterpret_cast<uint4 *>(rowbuf)[c] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    const unsigned row_bytes = 2u * (unsigned)cols;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        // offsets clamped into [0, stored]: a corrupt row_indices cannot send loads outside the buffers
        const int begin = min(max(__ldg(ri + row), 0), stored);
        const int end = min(__ldg(ri + row + 1), stored);
        const long long row0 = row * (long long)cols;
        const int off = vec_ok ? (int)(row0 & 7) : 0;
        unsigned char *base = reinterpret_cast<unsigned char *>(rowbuf + off);
        // twice the column in front of the unit that holds `begin`: its leading elements belong to the row before
        int col2 = -2 * (begin & 7);
        int parity = 0;
        for (int pos = begin & ~7; pos < end; pos += kRowThreads * 8, parity ^= 1) {
            const int first = pos + tid * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            unsigned w = 0u;
            const bool active = first < end;
            if (active) {
                v = __ldg(values + (first >> 3));
                w = __ldg(deltas + (first >> 3));
                const int lo = begin - first, hi = end - first;
                if (lo > 0 || hi < 8) {   // the unit straddles an end of the row: drop what lies outside
                    const int l = min(max(lo, 0), 8), h = min(max(hi, 0), 8);
                    unsigned m = l >= 8 ? 0u : (0xffffffffu << (4 * l));
                    if (h < 8) m &= ~(0xffffffffu << (4 * h));
                    w &= m;
                    unsigned *vw = reinterpret_cast<unsigned *>(&v);
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        vw[j] &= (((m >> (8 * j)) & 1u) * 0xffffu) | (((m >> (8 * j + 4)) & 1u) * 0xffff0000u);
                }
            }
            const unsigned ev = w & 0x0f0f0f0fu, od = (w >> 4) & 0x0f0f0f0fu;
            const unsigned pe = ev * 0x02020202u + 0x0c080400u, po = od * 0x02020202u;
            const unsigned ce = po * 256u + pe, co = pe + po + 0x02020202u;
            const unsigned mine = active ? (co >> 24) + 2u : 0u;   // twice the columns this unit advances
            unsigned inc = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned u = __shfl_up_sync(0xffffffffu, inc, o);
                if (lane >= o) inc += u;
            }
            if (lane == 31) warp_total[parity][warp] = inc;
            __syncthreads();
            unsigned before = 0u, all = 0u;
#pragma unroll
            for (int k = 0; k < kRowThreads / 32; ++k) {
                const unsigned t = warp_total[parity][k];
                if (k < warp) before += t;
                all += t;
            }
            const int a0 = col2 + (int)(before + inc - mine);   // twice the unit's base column
            col2 += (int)all;
            const unsigned *vw = reinterpret_cast<const unsigned *>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const unsigned lo16 = vw[j] & 0xffffu, hi16 = vw[j] >> 16;
                const unsigned be = (unsigned)(a0 + (int)((ce >> (8 * j)) & 0xffu));
                const unsigned bo = (unsigned)(a0 + (int)((co >> (8 * j)) & 0xffu));
                // +-0 (pads, masked elements) is not stored; offsets of malformed input stay inside the row
                if ((lo16 & 0x7fffu) != 0u && be < row_bytes) *reinterpret_cast<unsigned short *>(base + be) = (unsigned short)lo16;
                if ((hi16 & 0x7fffu) != 0u && bo < row_bytes) *reinterpret_cast<unsigned short *>(base + bo) = (unsigned short)hi16;
            }
        }
        __syncthreads();
        // flush the row and leave the buffer zeroed for the next one
        const int n_chunks = (off + cols + 7) >> 3;
        unsigned short *out = dense + (row0 - off);
        for (int c = tid; c < n_chunks; c += kRowThreads) {
            const uint4 q = reinterpret_cast<const uint4 *>(rowbuf)[c];
            reinterpret_cast<uint4 *>(rowbuf)[c] = make_uint4(0u, 0u, 0u, 0u);
            const int e0 = 8 * c;
            if (vec_ok && e0 >= off && e0 + 8 <= off + cols) {
                reinterpret_cast<uint4 *>(out)[c] = q;
            } else {
                const unsigned short *qh = reinterpret_cast<const unsigned short *>(&q);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (e0 + j >= off && e0 + j < off + cols) out[e0 + j] = qh[j];
            }
        }
        __syncthreads();
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
    const size_t row_smem = ((size_t)cols + 16) * sizeof(unsigned short);
    cudaError_t e;
    if (row_smem + 1024 <= (size_t)dev->max_smem_optin) {
        // a CTA per row with the row in shared memory; as many CTAs per SM as threads and shared memory allow
        if (row_smem > 48 * 1024) {
            e = cudaFuncSetAttribute(decompress_row_cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_smem);
            if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        }
        long long per_sm = (long long)((size_t)dev->max_smem_optin / (row_smem + 1024));
        if (per_sm > 2048 / kRowThreads) per_sm = 2048 / kRowThreads;
        long long grid = (long long)dev->sm_count * per_sm;
        if (grid > rows) grid = rows;
        decompress_row_cta_kernel<<<(unsigned)grid, kRowThreads, row_smem, s>>>(
            static_cast<const uint4 *>(values), static_cast<const unsigned *>(deltas), row_indices, (int)rows, (int)cols,
            (int)padded_count, static_cast<unsigned short *>(dense), aligned(dense, 16));
    } else {
        // rows too wide for shared memory: a warp per row with a window of the row
        const int smem = kWarps * kStage * (int)sizeof(unsigned short);
        e = cudaFuncSetAttribute(decompress_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        long long grid = (rows + kWarps - 1) / kWarps;
        const long long cap = (long long)dev->sm_count * 3;   // three CTAs per SM fit by shared memory
        if (grid > cap) grid = cap;
        decompress_rows_kernel<<<(unsigned)grid, kWarps * 32, smem, s>>>(
            static_cast<const uint4 *>(values), static_cast<const unsigned *>(deltas), row_indices, (int)rows, (int)cols,
            (int)padded_count, static_cast<unsigned short *>(dense), aligned(dense, 16));
    }
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "decompress launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}
