// MACKO fp16 SpMV for sm_100a.
//
// Computes what the reference kernel `macko_spmv<reuse_value_from_c>` computes
// (src/macko_spmv/cuda/kernels.cuh:34-124): y[r] = fp16(alpha * sum_k val_k * x[col_k] (+ beta*y[r]))
// with col_k = (sum of the 4-bit deltas of elements 0..k of the row) + k and fp32 accumulation.
// The design is new:
//   * a persistent grid (a fixed number of CTAs per SM); every warp owns a contiguous
//     range of rows, so each warp streams one contiguous span of `values` / `deltas`;
//   * a warp is split into 32/L groups of L lanes; each group walks one row at a time and
//     picks its next row from the warp's range as soon as it runs out of work, so rows of
//     different length inside a warp do not wait for each other;
//   * one step of a lane = 8 stored elements: one 128-bit load of values and one 32-bit load
//     of 8 deltas, both straight into registers; D steps are issued before any is consumed;
//   * the 8 column offsets of a lane are produced with byte-SIMD integer arithmetic
//     (two multiplies give the prefix sums of the even and odd nibbles), already scaled to
//     byte offsets into x; only the lane totals cross lanes (log2(L) shuffles);
//   * x lives in shared memory, framed by zero padding so that masked-out elements read
//     0 without per-element range checks; products use the fp16 x fp16 + fp32 fused
//     multiply-add of sm_100 (no conversion instructions);
//   * row boundaries that fall inside a lane's 8-element group are handled by masking the
//     group once per step, only in warps that actually contain such a lane.
#include "common.cuh"

#include <cuda_fp16.h>

namespace macko {
namespace {

constexpr int kThreads = 512;        // threads per CTA
constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kGroup = 8;            // stored elements per lane per step (128-bit value load)
constexpr int kXPadFront = 8;        // zero fp16 slots in front of x[0]   (16 bytes keeps x 16B-aligned)
constexpr int kXPadBack = 160;       // zero fp16 slots after x[cols-1]    (> 8 + 8*15 + 8)

__device__ __forceinline__ float fma_h(float acc, unsigned short a, unsigned short b)
{
    // sm_100 mixed-precision FMA: exact fp16 product added in fp32, round to nearest.
    asm("fma.rn.f32.f16 %0, %1, %2, %0;" : "+f"(acc) : "h"(a), "h"(b));
    return acc;
}

__device__ __forceinline__ uint4 ldg_stream_v4(const uint4 *p)
{
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}

__device__ __forceinline__ unsigned ldg_stream_u32(const unsigned *p)
{
    unsigned r;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}

__device__ __forceinline__ unsigned short lds_u16(unsigned addr)
{
    unsigned short r;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(r) : "r"(addr));
    return r;
}

// Zero the fp16 halves of a 128-bit group whose element index is outside [lo, hi).
__device__ __forceinline__ void mask_values(uint4 &v, int lo, int hi)
{
    unsigned *w = reinterpret_cast<unsigned *>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        unsigned m = 0;
        if (2 * j >= lo && 2 * j < hi) m |= 0x0000ffffu;
        if (2 * j + 1 >= lo && 2 * j + 1 < hi) m |= 0xffff0000u;
        w[j] &= m;
    }
}

template <int L, int D, bool XS>
__global__ void __launch_bounds__(kThreads, 2)
spmv_kernel(const uint4 *__restrict__ values, const unsigned *__restrict__ deltas,
            const int *__restrict__ ri, const __half *__restrict__ x, __half *__restrict__ y,
            int rows, int cols, float alpha, float beta)
{
    extern __shared__ __align__(16) unsigned char smem[];
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int lig = lane & (L - 1);          // lane in group
    const int group_lane0 = lane & ~(L - 1); // first lane of my group
    constexpr unsigned kLeaders = (L == 32) ? 0x1u : (L == 16) ? 0x00010001u : (L == 8) ? 0x01010101u : 0x11111111u;

    // ---- this warp's contiguous row range --------------------------------------------------
    const long long n_warps = (long long)gridDim.x * kWarpsPerCta;
    const long long warp_id = (long long)blockIdx.x * kWarpsPerCta + (tid >> 5);
    int row_next = (int)((long long)rows * warp_id / n_warps);
    const int row_hi = (int)((long long)rows * (warp_id + 1) / n_warps);

    // Window of 32 row offsets held one per lane; row r of the window is read by shuffle.
    int win_base = row_next;
    int ri_reg = 0;
    if (row_next < row_hi) ri_reg = __ldg(ri + min(win_base + lane, rows));

    // ---- stage x into shared memory ------------------------------------------------------
    unsigned xs_addr = 0;  // shared-window byte address of x[0]
    if (XS) {
        __half *xs = reinterpret_cast<__half *>(smem);
        const int n_total = kXPadFront + cols + kXPadBack;
        for (int i = tid; i < kXPadFront; i += kThreads) xs[i] = __ushort_as_half(0);
        for (int i = kXPadFront + cols + tid; i < n_total; i += kThreads) xs[i] = __ushort_as_half(0);
        if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            const uint4 *src = reinterpret_cast<const uint4 *>(x);
            uint4 *dst = reinterpret_cast<uint4 *>(xs + kXPadFront);
            const int n_vec = cols >> 3;
            for (int i = tid; i < n_vec; i += kThreads) dst[i] = __ldg(src + i);
            for (int i = (n_vec << 3) + tid; i < cols; i += kThreads) xs[kXPadFront + i] = x[i];
        } else {
            for (int i = tid; i < cols; i += kThreads) xs[kXPadFront + i] = x[i];
        }
        xs_addr = (unsigned)__cvta_generic_to_shared(xs + kXPadFront);
        __syncthreads();
    }

    // ---- per-group state -------------------------------------------------------------------
    int my_row = -1;   // row being walked by my group (-1: none)
    int begin = 0;     // first stored element of the row
    int end = 0;       // one past the last stored element
    int pos = 0;       // first element of the group's next step (multiple of 8)
    int sum2 = 0;      // 2 * (sum of deltas of the row consumed so far)
    float acc = 0.f;

    for (;;) {
        // ---- groups that ran out of work finish their row and take the next one -----------
        const bool need = pos >= end;
        const unsigned needmask = __ballot_sync(0xffffffffu, need);
        if (needmask) {
            float total = acc;
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (need) {
                if (my_row >= 0 && lig == 0) {
                    float r = alpha * total;
                    if (beta != 0.f) r += beta * __half2float(y[my_row]);
                    y[my_row] = __float2half_rn(r);
                }
                acc = 0.f;
            }
            const int avail = row_hi - row_next;
            if (avail <= 0) {
                if (needmask == 0xffffffffu) break;
                if (need) { my_row = -1; pos = 0; end = 0; begin = 0; }
            } else {
                const unsigned leaders = needmask & kLeaders;
                const int want = __popc(leaders);
                const int take = min(want, avail);
                if (row_next + take > win_base + 31) {  // warp-uniform
                    win_base = row_next;
                    ri_reg = __ldg(ri + min(win_base + lane, rows));
                }
                const int rank = __popc(leaders & ((1u << group_lane0) - 1u));
                const int nr = row_next + rank;
                const int b = __shfl_sync(0xffffffffu, ri_reg, (nr - win_base) & 31);
                const int e = __shfl_sync(0xffffffffu, ri_reg, (nr + 1 - win_base) & 31);
                if (need) {
                    if (rank < take) {
                        my_row = nr; begin = b; end = e; pos = b & ~(kGroup - 1); sum2 = 0;
                    } else {
                        my_row = -1; pos = 0; end = 0; begin = 0;
                    }
                }
                row_next += take;
            }
        }

        // ---- issue the loads of D steps -----------------------------------------------------
        uint4 v[D];
        unsigned w[D];
#pragma unroll
        for (int s = 0; s < D; ++s) {
            const int ord = pos + (s * L + lig) * kGroup;
            v[s] = make_uint4(0u, 0u, 0u, 0u);
            w[s] = 0u;
            if (ord < end) {
                v[s] = ldg_stream_v4(values + (ord >> 3));
                w[s] = ldg_stream_u32(deltas + (ord >> 3));
            }
        }

        // ---- consume them ---------------------------------------------------------------------
#pragma unroll
        for (int s = 0; s < D; ++s) {
            const int ord = pos + (s * L + lig) * kGroup;
            const int lo = begin - ord;  // elements [0, lo) of the group belong to the previous row
            const int hi = end - ord;    // elements [hi, 8) belong to the next row
            const bool partial = (hi > 0) && (lo > 0 || hi < kGroup);
            if (__any_sync(0xffffffffu, partial)) {
                if (partial) {
                    const int lo_c = max(lo, 0), hi_c = min(hi, kGroup);
                    unsigned m = 0xffffffffu << (4 * lo_c);
                    if (hi_c < kGroup) m &= ~(0xffffffffu << (4 * hi_c));
                    w[s] &= m;
                    mask_values(v[s], lo_c, hi_c);
                }
            }
            // Byte-SIMD prefix sums of the 8 deltas, scaled by 2 (byte offsets into fp16 x):
            // ce byte j = 2*(incl. prefix of element 2j)   + 2*(2j)
            // co byte j = 2*(incl. prefix of element 2j+1) + 2*(2j+1)
            const unsigned e2 = (w[s] << 1) & 0x1e1e1e1eu;
            const unsigned o2 = (w[s] >> 3) & 0x1e1e1e1eu;
            const unsigned pe = e2 * 0x01010101u;
            const unsigned po = o2 * 0x01010101u;
            const unsigned ce = pe + (po << 8) + 0x0c080400u;
            const unsigned co = pe + po + 0x0e0a0602u;
            const int tot2 = (int)((pe + po) >> 24);

            int inc = tot2;
#pragma unroll
            for (int o = 1; o < L; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, inc, o, L);
                if (lig >= o) inc += t;
            }
            const int group_tot2 = __shfl_sync(0xffffffffu, inc, L - 1, L);
            // byte offset (from x[0]) of "column -1 + element index" for element 0 of this lane
            int base2 = sum2 + (inc - tot2) + 2 * (ord - begin);
            base2 = min(max(base2, -2 * kXPadFront), 2 * cols);
            sum2 += group_tot2;

            const unsigned *vw = reinterpret_cast<const unsigned *>(&v[s]);
            if (XS) {
                const unsigned a0 = xs_addr + (unsigned)base2;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const unsigned oe = __byte_perm(ce, 0u, 0x4440u + j);
                    const unsigned oo = __byte_perm(co, 0u, 0x4440u + j);
                    const unsigned short xe = lds_u16(a0 + oe);
                    const unsigned short xo = lds_u16(a0 + oo);
                    acc = fma_h(acc, (unsigned short)(vw[j] & 0xffffu), xe);
                    acc = fma_h(acc, (unsigned short)(vw[j] >> 16), xo);
                }
            } else {
                const unsigned short *xg = reinterpret_cast<const unsigned short *>(x);
                const int cmax = cols - 1;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int ce_j = (base2 + (int)__byte_perm(ce, 0u, 0x4440u + j)) >> 1;
                    const int co_j = (base2 + (int)__byte_perm(co, 0u, 0x4440u + j)) >> 1;
                    const unsigned short xe = __ldg(xg + min(max(ce_j, 0), cmax));
                    const unsigned short xo = __ldg(xg + min(max(co_j, 0), cmax));
                    acc = fma_h(acc, (unsigned short)(vw[j] & 0xffffu), xe);
                    acc = fma_h(acc, (unsigned short)(vw[j] >> 16), xo);
                }
            }
        }
        pos += D * L * kGroup;
    }
}

template <int L, int D, bool XS>
int launch(const void *values, const void *deltas, const int32_t *ri, int rows, int cols,
           const void *x, void *y, float alpha, float beta, cudaStream_t stream,
           const DeviceInfo &dev, int ctas_per_sm)
{
    const size_t smem = XS ? (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half) : 0;
    auto kernel = spmv_kernel<L, D, XS>;
    if (smem > 48 * 1024) {
        // Idempotent and cheap; set on every call so that every device is covered.
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    int per_sm = ctas_per_sm > 0 ? ctas_per_sm : 2;
    if (smem > 0) per_sm = max(1, min(per_sm, (int)((size_t)dev.max_smem_optin / (smem + 1024))));
    // No more warps than row groups: a warp without rows would only stage x.
    const long long groups = ((long long)rows * L + 31) / 32;
    long long ctas = (long long)dev.sm_count * per_sm;
    const long long needed = (groups + kWarpsPerCta - 1) / kWarpsPerCta;
    if (needed < ctas) ctas = needed < 1 ? 1 : needed;
    kernel<<<(unsigned)ctas, kThreads, smem, stream>>>(
        static_cast<const uint4 *>(values), static_cast<const unsigned *>(deltas), ri,
        static_cast<const __half *>(x), static_cast<__half *>(y), rows, cols, alpha, beta);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "spmv launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}

template <int L, bool XS>
int launch_d(int D, const void *values, const void *deltas, const int32_t *ri, int rows, int cols,
             const void *x, void *y, float alpha, float beta, cudaStream_t stream,
             const DeviceInfo &dev, int ctas_per_sm)
{
    switch (D) {
        case 1: return launch<L, 1, XS>(values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        case 2: return launch<L, 2, XS>(values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        case 4: return launch<L, 4, XS>(values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        default: return fail(MACKO_ERR_INVALID_ARGUMENT, "steps_in_flight must be 1, 2 or 4 (got %d)", D);
    }
}

template <bool XS>
int launch_l(int L, int D, const void *values, const void *deltas, const int32_t *ri, int rows, int cols,
             const void *x, void *y, float alpha, float beta, cudaStream_t stream,
             const DeviceInfo &dev, int ctas_per_sm)
{
    switch (L) {
        case 4: return launch_d<4, XS>(D, values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        case 8: return launch_d<8, XS>(D, values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        case 16: return launch_d<16, XS>(D, values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        case 32: return launch_d<32, XS>(D, values, deltas, ri, rows, cols, x, y, alpha, beta, stream, dev, ctas_per_sm);
        default: return fail(MACKO_ERR_INVALID_ARGUMENT, "lanes_per_row must be 4, 8, 16 or 32 (got %d)", L);
    }
}

int check_args(const void *values, const void *deltas, const int32_t *ri, int64_t rows, int64_t cols,
               int64_t padded_count, const void *x, const void *y)
{
    if (rows < 0 || cols < 0 || padded_count < 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "negative size (rows=%lld cols=%lld P=%lld)",
                    (long long)rows, (long long)cols, (long long)padded_count);
    if (rows >= (1LL << 31) - 64 || cols >= (1LL << 30) || padded_count >= (1LL << 31))
        return fail(MACKO_ERR_SIZE_OVERFLOW, "rows=%lld cols=%lld P=%lld exceed 31-bit indexing",
                    (long long)rows, (long long)cols, (long long)padded_count);
    if (padded_count % 8 != 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "padded_count %lld is not a multiple of 8", (long long)padded_count);
    if (rows == 0) return MACKO_OK;
    if (!ri || !y) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices or y");
    if (cols > 0 && !x) return fail(MACKO_ERR_INVALID_ARGUMENT, "null x");
    if (padded_count > 0 && (!values || !deltas)) return fail(MACKO_ERR_INVALID_ARGUMENT, "null values or deltas");
    if (!aligned(values, 16)) return fail(MACKO_ERR_MISALIGNED, "values must be 16-byte aligned");
    if (!aligned(deltas, 4)) return fail(MACKO_ERR_MISALIGNED, "deltas must be 4-byte aligned");
    if (!aligned(ri, 4)) return fail(MACKO_ERR_MISALIGNED, "row_indices must be 4-byte aligned");
    if (!aligned(x, 2) || !aligned(y, 2)) return fail(MACKO_ERR_MISALIGNED, "x and y must be 2-byte aligned");
    return MACKO_OK;
}

}  // namespace
}  // namespace macko

extern "C" {

int macko_spmv_fp16_tuned(const void *values, const void *deltas, const int32_t *row_indices,
                          int64_t rows, int64_t cols, int64_t padded_count,
                          const void *x, void *y, float alpha, float beta, void *stream,
                          int lanes_per_row, int steps_in_flight, int x_in_shared, int ctas_per_sm)
{
    using namespace macko;
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, y);
    if (st != MACKO_OK) return st;
    if (rows == 0) return MACKO_OK;
    if (ctas_per_sm < 0) return fail(MACKO_ERR_INVALID_ARGUMENT, "ctas_per_sm must be >= 0");
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    if (x_in_shared && smem > (size_t)dev->max_smem_optin)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "x does not fit shared memory (cols=%lld)", (long long)cols);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (x_in_shared)
        return launch_l<true>(lanes_per_row, steps_in_flight, values, deltas, row_indices, (int)rows, (int)cols,
                              x, y, alpha, beta, s, *dev, ctas_per_sm);
    return launch_l<false>(lanes_per_row, steps_in_flight, values, deltas, row_indices, (int)rows, (int)cols,
                           x, y, alpha, beta, s, *dev, ctas_per_sm);
}

int macko_spmv_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, void *stream)
{
    using namespace macko;
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, y);
    if (st != MACKO_OK) return st;
    if (rows == 0) return MACKO_OK;
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;

    // Shape heuristics. Fewer lanes per row keep the x gathers of one instruction close
    // together (fewer shared-memory bank conflicts) and shorten the cross-lane scan, but
    // there must be enough row groups to fill every resident warp, and a row should fill
    // at least one step of its group.
    const long long resident_warps = (long long)dev->sm_count * 2 * kWarpsPerCta;
    const long long avg_row = padded_count / rows;
    int L = 32;
    while (L > 4 && (rows * (long long)(L / 2) / 32 >= resident_warps || avg_row <= (long long)L * kGroup / 2)) L >>= 1;
    int D = 4;
    if (avg_row <= (long long)L * kGroup * 2) D = 2;
    if (avg_row <= (long long)L * kGroup) D = 1;
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    const bool xs = smem <= (size_t)dev->max_smem_optin;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (xs)
        return launch_l<true>(L, D, values, deltas, row_indices, (int)rows, (int)cols, x, y, alpha, beta, s, *dev, 0);
    return launch_l<false>(L, D, values, deltas, row_indices, (int)rows, (int)cols, x, y, alpha, beta, s, *dev, 0);
}
}
