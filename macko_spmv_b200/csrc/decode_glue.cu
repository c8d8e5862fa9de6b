// The element-wise and attention steps between the matrix-vector products of a batch-1 decode step of a
// Llama-architecture transformer, as three kernels per block instead of some twenty library kernels (plus one per token):
//
//   add_rmsnorm      x += sum of the pending output vectors (the previous product's y, or the N partial y of a
//                    column-sharded layer), then out = rmsnorm(x) * weight
//   rope_attention   rotary embedding of q and k at position pos, k and v appended to the cache, softmax
//                    attention of q over cache rows 0..pos (one CTA per head)
//   silu_mul         out = silu(gate) * up
//   argmax           the greedy choice of the next token from the fp16 logits
//
// The reference measures tokens/s of a Hugging Face model whose projections are swapped for MACKO layers
// (python_scripts/util_run_pruned_llm.py:102-133, 159-207); the model code around the projections is the
// library's there. These kernels are that surrounding code for the decode loop of this package, so that a
// token costs eight launches per block. All of them launch with programmatic stream serialization: they
// signal their dependents at once and wait for their producer before they touch memory, so the next product
// kernel's early matrix loads run under them.
#include <cuda_fp16.h>

#include "common.cuh"

namespace macko {
namespace {

constexpr int kNormThreads = 512;

__device__ __forceinline__ void pdl_prologue()
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float block_sum(float v, float *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int n_warps = blockDim.x >> 5;
    float t = lane < n_warps ? scratch[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// One CTA. x (fp16, n elements) is the residual stream: x[i] <- x[i] + pending[0][i] + pending[1][i] + ...
// (fp32 sum in that order, rounded to fp16 once), then out[i] = x[i] * rsqrt(mean(x^2) + eps) * weight[i]
// with the rounded x, all in fp32, rounded to fp16. n_pending may be 0. The weight (a parameter, not the output
// of the kernel in front) is fetched before the wait for that kernel; a thread keeps its first eight elements
// in registers between the two passes (all of them when n <= 4096). With `peer_flags` the kernel first waits
// (bounded) for the slices of the other ranks in `pending`.
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(__half *__restrict__ x, const __half *__restrict__ pending, int n_pending, long long pending_stride,
                   const __half *__restrict__ weight, __half *__restrict__ out, int n, float eps,
                   unsigned *__restrict__ peer_flags, int world, unsigned spin_limit)
{
    __shared__ float scratch[32];
    const bool vec = (n & 7) == 0 && (pending_stride & 7) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(pending) |
                       reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    const int n_vec = vec ? n >> 3 : 0;
    asm volatile("griddepcontrol.launch_dependents;");
    uint4 w_first = make_uint4(0u, 0u, 0u, 0u);
    if ((int)threadIdx.x < n_vec) w_first = __ldg(reinterpret_cast<const uint4 *>(weight) + threadIdx.x);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (peer_flags != nullptr) {
        // `pending` is the exchange buffer of a row-sharded product launched with a deferred wait: the slices of
        // the other ranks are complete once their arrival counters have reached this rank's call counter (what
        // macko_peer_wait checks as a kernel of its own). Bounded: a rank that never arrives is recorded in
        // flags[world + 2] and the kernel carries on with what is there.
        if ((int)threadIdx.x < world) {
            const unsigned seq = peer_flags[world];
            unsigned seen = 0u;
            bool arrived = false;
            for (unsigned spin = 0; spin < spin_limit; ++spin) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(peer_flags + threadIdx.x) : "memory");
                if ((int)(seen - seq) >= 0) { arrived = true; break; }
            }
            if (!arrived) peer_flags[world + 2] = 1u + threadIdx.x;
        }
        __syncthreads();
    }
    float sq = 0.f;
    uint4 x_first = make_uint4(0u, 0u, 0u, 0u);
    if (vec) {
        for (int c = threadIdx.x; c < n_vec; c += kNormThreads) {
            uint4 xv = reinterpret_cast<const uint4 *>(x)[c];
            __half2 *xh = reinterpret_cast<__half2 *>(&xv);
            float f[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __half22float2(xh[j]);
                f[2 * j] = t.x;
                f[2 * j + 1] = t.y;
            }
            for (int p = 0; p < n_pending; ++p) {
                uint4 pv = __ldcg(reinterpret_cast<const uint4 *>(pending + (size_t)p * pending_stride) + c);
                const __half2 *ph = reinterpret_cast<const __half2 *>(&pv);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 t = __half22float2(ph[j]);
                    f[2 * j] += t.x;
                    f[2 * j + 1] += t.y;
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                xh[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
                const float2 t = __half22float2(xh[j]);
                sq += t.x * t.x + t.y * t.y;
            }
            if (n_pending > 0) reinterpret_cast<uint4 *>(x)[c] = xv;
            if (c == (int)threadIdx.x) x_first = xv;
        }
    } else {
        for (int i = threadIdx.x; i < n; i += kNormThreads) {
            float f = __half2float(x[i]);
            for (int p = 0; p < n_pending; ++p) f += __half2float(__ldcg(pending + (size_t)p * pending_stride + i));
            const __half h = __float2half_rn(f);
            if (n_pending > 0) x[i] = h;
            const float r = __half2float(h);
            sq += r * r;
        }
    }
    const float total = block_sum(sq, scratch);
    const float rstd = rsqrtf(total / (float)n + eps);
    // second pass: every thread handles the elements it wrote itself
    if (vec) {
        for (int c = threadIdx.x; c < n_vec; c += kNormThreads) {
            const bool first = c == (int)threadIdx.x;
            const uint4 xv = first ? x_first : reinterpret_cast<const uint4 *>(x)[c];
            const uint4 wv = first ? w_first : __ldg(reinterpret_cast<const uint4 *>(weight) + c);
            const __half2 *xh = reinterpret_cast<const __half2 *>(&xv);
            const __half2 *wh = reinterpret_cast<const __half2 *>(&wv);
            uint4 ov;
            __half2 *oh = reinterpret_cast<__half2 *>(&ov);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 a = __half22float2(xh[j]), w = __half22float2(wh[j]);
                oh[j] = __floats2half2_rn(a.x * rstd * w.x, a.y * rstd * w.y);
            }
            reinterpret_cast<uint4 *>(out)[c] = ov;
        }
    } else {
        for (int i = threadIdx.x; i < n; i += kNormThreads)
            out[i] = __float2half_rn(__half2float(x[i]) * rstd * __half2float(weight[i]));
    }
}

// out[i] = silu(gu[i]) * gu[n + i], fp32 arithmetic, rounded once.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half *__restrict__ gu, __half *__restrict__ out, int n)
{
    pdl_prologue();
    const int stride = gridDim.x * blockDim.x;
    const bool vec = (n & 7) == 0 && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (vec) {
        for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < (n >> 3); c += stride) {
            const uint4 gv = __ldcg(reinterpret_cast<const uint4 *>(gu) + c);
            const uint4 uv = __ldcg(reinterpret_cast<const uint4 *>(gu + n) + c);
            const __half2 *gh = reinterpret_cast<const __half2 *>(&gv);
            const __half2 *uh = reinterpret_cast<const __half2 *>(&uv);
            uint4 ov;
            __half2 *oh = reinterpret_cast<__half2 *>(&ov);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 g = __half22float2(gh[j]), u = __half22float2(uh[j]);
                oh[j] = __floats2half2_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
            }
            reinterpret_cast<uint4 *>(out)[c] = ov;
        }
    } else {
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
            const float g = __half2float(__ldcg(gu + i)), u = __half2float(__ldcg(gu + n + i));
            out[i] = __float2half_rn(g / (1.f + __expf(-g)) * u);
        }
    }
}

// Index of the largest of n fp16 values (the lowest index among equal ones; NaN never wins), as one int64: the
// greedy choice of the next token. One CTA.
__global__ void __launch_bounds__(1024)
argmax_kernel(const __half *__restrict__ v, int n, long long *__restrict__ out)
{
    __shared__ float best_s[32];
    __shared__ int idx_s[32];
    pdl_prologue();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    if ((n & 7) == 0 && (reinterpret_cast<uintptr_t>(v) & 15) == 0) {
        for (int c = threadIdx.x; c < (n >> 3); c += 1024) {
            const uint4 raw = __ldcg(reinterpret_cast<const uint4 *>(v) + c);
            const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 t = __half22float2(h[j]);
                if (t.x > best) { best = t.x; idx = 8 * c + 2 * j; }
                if (t.y > best) { best = t.y; idx = 8 * c + 2 * j + 1; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < n; i += 1024) {
            const float t = __half2float(__ldcg(v + i));
            if (t > best) { best = t; idx = i; }
        }
    }
    auto merge = [&](float ob, int oi) {
        if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { best_s[warp] = best; idx_s[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = best_s[lane];
        idx = idx_s[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
        if (lane == 0) *out = idx == 0x7fffffff ? 0 : idx;   // all -inf or NaN: index 0
    }
}

constexpr int kAttnWarps = 8;

// VPL consecutive fp16 values as one load or store (4, 8 or 16 bytes).
template <int VPL> struct HalfVec;
template <> struct HalfVec<2> { using type = unsigned; };
template <> struct HalfVec<4> { using type = uint2; };
template <> struct HalfVec<8> { using type = uint4; };

template <int VPL>
__device__ __forceinline__ void unpack_halfs(const typename HalfVec<VPL>::type &raw, float (&f)[VPL])
{
    const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
    for (int j = 0; j < VPL / 2; ++j) {
        const float2 t = __half22float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
    }
}

template <int VPL>
__device__ __forceinline__ typename HalfVec<VPL>::type pack_halfs(const float (&f)[VPL])
{
    typename HalfVec<VPL>::type raw;
    __half2 *h = reinterpret_cast<__half2 *>(&raw);
#pragma unroll
    for (int j = 0; j < VPL / 2; ++j) h[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
    return raw;
}

__device__ __forceinline__ float ld_cluster_f32(const float *local, unsigned cta_rank)
{
    // the same shared-memory variable in the CTA `cta_rank` of this cluster
    unsigned addr = (unsigned)__cvta_generic_to_shared(local), remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(cta_rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// One thread-block cluster per head (1, 2, 4 or 8 CTAs, by how many heads there are: the cluster's CTAs have
// consecutive blockIdx.x); head_dim = 32 * VPL, lane l holds dimensions VPL*l .. VPL*l + VPL - 1, so a cache row
// is one vector load per lane and the rotary partner of a dimension, head_dim / 2 away, sits 16 lanes away.
// qkv is [3][heads][head_dim] (q, k, v of the new token, not yet rotated), the cos/sin tables are
// [max_len][head_dim] with both halves equal, the caches are [heads][max_len][head_dim]. Every CTA rotates q and
// k for itself; the first one of the cluster stores k and v into cache row pos. The warps of the cluster take
// cache rows round robin, four rows per iteration with all loads issued first, each warp with an online softmax
// of its own (row pos, the new token, comes from shared memory, not from the cache row written here); the warps
// of a CTA are merged through shared memory, the CTAs of the cluster through distributed shared memory by the
// first CTA. Every thread of every CTA reaches both cluster barriers: there is no early exit.
template <int VPL>
__global__ void __launch_bounds__(kAttnWarps * 32, 1)
rope_attention_kernel(const __half *__restrict__ qkv, const __half *__restrict__ cos_table, const __half *__restrict__ sin_table,
                      const long long *__restrict__ pos_ptr, __half *__restrict__ k_cache, __half *__restrict__ v_cache,
                      __half *__restrict__ out, int heads, int max_len, float scale)
{
    constexpr int HD = 32 * VPL;
    constexpr int U = VPL >= 8 ? 2 : 4;   // cache rows in flight per warp
    using Vec = typename HalfVec<VPL>::type;
    __shared__ __align__(16) float q_s[HD], k_s[HD], v_s[HD];
    __shared__ float m_s[kAttnWarps], l_s[kAttnWarps];
    __shared__ __align__(16) float acc_s[kAttnWarps][HD];
    __shared__ float part_acc[HD], part_ml[2];   // this CTA's merged partial result, read by the cluster's first CTA
    pdl_prologue();
    unsigned crank, csize;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(crank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(csize));
    const int head = blockIdx.x / csize, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long pos64 = *pos_ptr;
    const int pos = (int)(pos64 < 0 ? 0 : (pos64 >= max_len ? max_len - 1 : pos64));   // a position outside the cache is clamped
    if (warp == 0) {
        const size_t at = (size_t)head * HD + VPL * lane;
        float qf[VPL], kf[VPL], vf[VPL], cf[VPL], sf[VPL];
        unpack_halfs<VPL>(__ldcg(reinterpret_cast<const Vec *>(qkv + at)), qf);
        unpack_halfs<VPL>(__ldcg(reinterpret_cast<const Vec *>(qkv + (size_t)heads * HD + at)), kf);
        const Vec vraw = __ldcg(reinterpret_cast<const Vec *>(qkv + (size_t)2 * heads * HD + at));
        unpack_halfs<VPL>(vraw, vf);
        unpack_halfs<VPL>(__ldg(reinterpret_cast<const Vec *>(cos_table + (size_t)pos * HD + VPL * lane)), cf);
        unpack_halfs<VPL>(__ldg(reinterpret_cast<const Vec *>(sin_table + (size_t)pos * HD + VPL * lane)), sf);
        float kr[VPL];
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            // rotate-half: the first half of the head pairs with -x[d + HD/2], the second with +x[d - HD/2]
            const float qp = __shfl_xor_sync(0xffffffffu, qf[j], 16), kp = __shfl_xor_sync(0xffffffffu, kf[j], 16);
            const float sign = lane < 16 ? -1.f : 1.f;
            kr[j] = __half2float(__float2half_rn(kf[j] * cf[j] + sign * kp * sf[j]));
            q_s[VPL * lane + j] = __half2float(__float2half_rn(qf[j] * cf[j] + sign * qp * sf[j])) * scale;
            k_s[VPL * lane + j] = kr[j];
            v_s[VPL * lane + j] = vf[j];
        }
        if (crank == 0) {
            const size_t row = ((size_t)head * max_len + pos) * HD + VPL * lane;
            *reinterpret_cast<Vec *>(k_cache + row) = pack_halfs<VPL>(kr);
            *reinterpret_cast<Vec *>(v_cache + row) = vraw;
        }
    }
    __syncthreads();
    float qf[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) qf[j] = q_s[VPL * lane + j];
    float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
    const __half *kc = k_cache + (size_t)head * max_len * HD + VPL * lane;
    const __half *vc = v_cache + (size_t)head * max_len * HD + VPL * lane;
    const int gw = (int)crank * kAttnWarps + warp, n_gw = (int)csize * kAttnWarps;
    for (int t0 = gw; t0 <= pos; t0 += U * n_gw) {
        Vec kraw[U], vraw[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = t0 + u * n_gw;
            if (t < pos) {
                kraw[u] = __ldcg(reinterpret_cast<const Vec *>(kc + (size_t)t * HD));
                vraw[u] = __ldcg(reinterpret_cast<const Vec *>(vc + (size_t)t * HD));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int t = t0 + u * n_gw;
            if (t > pos) break;   // warp-uniform
            float kf[VPL], vf[VPL];
            if (t == pos) {
#pragma unroll
                for (int j = 0; j < VPL; ++j) { kf[j] = k_s[VPL * lane + j]; vf[j] = v_s[VPL * lane + j]; }
            } else {
                unpack_halfs<VPL>(kraw[u], kf);
                unpack_halfs<VPL>(vraw[u], vf);
            }
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < VPL; ++j) s += qf[j] * kf[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            const float m_new = fmaxf(m, s);
            const float keep = __expf(m - m_new);   // 0 on a warp's first row (m = -inf)
            const float p = __expf(s - m_new);
            l = l * keep + p;
#pragma unroll
            for (int j = 0; j < VPL; ++j) acc[j] = acc[j] * keep + p * vf[j];
            m = m_new;
        }
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc_s[warp][VPL * lane + j] = acc[j];
    __syncthreads();
    // the CTA's partial result, not normalised: sum_w e^(m_w - M) acc_w, M, sum_w e^(m_w - M) l_w (a CTA
    // without rows leaves M = -inf and zeros)
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w]);
    for (int d = threadIdx.x; d < HD; d += kAttnWarps * 32) {
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float f = (m_s[w] == -INFINITY) ? 0.f : __expf(m_s[w] - mm);
            num += f * acc_s[w][d];
            den += f * l_s[w];
        }
        part_acc[d] = num;
        if (d == 0) { part_ml[0] = mm; part_ml[1] = den; }
    }
    if (csize > 1) cluster_barrier(); else __syncthreads();
    if (crank == 0) {
        for (int d = threadIdx.x; d < HD; d += kAttnWarps * 32) {
            float big = -INFINITY;
            for (unsigned r = 0; r < csize; ++r) big = fmaxf(big, csize > 1 ? ld_cluster_f32(&part_ml[0], r) : part_ml[0]);
            float num = 0.f, den = 0.f;
            for (unsigned r = 0; r < csize; ++r) {
                const float mr = csize > 1 ? ld_cluster_f32(&part_ml[0], r) : part_ml[0];
                const float f = (mr == -INFINITY) ? 0.f : __expf(mr - big);
                num += f * (csize > 1 ? ld_cluster_f32(&part_acc[d], r) : part_acc[d]);
                den += f * (csize > 1 ? ld_cluster_f32(&part_ml[1], r) : part_ml[1]);
            }
            out[(size_t)head * HD + d] = __float2half_rn(num / den);
        }
    }
    if (csize > 1) cluster_barrier();   // the other CTAs' shared memory stays until the first one has read it
}

template <typename T> struct Same { using type = T; };

// `cluster` > 1: thread-block clusters of that many CTAs along x (the grid is a multiple of it).
template <typename... Args>
int launch_pdl(const char *what, void (*kernel)(Args...), dim3 grid, dim3 block, int cluster, cudaStream_t stream,
               typename Same<Args>::type... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = cluster > 1 ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return MACKO_OK;
}

}  // namespace
}  // namespace macko

using namespace macko;

extern "C" {

static int add_rmsnorm_checked(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                               void *out, int64_t n, float eps, uint32_t *peer_flags, int world, uint32_t spin_limit,
                               void *stream)
{
    if (!x || !weight || !out || n <= 0 || n > (1 << 24) || n_pending < 0 || n_pending > 64 || (n_pending > 0 && !pending) ||
        (n_pending > 0 && pending_stride < n))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "add_rmsnorm: n=%lld n_pending=%d stride=%lld or a null pointer",
                    (long long)n, n_pending, (long long)pending_stride);
    return launch_pdl("add_rmsnorm", add_rmsnorm_kernel, dim3(1), dim3(kNormThreads), 1, static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(x), static_cast<const __half *>(pending), n_pending, (long long)pending_stride,
                      static_cast<const __half *>(weight), static_cast<__half *>(out), (int)n, eps,
                      reinterpret_cast<unsigned *>(peer_flags), world, (unsigned)(spin_limit == 0 ? (1u << 23) : spin_limit));
}

int macko_decode_add_rmsnorm(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                             void *out, int64_t n, float eps, void *stream)
{
    return add_rmsnorm_checked(x, pending, n_pending, pending_stride, weight, out, n, eps, nullptr, 0, 0, stream);
}

int macko_decode_add_rmsnorm_peer(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                                  void *out, int64_t n, float eps, uint32_t *local_flags, int world, uint32_t spin_limit,
                                  void *stream)
{
    if (!local_flags || world < 1 || world > 8 || !aligned(local_flags, 4))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "add_rmsnorm_peer: null or misaligned flags, or world %d outside 1..8", world);
    return add_rmsnorm_checked(x, pending, n_pending, pending_stride, weight, out, n, eps, local_flags, world, spin_limit, stream);
}

int macko_decode_silu_mul(const void *gate_up, void *out, int64_t n, void *stream)
{
    if (!gate_up || !out || n <= 0 || n > (1 << 28))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "silu_mul: n=%lld or a null pointer", (long long)n);
    const int ctas = (int)((n / 8 + 255) / 256) > 0 ? (int)((n / 8 + 255) / 256) : 1;
    return launch_pdl("silu_mul", silu_mul_kernel, dim3(ctas > 296 ? 296 : ctas), dim3(256), 1, static_cast<cudaStream_t>(stream),
                      static_cast<const __half *>(gate_up), static_cast<__half *>(out), (int)n);
}

int macko_decode_argmax(const void *values, int64_t n, int64_t *index, void *stream)
{
    if (!values || !index || n <= 0 || n > (1 << 30))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "argmax: n=%lld or a null pointer", (long long)n);
    return launch_pdl("argmax", argmax_kernel, dim3(1), dim3(1024), 1, static_cast<cudaStream_t>(stream),
                      static_cast<const __half *>(values), (int)n, reinterpret_cast<long long *>(index));
}

int macko_decode_rope_attention(const void *qkv, const void *cos_table, const void *sin_table, const int64_t *position,
                                void *k_cache, void *v_cache, void *out, int heads, int head_dim, int max_len, void *stream)
{
    if (!qkv || !cos_table || !sin_table || !position || !k_cache || !v_cache || !out || heads <= 0 || max_len <= 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "rope_attention: heads=%d max_len=%d or a null pointer", heads, max_len);
    if (head_dim != 64 && head_dim != 128 && head_dim != 256)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "rope_attention: head_dim %d (64, 128 and 256 are built)", head_dim);
    const void *ptrs[] = {qkv, cos_table, sin_table, k_cache, v_cache};
    for (const void *p : ptrs)
        if (!aligned(p, 16)) return fail(MACKO_ERR_MISALIGNED, "rope_attention: qkv, the tables and the caches must be 16-byte aligned");
    const float scale = 1.0f / sqrtf((float)head_dim);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // as many CTAs per head as keeps the grid within about one CTA per SM (clusters of up to 8 are portable)
    const DeviceInfo *dev = nullptr;
    if (int st = current_device_info(&dev)) return st;
    int cluster = 8;
    while (cluster > 1 && (long long)heads * cluster > dev->sm_count) cluster >>= 1;
    const dim3 grid((unsigned)(heads * cluster)), block(kAttnWarps * 32);
#define MACKO_ATTN(V)                                                                                                   \
    return launch_pdl("rope_attention", rope_attention_kernel<V>, grid, block, cluster, s, static_cast<const __half *>(qkv), \
                      static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table),                    \
                      reinterpret_cast<const long long *>(position), static_cast<__half *>(k_cache),                     \
                      static_cast<__half *>(v_cache), static_cast<__half *>(out), heads, max_len, scale)
    switch (head_dim) {
    case 64: MACKO_ATTN(2);
    case 128: MACKO_ATTN(4);
    default: MACKO_ATTN(8);
    }
#undef MACKO_ATTN
}

}  // extern "C"
