// The element-wise and attention steps between the matrix-vector products of a batch-1 decode step of a
// Llama-architecture transformer, as three kernels per block instead of some twenty library kernels:
//
//   add_rmsnorm      x += sum of the pending output vectors (the previous product's y, or the N partial y of a
//                    column-sharded layer), then out = rmsnorm(x) * weight
//   rope_attention   rotary embedding of q and k at position pos, k and v appended to the cache, softmax
//                    attention of q over cache rows 0..pos (one CTA per head)
//   silu_mul         out = silu(gate) * up
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
// with the rounded x, all in fp32, rounded to fp16. n_pending may be 0.
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(__half *__restrict__ x, const __half *__restrict__ pending, int n_pending, long long pending_stride,
                   const __half *__restrict__ weight, __half *__restrict__ out, int n, float eps)
{
    __shared__ float scratch[32];
    pdl_prologue();
    float sq = 0.f;
    const bool vec = (n & 7) == 0 && (pending_stride & 7) == 0 &&
                     ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(pending) |
                       reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (vec) {
        for (int c = threadIdx.x; c < (n >> 3); c += kNormThreads) {
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
    // second pass: every thread re-reads the elements it wrote itself
    if (vec) {
        for (int c = threadIdx.x; c < (n >> 3); c += kNormThreads) {
            const uint4 xv = reinterpret_cast<const uint4 *>(x)[c];
            const uint4 wv = __ldg(reinterpret_cast<const uint4 *>(weight) + c);
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

constexpr int kAttnWarps = 8;

// One CTA per head; head_dim = 32 * VPL, lane l holds dimensions l, l + 32, ... (the rotary partner of dimension d,
// d +- head_dim / 2, then sits in the same lane). qkv is [3][heads][head_dim] (q, k, v of the new token, not yet
// rotated), cos/sin tables are [max_len][head_dim] with both halves equal, caches are [heads][max_len][head_dim].
// Warp w takes cache rows w, w + 8, ... with an online softmax of its own; the eight partial results are merged
// at the end. Row pos (the new token) is taken from shared memory, not from the cache rows written here.
template <int VPL>
__global__ void __launch_bounds__(kAttnWarps * 32)
rope_attention_kernel(const __half *__restrict__ qkv, const __half *__restrict__ cos_table, const __half *__restrict__ sin_table,
                      const long long *__restrict__ pos_ptr, __half *__restrict__ k_cache, __half *__restrict__ v_cache,
                      __half *__restrict__ out, int heads, int max_len, float scale)
{
    constexpr int HD = 32 * VPL;
    __shared__ float q_s[HD], k_s[HD], v_s[HD];
    __shared__ float m_s[kAttnWarps], l_s[kAttnWarps];
    __shared__ float acc_s[kAttnWarps][HD];
    pdl_prologue();
    const int head = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    long long pos64 = *pos_ptr;
    const int pos = (int)(pos64 < 0 ? 0 : (pos64 >= max_len ? max_len - 1 : pos64));   // a position outside the cache is clamped
    if (warp == 0) {
        const __half *q = qkv + (size_t)head * HD;
        const __half *k = qkv + ((size_t)heads + head) * HD;
        const __half *v = qkv + ((size_t)2 * heads + head) * HD;
        float qf[VPL], kf[VPL];
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            qf[j] = __half2float(__ldcg(q + j * 32 + lane));
            kf[j] = __half2float(__ldcg(k + j * 32 + lane));
        }
#pragma unroll
        for (int j = 0; j < VPL; ++j) {
            const int d = j * 32 + lane;
            const float c = __half2float(__ldg(cos_table + (size_t)pos * HD + d));
            const float s = __half2float(__ldg(sin_table + (size_t)pos * HD + d));
            // rotate-half: first half pairs with -x[d + HD/2], second half with +x[d - HD/2]
            const float qr = (j < VPL / 2) ? -qf[j + VPL / 2] : qf[j - VPL / 2];
            const float kr = (j < VPL / 2) ? -kf[j + VPL / 2] : kf[j - VPL / 2];
            const __half kh = __float2half_rn(kf[j] * c + kr * s);
            const __half vh = __ldcg(v + d);
            q_s[d] = __half2float(__float2half_rn(qf[j] * c + qr * s)) * scale;
            k_s[d] = __half2float(kh);
            v_s[d] = __half2float(vh);
            k_cache[((size_t)head * max_len + pos) * HD + d] = kh;
            v_cache[((size_t)head * max_len + pos) * HD + d] = vh;
        }
    }
    __syncthreads();
    float qf[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) qf[j] = q_s[j * 32 + lane];
    float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc[j] = 0.f;
    const __half *kc = k_cache + (size_t)head * max_len * HD;
    const __half *vc = v_cache + (size_t)head * max_len * HD;
#pragma unroll 2
    for (int t = warp; t <= pos; t += kAttnWarps) {
        float kf[VPL], vf[VPL];
        if (t == pos) {
#pragma unroll
            for (int j = 0; j < VPL; ++j) { kf[j] = k_s[j * 32 + lane]; vf[j] = v_s[j * 32 + lane]; }
        } else {
#pragma unroll
            for (int j = 0; j < VPL; ++j) {
                kf[j] = __half2float(__ldcg(kc + (size_t)t * HD + j * 32 + lane));
                vf[j] = __half2float(__ldcg(vc + (size_t)t * HD + j * 32 + lane));
            }
        }
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < VPL; ++j) s += qf[j] * kf[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float m_new = fmaxf(m, s);
        const float keep = __expf(m - m_new);   // 0 on the first row (m = -inf)
        const float p = __expf(s - m_new);
        l = l * keep + p;
#pragma unroll
        for (int j = 0; j < VPL; ++j) acc[j] = acc[j] * keep + p * vf[j];
        m = m_new;
    }
    if (lane == 0) { m_s[warp] = m; l_s[warp] = l; }
#pragma unroll
    for (int j = 0; j < VPL; ++j) acc_s[warp][j * 32 + lane] = acc[j];
    __syncthreads();
    for (int d = threadIdx.x; d < HD; d += kAttnWarps * 32) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, m_s[w]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float f = (m_s[w] == -INFINITY) ? 0.f : __expf(m_s[w] - mm);
            num += f * acc_s[w][d];
            den += f * l_s[w];
        }
        out[(size_t)head * HD + d] = __float2half_rn(num / den);
    }
}

template <typename T> struct Same { using type = T; };

template <typename... Args>
int launch_pdl(const char *what, void (*kernel)(Args...), dim3 grid, dim3 block, cudaStream_t stream,
               typename Same<Args>::type... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, args...);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return MACKO_OK;
}

}  // namespace
}  // namespace macko

using namespace macko;

extern "C" {

int macko_decode_add_rmsnorm(void *x, const void *pending, int n_pending, int64_t pending_stride, const void *weight,
                             void *out, int64_t n, float eps, void *stream)
{
    if (!x || !weight || !out || n <= 0 || n > (1 << 24) || n_pending < 0 || n_pending > 64 || (n_pending > 0 && !pending) ||
        (n_pending > 0 && pending_stride < n))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "add_rmsnorm: n=%lld n_pending=%d stride=%lld or a null pointer",
                    (long long)n, n_pending, (long long)pending_stride);
    return launch_pdl("add_rmsnorm", add_rmsnorm_kernel, dim3(1), dim3(kNormThreads), static_cast<cudaStream_t>(stream),
                      static_cast<__half *>(x), static_cast<const __half *>(pending), n_pending, (long long)pending_stride,
                      static_cast<const __half *>(weight), static_cast<__half *>(out), (int)n, eps);
}

int macko_decode_silu_mul(const void *gate_up, void *out, int64_t n, void *stream)
{
    if (!gate_up || !out || n <= 0 || n > (1 << 28))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "silu_mul: n=%lld or a null pointer", (long long)n);
    const int ctas = (int)((n / 8 + 255) / 256) > 0 ? (int)((n / 8 + 255) / 256) : 1;
    return launch_pdl("silu_mul", silu_mul_kernel, dim3(ctas > 296 ? 296 : ctas), dim3(256), static_cast<cudaStream_t>(stream),
                      static_cast<const __half *>(gate_up), static_cast<__half *>(out), (int)n);
}

int macko_decode_rope_attention(const void *qkv, const void *cos_table, const void *sin_table, const int64_t *position,
                                void *k_cache, void *v_cache, void *out, int heads, int head_dim, int max_len, void *stream)
{
    if (!qkv || !cos_table || !sin_table || !position || !k_cache || !v_cache || !out || heads <= 0 || max_len <= 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "rope_attention: heads=%d max_len=%d or a null pointer", heads, max_len);
    const float scale = 1.0f / sqrtf((float)head_dim);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid((unsigned)heads), block(kAttnWarps * 32);
#define MACKO_ATTN(V)                                                                                                   \
    return launch_pdl("rope_attention", rope_attention_kernel<V>, grid, block, s, static_cast<const __half *>(qkv),      \
                      static_cast<const __half *>(cos_table), static_cast<const __half *>(sin_table),                    \
                      reinterpret_cast<const long long *>(position), static_cast<__half *>(k_cache),                     \
                      static_cast<__half *>(v_cache), static_cast<__half *>(out), heads, max_len, scale)
    switch (head_dim) {
    case 64: MACKO_ATTN(2);
    case 128: MACKO_ATTN(4);
    case 256: MACKO_ATTN(8);
    default: return fail(MACKO_ERR_INVALID_ARGUMENT, "rope_attention: head_dim %d (64, 128 and 256 are built)", head_dim);
    }
#undef MACKO_ATTN
}

}  // extern "C"
