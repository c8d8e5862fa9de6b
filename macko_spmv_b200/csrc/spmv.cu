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
//   * one unit of a lane = 8 stored elements: one 128-bit load of values and one 32-bit load
//     of 8 deltas, both straight into registers; 2, 4 or 6 units per lane are issued before any
//     is consumed, and the phases of the computation run over all of them (loads, prefix sums,
//     scans, gathers) so that independent work hides shuffle and shared-memory latency;
//   * the 8 column offsets of a unit are produced with byte-SIMD integer arithmetic
//     (two multiplies give the prefix sums of the even and odd nibbles), already scaled to
//     byte offsets into x; only lane totals cross lanes, two units per shuffle;
//   * the kernel is bound by instruction issue on the half-rate integer pipe and by shared-memory
//     wavefronts, not by HBM, so per element it spends three instructions and none on that pipe:
//     a dot-product instruction forms the address, one 16-bit shared load gathers x from a
//     zero-framed copy (masked-out elements read 0 without range checks), and the sm_100
//     fp16 x fp16 + fp32 fused multiply-add needs no conversions;
//   * row boundaries that fall inside a unit are handled by masking that unit, only in warps
//     that actually contain such a unit (one warp-wide reduction per iteration finds them);
//   * the first matrix loads of every warp are in flight before x is staged, and, when the caller
//     declares the matrix immutable, before the kernel waits for the previous kernel of the stream
//     (programmatic dependent launch), so the first HBM round trip overlaps that kernel's tail;
//   * a planned launch walks "virtual rows" (rows cut into segments of bounded length, sorted by
//     length and dealt to the warps in serpentine order) from side metadata built once per matrix,
//     which balances matrices with very uneven rows; the compressed buffers stay untouched.
#include "common.cuh"
#include "plan.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <type_traits>

namespace macko {
namespace {

constexpr int kThreads = 512;        // threads per CTA
constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kGroup = 8;            // stored elements per lane per sub-step (one 128-bit value load)
constexpr int kXPadFront = 32;       // zero fp16 slots in front of x[0] (64 bytes: keeps x 16B-aligned)
constexpr int kXPadBack = 160;       // zero fp16 slots after x[cols-1]  (> 8 * 16 + 8)

// acc += fp16(low or high half of vword) * fp16(low half of xbits): the sm_100 mixed-precision FMA
// (exact fp16 product accumulated in fp32, round to nearest); the halves are split inside the asm so
// that no repacking instructions are needed around it.
// Value types of the stored elements (x and y follow: fp16 for fp16 and int8 values, bf16 for bf16 values)
constexpr int kF16 = 0, kBF16 = 1, kI8 = 2;

template <int HALF, int VT = kF16>
__device__ __forceinline__ float fma_h(float acc, unsigned vword, unsigned xbits)
{
    if (VT == kBF16) {
        if (HALF)
            asm("{.reg .b16 l,h,xl,xh; mov.b32 {l,h}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.bf16 %0, h, xl, %0;}"
                : "+f"(acc) : "r"(vword), "r"(xbits));
        else
            asm("{.reg .b16 l,h,xl,xh; mov.b32 {l,h}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.bf16 %0, l, xl, %0;}"
                : "+f"(acc) : "r"(vword), "r"(xbits));
    } else {
        if (HALF)
            asm("{.reg .b16 l,h,xl,xh; mov.b32 {l,h}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, h, xl, %0;}"
                : "+f"(acc) : "r"(vword), "r"(xbits));
        else
            asm("{.reg .b16 l,h,xl,xh; mov.b32 {l,h}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, l, xl, %0;}"
                : "+f"(acc) : "r"(vword), "r"(xbits));
    }
    return acc;
}

// 16-bit storage type <-> fp32 for the y epilogue (fp16 or bf16 bits in an unsigned short)
template <int VT>
__device__ __forceinline__ unsigned short to_bits16(float f)
{
    if (VT == kBF16) return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    return __half_as_ushort(__float2half_rn(f));
}
template <int VT>
__device__ __forceinline__ float from_bits16(unsigned short b)
{
    if (VT == kBF16) return __bfloat162float(__ushort_as_bfloat16(b));
    return __half2float(__ushort_as_half(b));
}

// Four signed bytes -> their exact fp16 values, as two f16x2 words (elements 0,1 and 2,3): flip the sign bit
// (byte + 128 as an unsigned byte), put every byte under the exponent of 1024.0 (0x64xx = 1024 + byte) and
// subtract 1152.0: one permute and one packed subtraction per pair.
__device__ __forceinline__ void bytes_to_f16x2(unsigned w, unsigned &lo, unsigned &hi)
{
    const unsigned u = w ^ 0x80808080u;
    unsigned a = __byte_perm(u, 0x64646464u, 0x4140);
    unsigned b = __byte_perm(u, 0x64646464u, 0x4342);
    asm("sub.f16x2 %0, %0, %1;" : "+r"(a) : "r"(0x64806480u));
    asm("sub.f16x2 %0, %0, %1;" : "+r"(b) : "r"(0x64806480u));
    lo = a;
    hi = b;
}

__device__ __forceinline__ uint2 ldg_stream_v2(const uint2 *p)
{
    uint2 r;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
    return r;
}

// Zero the deltas and the int8 values (in v.x, v.y) of one 8-element unit outside element range [lo, hi).
__device__ __forceinline__ void mask_unit_bytes(uint4 &v, unsigned &w, int lo, int hi)
{
    lo = min(max(lo, 0), kGroup);
    hi = min(max(hi, 0), kGroup);
    unsigned m = lo >= kGroup ? 0u : (0xffffffffu << (4 * lo));
    if (hi < kGroup) m &= ~(0xffffffffu << (4 * hi));
    w &= m;
    unsigned keep[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 8; ++j) keep[j >> 2] |= (((m >> (4 * j)) & 1u) * 0xffu) << (8 * (j & 3));
    v.x &= keep[0];
    v.y &= keep[1];
}

// acc += fp16(half VH of vword) * fp16(half XH of xword)
template <int VH, int XH>
__device__ __forceinline__ float fma_hh(float acc, unsigned vword, unsigned xword)
{
    if (VH == 0 && XH == 0)
        asm("{.reg .b16 vl,vh,xl,xh; mov.b32 {vl,vh}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, vl, xl, %0;}" : "+f"(acc) : "r"(vword), "r"(xword));
    else if (VH == 0 && XH == 1)
        asm("{.reg .b16 vl,vh,xl,xh; mov.b32 {vl,vh}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, vl, xh, %0;}" : "+f"(acc) : "r"(vword), "r"(xword));
    else if (VH == 1 && XH == 0)
        asm("{.reg .b16 vl,vh,xl,xh; mov.b32 {vl,vh}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, vh, xl, %0;}" : "+f"(acc) : "r"(vword), "r"(xword));
    else
        asm("{.reg .b16 vl,vh,xl,xh; mov.b32 {vl,vh}, %1; mov.b32 {xl,xh}, %2; fma.rn.f32.f16 %0, vh, xh, %0;}" : "+f"(acc) : "r"(vword), "r"(xword));
    return acc;
}

// BV consecutive fp16 values (BV = 2, 4 or 8) from shared memory into BV/2 words
template <int BV>
__device__ __forceinline__ void lds_vec(unsigned addr, unsigned (&r)[BV / 2])
{
    if constexpr (BV == 2)
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r[0]) : "r"(addr));
    else if constexpr (BV == 4)
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
    else
        asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
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

__device__ __forceinline__ unsigned lds_u16(unsigned addr)
{
    unsigned r;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(r) : "r"(addr));
    return r;
}

// c + byte `J` of a: one integer dot-product instruction extracts the byte and adds the base, and it
// does not run on the (half-rate) integer ALU pipe the rest of the index arithmetic competes for.
template <int J, int M = 1>
__device__ __forceinline__ int add_byte(unsigned a, int c)
{
    return __dp4a(a, (unsigned)M << (8 * J), (unsigned)c);   // c + M * byte J of a
}

// Zero the deltas and the fp16 values of one 8-element unit outside element range [lo, hi).
__device__ __forceinline__ void mask_unit(uint4 &v, unsigned &w, int lo, int hi)
{
    lo = min(max(lo, 0), kGroup);
    hi = min(max(hi, 0), kGroup);
    unsigned m = lo >= kGroup ? 0u : (0xffffffffu << (4 * lo));
    if (hi < kGroup) m &= ~(0xffffffffu << (4 * hi));
    w &= m;
    unsigned *vw = reinterpret_cast<unsigned *>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned lo16 = ((m >> (8 * j)) & 1u) * 0xffffu;
        const unsigned hi16 = ((m >> (8 * j + 4)) & 1u) * 0xffff0000u;
        vw[j] &= (lo16 | hi16);
    }
}

// Where a row-sharded launch delivers its slice of y: the full-y buffer of every rank (peer-mapped
// device pointers) and every rank's flag words. world == 0 for an ordinary launch.
template <int V> struct Int { static constexpr int value = V; };

// A virtual row of a planned launch is done (called by the leader lane of its group): a whole row goes to
// y; a segment of a cut row leaves its fp32 sum in the plan, where plan_combine_kernel adds the segments of
// every cut row in segment order once the product kernel has finished.
__device__ __forceinline__ void plan_row_done(const PlanView &pl, unsigned o, float total, float alpha, float beta,
                                              unsigned short *__restrict__ y16, int rows)
{
    if (!(o & kPlanPartialBit)) {
        if (o < (unsigned)rows) {
            float r = alpha * total;
            if (beta != 0.f) r += beta * __half2float(__ushort_as_half(y16[o]));
            y16[o] = __half_as_ushort(__float2half_rn(r));
        }
        return;
    }
    const unsigned v = o & ~kPlanPartialBit;
    if (v < (unsigned)pl.n_virtual) pl.partial[v] = total;
}

// y[row] = fp16(alpha * (sum of the row's segment sums, in segment order) + beta * y[row]) for every cut row.
// Launched right behind the product kernel of a planned launch, as its programmatic dependent.
__global__ void __launch_bounds__(256)
plan_combine_kernel(const PlanView pl, float alpha, float beta, unsigned short *__restrict__ y16, int rows)
{
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= pl.n_split) return;
    const unsigned row = __ldg(pl.split_list + i);
    if (row >= (unsigned)rows) return;
    const int first = __ldg(pl.seg_first + row);
    const int n = min(__ldg(pl.seg_first + row + 1), pl.n_virtual) - first;
    float sum = 0.f;
    for (int k = 0; k < n; ++k) sum += __ldcg(pl.partial + first + k);
    float r = alpha * sum;
    if (beta != 0.f) r += beta * __half2float(__ushort_as_half(y16[row]));
    y16[row] = __half_as_ushort(__float2half_rn(r));
}

constexpr int kMaxPeers = 8;
constexpr unsigned kDefaultSpinLimit = 1u << 23;
struct Peers {
    __half *y[kMaxPeers];
    unsigned *flags[kMaxPeers];   // per rank: [0, world) arrival counters, [world] calls issued, [world+1] CTA ticket, [world+2] error
    long long row_offset;         // first row of this rank's block in the full y
    int world;
    int rank;
    unsigned spin_limit;          // polls of the arrival counters before the wait gives up
    int deferred;                 // publish and return: the caller enqueues macko_peer_wait where y is consumed
};

// Kernel variants without a scatter epilogue / without a plan take an empty structure in place of the tables:
// the parameter block of the plain product stays small.
struct NoPeers {};
struct NoPlan {};
template <bool P> using PeersArg = std::conditional_t<P, Peers, NoPeers>;
template <bool P> using PlanArg = std::conditional_t<P, PlanView, NoPlan>;

// First row of warp `w` of `n_warps` when the rows are dealt to the warps in blocks of K as evenly as they go:
// K * floor(n_blocks * w / n_warps), capped at rows. A 32-bit division whenever the product fits (every matrix of
// fewer than 2^32 / n_warps row blocks: a 64-bit division is some hundred instructions, in every warp of the grid).
template <int K>
__device__ __forceinline__ int block_boundary(int rows, unsigned w, unsigned n_warps)
{
    const unsigned n_blocks = ((unsigned)rows + K - 1) / K;
    unsigned b;
    if (__umulhi(n_blocks, n_warps) == 0u) b = n_blocks * w / n_warps;   // w <= n_warps: the product fits 32 bits
    else b = (unsigned)((unsigned long long)n_blocks * w / n_warps);
    const unsigned long long r = (unsigned long long)b * K;
    return (int)(r < (unsigned long long)rows ? r : (unsigned long long)rows);
}

// What a launch carries besides the reference's arguments.
struct Extra {
    unsigned flags;               // MACKO_SPMV_MATRIX_IMMUTABLE
    PlanView plan;                // planned launch: virtual rows instead of row_indices (PLAN kernels only)
};

// L     lanes per row (a warp walks 32/L rows at once)
// NPAIR pairs of sub-steps per iteration; a sub-step of a group is 8*L consecutive stored elements,
//       and the two sub-steps of a pair share one cross-lane scan (two 16-bit fields per register)
// XS    x staged in shared memory (else gathered from global memory with explicit clamping)
// PEER  the epilogue stores every y value into the full-y buffer of all ranks over NVLink and, once the
//       whole grid is done, bumps this rank's arrival counter on every rank (no collective call follows)
// BV    vectors multiplied at once (1, 2, 4 or 8): x is [batch][cols] and y is [batch][rows], batch <= BV.
//       The matrix is streamed once; shared memory holds the vectors interleaved (BV values per column),
//       so one vector load gathers a column of all of them.
// PLAN  rows come from a plan: virtual rows (begin, length, starting column, destination) sorted by length;
//       the segments of a long row leave fp32 partial sums that the last one to finish adds up in segment order
// VT    value type: kF16; kBF16 (values, x and y are bfloat16: same buffers, same decode); kI8 (values are
//       signed bytes, 8 per 64-bit load, x and y fp16: the reference's int8 variant, kernels.cuh:127-216);
//       fp32 accumulation in every case
// EARLY the caller has declared the matrix immutable: the first matrix loads are issued before the wait for the
//       previous kernel of the stream and before x is staged (a separate instantiation, so that the default
//       launch keeps the simpler code: wait, stage x, then walk the rows)
template <int L, int NPAIR, bool XS, bool PEER, int BV = 1, bool PLAN = false, int VT = kF16, bool EARLY = false>
__global__ void __launch_bounds__(kThreads, 2)
spmv_kernel(const uint4 *__restrict__ values, const unsigned *__restrict__ deltas,
            const int *__restrict__ ri, const __half *__restrict__ x, __half *__restrict__ y,
            int rows, int cols, int stored, float alpha, float beta, int batch, unsigned flags,
            const PeersArg<PEER> peers, const PlanArg<PLAN> plan)
{
    static_assert(BV == 1 || (XS && !PEER), "batched products gather from shared memory and have no scatter epilogue");
    static_assert(!PLAN || (XS && !PEER && BV == 1), "planned launches are built for the single-vector product with x in shared memory");
    static_assert(VT == kF16 || (!PEER && BV == 1 && !PLAN), "bfloat16 and int8 values are built for the plain single-vector product");
    static_assert(!EARLY || BV == 1, "early matrix loads are built for the single-vector product");
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int STEP = kGroup * L;   // elements per group per sub-step
    constexpr int D = 2 * NPAIR;       // sub-steps per iteration
    constexpr int K = 32 / L;          // rows a warp walks at once
    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int lig = lane & (L - 1);          // lane in group
    const int group_lane0 = lane & ~(L - 1); // first lane of my group
    constexpr unsigned kLeaders = (L == 32) ? 0x1u : (L == 16) ? 0x00010001u : (L == 8) ? 0x01010101u : 0x11111111u;
    unsigned short *y16 = reinterpret_cast<unsigned short *>(y);

    // Programmatic dependent launch: let the next kernel of the stream start occupying SMs as ours
    // drain. Memory written by earlier kernels of the stream (x, y, and the matrix unless the caller has
    // declared it immutable) is not touched before griddepcontrol.wait. Both are no-ops for a plain launch.
    asm volatile("griddepcontrol.launch_dependents;");
    if constexpr (!EARLY) asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- this warp's work: a contiguous row range dealt in blocks of K rows (so that the groups of a warp
    //      run out of rows together), or, planned, every n_warps-th block of K virtual rows of the sorted
    //      list, the direction alternating from round to round (longest first: the ends even out) ------------
    const long long n_warps = (long long)gridDim.x * kWarpsPerCta;
    const long long warp_id = (long long)blockIdx.x * kWarpsPerCta + (tid >> 5);
    int row_next, row_hi;   // plain: rows [row_next, row_hi); planned: positions in the warp's sequence
    if constexpr (PLAN) {
        const int V = plan.n_virtual;
        const int W = (int)n_warps, w = (int)warp_id;
        const int nb = (V + K - 1) / K;                 // blocks of K virtual rows
        const int full_rounds = nb / W;
        const int rest = nb - full_rounds * W;           // blocks of the last, partly filled round
        const int slot = (full_rounds & 1) ? W - 1 - w : w;
        const int count = full_rounds + (slot < rest ? 1 : 0);
        row_next = 0;
        row_hi = count * K;
        if (count > 0) {
            const int last_round = count - 1;
            const int last_blk = last_round * W + ((last_round & 1) ? W - 1 - w : w);
            if (last_blk == nb - 1) row_hi -= nb * K - V;   // the very last block may hold fewer than K
        }
    } else {
        row_next = block_boundary<K>(rows, (unsigned)warp_id, (unsigned)n_warps);
        row_hi = block_boundary<K>(rows, (unsigned)warp_id + 1u, (unsigned)n_warps);
    }
    // sorted index of position p of this warp's sequence (planned)
    auto sorted_index = [&](int p) -> int {
        const int W = (int)n_warps, w = (int)warp_id;
        const int round = p / K;
        return (round * W + ((round & 1) ? W - 1 - w : w)) * K + (p - round * K);
    };

    // PEER: rows of the whole CTA (its warps own consecutive ranges) and the staging area for their y
    int cta_row_lo = 0, cta_row_hi = 0;
    if constexpr (PEER) {
        const unsigned cta_w0 = blockIdx.x * kWarpsPerCta;
        cta_row_lo = block_boundary<K>(rows, cta_w0, (unsigned)n_warps);
        cta_row_hi = block_boundary<K>(rows, cta_w0 + kWarpsPerCta, (unsigned)n_warps);
    }
    __half *ystage = reinterpret_cast<__half *>(smem + (((size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half) + 15) & ~(size_t)15));

    // Window of 32 row offsets (planned: 32 virtual-row descriptors) held one per lane and read by shuffle.
    int win_base = row_next;
    int ri_reg = 0;      // plain: ri[win_base + lane]; planned: first stored element of the virtual row
    unsigned pk_reg = 0; // planned: length | starting column << kPlanLenBits
    auto load_window = [&]() {
        if constexpr (PLAN) {
            const int p = win_base + lane;
            uint2 d = make_uint2(0u, 0u);
            if (p < row_hi) d = __ldg(plan.desc + sorted_index(p));
            ri_reg = (int)d.x;
            pk_reg = d.y;
        } else {
            ri_reg = __ldg(ri + min(win_base + lane, rows));
        }
    };
    if (row_next < row_hi) load_window();

    // ---- per-group state ------------------------------------------------------------------------------
    constexpr int LOG_STEP = (L == 32) ? 8 : (L == 16) ? 7 : (L == 8) ? 6 : 5;
    int my_row = -1;   // plain: row being walked by my group (-1: none); planned: 0 while a virtual row is walked
    unsigned out_word = 0u;   // planned: destination of the virtual row (a row of y, or a partial-sum slot)
    int begin = 0;     // first stored element of the row
    int end = 0;       // one past the last stored element
    int pos = 0;       // first element of the group's next iteration (multiple of 8)
    // Byte address (shared window, or byte offset from x - kXPadFront when x stays in global memory) of
    // "column -1 + index in row" in front of the lane's unit of the next sub-step, less 14 per lane below
    // it in the group: the lane totals that go through the scan carry +14 each (see the decode below).
    // x_base (the shared-window address of the front padding) is known before x is staged.
    const int x_base = (XS || BV > 1) ? (int)__cvta_generic_to_shared(smem) : 0;
    const int x_fold = (BV == 1) ? x_base : 0;   // batched: offsets stay per-vector and are scaled by BV at the gather
    const unsigned lane_const = (unsigned)(x_fold + 2 * kXPadFront + 2 * lig);
    const unsigned a_max = (unsigned)(x_fold + 2 * (kXPadFront + cols));
    unsigned run = 0u;
    float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
    float accb[BV][2];   // batched: per vector, even and odd elements
#pragma unroll
    for (int b = 0; b < BV; ++b) accb[b][0] = accb[b][1] = 0.f;

    // Stages x into shared memory, framed by zeros (one CTA-wide barrier at its end).
    auto stage_x = [&]() {
    if (BV > 1) {
        __half *xs = reinterpret_cast<__half *>(smem);
        const int n_total = (kXPadFront + cols + kXPadBack) * BV;
        for (int i = tid; i < kXPadFront * BV; i += kThreads) xs[i] = __ushort_as_half(0);
        for (int i = (kXPadFront + cols) * BV + tid; i < n_total; i += kThreads) xs[i] = __ushort_as_half(0);
#pragma unroll
        for (int b = 0; b < BV; ++b) {
            const __half *xb = x + (size_t)b * cols;
#pragma unroll 4
            for (int c = tid; c < cols; c += kThreads)
                xs[(size_t)(kXPadFront + c) * BV + b] = b < batch ? xb[c] : __ushort_as_half(0);
        }
        __syncthreads();
    } else if (XS) {
        __half *xs = reinterpret_cast<__half *>(smem);
        const int n_total = kXPadFront + cols + kXPadBack;
#pragma unroll 1
        for (int i = tid; i < kXPadFront; i += kThreads) xs[i] = __ushort_as_half(0);
#pragma unroll 1
        for (int i = kXPadFront + cols + tid; i < n_total; i += kThreads) xs[i] = __ushort_as_half(0);
        if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
            // 16-byte asynchronous copies global -> shared: no registers, all of a thread's copies in flight
            // together, and the matrix loads issued above stay in flight beside them
            const int n_vec = cols >> 3;
            const unsigned dst0 = (unsigned)x_base + 2u * kXPadFront;
            const char *src0 = reinterpret_cast<const char *>(x);
#pragma unroll 1
            for (int i = tid; i < n_vec; i += kThreads)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + 16u * (unsigned)i), "l"(src0 + 16 * (size_t)i) : "memory");
#pragma unroll 1
            for (int i = (n_vec << 3) + tid; i < cols; i += kThreads) xs[kXPadFront + i] = x[i];
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
#pragma unroll 1
            for (int i = tid; i < cols; i += kThreads) xs[kXPadFront + i] = x[i];
        }
        __syncthreads();
    }
    };
    if constexpr (!EARLY) stage_x();
    bool first_pass = EARLY;
    for (;;) {
        bool done = false;
        // ---- groups that ran out of work finish their row and take the next one ---------------------
        const bool need = pos >= end;
        const unsigned needmask = __ballot_sync(0xffffffffu, need);
        if (needmask) {
            if constexpr (BV == 1) {
                float total = (acc0 + acc1) + (acc2 + acc3);
#pragma unroll
                for (int o = L / 2; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                if (need) {
                    if (my_row >= 0 && lig == 0) {
                        if constexpr (PLAN) {
                            plan_row_done(plan, out_word, total, alpha, beta, y16, rows);
                        } else if constexpr (PEER) {
                            ystage[my_row - cta_row_lo] = __float2half_rn(alpha * total);   // delivered in bulk at the end
                        } else {
                            float r = alpha * total;
                            if (beta != 0.f) r += beta * from_bits16<VT>(y16[my_row]);
                            y16[my_row] = to_bits16<VT>(r);
                        }
                    }
                    acc0 = acc1 = acc2 = acc3 = 0.f;
                }
            } else {
#pragma unroll
                for (int b = 0; b < BV; ++b) {
                    float total = accb[b][0] + accb[b][1];
#pragma unroll
                    for (int o = L / 2; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
                    if (need) {
                        if (my_row >= 0 && lig == 0 && b < batch) {
                            __half *yb = y + (size_t)b * rows;
                            float r = alpha * total;
                            if (beta != 0.f) r += beta * __half2float(yb[my_row]);
                            yb[my_row] = __float2half_rn(r);
                        }
                        accb[b][0] = accb[b][1] = 0.f;
                    }
                }
            }
            const int avail = row_hi - row_next;
            if (avail <= 0) {
                if (needmask == 0xffffffffu) done = true;
                if (need) { my_row = -1; pos = 0; end = 0; begin = 0; }
            } else {
                const unsigned leaders = needmask & kLeaders;
                const int want = __popc(leaders);
                const int take = min(want, avail);
                if (row_next + take > win_base + (PLAN ? 32 : 31)) {  // warp-uniform
                    win_base = row_next;
                    load_window();
                }
                const int rank = __popc(leaders & ((1u << group_lane0) - 1u));
                const int nr = row_next + rank;
                // offsets are clamped into [0, stored] so that corrupt row_indices (or a corrupt plan) cannot send
                // loads outside values/deltas
                int b, e;
                unsigned colbase2 = 0u;   // planned: twice the column sum in front of the segment (a byte offset into x)
                if constexpr (PLAN) {
                    b = min(max(__shfl_sync(0xffffffffu, ri_reg, (nr - win_base) & 31), 0), stored);
                    const unsigned pk = __shfl_sync(0xffffffffu, pk_reg, (nr - win_base) & 31);
                    e = min(b + (int)(pk & ((1u << kPlanLenBits) - 1u)), stored);
                    colbase2 = (pk >> kPlanLenBits) << 1;
                } else {
                    b = min(max(__shfl_sync(0xffffffffu, ri_reg, (nr - win_base) & 31), 0), stored);
                    e = min(__shfl_sync(0xffffffffu, ri_reg, (nr + 1 - win_base) & 31), stored);
                }
                if (need) {
                    if (rank < take) {
                        if constexpr (PLAN) {
                            my_row = 0;
                            out_word = __ldg(plan.out + sorted_index(nr));   // needed only when the virtual row ends
                        } else {
                            my_row = nr;
                        }
                        begin = b; end = e; pos = b & ~(kGroup - 1);
                        run = lane_const + colbase2 - 2u * (unsigned)(b & (kGroup - 1));   // the unit that holds `begin` starts before the row
                    } else {
                        my_row = -1; pos = 0; end = 0; begin = 0;
                    }
                }
                row_next += take;
            }
        }

        if constexpr (!EARLY) {
            if (done) break;
        }

        // ---- issue the loads of the whole iteration ------------------------------------------------------
        uint4 v[D];
        unsigned w[D];
        const int ord0 = pos + lig * kGroup;
        const int rem0 = end - ord0;    // elements of the row from the lane's first unit on
        const int lo0 = begin - ord0;   // > 0: leading elements of sub-step 0 belong to the previous row
        {
            const uint4 *vp = values + (ord0 >> 3);
            const unsigned *dp = deltas + (ord0 >> 3);
#pragma unroll
            for (int s = 0; s < D; ++s) {
                v[s] = make_uint4(0u, 0u, 0u, 0u);
                w[s] = 0u;
                if (s * STEP < rem0) {
                    if constexpr (VT == kI8) {
                        const uint2 t = ldg_stream_v2(reinterpret_cast<const uint2 *>(values) + (ord0 >> 3) + s * L);
                        v[s].x = t.x;
                        v[s].y = t.y;
                    } else {
                        v[s] = ldg_stream_v4(vp + s * L);
                    }
                    w[s] = ldg_stream_u32(dp + s * L);
                }
            }
        }

        // ---- first pass only: with the first matrix loads in flight, wait for the previous kernel of the
        //      stream (if that has not happened yet) and stage x into shared memory, framed by zeros. Every
        //      warp comes through here, also one without rows. ---------------------------------------------
        if constexpr (EARLY) {
            if (first_pass) {
                first_pass = false;
                asm volatile("griddepcontrol.wait;" ::: "memory");
                stage_x();
            }
        }
        if (done) break;

        // Which sub-steps hold a unit that straddles the first or the last element of a row, and how far the
        // longest row of the warp still reaches: two warp-wide reductions per iteration replace a vote per unit.
        unsigned mybits = 0u;
        if (rem0 > 0) {
            if (lo0 > 0) mybits = 1u;
            const int tail = rem0 & (STEP - 1);
            const unsigned s_end = (unsigned)rem0 >> LOG_STEP;
            if (tail > 0 && tail < kGroup && s_end < (unsigned)D) mybits |= 1u << s_end;
        }
        const unsigned straddle = __reduce_or_sync(0xffffffffu, mybits);
        const int max_rem = __reduce_max_sync(0xffffffffu, rem0);

#pragma unroll
        for (int p = 0; p < NPAIR; ++p) {
            // a pair in which no lane of the warp has an element left ends the iteration
            if (p > 0 && max_rem <= 2 * p * STEP) break;
            // Byte-SIMD prefix sums of the 8 deltas of a unit, scaled by 2 (byte offsets into fp16 x):
            //   ce byte j = 2*(inclusive prefix of element 2j)   + 2*(2j)
            //   co byte j = 2*(inclusive prefix of element 2j+1) + 2*(2j+1)
            // so the top byte of co is 2*(sum of the 8 deltas) + 14.
            unsigned ce[2], co[2];
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {
                const int s = 2 * p + hs;
                if (straddle & (1u << s)) {
                    if constexpr (VT == kI8) mask_unit_bytes(v[s], w[s], (s == 0) ? lo0 : 0, rem0 - s * STEP);
                    else mask_unit(v[s], w[s], (s == 0) ? lo0 : 0, rem0 - s * STEP);
                }
                const unsigned ev = w[s] & 0x0f0f0f0fu;
                const unsigned od = (w[s] >> 4) & 0x0f0f0f0fu;
                const unsigned pe = ev * 0x02020202u + 0x0c080400u;
                const unsigned po = od * 0x02020202u;
                ce[hs] = po * 256u + pe;
                co[hs] = pe + po + 0x02020202u;
            }
            // one scan for both sub-steps: lane totals packed as two 16-bit fields (each < 2^13)
            const unsigned t = (co[0] >> 24) | ((co[1] >> 8) & 0x00ff0000u);
            unsigned inc = t;
#pragma unroll
            for (int o = 1; o < L; o <<= 1) {
                const unsigned u = __shfl_up_sync(0xffffffffu, inc, o, L);
                if (lig >= o) inc += u;
            }
            const unsigned g = __shfl_sync(0xffffffffu, inc, L - 1, L);
            const unsigned ex = inc - t;
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {
                const int s = 2 * p + hs;
                // lane base = run + (low or high field of ex); the group advances by its field of g, which
                // holds 14 per lane where 16 (2 bytes x 8 elements) are due: 2*L more per sub-step
                const unsigned sel = hs ? 0x0100u : 0x0001u;
                const unsigned a0 = min(__dp2a_lo(ex, sel, run) + (unsigned)(2 * L * s), a_max);   // keeps malformed input inside the padded x
                run = __dp2a_lo(g, sel, run);
                unsigned vconv[4];   // int8: the unit's 8 values as four f16x2 words
                if constexpr (VT == kI8) {
                    bytes_to_f16x2(v[s].x, vconv[0], vconv[1]);
                    bytes_to_f16x2(v[s].y, vconv[2], vconv[3]);
                }
                const unsigned *vw = (VT == kI8) ? vconv : reinterpret_cast<const unsigned *>(&v[s]);
                if constexpr (BV > 1) {
                    const int ab = x_base + (int)a0 * BV;
                    auto element_pair = [&](auto jt) {
                        constexpr int J = decltype(jt)::value;
                        unsigned xe[BV / 2], xo[BV / 2];
                        lds_vec<BV>((unsigned)add_byte<J, BV>(ce[hs], ab), xe);
                        lds_vec<BV>((unsigned)add_byte<J, BV>(co[hs], ab), xo);
#pragma unroll
                        for (int b = 0; b < BV; b += 2) {
                            accb[b][0] = fma_hh<0, 0>(accb[b][0], vw[J], xe[b / 2]);
                            accb[b + 1][0] = fma_hh<0, 1>(accb[b + 1][0], vw[J], xe[b / 2]);
                            accb[b][1] = fma_hh<1, 0>(accb[b][1], vw[J], xo[b / 2]);
                            accb[b + 1][1] = fma_hh<1, 1>(accb[b + 1][1], vw[J], xo[b / 2]);
                        }
                    };
                    element_pair(Int<0>{});
                    element_pair(Int<1>{});
                    element_pair(Int<2>{});
                    element_pair(Int<3>{});
                } else {
                    unsigned xe[4], xo[4];
                    if (XS) {
                        xe[0] = lds_u16((unsigned)add_byte<0>(ce[hs], (int)a0));
                        xo[0] = lds_u16((unsigned)add_byte<0>(co[hs], (int)a0));
                        xe[1] = lds_u16((unsigned)add_byte<1>(ce[hs], (int)a0));
                        xo[1] = lds_u16((unsigned)add_byte<1>(co[hs], (int)a0));
                        xe[2] = lds_u16((unsigned)add_byte<2>(ce[hs], (int)a0));
                        xo[2] = lds_u16((unsigned)add_byte<2>(co[hs], (int)a0));
                        xe[3] = lds_u16((unsigned)add_byte<3>(ce[hs], (int)a0));
                        xo[3] = lds_u16((unsigned)add_byte<3>(co[hs], (int)a0));
                    } else {
                        const unsigned short *xg = reinterpret_cast<const unsigned short *>(x);
                        const int cmax = cols - 1;
                        auto gather = [&](int off2) -> unsigned {
                            return (unsigned)__ldg(xg + min(max((off2 >> 1) - kXPadFront, 0), cmax));
                        };
                        xe[0] = gather(add_byte<0>(ce[hs], (int)a0));
                        xo[0] = gather(add_byte<0>(co[hs], (int)a0));
                        xe[1] = gather(add_byte<1>(ce[hs], (int)a0));
                        xo[1] = gather(add_byte<1>(co[hs], (int)a0));
                        xe[2] = gather(add_byte<2>(ce[hs], (int)a0));
                        xo[2] = gather(add_byte<2>(co[hs], (int)a0));
                        xe[3] = gather(add_byte<3>(ce[hs], (int)a0));
                        xo[3] = gather(add_byte<3>(co[hs], (int)a0));
                    }
                    acc0 = fma_h<0, VT == kBF16 ? kBF16 : kF16>(acc0, vw[0], xe[0]);
                    acc1 = fma_h<1, VT == kBF16 ? kBF16 : kF16>(acc1, vw[0], xo[0]);
                    acc2 = fma_h<0, VT == kBF16 ? kBF16 : kF16>(acc2, vw[1], xe[1]);
                    acc3 = fma_h<1, VT == kBF16 ? kBF16 : kF16>(acc3, vw[1], xo[1]);
                    acc0 = fma_h<0, VT == kBF16 ? kBF16 : kF16>(acc0, vw[2], xe[2]);
                    acc1 = fma_h<1, VT == kBF16 ? kBF16 : kF16>(acc1, vw[2], xo[2]);
                    acc2 = fma_h<0, VT == kBF16 ? kBF16 : kF16>(acc2, vw[3], xe[3]);
                    acc3 = fma_h<1, VT == kBF16 ? kBF16 : kF16>(acc3, vw[3], xo[3]);
                }
            }
        }
        // every sub-step that was skipped lies behind the end of all rows of the warp: `run` is not used again before the next row resets it
        run += (unsigned)(2 * L * D);
        pos += D * STEP;
    }

    if constexpr (PEER) {
        // Every CTA writes the y values of its (contiguous) rows into this rank's own copy of the full y with
        // coalesced stores, makes them visible on this GPU and takes a ticket. The CTA that takes the last
        // ticket then forwards the rank's whole slice to the other ranks over NVLink and publishes it with one
        // system-scope fence: a system-scope fence in each of the CTAs costs 6-7 us per launch even on one GPU.
        __syncthreads();
        const int n_mine = cta_row_hi - cta_row_lo;
        {
            __half *dst = peers.y[peers.rank] + peers.row_offset + cta_row_lo;
            for (int i = tid; i < n_mine; i += kThreads) dst[i] = ystage[i];
        }
        __shared__ unsigned last_cta_seq;
        __shared__ unsigned is_last_cta;
        __syncthreads();
        if (tid == 0) {
            __threadfence();   // the CTA's stores (ordered before this by the barrier) are visible device-wide before its ticket
            const unsigned ticket = atomicAdd(peers.flags[peers.rank] + peers.world + 1, 1u);
            is_last_cta = ticket == gridDim.x - 1;
            if (is_last_cta) __threadfence();   // ... and the last CTA sees the stores of every CTA whose ticket it has seen
            last_cta_seq = 0u;
        }
        __syncthreads();
        if (is_last_cta) {
            // Forward this rank's slice (read around L1: other SMs wrote it) to every other rank; chunk c of the
            // slice goes to all peers before chunk c + kThreads, so the stores to different peers are in flight together.
            const unsigned short *src = reinterpret_cast<const unsigned short *>(peers.y[peers.rank] + peers.row_offset);
            bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
            for (int p = 0; p < peers.world; ++p)
                vec = vec && ((reinterpret_cast<uintptr_t>(peers.y[p] + peers.row_offset) & 15) == 0);
            if (vec) {
                const int chunks = rows >> 3;
                for (int c = tid; c < chunks; c += kThreads) {
                    const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(src) + c);
                    for (int p = 0; p < peers.world; ++p)
                        if (p != peers.rank) reinterpret_cast<uint4 *>(peers.y[p] + peers.row_offset)[c] = val;
                }
                for (int i = (chunks << 3) + tid; i < rows; i += kThreads) {
                    const unsigned short val = __ldcg(src + i);
                    for (int p = 0; p < peers.world; ++p)
                        if (p != peers.rank) reinterpret_cast<unsigned short *>(peers.y[p] + peers.row_offset)[i] = val;
                }
            } else {
                for (int i = tid; i < rows; i += kThreads) {
                    const unsigned short val = __ldcg(src + i);
                    for (int p = 0; p < peers.world; ++p)
                        if (p != peers.rank) reinterpret_cast<unsigned short *>(peers.y[p] + peers.row_offset)[i] = val;
                }
            }
            __syncthreads();   // inside a CTA-uniform branch: all forwarding stores are issued
            if (tid == 0) {
                // One system-scope fence, cumulative over what the barrier ordered before it (the forwarded slice),
                // then the arrival counters of all ranks as plain system-scope stores behind it: a release per
                // counter would wait for a round trip over NVLink each time.
                __threadfence_system();
                unsigned *mine = peers.flags[peers.rank];
                const unsigned seq = mine[peers.world] + 1u;
                mine[peers.world] = seq;
                mine[peers.world + 1] = 0u;
                for (int p = 0; p < peers.world; ++p)
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peers.flags[p] + peers.rank), "r"(seq) : "memory");
                last_cta_seq = seq;
            }
            __syncthreads();
        }
        // Unless the caller asked for a deferred wait, the CTA that finished last stays until the slices of all
        // other ranks have arrived, so the end of this kernel means that this rank's full y is complete. Its own
        // counters are already out, so no rank waits for a kernel that waits for it; the wait is bounded and
        // records who was missing.
        const unsigned seq = last_cta_seq;
        if (seq != 0u && !peers.deferred && tid < peers.world) {
            unsigned *mine = peers.flags[peers.rank];
            unsigned seen = 0u;
            bool arrived = false;
            for (unsigned spin = 0; spin < peers.spin_limit; ++spin) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine + tid) : "memory");
                if ((int)(seen - seq) >= 0) { arrived = true; break; }
            }
            if (!arrived) mine[peers.world + 2] = 1u + (unsigned)tid;
        }
    }
}

// One CTA: copies rows [row_offset, row_offset + rows) of this rank's full y into the full y of every other rank,
// makes them visible system-wide and publishes this rank's arrival counter everywhere: the exchange step of a
// row-sharded product as a kernel of its own, for callers that run it beside the next products (on another
// stream or graph branch) instead of at the tail of the product kernel.
__global__ void __launch_bounds__(kThreads) peer_forward_kernel(const Peers peers, int rows)
{
    const int tid = threadIdx.x;
    const unsigned short *src = reinterpret_cast<const unsigned short *>(peers.y[peers.rank] + peers.row_offset);
    bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0);
    for (int p = 0; p < peers.world; ++p)
        vec = vec && ((reinterpret_cast<uintptr_t>(peers.y[p] + peers.row_offset) & 15) == 0);
    const int chunks = vec ? rows >> 3 : 0;
    for (int c = tid; c < chunks; c += kThreads) {
        const uint4 val = __ldcg(reinterpret_cast<const uint4 *>(src) + c);
        for (int p = 0; p < peers.world; ++p)
            if (p != peers.rank) reinterpret_cast<uint4 *>(peers.y[p] + peers.row_offset)[c] = val;
    }
    for (int i = (chunks << 3) + tid; i < rows; i += kThreads) {
        const unsigned short val = __ldcg(src + i);
        for (int p = 0; p < peers.world; ++p)
            if (p != peers.rank) reinterpret_cast<unsigned short *>(peers.y[p] + peers.row_offset)[i] = val;
    }
    __syncthreads();
    if (tid == 0) {
        __threadfence_system();   // cumulative over what the barrier ordered before it: the forwarded slice is out
        unsigned *mine = peers.flags[peers.rank];
        const unsigned seq = mine[peers.world] + 1u;
        mine[peers.world] = seq;
        for (int p = 0; p < peers.world; ++p)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peers.flags[p] + peers.rank), "r"(seq) : "memory");
    }
}

// Waits (bounded) until every rank's arrival counter has reached this rank's own call counter, i.e.
// until all slices of the row-sharded products issued so far have landed in this rank's full y.
__global__ void peer_wait_kernel(unsigned *flags, int world, unsigned spin_limit)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int p = threadIdx.x;
    if (p >= world) return;
    const unsigned expected = flags[world];
    unsigned seen = 0;
    for (unsigned spin = 0; spin < spin_limit; ++spin) {
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flags + p) : "memory");
        if ((int)(seen - expected) >= 0) return;
    }
    flags[world + 2] = 1u + (unsigned)p;   // gave up: the host can read which rank never arrived
}

// Overlap of consecutive launches (programmatic dependent launch) can be switched off with
// MACKO_SPMV_PDL=0 in the environment, read once.
bool use_pdl()
{
    static const bool on = [] {
        const char *v = getenv("MACKO_SPMV_PDL");
        return !(v && v[0] == '0');
    }();
    return on;
}

template <int L, int NPAIR, bool XS, bool PEER, int BV, bool PLAN, int VT, bool EARLY>
int launch_variant(const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
                   const void *x, void *y, float alpha, float beta, cudaStream_t stream,
                   const DeviceInfo &dev, int ctas_per_sm, const Peers &peers, int batch, const Extra &extra);

// The instantiation with or without early matrix loads, by the immutable-matrix flag of the call.
template <int L, int NPAIR, bool XS, bool PEER = false, int BV = 1, bool PLAN = false, int VT = kF16>
int launch(const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
           const void *x, void *y, float alpha, float beta, cudaStream_t stream,
           const DeviceInfo &dev, int ctas_per_sm, const Peers &peers = Peers{}, int batch = 1, const Extra &extra = Extra{})
{
    if constexpr (BV == 1) {
        if (extra.flags & MACKO_SPMV_MATRIX_IMMUTABLE)
            return launch_variant<L, NPAIR, XS, PEER, BV, PLAN, VT, true>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta,
                                                                         stream, dev, ctas_per_sm, peers, batch, extra);
    }
    return launch_variant<L, NPAIR, XS, PEER, BV, PLAN, VT, false>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta,
                                                                  stream, dev, ctas_per_sm, peers, batch, extra);
}

template <int L, int NPAIR, bool XS, bool PEER, int BV, bool PLAN, int VT, bool EARLY>
int launch_variant(const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
                   const void *x, void *y, float alpha, float beta, cudaStream_t stream,
                   const DeviceInfo &dev, int ctas_per_sm, const Peers &peers, int batch, const Extra &extra)
{
    size_t smem = XS ? (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half) * BV : 0;
    if (PEER)  // staging area for a CTA's slice of y (a CTA never owns more rows than rows / #SMs + rounding)
        smem = ((smem + 15) & ~(size_t)15) + (size_t)(rows / dev.sm_count + kWarpsPerCta * 8 + 8) * sizeof(__half);
    if (smem > (size_t)dev.max_smem_optin)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "the launch needs %lld bytes of shared memory, the device offers %d (cols=%d)",
                    (long long)smem, dev.max_smem_optin, cols);
    auto kernel = spmv_kernel<L, NPAIR, XS, PEER, BV, PLAN, VT, EARLY>;
    if (smem > 48 * 1024) {
        // Idempotent and cheap; set on every call so that every device is covered.
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    int per_sm = ctas_per_sm > 0 ? ctas_per_sm : 2;
    if (smem > 0) per_sm = max(1, min(per_sm, (int)((size_t)dev.max_smem_optin / (smem + 1024))));
    // Always a whole number of CTAs per SM: with fewer CTAs than that, some SMs would hold twice the rows
    // of others. Only matrices with fewer row groups than CTAs get a smaller grid (one group per CTA).
    const long long work_rows = PLAN ? (long long)extra.plan.n_virtual : (long long)rows;
    const long long groups = (work_rows * L + 31) / 32;
    long long ctas = (long long)dev.sm_count * per_sm;
    if (groups < ctas) ctas = groups < 1 ? 1 : groups;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // A scatter launch that ends with a CTA waiting for other GPUs launches without the overlap: letting the
    // next kernel move in early only takes SM slots away from it (measured: slower). With a deferred wait the
    // kernel publishes and returns, and overlaps like any other.
    cfg.numAttrs = (use_pdl() && (!PEER || peers.deferred)) ? 1 : 0;
    PeersArg<PEER> peers_arg{};
    PlanArg<PLAN> plan_arg{};
    if constexpr (PEER) peers_arg = peers;
    if constexpr (PLAN) plan_arg = extra.plan;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel,
        static_cast<const uint4 *>(values), static_cast<const unsigned *>(deltas), ri,
        static_cast<const __half *>(x), static_cast<__half *>(y), rows, cols, (int)padded, alpha, beta, batch, extra.flags,
        peers_arg, plan_arg);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "spmv launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}

template <int L, bool XS, int VT>
int launch_d(int D, const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
             const void *x, void *y, float alpha, float beta, cudaStream_t stream,
             const DeviceInfo &dev, int ctas_per_sm, const Extra &extra)
{
    switch (D) {
        case 2: return launch<L, 1, XS, false, 1, false, VT>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, Peers{}, 1, extra);
        case 4: return launch<L, 2, XS, false, 1, false, VT>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, Peers{}, 1, extra);
        case 6: return launch<L, 3, XS, false, 1, false, VT>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, Peers{}, 1, extra);
        default: return fail(MACKO_ERR_INVALID_ARGUMENT, "steps_in_flight must be 2, 4 or 6 (got %d)", D);
    }
}

template <bool XS, int VT = kF16>
int launch_l(int L, int D, const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
             const void *x, void *y, float alpha, float beta, cudaStream_t stream,
             const DeviceInfo &dev, int ctas_per_sm, const Extra &extra = Extra{})
{
    switch (L) {
        case 4: return launch_d<4, XS, VT>(D, values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, extra);
        case 8: return launch_d<8, XS, VT>(D, values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, extra);
        case 16: return launch_d<16, XS, VT>(D, values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, extra);
        case 32: return launch_d<32, XS, VT>(D, values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, ctas_per_sm, extra);
        default: return fail(MACKO_ERR_INVALID_ARGUMENT, "lanes_per_row must be 4, 8, 16 or 32 (got %d)", L);
    }
}

// Lanes per row (L) and units in flight per lane (D) for a matrix, calibrated on B200 over row counts
// 4096..49152, row lengths 500..25000 stored elements and densities 0.1..0.9:
//   * fewer lanes per row keep the x gathers of one load instruction close together (fewer shared-memory bank
//     conflicts, the resource the kernel is bound by) and shorten the cross-lane scan, so the smallest L wins
//     that still (a) gives at least ~0.55 of the resident warps a block of rows and (b) walks a row in at most
//     ~64 sub-steps (a row is a serial chain of sub-steps; 16 sub-steps for very wide matrices, where a full
//     warp per row measured better);
//   * rows shorter than half a sub-step shrink the group further;
//   * six units in flight once a row holds more than three sub-steps, four above one, else two.
struct Shape { int L, D; };
Shape choose_shape(long long rows, long long cols, long long padded, int resident_warps)
{
    const long long avg_row = rows > 0 ? padded / rows : 0;
    const long long chain = cols > 16384 ? 16 : 64;
    int L = 32;
    for (int cand = 8; cand < 32; cand <<= 1) {
        const bool enough_blocks = rows * cand * 100 >= 55LL * 32 * resident_warps;
        const bool short_chain = avg_row <= chain * kGroup * cand;
        if (enough_blocks && short_chain) { L = cand; break; }
    }
    while (L > 4 && avg_row < (long long)L * kGroup / 2) L >>= 1;
    const int D = avg_row > 3LL * L * kGroup ? 6 : avg_row > (long long)L * kGroup ? 4 : 2;
    return {L, D};
}

// One launch for up to BV vectors. Lanes per row as in the single-vector product; fewer units in flight with
// more vectors, whose accumulators and gathered values take the registers.
template <int BV>
int launch_batched(const void *values, const void *deltas, const int32_t *ri, int rows, int cols, long long padded,
                   const void *x, void *y, int batch, float alpha, float beta, cudaStream_t stream, const DeviceInfo &dev)
{
    // lanes per row as for one vector (the kernel is built for 8 and 32 here), with the resident warps that
    // BV copies of x in shared memory leave
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half) * BV;
    const int ctas = smem * 2 + 2048 <= (size_t)dev.max_smem_optin ? 2 : 1;
    const Shape shape = choose_shape(rows, cols, padded, dev.sm_count * ctas * kWarpsPerCta);
    const bool wide = shape.L >= 16;   // 16 lanes per row are not built for several vectors: a warp per row is the closer choice
    if constexpr (BV <= 4) {
        if (shape.D >= 4)
            return wide ? launch<32, 2, true, false, BV>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, 0, Peers{}, batch)
                        : launch<8, 2, true, false, BV>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, 0, Peers{}, batch);
    }
    return wide ? launch<32, 1, true, false, BV>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, 0, Peers{}, batch)
                : launch<8, 1, true, false, BV>(values, deltas, ri, rows, cols, padded, x, y, alpha, beta, stream, dev, 0, Peers{}, batch);
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

namespace macko {
namespace {

int check_flags(uint32_t flags)
{
    if (flags & ~(uint32_t)MACKO_SPMV_MATRIX_IMMUTABLE)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", flags);
    return MACKO_OK;
}

// The default launch: shape from the chooser, x in shared memory when it fits.
template <int VT>
int spmv_default(const void *values, const void *deltas, const int32_t *row_indices,
                 int64_t rows, int64_t cols, int64_t padded_count,
                 const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream)
{
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, y);
    if (st == MACKO_OK) st = check_flags(flags);
    if (st != MACKO_OK) return st;
    if (rows == 0) return MACKO_OK;
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;

    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    const int ctas = smem * 2 + 2048 <= (size_t)dev->max_smem_optin ? 2 : 1;
    const Shape shape = choose_shape(rows, cols, padded_count, dev->sm_count * ctas * kWarpsPerCta);
    const int L = shape.L, D = shape.D;
    const bool xs = smem <= (size_t)dev->max_smem_optin;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    Extra extra = {};
    extra.flags = flags;
    if (xs)
        return launch_l<true, VT>(L, D, values, deltas, row_indices, (int)rows, (int)cols, padded_count, x, y, alpha, beta, s, *dev, 0, extra);
    return launch_l<false, VT>(L, D, values, deltas, row_indices, (int)rows, (int)cols, padded_count, x, y, alpha, beta, s, *dev, 0, extra);
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
    if (cols == 0) x_in_shared = 1;   // nothing to gather: the zero frame in shared memory serves every (malformed) element
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    if (x_in_shared && smem > (size_t)dev->max_smem_optin)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "x does not fit shared memory (cols=%lld)", (long long)cols);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (x_in_shared)
        return launch_l<true>(lanes_per_row, steps_in_flight, values, deltas, row_indices, (int)rows, (int)cols, padded_count,
                              x, y, alpha, beta, s, *dev, ctas_per_sm);
    return launch_l<false>(lanes_per_row, steps_in_flight, values, deltas, row_indices, (int)rows, (int)cols, padded_count,
                           x, y, alpha, beta, s, *dev, ctas_per_sm);
}

int macko_spmv_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, void *stream)
{
    return macko::spmv_default<macko::kF16>(values, deltas, row_indices, rows, cols, padded_count, x, y, alpha, beta, 0u, stream);
}

int macko_spmv_fp16_ex(const void *values, const void *deltas, const int32_t *row_indices,
                       int64_t rows, int64_t cols, int64_t padded_count,
                       const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream)
{
    return macko::spmv_default<macko::kF16>(values, deltas, row_indices, rows, cols, padded_count, x, y, alpha, beta, flags, stream);
}

int macko_spmv_bf16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream)
{
    return macko::spmv_default<macko::kBF16>(values, deltas, row_indices, rows, cols, padded_count, x, y, alpha, beta, flags, stream);
}

int macko_spmv_int8(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream)
{
    return macko::spmv_default<macko::kI8>(values, deltas, row_indices, rows, cols, padded_count, x, y, alpha, beta, flags, stream);
}

int macko_spmv_fp16_planned(const void *values, const void *deltas, const int32_t *row_indices,
                            int64_t rows, int64_t cols, int64_t padded_count,
                            const void *plan, const macko_spmv_plan_info *info,
                            const void *x, void *y, float alpha, float beta, uint32_t flags, void *stream)
{
    using namespace macko;
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, y);
    if (st == MACKO_OK) st = check_flags(flags);
    if (st != MACKO_OK) return st;
    if (!plan || !info) return fail(MACKO_ERR_INVALID_ARGUMENT, "null plan or plan info");
    if (!aligned(plan, 16)) return fail(MACKO_ERR_MISALIGNED, "plan must be 16-byte aligned");
    if (info->rows != rows || info->padded_count != padded_count || info->virtual_rows < rows ||
        info->segment_elements < 256 || info->segment_elements > kPlanMaxSegment || info->segment_elements % 256 != 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "the plan info does not describe this matrix (rows %lld/%lld, P %lld/%lld, %d virtual rows)",
                    (long long)info->rows, (long long)rows, (long long)info->padded_count, (long long)padded_count, info->virtual_rows);
    const PlanLayout lay = plan_layout(rows, padded_count, info->segment_elements);
    if (info->plan_bytes != lay.total || (long long)info->virtual_rows > lay.v_max)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "the plan info is inconsistent (bytes %lld, expected %lld)",
                    (long long)info->plan_bytes, (long long)lay.total);
    if (rows == 0) return MACKO_OK;
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    if (smem > (size_t)dev->max_smem_optin)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "cols=%lld does not fit shared memory in the planned launch", (long long)cols);
    char *base = const_cast<char *>(static_cast<const char *>(plan));
    Extra extra = {};
    extra.flags = flags;
    extra.plan.desc = reinterpret_cast<const uint2 *>(base + lay.desc);
    extra.plan.out = reinterpret_cast<const unsigned *>(base + lay.out);
    extra.plan.vrow = reinterpret_cast<const unsigned *>(base + lay.vrow);
    extra.plan.partial = reinterpret_cast<float *>(base + lay.partial);
    extra.plan.seg_first = reinterpret_cast<const int *>(base + lay.seg_first);
    extra.plan.split_list = reinterpret_cast<const unsigned *>(base + lay.split_list);
    extra.plan.n_split = info->split_rows;
    extra.plan.n_virtual = info->virtual_rows;
    if (info->split_rows < 0 || info->split_rows > rows)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "the plan info is inconsistent (%d cut rows of %lld)", info->split_rows, (long long)rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    st = launch<8, 3, true, false, 1, true>(values, deltas, row_indices, (int)rows, (int)cols, padded_count, x, y,
                                            alpha, beta, s, *dev, 0, Peers{}, 1, extra);
    if (st != MACKO_OK || info->split_rows == 0) return st;
    // the segments of the cut rows are added up by a second, tiny kernel that starts when the first has finished
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((info->split_rows + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = use_pdl() ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, plan_combine_kernel, extra.plan, alpha, beta, static_cast<unsigned short *>(y), (int)rows);
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "plan combine launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}

int macko_spmv_shape(int64_t rows, int64_t cols, int64_t padded_count, int sm_count,
                     int *lanes_per_row, int *steps_in_flight)
{
    using namespace macko;
    if (rows < 0 || cols < 0 || padded_count < 0 || sm_count <= 0 || !lanes_per_row || !steps_in_flight)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "bad argument to macko_spmv_shape");
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    const int ctas = smem * 2 + 2048 <= (size_t)227 * 1024 ? 2 : 1;
    const Shape shape = choose_shape(rows, cols, padded_count, sm_count * ctas * kWarpsPerCta);
    *lanes_per_row = shape.L;
    *steps_in_flight = shape.D;
    return MACKO_OK;
}

int macko_spmm_fp16(const void *values, const void *deltas, const int32_t *row_indices,
                    int64_t rows, int64_t cols, int64_t padded_count,
                    const void *x, void *y, int64_t batch, float alpha, float beta, void *stream)
{
    using namespace macko;
    if (batch < 0) return fail(MACKO_ERR_INVALID_ARGUMENT, "negative batch %lld", (long long)batch);
    if (batch == 0) return MACKO_OK;   // nothing to read or write: x and y may be null
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, y);
    if (st != MACKO_OK) return st;
    if (rows == 0) return MACKO_OK;
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t per_vector = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half);
    const char *xp = static_cast<const char *>(x);
    char *yp = static_cast<char *>(y);
    // Chunks of up to 8 vectors per pass over the matrix, fewer when that many copies of x do not fit
    // shared memory; what is left over goes through the single-vector product.
    int64_t done = 0;
    while (done < batch) {
        const int64_t left = batch - done;
        int bv = left >= 5 ? 8 : left >= 3 ? 4 : left >= 2 ? 2 : 1;
        while (bv > 1 && per_vector * bv > (size_t)dev->max_smem_optin) bv >>= 1;
        const int now = (int)(left < bv ? left : bv);
        const void *xc = xp + (size_t)done * cols * sizeof(__half);
        void *yc = yp + (size_t)done * rows * sizeof(__half);
        const int r = (int)rows, c = (int)cols;
        switch (bv) {
            case 8: st = launch_batched<8>(values, deltas, row_indices, r, c, padded_count, xc, yc, now, alpha, beta, s, *dev); break;
            case 4: st = launch_batched<4>(values, deltas, row_indices, r, c, padded_count, xc, yc, now, alpha, beta, s, *dev); break;
            case 2: st = launch_batched<2>(values, deltas, row_indices, r, c, padded_count, xc, yc, now, alpha, beta, s, *dev); break;
            default: st = macko_spmv_fp16(values, deltas, row_indices, rows, cols, padded_count, xc, yc, alpha, beta, stream); break;
        }
        if (st != MACKO_OK) return st;
        done += now;
    }
    return MACKO_OK;
}

int macko_spmv_fp16_scatter_ex(const void *values, const void *deltas, const int32_t *row_indices,
                               int64_t rows, int64_t cols, int64_t padded_count, const void *x,
                               void *const *peer_y, int64_t row_offset, uint32_t *const *peer_flags,
                               int rank, int world, uint32_t flags, uint32_t spin_limit, void *stream)
{
    using namespace macko;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "rank %d / world %d outside 1..%d", rank, world, kMaxPeers);
    if (!peer_y || !peer_flags || row_offset < 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "null peer tables or negative row offset");
    if (flags & ~(uint32_t)(MACKO_SPMV_MATRIX_IMMUTABLE | MACKO_SCATTER_DEFERRED_WAIT))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "unknown flag bits 0x%x", flags);
    Peers peers = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_y[p] || !peer_flags[p]) return fail(MACKO_ERR_INVALID_ARGUMENT, "null pointer for rank %d", p);
        if (!aligned(peer_y[p], 2) || !aligned(peer_flags[p], 4))
            return fail(MACKO_ERR_MISALIGNED, "peer buffers need 2-byte (y) and 4-byte (flags) alignment");
        peers.y[p] = static_cast<__half *>(peer_y[p]);
        peers.flags[p] = peer_flags[p];
    }
    peers.row_offset = row_offset;
    peers.world = world;
    peers.rank = rank;
    peers.spin_limit = spin_limit == 0 ? kDefaultSpinLimit : spin_limit;
    peers.deferred = (flags & MACKO_SCATTER_DEFERRED_WAIT) ? 1 : 0;
    int st = check_args(values, deltas, row_indices, rows, cols, padded_count, x, peer_y[rank]);
    if (st != MACKO_OK) return st;
    const DeviceInfo *dev = nullptr;
    st = current_device_info(&dev);
    if (st != MACKO_OK) return st;
    // x and the CTA's slice of y share the CTA's shared memory (launch() refuses what does not fit)
    const size_t smem = (size_t)(kXPadFront + cols + kXPadBack) * sizeof(__half) +
                        (size_t)(rows / dev->sm_count + kWarpsPerCta * 8 + 16) * sizeof(__half);
    if (smem > (size_t)dev->max_smem_optin)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "cols=%lld (plus the y staging of %lld rows) does not fit shared memory in the scatter variant",
                    (long long)cols, (long long)rows);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // rows == 0 still has to signal: launch the kernel with an empty range (one CTA)
    const int ctas = smem * 2 + 4096 <= (size_t)dev->max_smem_optin ? 2 : 1;
    Shape shape = choose_shape(rows, cols, padded_count, dev->sm_count * ctas * kWarpsPerCta);
    if (shape.L < 8) shape.L = 8;   // the scatter variant is built for 8, 16 and 32 lanes per row
    const int r = (int)rows, c = (int)cols;
    Extra extra = {};
    extra.flags = flags & MACKO_SPMV_MATRIX_IMMUTABLE;
#define MACKO_SCATTER(LL, NP) \
    launch<LL, NP, true, true>(values, deltas, row_indices, r, c, padded_count, x, nullptr, 1.f, 0.f, s, *dev, 0, peers, 1, extra)
    switch (shape.L * 10 + shape.D) {
        case 82: return MACKO_SCATTER(8, 1);
        case 84: return MACKO_SCATTER(8, 2);
        case 86: return MACKO_SCATTER(8, 3);
        case 162: return MACKO_SCATTER(16, 1);
        case 164: return MACKO_SCATTER(16, 2);
        case 166: return MACKO_SCATTER(16, 3);
        case 322: return MACKO_SCATTER(32, 1);
        case 324: return MACKO_SCATTER(32, 2);
        default: return MACKO_SCATTER(32, 3);
    }
#undef MACKO_SCATTER
}

int macko_spmv_fp16_scatter(const void *values, const void *deltas, const int32_t *row_indices,
                            int64_t rows, int64_t cols, int64_t padded_count, const void *x,
                            void *const *peer_y, int64_t row_offset, uint32_t *const *peer_flags,
                            int rank, int world, void *stream)
{
    return macko_spmv_fp16_scatter_ex(values, deltas, row_indices, rows, cols, padded_count, x, peer_y, row_offset,
                                      peer_flags, rank, world, 0u, 0u, stream);
}

int macko_peer_forward(void *const *peer_y, int64_t row_offset, int64_t rows, uint32_t *const *peer_flags,
                       int rank, int world, void *stream)
{
    using namespace macko;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "rank %d / world %d outside 1..%d", rank, world, kMaxPeers);
    if (!peer_y || !peer_flags || row_offset < 0 || rows < 0 || rows >= (1LL << 31))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "null peer tables, negative row offset or bad row count");
    Peers peers = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_y[p] || !peer_flags[p]) return fail(MACKO_ERR_INVALID_ARGUMENT, "null pointer for rank %d", p);
        if (!aligned(peer_y[p], 2) || !aligned(peer_flags[p], 4))
            return fail(MACKO_ERR_MISALIGNED, "peer buffers need 2-byte (y) and 4-byte (flags) alignment");
        peers.y[p] = static_cast<__half *>(peer_y[p]);
        peers.flags[p] = peer_flags[p];
    }
    peers.row_offset = row_offset;
    peers.world = world;
    peers.rank = rank;
    peer_forward_kernel<<<1, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(peers, (int)rows);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "peer forward launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}

int macko_peer_wait_limited(uint32_t *local_flags, int world, uint32_t spin_limit, void *stream)
{
    using namespace macko;
    if (!local_flags || world < 1 || world > kMaxPeers)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "null flags or world %d outside 1..%d", world, kMaxPeers);
    if (!aligned(local_flags, 4)) return fail(MACKO_ERR_MISALIGNED, "flags must be 4-byte aligned");
    peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(local_flags, world,
                                                                        spin_limit == 0 ? kDefaultSpinLimit : spin_limit);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "peer wait launch: %s", cudaGetErrorString(e));
    return MACKO_OK;
}

int macko_peer_wait(uint32_t *local_flags, int world, void *stream)
{
    return macko_peer_wait_limited(local_flags, world, 0u, stream);
}
}
