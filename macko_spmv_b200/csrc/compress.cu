// GPU compressor producing MACKO buffers bit-identical to the reference host encoder
// `compress_rows_cpu` (src/macko_spmv/cuda/cpu_compressor.cuh:6-73).
//
// The reference walks every row with a running zero counter. The same output follows from a
// closed form that parallelises: a true non-zero at column c whose previous non-zero of the
// row (or -1) is at c0 has gap g = c - c0 - 1; it emits floor(g/16) pads, sitting on columns
// c0+16, c0+32, ... (value = the +-0 found there, delta 15), then itself with delta g mod 16.
// Zeros after the last non-zero of a row emit nothing. NaNs are stored as 0x7fff, -0.0 counts
// as zero (cpu_compressor.cuh:26-27,36).
//
// Phase 1 (count):  one warp per row -> stored elements per row -> prefix sum = row_indices.
// Phase 2 (emit):   one warp per row -> values and packed deltas in one pass (emit_rows_packed_kernel);
//                   the built-in-scratch entry point and the int8 encoder write one delta per byte into
//                   scratch and a final pass packs two per byte and zeroes the tail up to P.
// A warp reads 256 columns per step (one 128-bit load per lane, aligned on the matrix
// allocation, not on the row, so odd column counts still use vector loads).
#include "common.cuh"

#include <cuda_fp16.h>

#include <mutex>

namespace macko {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kThreads = kWarpsPerCta * 32;
constexpr int kColsPerLane = 8;
constexpr int kColsPerStep = 32 * kColsPerLane;
constexpr int kUnroll = 4;        // steps whose loads are in flight together
constexpr int kStageElems = 320;  // stored elements of one step that fit the per-warp staging area

// Warps of the emit kernel (and the pack kernel) that had to refuse a store because row_indices pointed
// beyond the padded count they were given: non-zero means that the outputs of that call are incomplete.
// Per device, read and cleared by macko_compress_overflow().
static __device__ unsigned g_compress_overflow;

// Every NaN is stored as 0x7fff (what the reference's float round trip makes of it, cpu_compressor.cuh:26,36).
// `nan_above` is the bit pattern of +infinity of the value type: 0x7c00 for fp16, 0x7f80 for bfloat16.
__device__ __forceinline__ unsigned short canonical(unsigned short h, unsigned nan_above)
{
    return ((h & 0x7fffu) > nan_above) ? (unsigned short)0x7fffu : h;
}

// Loads the 8 fp16 of this lane for the step starting at global element index g0 (a multiple of 8
// relative to the allocation start on the vector path) as four packed words; elements outside the
// allocation read as zero. Which of the 8 belong to the row is decided by row_bits().
__device__ __forceinline__ void load8(const unsigned short *dense, unsigned g0, unsigned total, bool vec_ok,
                                      unsigned (&w)[4])
{
    if (vec_ok && g0 + 8u <= total) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(dense + g0));
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const unsigned g = g0 + 2u * j;
            const unsigned lo16 = g < total ? (unsigned)__ldg(dense + g) : 0u;
            const unsigned hi16 = g + 1u < total ? (unsigned)__ldg(dense + g + 1u) : 0u;
            w[j] = lo16 | (hi16 << 16);
        }
    }
}

// Bit i set <=> element g0 + i lies inside the row [lo, hi).
__device__ __forceinline__ unsigned row_bits(unsigned g0, unsigned lo, unsigned hi)
{
    const unsigned a = g0 >= lo ? 0u : min(lo - g0, 8u), b = g0 >= hi ? 0u : min(hi - g0, 8u);
    return ((1u << b) - 1u) & ~((1u << a) - 1u);
}

// Bit i set <=> fp16 element i of the four packed words is not +-0.
__device__ __forceinline__ unsigned nonzero_bits(const unsigned (&w)[4])
{
    unsigned nz = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned t = __vsetne2(w[j] & 0x7fff7fffu, 0u);   // 1 per non-zero halfword
        nz |= ((t & 1u) | (t >> 15)) << (2 * j);
    }
    return nz & 0xffu;
}

// Column (row-relative) of the last non-zero strictly before this lane's 8 columns.
__device__ __forceinline__ int prev_nonzero_before_lane(unsigned any, int lane, int my_last_col, int carry)
{
    const unsigned lower = any & ((1u << lane) - 1u);
    const int src = lower ? 31 - __clz(lower) : lane;
    const int got = __shfl_sync(0xffffffffu, my_last_col, src);
    return lower ? got : carry;
}

template <bool EMIT>
__global__ void __launch_bounds__(kThreads)
compress_rows_kernel(const unsigned short *__restrict__ dense, int rows, int cols, bool vec_ok,
                     int *__restrict__ row_counts_out,           // !EMIT: count of row r at [r+1]
                     const int *__restrict__ row_indices,        // EMIT
                     unsigned short *__restrict__ values,        // EMIT
                     unsigned char *__restrict__ nibbles,        // EMIT: one delta per byte
                     int limit,                                  // EMIT: slots in values / nibbles (P)
                     unsigned nan_above)                         // EMIT: +infinity of the value type
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= rows) return;
    // element indices fit 32 bits: the entry points refuse matrices of 2^31 elements or more, and a walk ends
    // less than 2048 elements behind its row
    const unsigned total = (unsigned)rows * (unsigned)cols;
    const unsigned row_lo = (unsigned)row * (unsigned)cols;
    const unsigned row_hi = row_lo + (unsigned)cols;
    // First step starts at the 8-element boundary at or below the row start.
    const unsigned first = vec_ok ? (row_lo & ~7u) : row_lo;

    int carry_prev = -1;   // column of the last non-zero seen so far in this row
    int count = 0;         // !EMIT: stored elements seen by this lane
    int out = EMIT ? row_indices[row] : 0;  // EMIT: next output slot of the warp
    // EMIT: output slots come from row_indices, which the caller may have paired with a too small P (or
    // with a matrix that changed since the count): every store is checked against `limit` and refused
    // stores are counted, so an inconsistent call cannot write outside values / the scratch.
    bool refused = false;

    // EMIT: the stored elements of one step are gathered in shared memory and written out with
    // coalesced stores (every lane writing its own few elements would issue many tiny stores).
    __shared__ unsigned short stage_v[EMIT ? kWarpsPerCta : 1][EMIT ? kStageElems : 1];
    __shared__ unsigned char stage_n[EMIT ? kWarpsPerCta : 1][EMIT ? kStageElems : 1];
    const int wslot = EMIT ? (int)(threadIdx.x >> 5) : 0;

    for (unsigned group0 = first; group0 < row_hi; group0 += (unsigned)(kUnroll * kColsPerStep)) {
        // all loads of kUnroll steps are issued before the first one is consumed
        unsigned ws[kUnroll][4];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            load8(dense, group0 + (unsigned)(u * kColsPerStep + lane * kColsPerLane), total, vec_ok, ws[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const unsigned g0 = group0 + (unsigned)(u * kColsPerStep + lane * kColsPerLane);
            const unsigned (&w)[4] = ws[u];
            const int c0 = (int)(g0 - row_lo);  // column of element 0; may be negative on the first step
            const unsigned nz = nonzero_bits(w) & row_bits(g0, row_lo, row_hi);
            const unsigned any = __ballot_sync(0xffffffffu, nz != 0);
            if (any == 0) continue;  // warp-uniform
            const int my_last = c0 + (31 - __clz(nz | 1u));
            int prev = prev_nonzero_before_lane(any, lane, my_last, carry_prev);
            carry_prev = __shfl_sync(0xffffffffu, my_last, 31 - __clz(any));

            // stored elements emitted by this lane in this step: one per non-zero, plus the pads in
            // front of its first non-zero (later ones follow within 8 columns, so they need none)
            int mine = __popc(nz);
            if (nz) mine += (c0 + (__ffs(nz) - 1) - prev - 1) >> 4;
            if (!EMIT) {
                count += mine;
            } else {
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, incl, o);
                    if (lane >= o) incl += t;
                }
                const int step_total = __shfl_sync(0xffffffffu, incl, 31);
                const bool staged = step_total <= kStageElems;   // warp-uniform; long pad runs go direct
                int k = staged ? incl - mine : out + incl - mine;
                unsigned short *vdst = staged ? stage_v[wslot] : values;
                unsigned char *ndst = staged ? stage_n[wslot] : nibbles;
                // staged slots are below step_total <= kStageElems by construction; direct slots are checked
                const unsigned cap = staged ? (unsigned)kStageElems : (unsigned)limit;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (nz & (1u << i)) {
                        const int c = c0 + i;
                        for (int p = prev + 16; p < c; p += 16) {  // pads keep the sign of the zero they sit on
                            if ((unsigned)k < cap) {
                                vdst[k] = __ldg(dense + row_lo + p);
                                ndst[k] = 15;
                            } else {
                                refused = true;
                            }
                            ++k;
                        }
                        if ((unsigned)k < cap) {
                            vdst[k] = canonical((unsigned short)((w[i >> 1] >> (16 * (i & 1))) & 0xffffu), nan_above);
                            ndst[k] = (unsigned char)((c - prev - 1) & 15);
                        } else {
                            refused = true;
                        }
                        ++k;
                        prev = c;
                    }
                }
                if (staged) {
                    __syncwarp();
                    for (int i = lane; i < step_total; i += 32) {
                        if ((unsigned)(out + i) < (unsigned)limit) {
                            values[out + i] = stage_v[wslot][i];
                            nibbles[out + i] = stage_n[wslot][i];
                        } else {
                            refused = true;
                        }
                    }
                    __syncwarp();
                }
                out += step_total;
            }
        }
    }
    if (!EMIT) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
        if (lane == 0) row_counts_out[row + 1] = count;
    } else {
        if (__any_sync(0xffffffffu, refused) && lane == 0) atomicAdd(&g_compress_overflow, 1u);
    }
}

// ---- emit with packed deltas ---------------------------------------------------------------------------
// The emit phase of macko_compress_emit / _emit_bf16: values and the packed 4-bit deltas in one pass, no scratch
// and no packing pass. A warp walks its row as above and appends what a step stores to a small ring in shared
// memory whose slot j stands for output slot ring_base + j, ring_base a multiple of 8. Whenever the ring could
// not take another step, all complete groups of 8 slots leave: the values as one 16-byte store, their 8 deltas packed into one 32-bit
// store. The first and the last group of a row may be shared with the neighbouring rows (rows start at
// arbitrary slots): their values leave one by one and their nibbles are merged into the word with atomicOr,
// which is why the caller clears `deltas` before the launch. Pads: only a lane's first non-zero of a step can
// have pads in front of it (later ones are less than 8 columns apart). The run in front of the first non-zero
// of the whole step can be as long as the row and is written by the warp together, 256 pads at a time; the
// others (at most 15 per lane, 16 per step) by their lane. The warp of the last row also clears values[n, P).
constexpr int kRing = 544;   // room for two appends: what stays after a flush (< 8), then twice 256 non-zeros + 16 pads
constexpr int kRingFlushAbove = kRing - 272;   // a step (or a batch of 256 pads) always fits below kRing

// The 8 deltas of bytes b0..b7 (each < 16) as 8 nibbles, the first in the low nibble.
__device__ __forceinline__ unsigned pack_nibbles(uint2 b)
{
    b.x &= 0x0f0f0f0fu;   // ring entries of another row hold anything
    b.y &= 0x0f0f0f0fu;
    unsigned x = (b.x | (b.x >> 4)) & 0x00ff00ffu;
    x = (x | (x >> 8)) & 0xffffu;
    unsigned y = (b.y | (b.y >> 4)) & 0x00ff00ffu;
    y = (y | (y >> 8)) & 0xffffu;
    return x | (y << 16);
}

template <typename V>
struct EmitRing {
    V *sv;                  // values of the ring's slots
    unsigned char *sn;      // their deltas, one per byte
    int base;               // output slot of ring slot 0 (a multiple of 8)
    int fill;               // ring slots in use (warp-uniform)
    int own_lo;             // first output slot that belongs to this row
    bool refused;
};

// Writes out the complete groups of 8 ring slots (`last`: the incomplete one as well), keeps the rest.
template <typename V>
__device__ __forceinline__ void ring_flush(EmitRing<V> &r, V *__restrict__ values, unsigned *__restrict__ deltas32,
                                           int limit, bool vec_v, bool last, int lane)
{
    __syncwarp();
    const int n_full = r.fill >> 3;
    const int n_groups = n_full + ((last && (r.fill & 7)) ? 1 : 0);
    for (int c = lane; c < n_groups; c += 32) {
        const int slot0 = r.base + 8 * c;
        const int lo = max(r.own_lo - slot0, 0);                 // first ring entry of the group that is this row's
        const int hi = c < n_full ? 8 : (r.fill & 7);            // one past its last
        if (lo >= hi) continue;
        const uint2 nb = *reinterpret_cast<const uint2 *>(r.sn + 8 * c);
        unsigned packed = pack_nibbles(nb);
        if (lo == 0 && hi == 8 && slot0 + 8 <= limit) {
            if (vec_v && sizeof(V) == 2) {
                *reinterpret_cast<uint4 *>(values + slot0) = *reinterpret_cast<const uint4 *>(r.sv + 8 * c);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) values[slot0 + j] = r.sv[8 * c + j];
            }
            deltas32[slot0 >> 3] = packed;
        } else {
            unsigned mask = 0xffffffffu << (4 * lo);
            if (hi < 8) mask &= ~(0xffffffffu << (4 * hi));
            for (int j = lo; j < hi; ++j) {
                if (slot0 + j < limit) {
                    values[slot0 + j] = r.sv[8 * c + j];
                } else {
                    mask &= ~(0xfu << (4 * j));
                    r.refused = true;
                }
            }
            if ((packed & mask) != 0u && slot0 < limit) atomicOr(deltas32 + (slot0 >> 3), packed & mask);
        }
    }
    __syncwarp();
    // the incomplete group moves to the front
    const int rest = r.fill & 7;
    V keep_v = 0;
    unsigned char keep_n = 0;
    if (lane < rest) { keep_v = r.sv[8 * n_full + lane]; keep_n = r.sn[8 * n_full + lane]; }
    __syncwarp();
    if (lane < rest) { r.sv[lane] = keep_v; r.sn[lane] = keep_n; }
    r.base += 8 * n_full;
    r.fill = rest;
    __syncwarp();
}

__global__ void __launch_bounds__(kThreads)
emit_rows_packed_kernel(const unsigned short *__restrict__ dense, int rows, int cols, bool vec_ok,
                        const int *__restrict__ row_indices, unsigned short *__restrict__ values,
                        unsigned *__restrict__ deltas32, int limit, unsigned nan_above, bool vec_v)
{
    __shared__ __align__(16) unsigned short ring_v[kWarpsPerCta][kRing];
    __shared__ __align__(8) unsigned char ring_n[kWarpsPerCta][kRing];
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= rows) return;
    // element indices fit 32 bits: the entry points refuse matrices of 2^31 elements or more, and a walk ends
    // less than 2048 elements behind its row
    const unsigned total = (unsigned)rows * (unsigned)cols;
    const unsigned row_lo = (unsigned)row * (unsigned)cols;
    const unsigned row_hi = row_lo + (unsigned)cols;
    const unsigned first = vec_ok ? (row_lo & ~7u) : row_lo;

    EmitRing<unsigned short> ring;
    ring.sv = ring_v[threadIdx.x >> 5];
    ring.sn = ring_n[threadIdx.x >> 5];
    const int out0 = min(max(row_indices[row], 0), limit);   // a corrupt offset cannot leave the buffers
    ring.base = out0 & ~7;
    ring.fill = out0 & 7;
    ring.own_lo = out0;
    ring.refused = row_indices[row] != out0;
    int carry_prev = -1;   // column of the last non-zero seen so far in this row

    for (unsigned group0 = first; group0 < row_hi; group0 += (unsigned)(kUnroll * kColsPerStep)) {
        unsigned ws[kUnroll][4];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
            load8(dense, group0 + (unsigned)(u * kColsPerStep + lane * kColsPerLane), total, vec_ok, ws[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const unsigned g0 = group0 + (unsigned)(u * kColsPerStep + lane * kColsPerLane);
            const unsigned (&w)[4] = ws[u];
            const int c0 = (int)(g0 - row_lo);  // column of element 0; may be negative on the first step
            unsigned nz = nonzero_bits(w);
            if (g0 < row_lo || g0 + 8u > row_hi) nz &= row_bits(g0, row_lo, row_hi);
            const unsigned any = __ballot_sync(0xffffffffu, nz != 0);
            if (any == 0) continue;  // warp-uniform
            const int my_last = c0 + (31 - __clz(nz | 1u));
            const int prev = prev_nonzero_before_lane(any, lane, my_last, carry_prev);
            const int c_first = c0 + __ffs(nz) - 1;   // meaningless when nz == 0
            int npad = nz ? (c_first - prev - 1) >> 4 : 0;

            // the pads in front of the step's first non-zero: the zeros behind carry_prev, by the whole warp
            const int leader = __ffs(any) - 1;
            const int lead_pads = __shfl_sync(0xffffffffu, npad, leader);
            if (lane == leader) npad = 0;
            for (int b0 = 0; b0 < lead_pads; b0 += 256) {
                const int n = min(256, lead_pads - b0);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int i = lane + 32 * q;
                    if (i < n) {
                        ring.sv[ring.fill + i] = __ldg(dense + row_lo + carry_prev + 16 * (b0 + i + 1));   // the +-0 it sits on
                        ring.sn[ring.fill + i] = 15;
                    }
                }
                ring.fill += n;
                if (ring.fill > kRingFlushAbove) ring_flush(ring, values, deltas32, limit, vec_v, false, lane);
            }
            carry_prev = __shfl_sync(0xffffffffu, my_last, 31 - __clz(any));

            const int mine = npad + __popc(nz);
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            const int step_total = __shfl_sync(0xffffffffu, incl, 31);
            int k = ring.fill + incl - mine;
            for (int q = 1; q <= npad; ++q) {           // rare: a gap of 16 or more zeros inside the step
                ring.sv[k] = __ldg(dense + row_lo + prev + 16 * q);
                ring.sn[k] = 15;
                ++k;
            }
            int before = prev;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (nz & (1u << i)) {
                    ring.sv[k] = canonical((unsigned short)((w[i >> 1] >> (16 * (i & 1))) & 0xffffu), nan_above);
                    ring.sn[k] = (unsigned char)((c0 + i - before - 1) & 15);
                    ++k;
                    before = c0 + i;
                }
            }
            ring.fill += step_total;
            if (ring.fill > kRingFlushAbove) ring_flush(ring, values, deltas32, limit, vec_v, false, lane);
        }
    }
    ring_flush(ring, values, deltas32, limit, vec_v, true, lane);
    if (row == rows - 1) {
        // everything from n = row_indices[rows] to the padded count is zero (the deltas already are)
        const int n = row_indices[rows];
        if (n < 0 || n > limit) ring.refused = true;   // row_indices and P do not belong together
        for (int i = max(n, 0) + lane; i < limit; i += 32) values[i] = 0;
    }
    if (__any_sync(0xffffffffu, ring.refused) && lane == 0) atomicAdd(&g_compress_overflow, 1u);
}

// In-place inclusive prefix sum over counts[1..rows]; counts[0] = 0. One CTA, four rows per thread
// and iteration.
__global__ void __launch_bounds__(1024) scan_rows_kernel(int *__restrict__ ri, int rows)
{
    __shared__ int warp_sums[32];
    __shared__ int carry_s;
    constexpr int kPerThread = 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { ri[0] = 0; carry_s = 0; }
    __syncthreads();
    for (int base = 0; base < rows; base += 1024 * kPerThread) {
        const int i0 = base + tid * kPerThread;
        int v[kPerThread];
        int mine = 0;
#pragma unroll
        for (int k = 0; k < kPerThread; ++k) {
            v[k] = i0 + k < rows ? ri[i0 + k + 1] : 0;
            mine += v[k];
            v[k] = mine;            // inclusive within the thread
        }
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += t;
        }
        if (lane == 31) warp_sums[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            int s = warp_sums[lane];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, s, o);
                if (lane >= o) s += t;
            }
            warp_sums[lane] = s;  // inclusive over warps
        }
        __syncthreads();
        const int before = carry_s + (warp ? warp_sums[warp - 1] : 0) + incl - mine;
#pragma unroll
        for (int k = 0; k < kPerThread; ++k)
            if (i0 + k < rows) ri[i0 + k + 1] = before + v[k];
        __syncthreads();
        if (tid == 0) carry_s += warp_sums[31];
        __syncthreads();
    }
}

// Packs 8 one-per-byte deltas into 4 bytes, zeroing everything at or beyond n = ri[rows];
// also zeroes values[n..P).
template <typename V>
__global__ void __launch_bounds__(256)
pack_kernel(const uint2 *__restrict__ nibbles8, const int *__restrict__ ri, int rows, int groups,
            unsigned *__restrict__ deltas32, V *__restrict__ values)
{
    const int g = blockIdx.x * 256 + threadIdx.x;
    if (g >= groups) return;   // every read and write below stays under 8 * groups = P
    const int n = ri[rows];
    if (g == 0 && (n < 0 || n > 8 * groups)) atomicAdd(&g_compress_overflow, 1u);   // row_indices and P do not belong together
    const int k0 = g * 8;
    unsigned packed = 0;
    if (k0 < n) {
        const uint2 b = nibbles8[g];
        const unsigned w[2] = {b.x, b.y};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const unsigned d = (w[i >> 2] >> (8 * (i & 3))) & 15u;
            if (k0 + i < n) packed |= d << (4 * i);
        }
    }
    deltas32[g] = packed;
    if (k0 + 8 > n) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (k0 + i >= n) values[k0 + i] = 0;
    }
}

// ---- int8 values ---------------------------------------------------------------------------------------
// The reference's int8 encoder (src/macko_spmv/cuda/cpu_compressor.cuh:75-117) differs from the fp16 one in
// two ways: a value is one signed byte, and trailing pads stay: a run of t zeros at the end of a row (or a
// whole empty row, t = cols) still emits floor(t / 16) pads (value 0, delta 15). Same walk as above, one warp
// per row, 8 columns per lane and step (one 64-bit load when the matrix is 8-byte aligned).
__device__ __forceinline__ void load8_bytes(const signed char *dense, unsigned g0, unsigned total, bool vec_ok,
                                            unsigned (&w)[2])
{
    if (vec_ok && g0 + 8u <= total) {
        const uint2 v = __ldg(reinterpret_cast<const uint2 *>(dense + g0));
        w[0] = v.x; w[1] = v.y;
    } else {
        w[0] = w[1] = 0u;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const unsigned g = g0 + j;
            const unsigned b = g < total ? (unsigned)(unsigned char)__ldg(dense + g) : 0u;
            w[j >> 2] |= b << (8 * (j & 3));
        }
    }
}

__device__ __forceinline__ unsigned nonzero_bytes(const unsigned (&w)[2])
{
    unsigned nz = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) nz |= (((w[j >> 2] >> (8 * (j & 3))) & 0xffu) != 0u ? 1u : 0u) << j;
    return nz;
}

template <bool EMIT>
__global__ void __launch_bounds__(kThreads)
compress_rows_int8_kernel(const signed char *__restrict__ dense, int rows, int cols, bool vec_ok,
                          int *__restrict__ row_counts_out, const int *__restrict__ row_indices,
                          signed char *__restrict__ values, unsigned char *__restrict__ nibbles, int limit)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
    if (row >= rows) return;
    // element indices fit 32 bits: the entry points refuse matrices of 2^31 elements or more, and a walk ends
    // less than 2048 elements behind its row
    const unsigned total = (unsigned)rows * (unsigned)cols;
    const unsigned row_lo = (unsigned)row * (unsigned)cols;
    const unsigned row_hi = row_lo + (unsigned)cols;
    const unsigned first = vec_ok ? (row_lo & ~7u) : row_lo;
    int carry_prev = -1;
    int count = 0;
    int out = EMIT ? row_indices[row] : 0;
    bool refused = false;
    for (unsigned group0 = first; group0 < row_hi; group0 += (unsigned)kColsPerStep) {
        const unsigned g0 = group0 + (unsigned)(lane * kColsPerLane);
        unsigned w[2];
        load8_bytes(dense, g0, total, vec_ok, w);
        const int c0 = (int)(g0 - row_lo);
        const unsigned nz = nonzero_bytes(w) & row_bits(g0, row_lo, row_hi);
        const unsigned any = __ballot_sync(0xffffffffu, nz != 0);
        if (any == 0) continue;
        const int my_last = c0 + (31 - __clz(nz | 1u));
        int prev = prev_nonzero_before_lane(any, lane, my_last, carry_prev);
        carry_prev = __shfl_sync(0xffffffffu, my_last, 31 - __clz(any));
        int mine = __popc(nz);
        if (nz) mine += (c0 + (__ffs(nz) - 1) - prev - 1) >> 4;
        if (!EMIT) {
            count += mine;
        } else {
            int incl = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += t;
            }
            int k = out + incl - mine;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (nz & (1u << i)) {
                    const int c = c0 + i;
                    for (int p = prev + 16; p < c; p += 16) {
                        if ((unsigned)k < (unsigned)limit) { values[k] = 0; nibbles[k] = 15; } else refused = true;
                        ++k;
                    }
                    if ((unsigned)k < (unsigned)limit) {
                        values[k] = (signed char)((w[i >> 2] >> (8 * (i & 3))) & 0xffu);
                        nibbles[k] = (unsigned char)((c - prev - 1) & 15);
                    } else {
                        refused = true;
                    }
                    ++k;
                    prev = c;
                }
            }
            out += __shfl_sync(0xffffffffu, incl, 31);
        }
    }
    // pads inside the zeros behind the last non-zero (the whole row when it has none)
    const int trailing = (cols - 1 - carry_prev) >> 4;
    if (!EMIT) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
        if (lane == 0) row_counts_out[row + 1] = count + trailing;
    } else {
        for (int i = lane; i < trailing; i += 32) {
            if ((unsigned)(out + i) < (unsigned)limit) { values[out + i] = 0; nibbles[out + i] = 15; } else refused = true;
        }
        if (__any_sync(0xffffffffu, refused) && lane == 0) atomicAdd(&g_compress_overflow, 1u);
    }
}

int check_dense(const void *dense, int64_t rows, int64_t cols, uintptr_t element_bytes = 2)
{
    if (rows < 0 || cols < 0) return fail(MACKO_ERR_INVALID_ARGUMENT, "negative size (rows=%lld cols=%lld)", (long long)rows, (long long)cols);
    if (rows > 0 && cols > 0 && rows > ((1LL << 31) - 1) / cols)
        return fail(MACKO_ERR_SIZE_OVERFLOW, "rows*cols = %lld*%lld does not fit 31 bits", (long long)rows, (long long)cols);
    if (rows >= (1LL << 31) - 1) return fail(MACKO_ERR_SIZE_OVERFLOW, "too many rows");
    if (rows * cols > 0 && !dense) return fail(MACKO_ERR_INVALID_ARGUMENT, "null dense matrix");
    if (!aligned(dense, element_bytes)) return fail(MACKO_ERR_MISALIGNED, "dense must be aligned to its element size");
    return MACKO_OK;
}

int launch_error(const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return MACKO_OK;
}


// ---- scratch for macko_compress_emit_static ------------------------------------------------------
// One delta per byte for up to kStaticScratchBytes stored elements. The array lives in the module's
// global memory: every device that loads the library carries it until the process exits.
constexpr long long kStaticScratchBytes = 16ll << 20;
static __device__ __align__(256) unsigned char g_emit_scratch[kStaticScratchBytes];

// Device address of g_emit_scratch on the current device. In host code the array's name only stands
// in for the symbol; the address a kernel may use has to be asked for, once per device, while that
// device is current.
int static_scratch_address(unsigned char **out)
{
    static unsigned char *addr[kMaxDevices] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(MACKO_ERR_CUDA, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!addr[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_emit_scratch);
        if (e != cudaSuccess || !p)
            return fail(MACKO_ERR_CUDA, "cudaGetSymbolAddress(g_emit_scratch): %s", cudaGetErrorString(e));
        addr[dev] = static_cast<unsigned char *>(p);
    }
    *out = addr[dev];
    return MACKO_OK;
}

}  // namespace

int launch_row_scan(int *counts, int rows, cudaStream_t stream)
{
    scan_rows_kernel<<<1, 1024, 0, stream>>>(counts, rows);
    return launch_error("row scan launch");
}

}  // namespace macko

extern "C" {

int macko_compress_count(const void *dense, int64_t rows, int64_t cols, int32_t *row_indices, void *stream)
{
    using namespace macko;
    int st = check_dense(dense, rows, cols);
    if (st != MACKO_OK) return st;
    if (!row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices");
    if (!aligned(row_indices, 4)) return fail(MACKO_ERR_MISALIGNED, "row_indices must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows > 0) {
        const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        compress_rows_kernel<false><<<grid, kThreads, 0, s>>>(
            static_cast<const unsigned short *>(dense), (int)rows, (int)cols, aligned(dense, 16),
            row_indices, nullptr, nullptr, nullptr, 0, 0u);
        st = launch_error("compress count launch");
        if (st != MACKO_OK) return st;
    }
    return launch_row_scan(row_indices, (int)rows, s);
}

int64_t macko_compress_workspace_bytes(int64_t padded_count) { return padded_count < 0 ? 0 : padded_count; }

static int compress_emit_typed(const void *dense, int64_t rows, int64_t cols, const int32_t *row_indices,
                               int64_t padded_count, void *values, void *deltas,
                               void *workspace, int64_t workspace_bytes, void *stream, unsigned nan_above)
{
    using namespace macko;
    int st = check_dense(dense, rows, cols);
    if (st != MACKO_OK) return st;
    if (!row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices");
    if (padded_count < 0 || padded_count % 8 != 0 || padded_count >= (1LL << 31))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "padded_count %lld must be a non-negative multiple of 8 below 2^31", (long long)padded_count);
    if (padded_count == 0) return MACKO_OK;
    if (!values || !deltas || !workspace) return fail(MACKO_ERR_INVALID_ARGUMENT, "null output or workspace");
    if (!aligned(values, 2) || !aligned(deltas, 4) || !aligned(workspace, 8))
        return fail(MACKO_ERR_MISALIGNED, "values needs 2-, deltas 4-, workspace 8-byte alignment");
    if (workspace_bytes < macko_compress_workspace_bytes(padded_count))
        return fail(MACKO_ERR_WORKSPACE, "workspace has %lld bytes, %lld needed", (long long)workspace_bytes,
                    (long long)macko_compress_workspace_bytes(padded_count));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Boundary groups of neighbouring rows merge their nibbles into one word: the deltas start at zero. The
    // workspace is not used any more by this entry point (its size is still checked: callers size it once).
    cudaError_t e = cudaMemsetAsync(deltas, 0, (size_t)padded_count / 2, s);
    if (e == cudaSuccess && rows == 0) e = cudaMemsetAsync(values, 0, (size_t)padded_count * 2, s);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "clearing the outputs: %s", cudaGetErrorString(e));
    if (rows > 0) {
        const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        emit_rows_packed_kernel<<<grid, kThreads, 0, s>>>(
            static_cast<const unsigned short *>(dense), (int)rows, (int)cols, aligned(dense, 16), row_indices,
            static_cast<unsigned short *>(values), static_cast<unsigned *>(deltas), (int)padded_count, nan_above,
            aligned(values, 16));
        st = launch_error("compress emit launch");
        if (st != MACKO_OK) return st;
    }
    return MACKO_OK;
}

int macko_compress_emit(const void *dense, int64_t rows, int64_t cols, const int32_t *row_indices,
                        int64_t padded_count, void *values, void *deltas,
                        void *workspace, int64_t workspace_bytes, void *stream)
{
    return compress_emit_typed(dense, rows, cols, row_indices, padded_count, values, deltas, workspace, workspace_bytes,
                               stream, 0x7c00u);
}

int macko_compress_emit_bf16(const void *dense, int64_t rows, int64_t cols, const int32_t *row_indices,
                             int64_t padded_count, void *values, void *deltas,
                             void *workspace, int64_t workspace_bytes, void *stream)
{
    return compress_emit_typed(dense, rows, cols, row_indices, padded_count, values, deltas, workspace, workspace_bytes,
                               stream, 0x7f80u);
}

int macko_compress_count_int8(const void *dense, int64_t rows, int64_t cols, int32_t *row_indices, void *stream)
{
    using namespace macko;
    int st = check_dense(dense, rows, cols, 1);
    if (st != MACKO_OK) return st;
    if (!row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices");
    if (!aligned(row_indices, 4)) return fail(MACKO_ERR_MISALIGNED, "row_indices must be 4-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows > 0) {
        const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        compress_rows_int8_kernel<false><<<grid, kThreads, 0, s>>>(
            static_cast<const signed char *>(dense), (int)rows, (int)cols, aligned(dense, 8), row_indices, nullptr, nullptr,
            nullptr, 0);
        st = launch_error("int8 compress count launch");
        if (st != MACKO_OK) return st;
    }
    return launch_row_scan(row_indices, (int)rows, s);
}

int macko_compress_emit_int8(const void *dense, int64_t rows, int64_t cols, const int32_t *row_indices,
                             int64_t padded_count, void *values, void *deltas,
                             void *workspace, int64_t workspace_bytes, void *stream)
{
    using namespace macko;
    int st = check_dense(dense, rows, cols, 1);
    if (st != MACKO_OK) return st;
    if (!row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices");
    if (padded_count < 0 || padded_count % 8 != 0 || padded_count >= (1LL << 31))
        return fail(MACKO_ERR_INVALID_ARGUMENT, "padded_count %lld must be a non-negative multiple of 8 below 2^31", (long long)padded_count);
    if (padded_count == 0) return MACKO_OK;
    if (!values || !deltas || !workspace) return fail(MACKO_ERR_INVALID_ARGUMENT, "null output or workspace");
    if (!aligned(deltas, 4) || !aligned(workspace, 8))
        return fail(MACKO_ERR_MISALIGNED, "deltas needs 4-, workspace 8-byte alignment");
    if (workspace_bytes < macko_compress_workspace_bytes(padded_count))
        return fail(MACKO_ERR_WORKSPACE, "workspace has %lld bytes, %lld needed", (long long)workspace_bytes,
                    (long long)macko_compress_workspace_bytes(padded_count));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows > 0) {
        const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        compress_rows_int8_kernel<true><<<grid, kThreads, 0, s>>>(
            static_cast<const signed char *>(dense), (int)rows, (int)cols, aligned(dense, 8), nullptr, row_indices,
            static_cast<signed char *>(values), static_cast<unsigned char *>(workspace), (int)padded_count);
        st = launch_error("int8 compress emit launch");
        if (st != MACKO_OK) return st;
    }
    const int groups = (int)(padded_count / 8);
    pack_kernel<signed char><<<(groups + 255) / 256, 256, 0, s>>>(
        static_cast<const uint2 *>(workspace), row_indices, (int)rows, groups,
        static_cast<unsigned *>(deltas), static_cast<signed char *>(values));
    return launch_error("int8 pack launch");
}

int macko_compress_overflow(uint32_t *count, void *stream)
{
    using namespace macko;
    if (!count) return fail(MACKO_ERR_INVALID_ARGUMENT, "null count");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned seen = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(&seen, g_compress_overflow, sizeof(seen), 0, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e == cudaSuccess && seen != 0) {
        const unsigned zero = 0;
        e = cudaMemcpyToSymbolAsync(g_compress_overflow, &zero, sizeof(zero), 0, cudaMemcpyHostToDevice, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    }
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "reading the compressor's overflow word: %s", cudaGetErrorString(e));
    *count = seen;
    return MACKO_OK;
}

int64_t macko_compress_static_capacity(void) { return macko::kStaticScratchBytes; }

int macko_compress_emit_static(const void *dense, int64_t rows, int64_t cols, const int32_t *row_indices,
                               int64_t padded_count, void *values, void *deltas, void *stream)
{
    using namespace macko;
    int st = check_dense(dense, rows, cols);
    if (st != MACKO_OK) return st;
    if (!row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null row_indices");
    if (padded_count < 0 || padded_count % 8 != 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "padded_count %lld must be a non-negative multiple of 8", (long long)padded_count);
    if (padded_count > kStaticScratchBytes)
        return fail(MACKO_ERR_WORKSPACE,
                    "padded_count %lld exceeds the built-in scratch of %lld stored elements; "
                    "use macko_compress_emit with a caller-provided workspace",
                    (long long)padded_count, (long long)kStaticScratchBytes);
    if (padded_count == 0) return MACKO_OK;
    if (!values || !deltas) return fail(MACKO_ERR_INVALID_ARGUMENT, "null output");
    if (!aligned(values, 2) || !aligned(deltas, 4))
        return fail(MACKO_ERR_MISALIGNED, "values needs 2-, deltas 4-byte alignment");
    unsigned char *scratch = nullptr;
    st = static_scratch_address(&scratch);   // first call on a device: resolves the symbol
    if (st != MACKO_OK) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Nothing in the scratch has to start at zero: the emit kernel writes every slot below
    // n = row_indices[rows] and the pack kernel reads no slot at or above n.
    if (rows > 0) {
        const unsigned grid = (unsigned)((rows + kWarpsPerCta - 1) / kWarpsPerCta);
        compress_rows_kernel<true><<<grid, kThreads, 0, s>>>(
            static_cast<const unsigned short *>(dense), (int)rows, (int)cols, aligned(dense, 16),
            nullptr, row_indices, static_cast<unsigned short *>(values), scratch, (int)padded_count, 0x7c00u);
        st = launch_error("compress emit (static scratch) launch");
        if (st != MACKO_OK) return st;
    }
    const int groups = (int)(padded_count / 8);
    pack_kernel<unsigned short><<<(groups + 255) / 256, 256, 0, s>>>(
        reinterpret_cast<const uint2 *>(scratch), row_indices, (int)rows, groups,
        static_cast<unsigned *>(deltas), static_cast<unsigned short *>(values));
    return launch_error("pack (static scratch) launch");
}
}
