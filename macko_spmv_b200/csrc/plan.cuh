// Side metadata of a planned SpMV launch ("plan"): the rows of a compressed matrix cut into virtual rows of
// bounded length, sorted by length. It is derived from row_indices and deltas once per matrix and leaves the
// three MACKO buffers untouched (the reference has no such structure: its kernel walks one row per warp,
// src/macko_spmv/cuda/kernels.cuh:41-60).
//
// A virtual row is a run of stored elements of one row: the whole row when it is short, else a segment
// [a0 + j*S, a0 + (j+1)*S) of it, a0 = the row's first element rounded down to a multiple of 8, so that every
// segment but the first starts on an 8-element unit. For each one the plan keeps where it starts, how long it
// is, the column sum in front of it (sum of delta + 1 over the row's elements before the segment: what the
// decode needs to continue in the middle of a row) and where its result goes.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace macko {

constexpr int kPlanLenBits = 12;                         // a virtual row holds fewer than 4096 stored elements
constexpr int kPlanMaxSegment = 3840;                    // largest segment length (a multiple of 256)
constexpr int kPlanDefaultSegment = 1536;
constexpr int kPlanBuckets = 64;                         // length classes: 64-element sub-steps spanned, 0..60
constexpr unsigned kPlanPartialBit = 0x80000000u;        // destination word: a partial-sum slot, not a row of y

// Pointers into a plan buffer, as the SpMV kernel sees it.
struct PlanView {
    const uint2 *desc;      // sorted: {first stored element, length | column sum in front << kPlanLenBits}
    const unsigned *out;    // sorted: row of y, or kPlanPartialBit | natural index of the segment
    const unsigned *vrow;   // natural order: row of each virtual row
    float *partial;         // natural order: fp32 sums of the segments of rows cut into several
    const int *seg_first;   // [rows + 1] natural index of the first virtual row of each row
    const unsigned *split_list;   // rows cut into several segments (in no particular order)
    int n_split;
    int n_virtual;
};

// Byte offsets of the sections of a plan buffer for a matrix of `rows` rows and `padded` stored elements cut
// into segments of `seg` elements. Pure arithmetic, shared by the builder and the launcher.
struct PlanLayout {
    long long v_max;        // upper bound of the number of virtual rows
    long long header, seg_first, split_list, desc, out, vrow, partial, tmp_begin, tmp_pk, tmp_out, block_hist, total;
};

inline PlanLayout plan_layout(long long rows, long long padded, int seg)
{
    auto up = [](long long b) { return (b + 255) & ~255LL; };
    PlanLayout l{};
    // every row gives at least one virtual row; a row of n elements starting at offset o (< 8) inside its first
    // unit gives ceil((o + n) / seg) <= 1 + (n + 7) / seg
    l.v_max = rows + (padded + 8 * rows) / seg + 1;
    const long long blocks = (l.v_max + 1023) / 1024;
    long long at = 0;
    l.header = at;      at = up(at + 64);
    l.seg_first = at;   at = up(at + 4 * (rows + 1));
    l.split_list = at;  at = up(at + 4 * (rows + 1));
    l.desc = at;        at = up(at + 8 * l.v_max);
    l.out = at;         at = up(at + 4 * l.v_max);
    l.vrow = at;        at = up(at + 4 * l.v_max);
    l.partial = at;     at = up(at + 4 * l.v_max);
    l.tmp_begin = at;   at = up(at + 4 * l.v_max);
    l.tmp_pk = at;      at = up(at + 4 * l.v_max);
    l.tmp_out = at;     at = up(at + 4 * l.v_max);
    l.block_hist = at;  at = up(at + 4 * (blocks + 1) * kPlanBuckets);
    l.total = at;
    return l;
}

// Length class of a virtual row: 64-element sub-steps between the unit its first element sits in and its end.
__host__ __device__ inline int plan_length_class(int begin, int len)
{
    return ((begin & 7) + len + 63) >> 6;
}

}  // namespace macko
