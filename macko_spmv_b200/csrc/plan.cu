// Builds the plan of a compressed matrix on the GPU (see plan.cuh): rows -> virtual rows of at most `seg`
// stored elements, each with the column sum in front of it, stably sorted by length class (longest first).
// One-off work per matrix: five small kernels and one read-back of the counts.
#include "common.cuh"
#include "plan.cuh"

namespace macko {
namespace {

__device__ __forceinline__ void row_span(const int *__restrict__ ri, int row, int stored, int &b, int &e)
{
    b = min(max(__ldg(ri + row), 0), stored);
    e = min(max(__ldg(ri + row + 1), b), stored);
}

// Virtual rows per row -> seg_first[row + 1]; longest row and number of split rows -> header.
__global__ void __launch_bounds__(256)
plan_count_kernel(const int *__restrict__ ri, int rows, int stored, int seg, int *__restrict__ seg_first,
                  unsigned *__restrict__ header)
{
    const int row = blockIdx.x * 256 + threadIdx.x;
    if (row >= rows) return;
    int b, e;
    row_span(ri, row, stored, b, e);
    const int n = e - b;
    const int nseg = n > 0 ? (e - (b & ~7) + seg - 1) / seg : 1;
    seg_first[row + 1] = nseg;
    atomicMax(header + 1, (unsigned)n);
    if (nseg > 1) atomicAdd(header + 2, 1u);
}

// One warp per row: the descriptors of its virtual rows in natural order. A row cut into several segments
// is walked once over its deltas (256 per step) to get the column sum in front of every segment.
__global__ void __launch_bounds__(256)
plan_segments_kernel(const unsigned *__restrict__ deltas32, const int *__restrict__ ri, int rows, int stored, int seg,
                     const int *__restrict__ seg_first, int *__restrict__ tmp_begin, unsigned *__restrict__ tmp_pk,
                     unsigned *__restrict__ tmp_out, unsigned *__restrict__ vrow, unsigned *__restrict__ split_list,
                     unsigned *__restrict__ header)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;
    int b, e;
    row_span(ri, row, stored, b, e);
    const int first = seg_first[row];
    const int nseg = seg_first[row + 1] - first;
    if (nseg <= 1) {
        if (lane == 0) {
            tmp_begin[first] = b;
            tmp_pk[first] = (unsigned)(e - b);
            tmp_out[first] = (unsigned)row;
            vrow[first] = (unsigned)row;
        }
        return;
    }
    if (lane == 0) split_list[atomicAdd(header + 3, 1u)] = (unsigned)row;   // the rows the combining pass has to visit
    const int a0 = b & ~7;
    unsigned running = 0;   // sum of (delta + 1) over the row's elements in front of the current step
    for (int base = a0; base < e; base += 256) {
        if ((base - a0) % seg == 0 && lane == 0) {
            const int j = (base - a0) / seg;
            const int sb = max(b, base), se = min(e, base + seg);
            tmp_begin[first + j] = sb;
            tmp_pk[first + j] = (unsigned)(se - sb) | (running << kPlanLenBits);
            tmp_out[first + j] = kPlanPartialBit | (unsigned)(first + j);
            vrow[first + j] = (unsigned)row;
        }
        const int k0 = base + 8 * lane;
        unsigned mine = 0;
        if (k0 < e) {
            const unsigned w = __ldg(deltas32 + (k0 >> 3));
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (k0 + i >= b && k0 + i < e) mine += ((w >> (4 * i)) & 15u) + 1u;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
        running += mine;
    }
}

__device__ __forceinline__ int bucket_of(int begin, unsigned pk)
{
    const int cls = min(plan_length_class(begin, (int)(pk & ((1u << kPlanLenBits) - 1u))), kPlanBuckets - 1);
    return kPlanBuckets - 1 - cls;   // ascending bucket = descending length
}

// Stable counting sort by bucket, step 1: histogram of every block of 1024 virtual rows.
__global__ void __launch_bounds__(1024)
plan_hist_kernel(const int *__restrict__ seg_first, int rows, const int *__restrict__ tmp_begin,
                 const unsigned *__restrict__ tmp_pk, unsigned *__restrict__ block_hist)
{
    __shared__ unsigned hist[kPlanBuckets];
    if (threadIdx.x < kPlanBuckets) hist[threadIdx.x] = 0;
    __syncthreads();
    const int n = seg_first[rows];
    const int v = blockIdx.x * 1024 + threadIdx.x;
    if (v < n) atomicAdd(&hist[bucket_of(tmp_begin[v], tmp_pk[v])], 1u);
    __syncthreads();
    if (threadIdx.x < kPlanBuckets) block_hist[(size_t)blockIdx.x * kPlanBuckets + threadIdx.x] = hist[threadIdx.x];
}

// Step 2 (one CTA of kPlanBuckets threads): block_hist[block][bucket] -> first sorted index of that block's
// members of that bucket. Also writes the number of virtual rows into the header.
__global__ void __launch_bounds__(kPlanBuckets)
plan_offsets_kernel(unsigned *__restrict__ block_hist, int blocks, const int *__restrict__ seg_first, int rows,
                    unsigned *__restrict__ header)
{
    __shared__ unsigned totals[kPlanBuckets];
    const int d = threadIdx.x;
    unsigned run = 0;
    for (int blk = 0; blk < blocks; ++blk) {
        const unsigned t = block_hist[(size_t)blk * kPlanBuckets + d];
        block_hist[(size_t)blk * kPlanBuckets + d] = run;
        run += t;
    }
    totals[d] = run;
    __syncthreads();
    unsigned base = 0;
    for (int k = 0; k < d; ++k) base += totals[k];
    for (int blk = 0; blk < blocks; ++blk) block_hist[(size_t)blk * kPlanBuckets + d] += base;
    if (d == 0) header[0] = (unsigned)seg_first[rows];
}

// Step 3: every virtual row to its sorted place; members of one bucket keep their natural order.
__global__ void __launch_bounds__(1024)
plan_scatter_kernel(const int *__restrict__ seg_first, int rows, const int *__restrict__ tmp_begin,
                    const unsigned *__restrict__ tmp_pk, const unsigned *__restrict__ tmp_out,
                    const unsigned *__restrict__ block_hist, uint2 *__restrict__ desc, unsigned *__restrict__ out)
{
    __shared__ unsigned cnt[32][kPlanBuckets];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 32 * kPlanBuckets; i += 1024) (&cnt[0][0])[i] = 0;
    __syncthreads();
    const int n = seg_first[rows];
    const int v = blockIdx.x * 1024 + tid;
    const bool live = v < n;
    int begin = 0;
    unsigned pk = 0;
    int d = kPlanBuckets;   // lanes without a virtual row form a class of their own
    if (live) {
        begin = tmp_begin[v];
        pk = tmp_pk[v];
        d = bucket_of(begin, pk);
    }
    const unsigned same = __match_any_sync(0xffffffffu, d);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (live && rank_in_warp == 0) cnt[warp][d] = (unsigned)__popc(same);
    __syncthreads();
    if (tid < kPlanBuckets) {   // exclusive prefix over the warps of the block, per bucket
        unsigned run = 0;
        for (int w = 0; w < 32; ++w) {
            const unsigned t = cnt[w][tid];
            cnt[w][tid] = run;
            run += t;
        }
    }
    __syncthreads();
    if (live) {
        const unsigned at = block_hist[(size_t)blockIdx.x * kPlanBuckets + d] + cnt[warp][d] + (unsigned)rank_in_warp;
        desc[at] = make_uint2((unsigned)begin, pk);
        out[at] = tmp_out[v];
    }
}

}  // namespace

int check_plan_args(int64_t rows, int64_t cols, int64_t padded_count, int32_t segment_elements, int *seg_out)
{
    if (rows < 0 || cols < 0 || padded_count < 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "negative size (rows=%lld cols=%lld P=%lld)", (long long)rows,
                    (long long)cols, (long long)padded_count);
    if (rows >= (1LL << 30) || padded_count >= (1LL << 31) || cols >= (1LL << (32 - kPlanLenBits)))
        return fail(MACKO_ERR_SIZE_OVERFLOW, "rows=%lld cols=%lld P=%lld are beyond what a plan can index",
                    (long long)rows, (long long)cols, (long long)padded_count);
    const int seg = segment_elements == 0 ? kPlanDefaultSegment : segment_elements;
    if (seg < 256 || seg > kPlanMaxSegment || seg % 256 != 0)
        return fail(MACKO_ERR_INVALID_ARGUMENT, "segment_elements must be 0 or a multiple of 256 in [256, %d] (got %d)",
                    kPlanMaxSegment, segment_elements);
    *seg_out = seg;
    return MACKO_OK;
}

}  // namespace macko

extern "C" {

int64_t macko_spmv_plan_bytes(int64_t rows, int64_t cols, int64_t padded_count, int32_t segment_elements)
{
    using namespace macko;
    int seg = 0;
    if (check_plan_args(rows, cols, padded_count, segment_elements, &seg) != MACKO_OK) return -1;
    return plan_layout(rows, padded_count, seg).total;
}

int macko_spmv_plan(const void *deltas, const int32_t *row_indices, int64_t rows, int64_t cols, int64_t padded_count,
                    int32_t segment_elements, void *plan, int64_t plan_bytes, macko_spmv_plan_info *info, void *stream)
{
    using namespace macko;
    int seg = 0;
    int st = check_plan_args(rows, cols, padded_count, segment_elements, &seg);
    if (st != MACKO_OK) return st;
    if (!plan || !info || !row_indices) return fail(MACKO_ERR_INVALID_ARGUMENT, "null plan, info or row_indices");
    if (padded_count > 0 && !deltas) return fail(MACKO_ERR_INVALID_ARGUMENT, "null deltas");
    if (!aligned(plan, 16) || !aligned(deltas, 4) || !aligned(row_indices, 4))
        return fail(MACKO_ERR_MISALIGNED, "plan needs 16-, deltas and row_indices 4-byte alignment");
    const PlanLayout lay = plan_layout(rows, padded_count, seg);
    if (plan_bytes < lay.total)
        return fail(MACKO_ERR_WORKSPACE, "plan buffer has %lld bytes, %lld needed", (long long)plan_bytes, (long long)lay.total);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    char *base = static_cast<char *>(plan);
    unsigned *header = reinterpret_cast<unsigned *>(base + lay.header);
    int *seg_first = reinterpret_cast<int *>(base + lay.seg_first);
    unsigned *split_list = reinterpret_cast<unsigned *>(base + lay.split_list);
    uint2 *desc = reinterpret_cast<uint2 *>(base + lay.desc);
    unsigned *out = reinterpret_cast<unsigned *>(base + lay.out);
    unsigned *vrow = reinterpret_cast<unsigned *>(base + lay.vrow);
    int *tmp_begin = reinterpret_cast<int *>(base + lay.tmp_begin);
    unsigned *tmp_pk = reinterpret_cast<unsigned *>(base + lay.tmp_pk);
    unsigned *tmp_out = reinterpret_cast<unsigned *>(base + lay.tmp_out);
    unsigned *block_hist = reinterpret_cast<unsigned *>(base + lay.block_hist);
    const int blocks = (int)((lay.v_max + 1023) / 1024);
    const int r = (int)rows, stored = (int)padded_count;

    cudaError_t e = cudaMemsetAsync(header, 0, 64, s);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "plan memset: %s", cudaGetErrorString(e));
    if (rows > 0)
        plan_count_kernel<<<(r + 255) / 256, 256, 0, s>>>(row_indices, r, stored, seg, seg_first, header);
    st = launch_row_scan(seg_first, r, s);
    if (st != MACKO_OK) return st;
    if (rows > 0)
        plan_segments_kernel<<<(r + 7) / 8, 256, 0, s>>>(static_cast<const unsigned *>(deltas), row_indices, r, stored, seg,
                                                         seg_first, tmp_begin, tmp_pk, tmp_out, vrow, split_list, header);
    plan_hist_kernel<<<blocks, 1024, 0, s>>>(seg_first, r, tmp_begin, tmp_pk, block_hist);
    plan_offsets_kernel<<<1, kPlanBuckets, 0, s>>>(block_hist, blocks, seg_first, r, header);
    plan_scatter_kernel<<<blocks, 1024, 0, s>>>(seg_first, r, tmp_begin, tmp_pk, tmp_out, block_hist, desc, out);
    e = cudaGetLastError();
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "plan launch: %s", cudaGetErrorString(e));
    unsigned host_header[4] = {0, 0, 0, 0};
    e = cudaMemcpyAsync(host_header, header, sizeof(host_header), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return fail(MACKO_ERR_CUDA, "plan read-back: %s", cudaGetErrorString(e));

    *info = macko_spmv_plan_info{};
    info->plan_bytes = lay.total;
    info->rows = rows;
    info->padded_count = padded_count;
    info->virtual_rows = (int32_t)host_header[0];
    info->segment_elements = seg;
    info->longest_row = (int32_t)host_header[1];
    info->split_rows = (int32_t)host_header[2];
    // Worth it when rows are long enough to be cut (a row is a serial chain of sub-steps for the lanes that walk
    // it) or when some rows are far longer than the average (the plain launch gives every warp the same number
    // of rows, not the same number of elements).
    const long long mean = rows > 0 ? padded_count / rows : 0;
    info->recommended = (info->longest_row > 2 * seg && (long long)info->longest_row >= 3 * mean) ? 1 : 0;
    return MACKO_OK;
}
}
