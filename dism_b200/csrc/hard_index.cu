// Position index: the positions of one side of every (batch, head), sorted by
// (label bucket, position).  One CTA per (batch, head) runs a stable two-pass counting sort
// (64 bins per pass, 4096 buckets in all); with that many buckets a bucket almost always holds a
// single label, so a row's partners are one contiguous, position-ordered range of the index.
#include "dism_common.cuh"

namespace dism {

constexpr int INDEX_THREADS = 1024;
constexpr int PASS_BINS = 64;
static_assert(PASS_BINS * PASS_BINS == BUCKETS, "two passes cover the bucket number");

// One stable counting pass over n items of this (batch, head).  FIRST reads labels in position
// order and sorts by the low six bucket bits; the second pass reads the first pass's entries and
// sorts by the high six bits.
template <bool FIRST>
__device__ __forceinline__ void counting_pass(const int* __restrict__ labels, const int2* __restrict__ source,
                                              int2* __restrict__ target, int* __restrict__ previous, int n, int* base,
                                              int* total, unsigned short (*counts)[PASS_BINS]) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < PASS_BINS) total[tid] = 0;
    __syncthreads();
    for (int at = tid; at < n; at += INDEX_THREADS) {
        const int bucket = bucket_of(FIRST ? labels[at] : source[at].y);
        atomicAdd(&total[FIRST ? bucket & (PASS_BINS - 1) : bucket >> 6], 1);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the 64 bin sizes, two per lane
        const int a = total[2 * lane], b = total[2 * lane + 1];
        int prefix = a + b;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        prefix -= a + b;
        base[2 * lane] = prefix;
        base[2 * lane + 1] = prefix + a;
    }
    __syncthreads();
    for (int chunk = 0; chunk < n; chunk += INDEX_THREADS) {
        const int at = chunk + tid;
        const bool valid = at < n;
        int2 item = make_int2(0, 0);
        if (valid) item = FIRST ? make_int2(at, labels[at]) : source[at];
        const int bucket = bucket_of(item.y);
        const int bin = valid ? (FIRST ? bucket & (PASS_BINS - 1) : bucket >> 6) : PASS_BINS;  // invalid lanes pair up only with each other
        for (int e = tid; e < (INDEX_THREADS / 32) * PASS_BINS; e += INDEX_THREADS) (&counts[0][0])[e] = 0;
        __syncthreads();
        const unsigned peers = __match_any_sync(FULL, bin);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (valid && rank == 0) counts[warp][bin] = (unsigned short)__popc(peers);
        __syncthreads();
        if (tid < PASS_BINS) {  // exclusive prefix over the warps, which are in input order
            int running = 0;
            for (int w = 0; w < INDEX_THREADS / 32; ++w) {
                const int c = counts[w][tid];
                counts[w][tid] = (unsigned short)running;
                running += c;
            }
            total[tid] = running;
        }
        __syncthreads();
        if (valid) {
            const int to = base[bin] + counts[warp][bin] + rank;
            target[to] = item;
            if (!FIRST) previous[to] = item.x > 0 ? labels[item.x - 1] : 0;
        }
        __syncthreads();
        if (tid < PASS_BINS) base[tid] += total[tid];
        __syncthreads();
    }
}

// Where one side's index goes, and the labels it is built from.
struct IndexSide {
    const int* labels;
    int2 *entries, *scratch;
    int *previous, *starts;
};

// blockIdx.y picks the side: both sides of a readout are built by one launch, two CTAs to an SM.
__global__ __launch_bounds__(INDEX_THREADS, 2) void build_index_kernel(const IndexSide side0, const IndexSide side1, int n) {
    const IndexSide& side = blockIdx.y ? side1 : side0;
    const int* __restrict__ labels = side.labels;
    int2* __restrict__ entries = side.entries;
    int2* __restrict__ scratch = side.scratch;
    int* __restrict__ previous = side.previous;
    int* __restrict__ starts = side.starts;
    __shared__ int base[PASS_BINS], total[PASS_BINS];
    __shared__ unsigned short counts[INDEX_THREADS / 32][PASS_BINS];
    __shared__ int histogram[BUCKETS];
    __shared__ int warp_sum[INDEX_THREADS / 32];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    labels += int64_t(blockIdx.x) * n;
    entries += int64_t(blockIdx.x) * n;
    scratch += int64_t(blockIdx.x) * n;
    previous += int64_t(blockIdx.x) * n;
    starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    // bucket starts: histogram of all 4096 buckets and its exclusive scan (four buckets per thread)
    for (int e = tid; e < BUCKETS; e += INDEX_THREADS) histogram[e] = 0;
    __syncthreads();
    for (int at = tid; at < n; at += INDEX_THREADS) atomicAdd(&histogram[bucket_of(labels[at])], 1);
    __syncthreads();
    {
        constexpr int PER = BUCKETS / INDEX_THREADS;
        int local[PER], sum = 0;
#pragma unroll
        for (int e = 0; e < PER; ++e) { local[e] = sum; sum += histogram[tid * PER + e]; }
        int prefix = sum;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        if (lane == 31) warp_sum[warp] = prefix;
        __syncthreads();
        if (warp == 0) {
            const int mine = warp_sum[lane];
            int scan = mine;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, scan, s);
                if (lane >= s) scan += other;
            }
            warp_sum[lane] = scan - mine;
        }
        __syncthreads();
        const int before = warp_sum[warp] + prefix - sum;
#pragma unroll
        for (int e = 0; e < PER; ++e) starts[tid * PER + e] = before + local[e];
        if (tid == INDEX_THREADS - 1) starts[BUCKETS] = n;
    }
    __syncthreads();
    counting_pass<true>(labels, nullptr, scratch, nullptr, n, base, total, counts);
    __syncthreads();
    counting_pass<false>(labels, scratch, entries, previous, n, base, total, counts);
}

// Per side: entries int2 [BH, N], sort scratch int2 [BH, N], previous int [BH, N], starts int [BH, BUCKETS + 1].
size_t index_bytes(int batch_heads, int n, int sides) {
    size_t one = size_t(batch_heads) * n * (2 * sizeof(int2) + sizeof(int)) + size_t(batch_heads) * (BUCKETS + 1) * sizeof(int);
    one = (one + 255) & ~size_t(255);
    return one * sides;
}

SideIndex side_index(void* workspace, int batch_heads, int n, int side, int sides) {
    const size_t one = index_bytes(batch_heads, n, 1);
    char* p = static_cast<char*>(workspace) + one * side;
    (void)sides;
    const size_t items = size_t(batch_heads) * n;
    return SideIndex{reinterpret_cast<const int2*>(p), reinterpret_cast<const int*>(p + items * (2 * sizeof(int2) + sizeof(int))),
                     reinterpret_cast<const int*>(p + items * 2 * sizeof(int2))};
}

static IndexSide index_side(const int* labels, void* workspace, int batch_heads, int n, int side, int sides) {
    const SideIndex index = side_index(workspace, batch_heads, n, side, sides);
    int2* entries = const_cast<int2*>(index.entries);
    return IndexSide{labels, entries, entries + size_t(batch_heads) * n, const_cast<int*>(index.previous), const_cast<int*>(index.starts)};
}

cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream) {
    const IndexSide target = index_side(labels, workspace, batch_heads, n, side, sides);
    KernelTimer timer("build_index", stream);
    build_index_kernel<<<dim3(batch_heads, 1), INDEX_THREADS, 0, stream>>>(target, target, n);
    return cudaGetLastError();
}

cudaError_t launch_build_index_pair(const int* labels0, const int* labels1, int batch_heads, int n, void* workspace,
                                    cudaStream_t stream) {
    KernelTimer timer("build_index", stream);
    build_index_kernel<<<dim3(batch_heads, 2), INDEX_THREADS, 0, stream>>>(index_side(labels0, workspace, batch_heads, n, 0, 2),
                                                                             index_side(labels1, workspace, batch_heads, n, 1, 2), n);
    return cudaGetLastError();
}

}  // namespace dism
