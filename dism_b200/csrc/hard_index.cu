// Position index: the positions of one side of every (batch, head), sorted by
// (label bucket, position) with a stable counting sort, one CTA per (batch, head).
#include "dism_common.cuh"

namespace dism {

constexpr int INDEX_THREADS = 1024;

__global__ __launch_bounds__(INDEX_THREADS) void build_index_kernel(const int* __restrict__ labels, int n,
                                                                    int2* __restrict__ entries,
                                                                    int* __restrict__ starts) {
    __shared__ int base[BUCKETS], total[BUCKETS];
    __shared__ unsigned short counts[INDEX_THREADS / 32][BUCKETS];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    labels += int64_t(blockIdx.x) * n;
    entries += int64_t(blockIdx.x) * n;
    starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    if (tid < BUCKETS) total[tid] = 0;
    __syncthreads();
    for (int pos = tid; pos < n; pos += INDEX_THREADS) atomicAdd(&total[bucket_of(labels[pos])], 1);
    __syncthreads();
    if (warp == 0) {  // exclusive scan of the 256 bucket sizes, 8 per lane
        int local[BUCKETS / 32], sum = 0;
#pragma unroll
        for (int e = 0; e < BUCKETS / 32; ++e) { local[e] = sum; sum += total[lane * (BUCKETS / 32) + e]; }
        int prefix = sum;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        prefix -= sum;
#pragma unroll
        for (int e = 0; e < BUCKETS / 32; ++e) {
            base[lane * (BUCKETS / 32) + e] = prefix + local[e];
            starts[lane * (BUCKETS / 32) + e] = prefix + local[e];
        }
        if (lane == 31) starts[BUCKETS] = n;
    }
    __syncthreads();
    for (int chunk = 0; chunk < n; chunk += INDEX_THREADS) {
        const int pos = chunk + tid;
        const bool valid = pos < n;
        const int label = valid ? labels[pos] : 0;
        const int bucket = valid ? bucket_of(label) : BUCKETS;  // invalid lanes match only each other
        for (int e = tid; e < (INDEX_THREADS / 32) * BUCKETS; e += INDEX_THREADS) (&counts[0][0])[e] = 0;
        __syncthreads();
        const unsigned peers = __match_any_sync(FULL, bucket);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        if (valid && rank == 0) counts[warp][bucket] = (unsigned short)__popc(peers);
        __syncthreads();
        if (tid < BUCKETS) {  // exclusive prefix over the warps, in position order
            int running = 0;
            for (int w = 0; w < INDEX_THREADS / 32; ++w) {
                const int c = counts[w][tid];
                counts[w][tid] = (unsigned short)running;
                running += c;
            }
            total[tid] = running;
        }
        __syncthreads();
        if (valid) entries[base[bucket] + counts[warp][bucket] + rank] = make_int2(pos, label);
        __syncthreads();
        if (tid < BUCKETS) base[tid] += total[tid];
        __syncthreads();
    }
}

size_t index_bytes(int batch_heads, int n, int sides) {
    size_t one = size_t(batch_heads) * n * sizeof(int2) + size_t(batch_heads) * (BUCKETS + 1) * sizeof(int);
    one = (one + 255) & ~size_t(255);
    return one * sides;
}

SideIndex side_index(void* workspace, int batch_heads, int n, int side, int sides) {
    const size_t one = index_bytes(batch_heads, n, 1);
    char* p = static_cast<char*>(workspace) + one * side;
    (void)sides;
    return SideIndex{reinterpret_cast<const int2*>(p),
                     reinterpret_cast<const int*>(p + size_t(batch_heads) * n * sizeof(int2))};
}

cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream) {
    SideIndex index = side_index(workspace, batch_heads, n, side, sides);
    KernelTimer timer("build_index", stream);
    build_index_kernel<<<batch_heads, INDEX_THREADS, 0, stream>>>(labels, n, const_cast<int2*>(index.entries),
                                                                  const_cast<int*>(index.starts));
    return cudaGetLastError();
}

}  // namespace dism
