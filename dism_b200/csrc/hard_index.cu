// Position index: the positions of one side of every (batch, head), sorted by
// (label bucket, position).  One CTA per (batch, head, side) runs a stable two-pass counting sort
// (64 bins per pass, 4096 buckets in all); with that many buckets a bucket almost always holds a
// single label, so a row's partners are one contiguous, position-ordered range of the index.
// Every entry travels with the label one position before it, which the readout kernels compare to
// find pairs whose run is longer than one.
//
// A pass moves the items in rounds of eight per thread.  Inside a round every warp-sized group of
// consecutive items (a slot) counts its items per bin with seven warp votes; an exclusive prefix of
// those counts over the slots, which are in input order, gives each item its place.  The prefix is
// the only serial part: sixteen slots per thread and one exchange of part totals per round.  Items
// are first put in order in shared memory and leave from there, so that consecutive threads write
// consecutive entries: a scattered 8-byte store costs the SM a cycle per lane.
#include <cooperative_groups.h>

#include "dism_common.cuh"

namespace dism {

constexpr int PASS_BINS = 64, PER_THREAD = 8, SLOTS_PER_PART = 16;
static_assert(PASS_BINS * PASS_BINS == BUCKETS, "two passes cover the bucket number");

// Where one side's index goes, and the labels it is built from.
struct IndexSide {
    const int* labels;
    int2 *entries, *scratch;
    int *previous, *scratch_previous, *starts;
};

template <int THREADS>
struct IndexShared {
    static constexpr int ITEMS = THREADS * PER_THREAD, SLOTS = ITEMS / 32, PARTS = SLOTS / SLOTS_PER_PART;
    static_assert(PARTS * PASS_BINS == THREADS, "one thread per (bin, part) of the slot prefix");
    union {
        int histogram[BUCKETS];                    // bucket sizes, until the pass bases are known
        unsigned short counts[SLOTS][PASS_BINS];   // then: items per (slot, bin) of a round, turned into their exclusive prefix
    };
    int2 staged[ITEMS];            // the round's items in output order
    int staged_previous[ITEMS];
    int part_total[PARTS][PASS_BINS];
    int base[2][PASS_BINS];        // per pass: where the next item of a bin goes
    int local_base[PASS_BINS];     // where a bin starts inside the round
    int warp_sum[32];
};

// One stable counting pass over the items low .. high-1 of this (batch, head), which go to the places shared.base
// holds for their bins.  FIRST reads labels in position
// order and sorts by the low six bucket bits; the second pass reads the first pass's entries and
// sorts by the high six bits.
template <bool FIRST, int THREADS>
__device__ __forceinline__ void counting_pass(const int* __restrict__ labels, const int2* __restrict__ source,
                                              const int* __restrict__ source_previous, int2* __restrict__ target,
                                              int* __restrict__ target_previous, int low, int high, IndexShared<THREADS>& shared) {
    using Shared = IndexShared<THREADS>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int* base = shared.base[FIRST ? 0 : 1];
    const int scan_bin = tid & (PASS_BINS - 1), scan_part = tid / PASS_BINS;
    auto bin_of = [](int label) {
        const int bucket = bucket_of(label);
        return FIRST ? bucket & (PASS_BINS - 1) : bucket >> 6;
    };
    for (int round = low; round < high; round += Shared::ITEMS) {
        int2 item[PER_THREAD];
        int before_item[PER_THREAD];
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {  // all loads first: they are in flight together
            const int at = round + c * THREADS + tid;
            item[c] = make_int2(0, 0);
            before_item[c] = 0;
            if (at < high) {  // the first pass's output was written in this launch, maybe by another CTA: read it past L1
                item[c] = FIRST ? make_int2(at, __ldg(labels + at)) : __ldcg(source + at);
                before_item[c] = FIRST ? (at > 0 ? __ldg(labels + at - 1) : 0) : __ldcg(source_previous + at);
            }
        }
        unsigned places[PER_THREAD / 2] = {};  // per item sixteen bits: its bin, and above it its rank among the slot's items of that bin
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {
            const int at = round + c * THREADS + tid, slot = c * (THREADS / 32) + warp;
            const bool valid = at < high;
            const int bin = valid ? bin_of(item[c].y) : PASS_BINS;  // invalid lanes pair up only with each other
            reinterpret_cast<unsigned*>(shared.counts[slot])[lane] = 0u;  // the slot's 64 counters, two per lane
            if (round + c * THREADS >= high) continue;  // a slot past the end of the items (the same test in every thread)
            __syncwarp();
            unsigned peers = FULL;  // the lanes with this lane's bin: one vote per bit (cheaper than a warp match)
#pragma unroll
            for (int bit = 0; bit < 7; ++bit) {
                const unsigned vote = __ballot_sync(FULL, (bin >> bit) & 1);
                peers &= (bin >> bit) & 1 ? vote : ~vote;
            }
            const int rank = __popc(peers & ((1u << lane) - 1u));
            if (valid && rank == 0) shared.counts[slot][bin] = (unsigned short)__popc(peers);
            places[c >> 1] |= unsigned(bin | rank << 8) << (16 * (c & 1));
        }
        __syncthreads();
        // exclusive prefix of this thread's sixteen slots of one bin, then of the parts
        int running = 0;
        unsigned short before[SLOTS_PER_PART];
#pragma unroll
        for (int e = 0; e < SLOTS_PER_PART; ++e) {
            before[e] = (unsigned short)running;
            running += shared.counts[scan_part * SLOTS_PER_PART + e][scan_bin];
        }
        shared.part_total[scan_part][scan_bin] = running;
        __syncthreads();
        int offset = 0, all = 0;
#pragma unroll
        for (int part = 0; part < Shared::PARTS; ++part) {
            const int x = shared.part_total[part][scan_bin];
            if (part < scan_part) offset += x;
            all += x;
        }
#pragma unroll
        for (int e = 0; e < SLOTS_PER_PART; ++e) shared.counts[scan_part * SLOTS_PER_PART + e][scan_bin] = (unsigned short)(offset + before[e]);
        if (warp == 0) {  // where each bin starts inside the round: two bins per lane
            int first = 0, second = 0;
#pragma unroll
            for (int part = 0; part < Shared::PARTS; ++part) {
                first += shared.part_total[part][2 * lane];
                second += shared.part_total[part][2 * lane + 1];
            }
            int prefix = first + second;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, prefix, s);
                if (lane >= s) prefix += other;
            }
            shared.local_base[2 * lane] = prefix - first - second;
            shared.local_base[2 * lane + 1] = prefix - second;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {
            const int at = round + c * THREADS + tid, slot = c * (THREADS / 32) + warp;
            if (at >= high) continue;
            const unsigned place = places[c >> 1] >> (16 * (c & 1));
            const int bin = place & 255;
            const int to = shared.local_base[bin] + shared.counts[slot][bin] + ((place >> 8) & 255);
            shared.staged[to] = item[c];
            shared.staged_previous[to] = before_item[c];
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {
            const int i = c * THREADS + tid;
            if (round + i >= high) continue;
            const int2 entry = shared.staged[i];
            const int bin = bin_of(entry.y);
            const int to = base[bin] + i - shared.local_base[bin];
            target[to] = entry;
            target_previous[to] = shared.staged_previous[i];
        }
        __syncthreads();
        if (scan_part == Shared::PARTS - 1) base[scan_bin] += all;  // next read after the next round's barriers
    }
    __syncthreads();
}

// blockIdx.y picks the side: both sides of a readout are built by one launch.
template <int THREADS>
__global__ __launch_bounds__(THREADS, THREADS == 512 ? 2 : 1) void build_index_kernel(const IndexSide side0, const IndexSide side1, int n, const unsigned* choice) {
    if (!route_open(choice)) return;
    const IndexSide& side = blockIdx.y ? side1 : side0;
    const int* __restrict__ labels = side.labels;
    int2* __restrict__ entries = side.entries;
    int2* __restrict__ scratch = side.scratch;
    int* __restrict__ previous = side.previous;
    int* __restrict__ scratch_previous = side.scratch_previous;
    int* __restrict__ starts = side.starts;
    extern __shared__ __align__(16) unsigned char index_storage[];
    IndexShared<THREADS>& shared = *reinterpret_cast<IndexShared<THREADS>*>(index_storage);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    labels += int64_t(blockIdx.x) * n;
    entries += int64_t(blockIdx.x) * n;
    scratch += int64_t(blockIdx.x) * n;
    previous += int64_t(blockIdx.x) * n;
    scratch_previous += int64_t(blockIdx.x) * n;
    starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    // bucket starts: histogram of all 4096 buckets and its exclusive scan
    for (int e = tid; e < BUCKETS; e += THREADS) shared.histogram[e] = 0;
    __syncthreads();
    for (int at = tid; at < n; at += THREADS) atomicAdd(&shared.histogram[bucket_of(__ldg(labels + at))], 1);
    __syncthreads();
    {
        constexpr int PER = BUCKETS / THREADS;
        int local[PER], sum = 0;
#pragma unroll
        for (int e = 0; e < PER; ++e) { local[e] = sum; sum += shared.histogram[tid * PER + e]; }
        int prefix = sum;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        if (lane == 31) shared.warp_sum[warp] = prefix;
        __syncthreads();
        if (warp == 0) {
            const int mine = lane < THREADS / 32 ? shared.warp_sum[lane] : 0;
            int scan = mine;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, scan, s);
                if (lane >= s) scan += other;
            }
            shared.warp_sum[lane] = scan - mine;
        }
        __syncthreads();
        const int before = shared.warp_sum[warp] + prefix - sum;
#pragma unroll
        for (int e = 0; e < PER; ++e) starts[tid * PER + e] = before + local[e];
        if (tid == THREADS - 1) starts[BUCKETS] = n;
    }
    // where each pass's bins begin: bin sizes are sums of bucket sizes (low six bits, then high six bits)
    if (warp < 4) {
        const int pass = warp >> 1, bin = (warp & 1) * 32 + lane;
        int size = 0;
        for (int e = 0; e < PASS_BINS; ++e) {
            const int turned = (e + lane) & (PASS_BINS - 1);  // lanes start at different columns: no two in one bank
            size += shared.histogram[pass ? bin * PASS_BINS + turned : turned * PASS_BINS + bin];
        }
        int prefix = size;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        shared.base[pass][bin] = prefix - size;
        if (lane == 31) shared.part_total[0][warp] = prefix;  // the first half's size, for the second half
    }
    __syncthreads();
    if (warp < 4 && (warp & 1)) shared.base[warp >> 1][32 + lane] += shared.part_total[0][warp - 1];
    __syncthreads();
    counting_pass<true, THREADS>(labels, nullptr, nullptr, scratch, scratch_previous, 0, n, shared);
    counting_pass<false, THREADS>(labels, scratch, scratch_previous, entries, previous, 0, n, shared);
}

// The same sort by a cluster of CTAs, for launches with few (batch, head, side) slices: CTA r of the cluster takes the
// r-th part of the items in each pass.  What a CTA must know of the others goes through distributed shared memory:
// the sizes of its peers' bins (its items follow those of the CTAs before it, bin by bin) and, for the bucket starts,
// the peers' bucket histograms.  The second pass reads what the whole cluster wrote in the first, so the parts' bin
// sizes of the second pass are counted in between.  All waiting is the hardware's cluster barrier.
constexpr int CLUSTER_THREADS = 1024;
struct IndexClusterShared {
    IndexShared<CLUSTER_THREADS> sort;
    int histogram[BUCKETS];      // this CTA's part of the bucket histogram (kept while the peers read it)
    int bins[3][PASS_BINS];      // this CTA's bin sizes: first pass, second pass by original part, second pass by its part of the first pass's output
};

__global__ __launch_bounds__(CLUSTER_THREADS, 1) void build_index_cluster_kernel(const IndexSide side0, const IndexSide side1, int n, const unsigned* choice) {
    if (!route_open(choice)) return;  // (every CTA of a cluster reads the same word, so none waits for another)
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int parts = cluster.num_blocks(), part = cluster.block_rank(), slice = blockIdx.x / parts;
    const IndexSide& side = blockIdx.y ? side1 : side0;
    const int* __restrict__ labels = side.labels + int64_t(slice) * n;
    int2* entries = side.entries + int64_t(slice) * n;
    int2* scratch = side.scratch + int64_t(slice) * n;
    int* previous = side.previous + int64_t(slice) * n;
    int* scratch_previous = side.scratch_previous + int64_t(slice) * n;
    int* starts = side.starts + int64_t(slice) * (BUCKETS + 1);
    extern __shared__ __align__(16) unsigned char index_storage[];
    IndexClusterShared& shared = *reinterpret_cast<IndexClusterShared*>(index_storage);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int share = ((n + parts - 1) / parts + 31) & ~31, low = min(n, part * share), high = min(n, low + share);

    // this part's bucket histogram and its bin sizes for both passes
    for (int e = tid; e < BUCKETS; e += CLUSTER_THREADS) shared.histogram[e] = 0;
    __syncthreads();
    for (int at = low + tid; at < high; at += CLUSTER_THREADS) atomicAdd(&shared.histogram[bucket_of(__ldg(labels + at))], 1);
    __syncthreads();
    if (warp < 4) {
        const int pass = warp >> 1, bin = (warp & 1) * 32 + lane;
        int size = 0;
        for (int e = 0; e < PASS_BINS; ++e) {
            const int turned = (e + lane) & (PASS_BINS - 1);  // lanes start at different columns: no two in one bank
            size += shared.histogram[pass ? bin * PASS_BINS + turned : turned * PASS_BINS + bin];
        }
        shared.bins[pass][bin] = size;
    }
    cluster.sync();

    // bucket starts, by the first CTA: an exclusive scan of the whole cluster's histogram, four buckets per thread
    if (part == 0) {
        constexpr int PER = BUCKETS / CLUSTER_THREADS;
        int local[PER], sum = 0;
#pragma unroll
        for (int e = 0; e < PER; ++e) {
            int size = 0;
            for (int r = 0; r < parts; ++r) size += cluster.map_shared_rank(shared.histogram, r)[tid * PER + e];
            local[e] = sum;
            sum += size;
        }
        int prefix = sum;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int other = __shfl_up_sync(FULL, prefix, s);
            if (lane >= s) prefix += other;
        }
        if (lane == 31) shared.sort.warp_sum[warp] = prefix;
        __syncthreads();
        if (warp == 0) {
            const int mine = shared.sort.warp_sum[lane];
            int scan = mine;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, scan, s);
                if (lane >= s) scan += other;
            }
            shared.sort.warp_sum[lane] = scan - mine;
        }
        __syncthreads();
        const int before = shared.sort.warp_sum[warp] + prefix - sum;
#pragma unroll
        for (int e = 0; e < PER; ++e) starts[tid * PER + e] = before + local[e];
        if (tid == CLUSTER_THREADS - 1) starts[BUCKETS] = n;
    }
    // Where this part's items of a bin go: after the bins before it (sizes over the whole cluster) and after the same
    // bin's items of the parts before it.  `mine` picks the per-part sizes: 0 for the first pass, 2 for the second.
    auto place_bins = [&](int pass, int mine) {
        if (warp < 2) {
            const int bin = warp * 32 + lane;
            int all = 0, before = 0;
            for (int r = 0; r < parts; ++r) {
                all += cluster.map_shared_rank(&shared.bins[pass][0], r)[bin];
                if (r < part) before += cluster.map_shared_rank(&shared.bins[mine][0], r)[bin];
            }
            int prefix = all;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, prefix, s);
                if (lane >= s) prefix += other;
            }
            shared.sort.base[pass][bin] = prefix - all + before;
            if (lane == 31) shared.sort.part_total[0][warp] = prefix;  // the first half's size, for the second half
        }
        __syncthreads();
        if (warp == 1) shared.sort.base[pass][32 + lane] += shared.sort.part_total[0][0];
        __syncthreads();
    };
    place_bins(0, 0);
    counting_pass<true, CLUSTER_THREADS>(labels, nullptr, nullptr, scratch, scratch_previous, low, high, shared.sort);
    __threadfence();
    cluster.sync();  // the first pass's output is complete

    // bin sizes of this part of the first pass's output
    if (tid < PASS_BINS) shared.bins[2][tid] = 0;
    __syncthreads();
    for (int at = low + tid; at < high; at += CLUSTER_THREADS) atomicAdd(&shared.bins[2][bucket_of(__ldcg(scratch + at).y) >> 6], 1);
    cluster.sync();
    place_bins(1, 2);
    counting_pass<false, CLUSTER_THREADS>(labels, scratch, scratch_previous, entries, previous, low, high, shared.sort);
    cluster.sync();  // no CTA leaves while a peer may still read its shared memory
}

// Per side: entries int2 [BH, N], sort scratch int2 [BH, N], previous int [BH, N], its sort scratch int [BH, N],
// starts int [BH, BUCKETS + 1].
size_t index_bytes(int batch_heads, int n, int sides) {
    size_t one = size_t(batch_heads) * n * (2 * sizeof(int2) + 2 * sizeof(int)) + size_t(batch_heads) * (BUCKETS + 1) * sizeof(int);
    one = (one + 255) & ~size_t(255);
    return one * sides;
}

SideIndex side_index(void* workspace, int batch_heads, int n, int side, int sides) {
    const size_t one = index_bytes(batch_heads, n, 1);
    char* p = static_cast<char*>(workspace) + one * side;
    (void)sides;
    const size_t items = size_t(batch_heads) * n;
    return SideIndex{reinterpret_cast<const int2*>(p), reinterpret_cast<const int*>(p + items * (2 * sizeof(int2) + 2 * sizeof(int))),
                     reinterpret_cast<const int*>(p + items * 2 * sizeof(int2))};
}

static IndexSide index_side(const int* labels, void* workspace, int batch_heads, int n, int side, int sides) {
    const SideIndex index = side_index(workspace, batch_heads, n, side, sides);
    int2* entries = const_cast<int2*>(index.entries);
    int* previous = const_cast<int*>(index.previous);
    return IndexSide{labels, entries, entries + size_t(batch_heads) * n, previous, previous + size_t(batch_heads) * n, const_cast<int*>(index.starts)};
}

// Very few slices: a cluster of CTAs per slice.  Few: the widest CTA, which finishes a slice soonest.  Many: narrower
// CTAs, several to an SM.
static void run_build_index(const IndexSide& side0, const IndexSide& side1, int batch_heads, int sides, int n, const unsigned* choice,
                            cudaStream_t stream) {
    static const bool ready = [] {  // shared memory beyond 48 KiB has to be asked for once per kernel
        return cudaFuncSetAttribute(build_index_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(IndexShared<1024>))) == cudaSuccess &&
               cudaFuncSetAttribute(build_index_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(IndexShared<512>))) == cudaSuccess;
    }();
    (void)ready;
    const int sms = device_sm_count(), slices = batch_heads * sides;
    int parts = 1;  // CTAs per slice: as many as keep the launch within one CTA per SM, a power of two up to eight
    while (parts < 8 && slices * parts * 2 <= sms && n / (parts * 2) >= 8192) parts *= 2;  // (at 8192 positions a slice the cluster is no faster than one CTA)
    if (parts > 1) {
        static const bool cluster_ready = cudaFuncSetAttribute(build_index_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                               int(sizeof(IndexClusterShared))) == cudaSuccess;
        (void)cluster_ready;
        cudaLaunchConfig_t config{};
        config.gridDim = dim3(batch_heads * parts, sides);
        config.blockDim = dim3(CLUSTER_THREADS);
        config.dynamicSmemBytes = sizeof(IndexClusterShared);
        config.stream = stream;
        cudaLaunchAttribute attribute{};
        attribute.id = cudaLaunchAttributeClusterDimension;
        attribute.val.clusterDim.x = parts;
        attribute.val.clusterDim.y = 1;
        attribute.val.clusterDim.z = 1;
        config.attrs = &attribute;
        config.numAttrs = 1;
        cudaLaunchKernelEx(&config, build_index_cluster_kernel, side0, side1, n, choice);
    } else if (slices <= sms) {
        build_index_kernel<1024><<<dim3(batch_heads, sides), 1024, sizeof(IndexShared<1024>), stream>>>(side0, side1, n, choice);
    } else {
        build_index_kernel<512><<<dim3(batch_heads, sides), 512, sizeof(IndexShared<512>), stream>>>(side0, side1, n, choice);
    }
}

cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream) {
    const IndexSide target = index_side(labels, workspace, batch_heads, n, side, sides);
    KernelTimer timer("build_index", stream);
    run_build_index(target, target, batch_heads, 1, n, nullptr, stream);  // (the longest-match entry is not routed)
    return cudaGetLastError();
}

cudaError_t launch_build_index_pair(const int* labels0, const int* labels1, int batch_heads, int n, void* workspace,
                                    cudaStream_t stream) {
    KernelTimer timer("build_index", stream);
    run_build_index(index_side(labels0, workspace, batch_heads, n, 0, 2), index_side(labels1, workspace, batch_heads, n, 1, 2),
                    batch_heads, 2, n, route_word(), stream);
    return cudaGetLastError();
}

}  // namespace dism
