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

// One stable counting pass over n items of this (batch, head).  FIRST reads labels in position
// order and sorts by the low six bucket bits; the second pass reads the first pass's entries and
// sorts by the high six bits.
template <bool FIRST, int THREADS>
__device__ __forceinline__ void counting_pass(const int* __restrict__ labels, const int2* __restrict__ source,
                                              const int* __restrict__ source_previous, int2* __restrict__ target,
                                              int* __restrict__ target_previous, int n, IndexShared<THREADS>& shared) {
    using Shared = IndexShared<THREADS>;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int* base = shared.base[FIRST ? 0 : 1];
    const int scan_bin = tid & (PASS_BINS - 1), scan_part = tid / PASS_BINS;
    auto bin_of = [](int label) {
        const int bucket = bucket_of(label);
        return FIRST ? bucket & (PASS_BINS - 1) : bucket >> 6;
    };
    for (int round = 0; round < n; round += Shared::ITEMS) {
        int2 item[PER_THREAD];
        int before_item[PER_THREAD];
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {  // all loads first: they are in flight together
            const int at = round + c * THREADS + tid;
            item[c] = make_int2(0, 0);
            before_item[c] = 0;
            if (at < n) {
                item[c] = FIRST ? make_int2(at, __ldg(labels + at)) : source[at];
                before_item[c] = FIRST ? (at > 0 ? __ldg(labels + at - 1) : 0) : source_previous[at];
            }
        }
        unsigned places[PER_THREAD / 2] = {};  // per item sixteen bits: its bin, and above it its rank among the slot's items of that bin
#pragma unroll
        for (int c = 0; c < PER_THREAD; ++c) {
            const int at = round + c * THREADS + tid, slot = c * (THREADS / 32) + warp;
            const bool valid = at < n;
            const int bin = valid ? bin_of(item[c].y) : PASS_BINS;  // invalid lanes pair up only with each other
            reinterpret_cast<unsigned*>(shared.counts[slot])[lane] = 0u;  // the slot's 64 counters, two per lane
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
            if (at >= n) continue;
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
            if (round + i >= n) continue;
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
__global__ __launch_bounds__(THREADS, THREADS == 512 ? 2 : 1) void build_index_kernel(const IndexSide side0, const IndexSide side1, int n) {
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
    counting_pass<true, THREADS>(labels, nullptr, nullptr, scratch, scratch_previous, n, shared);
    counting_pass<false, THREADS>(labels, scratch, scratch_previous, entries, previous, n, shared);
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

// Few CTAs: the widest CTA, which finishes a slice soonest.  Many: narrower CTAs, several to an SM.
static void run_build_index(const IndexSide& side0, const IndexSide& side1, int batch_heads, int sides, int n, cudaStream_t stream) {
    static const bool ready = [] {  // shared memory beyond 48 KiB has to be asked for once per kernel
        return cudaFuncSetAttribute(build_index_kernel<1024>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(IndexShared<1024>))) == cudaSuccess &&
               cudaFuncSetAttribute(build_index_kernel<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(IndexShared<512>))) == cudaSuccess;
    }();
    (void)ready;
    if (batch_heads * sides <= device_sm_count())
        build_index_kernel<1024><<<dim3(batch_heads, sides), 1024, sizeof(IndexShared<1024>), stream>>>(side0, side1, n);
    else
        build_index_kernel<512><<<dim3(batch_heads, sides), 512, sizeof(IndexShared<512>), stream>>>(side0, side1, n);
}

cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream) {
    const IndexSide target = index_side(labels, workspace, batch_heads, n, side, sides);
    KernelTimer timer("build_index", stream);
    run_build_index(target, target, batch_heads, 1, n, stream);
    return cudaGetLastError();
}

cudaError_t launch_build_index_pair(const int* labels0, const int* labels1, int batch_heads, int n, void* workspace,
                                    cudaStream_t stream) {
    KernelTimer timer("build_index", stream);
    run_build_index(index_side(labels0, workspace, batch_heads, n, 0, 2), index_side(labels1, workspace, batch_heads, n, 1, 2),
                    batch_heads, 2, n, stream);
    return cudaGetLastError();
}

}  // namespace dism
