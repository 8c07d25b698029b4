// Skeleton shared by the three row-owned kernels of the hard path (forward, query-major backward,
// key-major backward).
//
// A CTA takes 256 consecutive rows of one (batch, head).  Rows differ a lot in how many partners
// they have (a popular label has a big bucket), so the CTA first orders its rows by an estimate
// of that load and its warps then pull groups of eight similar rows from the ordered list: the
// eight lane groups of a warp stay busy for about the same number of rounds, and heavy groups
// do not hold up the rest of the CTA.  Which warp handles a row never changes the row's result:
// a row is always accumulated by one lane group, partners in ascending position.
#pragma once
#include "dism_common.cuh"

namespace dism {

constexpr int TASK_ROWS = 256;  // rows per CTA task (sequence lengths are multiples of 256)
constexpr int LOAD_BINS = 32;

struct RowContext {  // what a task's rows share
    const int *iq, *ik, *boundary;
    const float *lut, *dlut, *lse2;
    SideIndex index;  // position index of the partner side
    int64_t vec0;     // (b, 0, h) in units of one vector
    int n, heads, bh;
};

struct RowsShared {
    int order[TASK_ROWS];
    int bin_count[LOAD_BINS], bin_start[LOAD_BINS];
    int next_group;
};

// lane r < OWN carries the search state of the warp's r-th row
struct SearchRow {
    int row;
    int label;     // label of the owned row
    int previous;  // label of the owned side at row - 1 (the diagonal predecessor's own-side label)
    int cursor, end;
};

// One round of partner search for the warp's OWN rows.  Each row reads its next 32 bucket
// entries (all eight loads are issued before any is used), keeps the causal entries with its
// label, and queues them in ascending position with the log2 weight of their run length
// (minus the partner's log2 normaliser when `shift_by_position` is given).  Returns in lane r
// the number queued for row r.  QUERY_MAJOR: owned rows are queries and partners are keys;
// otherwise owned rows are keys and partners are queries.
template <bool QUERY_MAJOR, bool EXTRA>
__device__ __forceinline__ int find_partners(PairQueue<EXTRA>* queue, const RowContext& ctx,
                                             const float* __restrict__ shift_by_position, SearchRow& mine, int lane) {
    const int* other_side = QUERY_MAJOR ? ctx.ik : ctx.iq;
    int2 entry[OWN];
    bool valid[OWN];
#pragma unroll
    for (int r = 0; r < OWN; ++r) {
        const int from = __shfl_sync(FULL, mine.cursor, r), to = __shfl_sync(FULL, mine.end, r);
        valid[r] = from + lane < to;
        entry[r] = make_int2(QUERY_MAJOR ? 0x7fffffff : -1, 0);
        if (valid[r]) entry[r] = __ldg(ctx.index.entries + from + lane);
    }
    int neighbour[OWN];
    float shift[OWN];
    bool hit[OWN];
#pragma unroll
    for (int r = 0; r < OWN; ++r) {
        const int row = __shfl_sync(FULL, mine.row, r), wanted = __shfl_sync(FULL, mine.label, r);
        const bool causal = QUERY_MAJOR ? entry[r].x <= row : entry[r].x >= row;
        hit[r] = valid[r] && causal && entry[r].y == wanted;
        // the other side's label one step up the diagonal, and the partner's normaliser
        neighbour[r] = 0;
        shift[r] = 0.f;
        if (hit[r] && entry[r].x > 0) neighbour[r] = __ldg(other_side + entry[r].x - 1);
        if (hit[r] && shift_by_position) shift[r] = __ldg(shift_by_position + entry[r].x);
        // keys ascend inside a bucket: a position beyond the row ends the row's search
        const unsigned beyond = QUERY_MAJOR ? __ballot_sync(FULL, valid[r] && entry[r].x > row) : 0u;
        const int from = __shfl_sync(FULL, mine.cursor, r), to = __shfl_sync(FULL, mine.end, r);
        if (lane == r && from < to) mine.cursor = beyond ? to : from + 32;
    }
    const float weight_one = __ldg(ctx.lut + 1), extra_one = EXTRA ? __ldg(ctx.dlut + 1) : 0.f;
    int queued = 0;
#pragma unroll
    for (int r = 0; r < OWN; ++r) {
        const int row = __shfl_sync(FULL, mine.row, r), previous = __shfl_sync(FULL, mine.previous, r);
        float weight = weight_one, extra = extra_one;
        if (hit[r] && entry[r].x > 0 && row > 0 && neighbour[r] == previous) {  // the run is longer than one
            const int i = QUERY_MAJOR ? row : entry[r].x, j = QUERY_MAJOR ? entry[r].x : row;
            const int length = 1 + run_length(ctx.iq, ctx.ik, ctx.boundary, ctx.n, i - 1, j - 1);
            weight = __ldg(ctx.lut + length);
            if (EXTRA) extra = __ldg(ctx.dlut + length);
        }
        const unsigned mask = __ballot_sync(FULL, hit[r]);
        if (hit[r]) {
            const int slot = __popc(mask & ((1u << lane) - 1u));
            queue->position[r][slot] = entry[r].x;
            queue->weight[r][slot] = weight - shift[r];
            if (EXTRA) queue->extra[r][slot] = extra;
        }
        if (lane == r) queued = __popc(mask);
    }
    return queued;
}

template <class Policy>
struct RowsKernelShared {
    RowsShared rows;
    PairQueue<Policy::EXTRA> queue[WARPS];
    GatherRing<8, Policy::VPL> ring[WARPS];
};

// Policy supplies: QUERY_MAJOR, EXTRA, VPL, R; Args with the common fields used below;
// per-lane state with begin(), pair(), finish(); the two gathered tensors.
template <class Policy>
__global__ __launch_bounds__(WARPS * 32) void rows_kernel(const typename Policy::Args a) {
    constexpr bool QM = Policy::QUERY_MAJOR;
    constexpr int VPL = Policy::VPL, R = Policy::R;
    extern __shared__ __align__(16) unsigned char storage[];
    auto& shared = *reinterpret_cast<RowsKernelShared<Policy>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group = lane >> 2, part = lane & 3;
    const bool has_r = part * 8 < R;  // this lane holds a slice of the R-wide vectors
    auto* queue = shared.queue + warp;
    const int blocks = a.n / TASK_ROWS;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        // (batch, head) major keeps the gathered vectors of the CTAs in flight inside L2; within a
        // (batch, head) the blocks with the most causal partners go first.
        const int bh = task / blocks, rank = task % blocks, block = QM ? blocks - 1 - rank : rank;
        const int b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        RowContext ctx;
        ctx.iq = a.iq + int64_t(bh) * a.n;
        ctx.ik = a.ik + int64_t(bh) * a.n;
        ctx.boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
        ctx.lut = a.lut + int64_t(h) * a.lut_stride;
        ctx.dlut = a.dlut ? a.dlut + int64_t(h) * a.lut_stride : nullptr;
        ctx.lse2 = a.lse2 ? a.lse2 + int64_t(bh) * a.n : nullptr;
        ctx.index = SideIndex{a.index.entries + int64_t(bh) * a.n, a.index.starts + int64_t(bh) * (BUCKETS + 1)};
        ctx.vec0 = int64_t(b) * a.n * a.heads + h;
        ctx.n = a.n;
        ctx.heads = a.heads;
        ctx.bh = bh;
        const int* own_labels = QM ? ctx.iq : ctx.ik;

        // ---- order the task's rows by estimated load, heaviest first -------------------------------
        __syncthreads();
        if (threadIdx.x < LOAD_BINS) shared.rows.bin_count[threadIdx.x] = 0;
        if (threadIdx.x == 0) shared.rows.next_group = 0;
        __syncthreads();
        const int my_row = block * TASK_ROWS + threadIdx.x;
        int bin = 0;
        if (active) {
            const int bucket = bucket_of(__ldg(own_labels + my_row));
            const int size = __ldg(ctx.index.starts + bucket + 1) - __ldg(ctx.index.starts + bucket);
            // about size * (causal share of the sequence) entries lie on the causal side
            const int64_t estimate = int64_t(size) * (QM ? my_row + 1 : a.n - my_row) / a.n;
            bin = estimate <= 0 ? 0 : min(LOAD_BINS - 1, 32 - __clz(int(estimate)));
        }
        const int rank_in_bin = atomicAdd(&shared.rows.bin_count[bin], 1);
        __syncthreads();
        if (warp == 0) {  // descending bins: exclusive scan from the top
            const int count = shared.rows.bin_count[LOAD_BINS - 1 - lane];
            int prefix = count;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, prefix, s);
                if (lane >= s) prefix += other;
            }
            shared.rows.bin_start[LOAD_BINS - 1 - lane] = prefix - count;
        }
        __syncthreads();
        shared.rows.order[shared.rows.bin_start[bin] + rank_in_bin] = my_row;
        __syncthreads();

        // ---- warps pull groups of eight rows ----------------------------------------------------------
        for (;;) {
            int chosen = 0;
            if (lane == 0) chosen = atomicAdd(&shared.rows.next_group, 1);
            chosen = __shfl_sync(FULL, chosen, 0);
            if (chosen >= TASK_ROWS / OWN) break;
            const int row = shared.rows.order[chosen * OWN + group];  // the row this lane group accumulates
            Policy state;
            state.begin(a, ctx, row, part, has_r, active);
            if (active) {
                SearchRow search;
                search.row = shared.rows.order[chosen * OWN + (lane & (OWN - 1))];
                search.label = __ldg(own_labels + search.row);
                search.previous = search.row ? __ldg(own_labels + search.row - 1) : 0;
                partner_range<QM>(ctx.index, search.label, search.row, search.cursor, search.end);
                while (__ballot_sync(FULL, lane < OWN && search.cursor < search.end)) {
                    __syncwarp();
                    const int queued = find_partners<QM, Policy::EXTRA>(queue, ctx, QM ? nullptr : ctx.lse2, search, lane);
                    __syncwarp();
                    const int mine = __shfl_sync(FULL, queued, group);
                    const int rounds = __reduce_max_sync(FULL, mine);
                    drain_partners<8, VPL>(
                        queue->position[group], mine, rounds, shared.ring + warp,
                        Policy::gather_a(a) + ctx.vec0 * R + part * 8, int64_t(a.heads) * R, has_r,
                        Policy::gather_b(a) + ctx.vec0 * (VPL * 4) + part * VPL, int64_t(a.heads) * (VPL * 4), lane,
                        [&](bool live, int slot, const float(&va)[8], const float(&vb)[VPL]) {
                            const float weight = live ? queue->weight[group][slot] : 0.f;
                            const float extra = (Policy::EXTRA && live) ? queue->extra[group][slot] : 0.f;
                            state.pair(live, weight, extra, va, vb);
                        });
                }
            }
            state.finish(a, ctx, row, part, has_r, active);
        }
    }
}

template <class Policy>
cudaError_t launch_rows_kernel(const typename Policy::Args& args, int ctas, cudaStream_t stream) {
    auto kernel = rows_kernel<Policy>;
    const int shared = sizeof(RowsKernelShared<Policy>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    int resident = 1;
    status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, WARPS * 32, shared);
    if (status != cudaSuccess) return status;
    int grid = ctas ? ctas : device_sm_count() * (resident > 0 ? resident : 1);
    if (grid > args.tasks) grid = args.tasks;
    {
        KernelTimer timer(Policy::name(), stream);
        kernel<<<grid, WARPS * 32, shared, stream>>>(args);
    }
    return cudaGetLastError();
}

}  // namespace dism
