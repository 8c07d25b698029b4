// Skeleton shared by the three row-owned kernels of the hard path (forward, query-major backward,
// key-major backward).
//
// A row with very many partners (a popular label in a long sequence) would keep one lane group
// busy long after everything else has finished, so such rows are taken out of the groups: a whole
// warp handles one of them, its eight lane groups each reduce one contiguous eighth of the
// partner range, and the eight partial results are merged in a fixed shuffle tree.
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
constexpr int LOAD_BINS = 64;
constexpr int HEAVY_ROW = 256;  // rows with at least this many partners are shared by a whole warp

struct RowContext {  // what a task's rows share
    const int *iq, *ik, *boundary;
    const float *lut, *dlut, *lse2;
    SideIndex index;  // position index of the partner side
    int64_t vec0;     // (b, 0, h) in units of one vector
    int n, heads, bh;
    int begin, end;   // the document of the task's rows: [begin, end) within the sequence
};

struct RowsShared {
    int order[TASK_ROWS];                       // local row numbers, heaviest first
    int label[TASK_ROWS], previous[TASK_ROWS];  // own-side labels of the row and of the row before it
    int first[TASK_ROWS], last[TASK_ROWS];      // the row's bucket range in the partner index
    int bin_count[LOAD_BINS], bin_start[LOAD_BINS];
    int next_group;
    int heavy[TASK_ROWS];  // local numbers of the rows handled one per warp
    int heavy_count;
};

// Search state of one owned row, replicated in the four lanes of its group.
struct SearchRow {
    int row;
    int label;     // label of the owned row
    int previous;  // label of the owned side at row - 1 (the diagonal predecessor's own-side label)
    int cursor, end;
    int queued;    // partners waiting in the group's queue
};

constexpr int QUEUE_DEPTH = 48;  // a scan step adds at most 32 partners and runs only with room for them

// Per-warp queues: one per owned row, partners in ascending position with their log2 weight
// (and, for the query-major backward, the dlog weight).
template <bool EXTRA>
struct PartnerQueues {
    int position[OWN][QUEUE_DEPTH];
    float weight[OWN][QUEUE_DEPTH];
    float extra[EXTRA ? OWN : 1][QUEUE_DEPTH];
};

// One scan step of a lane group: its row's next 32 bucket entries, eight per lane.  Entries with
// the row's label on the causal side are appended to the group's queue in ascending position.
// Only positions are recorded here; weights are filled in by finish_partners() for the whole
// queue at once, so that the dependent loads of many partners overlap.
// Every lane of the warp calls this (the prefix sums use full-warp shuffles); `scan` says whether
// this lane's group takes part.
template <bool QUERY_MAJOR, bool EXTRA>
__device__ __forceinline__ void scan_partners(PartnerQueues<EXTRA>* queue, const int2* __restrict__ entries,
                                              SearchRow& mine, bool scan, int group, int part, int lane) {
    int2 entry[8];
    const int base = mine.cursor + part * 8;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        entry[e] = make_int2(QUERY_MAJOR ? 0x7fffffff : -1, 0);
        if (scan && base + e < mine.end) entry[e] = __ldg(entries + base + e);
    }
    unsigned hits = 0;
    bool beyond = false;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const bool inside = scan && base + e < mine.end;
        const bool causal = QUERY_MAJOR ? entry[e].x <= mine.row : entry[e].x >= mine.row;
        if (inside && causal && entry[e].y == mine.label) hits |= 1u << e;
        if (QUERY_MAJOR && inside && !causal) beyond = true;  // keys ascend: nothing causal follows
    }
    const int count = __popc(hits);
    const int first = lane & ~3;
    const int c0 = __shfl_sync(FULL, count, first), c1 = __shfl_sync(FULL, count, first + 1);
    const int c2 = __shfl_sync(FULL, count, first + 2), c3 = __shfl_sync(FULL, count, first + 3);
    const unsigned ended = __ballot_sync(FULL, beyond);
    int slot = mine.queued + (part > 0 ? c0 : 0) + (part > 1 ? c1 : 0) + (part > 2 ? c2 : 0);
#pragma unroll
    for (int e = 0; e < 8; ++e)
        if (hits & (1u << e)) queue->position[group][slot++] = entry[e].x;
    if (scan) {
        mine.queued += c0 + c1 + c2 + c3;
        mine.cursor = ((ended >> first) & 15u) ? mine.end : min(mine.cursor + 32, mine.end);
    }
}

// Fills in the weights of the queued partners, four per group at a time (one per lane).  A run
// is longer than one only when the diagonal predecessor matches too; those partners are then
// handled one after the other by the whole warp, which walks 32 cells of the diagonal per step.
// Every lane of the warp calls this.
template <bool QUERY_MAJOR, bool EXTRA>
__device__ __forceinline__ void finish_partners(PartnerQueues<EXTRA>* queue, const RowContext& ctx,
                                                const float* __restrict__ shift_by_position, const SearchRow& mine,
                                                int group, int part, int lane) {
    const int* other_side = QUERY_MAJOR ? ctx.ik : ctx.iq;
    const float weight_one = __ldg(ctx.lut + 1), extra_one = EXTRA ? __ldg(ctx.dlut + 1) : 0.f;
    unsigned long long longer = 0;  // slots of this lane whose run continues up the diagonal
#pragma unroll 2
    for (int slot = part; slot < mine.queued; slot += 4) {
        const int position = queue->position[group][slot];
        const int neighbour = position > 0 ? __ldg(other_side + position - 1) : 0;
        const float shift = shift_by_position ? __ldg(shift_by_position + position) : 0.f;
        if (position > ctx.begin && mine.row > ctx.begin && neighbour == mine.previous) longer |= 1ull << slot;
        queue->weight[group][slot] = weight_one - shift;
        if (EXTRA) queue->extra[group][slot] = extra_one;
    }
    for (unsigned waiting = __ballot_sync(FULL, longer != 0); waiting; waiting = __ballot_sync(FULL, longer != 0)) {
        const int owner = __ffs(waiting) - 1;
        int slot = 0, position = 0;
        if (lane == owner) {
            slot = __ffsll((long long)longer) - 1;
            longer &= longer - 1;
            position = queue->position[group][slot];
        }
        position = __shfl_sync(FULL, position, owner);
        const int row = __shfl_sync(FULL, mine.row, owner);
        const int i = QUERY_MAJOR ? row : position, j = QUERY_MAJOR ? position : row;
        const int length = run_length(ctx.iq, ctx.ik, ctx.boundary, ctx.n, i, j, lane, ctx.begin);
        if (lane == owner) {
            const float shift = shift_by_position ? __ldg(shift_by_position + position) : 0.f;
            queue->weight[group][slot] = __ldg(ctx.lut + length) - shift;
            if (EXTRA) queue->extra[group][slot] = __ldg(ctx.dlut + length);
        }
    }
}

template <class Policy>
struct RowsKernelShared {
    RowsShared rows;
    PartnerQueues<Policy::EXTRA> queue[WARPS];
    GatherRing<8, Policy::VPL> ring[WARPS];
};

// Policy supplies: QUERY_MAJOR, EXTRA, VPL, R, MIN_CTAS (resident CTAs per SM to compile for); Args with the common fields used below;
// per-lane state with begin(), pair(), finish(); the two gathered tensors.
template <class Policy>
__global__ __launch_bounds__(WARPS * 32, Policy::MIN_CTAS) void rows_kernel(const typename Policy::Args a) {
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
        RowContext ctx;
        ctx.begin = 0;
        ctx.end = a.n;
        int hard_row = b;
        if (a.documents) {  // packed: one batch row, documents and hard training rows are 256-aligned spans
            const int2 document = __ldg(a.documents + block);
            ctx.begin = document.x;
            ctx.end = document.y;
            hard_row = (block * TASK_ROWS) / (a.n / a.hard_rows);
        }
        const bool active = a.hard[hard_row * a.heads + h];
        ctx.iq = a.iq + int64_t(bh) * a.n;
        ctx.ik = a.ik + int64_t(bh) * a.n;
        ctx.boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
        ctx.lut = a.lut + int64_t(h) * a.lut_stride;
        ctx.dlut = a.dlut ? a.dlut + int64_t(h) * a.lut_stride : nullptr;
        ctx.lse2 = a.lse2 ? a.lse2 + int64_t(bh) * a.n : nullptr;
        ctx.index = SideIndex{a.index.entries + int64_t(bh) * a.n, a.index.starts + int64_t(bh) * (BUCKETS + 1), nullptr};
        ctx.vec0 = int64_t(b) * a.n * a.heads + h;
        ctx.n = a.n;
        ctx.heads = a.heads;
        ctx.bh = bh;
        const int* own_labels = QM ? ctx.iq : ctx.ik;

        // ---- order the task's rows by estimated load, heaviest first -------------------------------
        __syncthreads();
        if (threadIdx.x < LOAD_BINS) shared.rows.bin_count[threadIdx.x] = 0;
        if (threadIdx.x == 0) shared.rows.next_group = shared.rows.heavy_count = 0;
        __syncthreads();
        const int my_row = block * TASK_ROWS + threadIdx.x;
        int bin = 0;
        if (active) {
            // every thread prepares one row's search: labels and bucket range go to shared memory, so
            // the lane groups start from there instead of from a chain of dependent global loads
            const int label = __ldg(own_labels + my_row);
            int first, last;
            partner_range<QM>(ctx.index, label, my_row, first, last, ctx.begin, ctx.end < a.n ? ctx.end : 0x7fffffff);
            shared.rows.label[threadIdx.x] = label;
            shared.rows.previous[threadIdx.x] = my_row > ctx.begin ? __ldg(own_labels + my_row - 1) : 0;
            shared.rows.first[threadIdx.x] = first;
            shared.rows.last[threadIdx.x] = last;
            // the causal range is, up to bucket collisions, the row's partner count: exact bins for
            // small counts, steps of 16 above
            const int count = last - first;
            bin = count < 48 ? count : min(LOAD_BINS - 1, 48 + (count - 48) / 16);
            if (count >= HEAVY_ROW) {  // handled by a whole warp later: an empty row as far as the groups go
                shared.rows.heavy[atomicAdd(&shared.rows.heavy_count, 1)] = threadIdx.x;
                shared.rows.first[threadIdx.x] = -1 - first;  // marks the row; the range is recovered from it
                bin = 0;
            }
        }
        const int rank_in_bin = atomicAdd(&shared.rows.bin_count[bin], 1);
        __syncthreads();
        if (warp == 0) {  // descending bins: exclusive scan from the top, two bins per lane
            const int heavy = shared.rows.bin_count[LOAD_BINS - 1 - 2 * lane];
            const int light = shared.rows.bin_count[LOAD_BINS - 2 - 2 * lane];
            int prefix = heavy + light;
#pragma unroll
            for (int s = 1; s < 32; s <<= 1) {
                const int other = __shfl_up_sync(FULL, prefix, s);
                if (lane >= s) prefix += other;
            }
            prefix -= heavy + light;
            shared.rows.bin_start[LOAD_BINS - 1 - 2 * lane] = prefix;
            shared.rows.bin_start[LOAD_BINS - 2 - 2 * lane] = prefix + heavy;
        }
        __syncthreads();
        shared.rows.order[shared.rows.bin_start[bin] + rank_in_bin] = threadIdx.x;
        __syncthreads();

        // ---- warps pull work items: first the groups of eight rows, then the heavy rows ---------------------
        for (;;) {
            int chosen = 0;
            if (lane == 0) chosen = atomicAdd(&shared.rows.next_group, 1);
            chosen = __shfl_sync(FULL, chosen, 0);
            const int shared_item = chosen - TASK_ROWS / OWN;  // >= 0: one heavy row for the whole warp
            if (shared_item >= shared.rows.heavy_count) break;
            const bool whole_warp = shared_item >= 0;
            const int local = whole_warp ? shared.rows.heavy[shared_item] : shared.rows.order[chosen * OWN + group];
            const int row = block * TASK_ROWS + local;  // the row this lane group works on
            const int first = shared.rows.first[local], last = shared.rows.last[local];
            // a heavy row (marked by a negative start) is skipped by its group and done by a whole warp later
            const bool mine_to_do = active && (whole_warp || first >= 0);
            Policy state;
            state.begin(a, ctx, row, part, has_r, mine_to_do, !whole_warp || group == 0);
            if (active) {
                SearchRow search;
                search.row = row;
                search.label = shared.rows.label[local];
                search.previous = shared.rows.previous[local];
                search.cursor = search.end = 0;
                if (whole_warp) {  // an eighth of the partner range per lane group
                    const int from = -1 - first, share = (last - from + OWN - 1) / OWN;
                    search.cursor = min(from + group * share, last);
                    search.end = min(search.cursor + share, last);
                } else if (first >= 0) {
                    search.cursor = first;
                    search.end = last;
                }
                search.queued = 0;
                for (;;) {
                    // scan while some group can take 32 more; otherwise weigh and drain every queue
                    const bool scan = search.cursor < search.end && search.queued <= QUEUE_DEPTH - 32;
                    if (__ballot_sync(FULL, scan)) {
                        scan_partners<QM, Policy::EXTRA>(queue, ctx.index.entries, search, scan, group, part, lane);
                        continue;
                    }
                    if (!__ballot_sync(FULL, search.queued > 0)) break;
                    __syncwarp();
                    finish_partners<QM, Policy::EXTRA>(queue, ctx, QM ? nullptr : ctx.lse2, search, group, part, lane);
                    __syncwarp();
                    const int mine = search.queued, rounds = __reduce_max_sync(FULL, mine);
                    drain_partners<8, VPL>(
                        queue->position[group], mine, rounds, shared.ring + warp,
                        Policy::gather_a(a) + ctx.vec0 * R + part * 8, int64_t(a.heads) * R, has_r,
                        Policy::gather_b(a) + ctx.vec0 * (VPL * 4) + part * VPL, int64_t(a.heads) * (VPL * 4), lane,
                        [&](bool live, int slot, const float(&va)[8], const float(&vb)[VPL]) {
                            const float weight = live ? queue->weight[group][slot] : 0.f;
                            const float extra = (Policy::EXTRA && live) ? queue->extra[group][slot] : 0.f;
                            state.pair(live, weight, extra, va, vb);
                        });
                    search.queued = 0;
                    __syncwarp();
                }
                if (whole_warp) state.merge_groups();
            }
            if (whole_warp ? group == 0 : (!active || first >= 0)) state.finish(a, ctx, row, part, has_r, active);
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
