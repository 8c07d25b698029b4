// Hard forward for dense labels: consecutive-position tiles.
//
// The label-block kernel (hard_forward_blocks.cuh) pays per matching pair and, for pairs whose run
// is longer than one, per step of the diagonal walk.  When a large share of all causal pairs match
// (all labels equal, a tiny vocabulary, a periodic stream) that is far more than the N^2/2 pairs
// cost when they are simply all visited, which is what the reference's tile kernel does
// (dism_v3/src/hard_forward.cu:27-118 on the strip rectangle of hard_summary / hard_chunk).  The
// plan kernel therefore counts the label-matching pairs of every (batch, head) from the bucket
// sizes of the two indices and sends a slice whose count reaches N^2/10 here; the label-block
// kernel then finds no tiles for that slice.
//
// Run lengths need no rectangle.  L(i, j) = 1 + L(i-1, j-1) on a match, so the run lengths of a
// block of sixteen query rows follow from those of the row above it: one key column per lane, sixteen
// steps, each taking the neighbouring lane's previous value.  A CTA owns a contiguous range of sixteen-row blocks
// of one (batch, head) and sweeps it downwards, handing the last row's lengths to the next block
// through a scratch row; the row above a chunk's first block comes from a walk along whole
// diagonals that the grid does before the sweeps (dense_route.cuh).  Within a block the eight warps split the key columns into eight contiguous
// ranges and work through them thirty-two at a time: the lanes first turn their columns' run lengths
// into log2 weights in shared memory, then the
// warp does what a fused attention kernel does on sixteen-by-sixteen tiles (scores = SQ.SK^T,
// online maximum from the weights, acc += (P o S).V, all bf16 mma.sync), and the warps' partial
// rows are merged with the reference's normalisation (maximum starts at 0, denominator at 1).
#pragma once
#include <cooperative_groups.h>

#include "hard_forward_blocks.cuh"

namespace dism {

struct DenseArgs {
    const __nv_bfloat16 *sq, *sk, *v;
    const int *iq, *ik;
    const uint8_t* hard;
    const int2* documents;  // packed layouts: (first position, end) of the document of every 256-position block; else null
    int hard_rows;          // packed layouts: training rows the hard flags are given for
    const float* lut;
    const int* route;  // [BH]
    int* rows;         // [BH, chunks, 3, N]: the row above the chunk, then the two rows the sweep alternates between
    __nv_bfloat16* out;
    float* lse2;
    int batch, heads, n, lut_stride, chunks;
    const unsigned* choice;  // route word of a captured graph, or null
};

template <int R, int DV>
struct alignas(16) DenseStage {
    __nv_bfloat16 sk[DENSE_COLUMNS][R + 8];
    __nv_bfloat16 v[DENSE_COLUMNS][DV + 8];
};
template <int R, int DV>
struct alignas(16) DenseWarpShared {
    union {
        DenseStage<R, DV> stage[2];
        struct {
            float acc[DENSE_ROWS][DV];
            float maximum[DENSE_ROWS], denominator[DENSE_ROWS];
        } partial;  // the warp's share of a block's rows, handed to the merge
    };
    float weight[DENSE_ROWS][DENSE_COLUMNS + 1];  // log2 weights of the current columns
};

// The sweep of one chunk of one (batch, head) by the whole CTA.
template <int R, int DV>
__device__ __forceinline__ void hard_forward_dense_chunk(const DenseArgs& a, int bh, int chunk) {
    constexpr int KSTEPS = R / 16, VTILES = DV / 8;
    static_assert(sizeof(DenseWarpShared<R, DV>) >= sizeof(float) * DENSE_ROWS * (DV + 2), "the partial rows fit in the warp's stages");
    extern __shared__ __align__(16) unsigned char storage[];
    auto* shared = reinterpret_cast<DenseWarpShared<R, DV>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    auto& mine = shared[warp];
    const int b = bh / a.heads, h = bh % a.heads, n = a.n;
    const int64_t vec0 = int64_t(b) * n * a.heads + h;
    const int* __restrict__ iq = a.iq + int64_t(bh) * n;
    const int* __restrict__ ik = a.ik + int64_t(bh) * n;
    const float* __restrict__ lut = a.lut + int64_t(h) * a.lut_stride;
    int* rows = a.rows + (int64_t(bh) * a.chunks + chunk) * 3 * n;
    const int first_block = dense_chunk_start(chunk, a.chunks, n), last_block = dense_chunk_start(chunk + 1, a.chunks, n);
    const unsigned sk_stride = unsigned(a.heads) * R * 2, v_stride = unsigned(a.heads) * DV * 2;
    const char* sk_lane = reinterpret_cast<const char*>(a.sk + vec0 * R) + (lane % (R / 8)) * 16;
    const char* v_lane = reinterpret_cast<const char*>(a.v + vec0 * DV) + (lane % (DV / 8)) * 16;

    auto stage_columns = [&](DenseStage<R, DV>& stage, int c0) {  // rows c0 .. c0 + 31 of sk and v (all below n)
        constexpr int SK_ROWS = 32 / (R / 8), V_ROWS = 32 / (DV / 8);
#pragma unroll
        for (int key = lane / (R / 8); key < DENSE_COLUMNS; key += SK_ROWS)
            cp_async16_or_zeros(&stage.sk[key][(lane % (R / 8)) * 8], sk_lane + uint64_t(unsigned(c0 + key)) * sk_stride, 16);
#pragma unroll
        for (int key = lane / (DV / 8); key < DENSE_COLUMNS; key += V_ROWS)
            cp_async16_or_zeros(&stage.v[key][(lane % (DV / 8)) * 8], v_lane + uint64_t(unsigned(c0 + key)) * v_stride, 16);
        cp_async_commit();
    };

    for (int block = first_block; block < last_block; ++block) {
        const int i0 = block * DENSE_ROWS;
        const int* previous_row = block == first_block ? rows : rows + (1 + (block & 1)) * int64_t(n);  // L(i0 - 1, .)
        int* next_row = rows + (1 + ((block + 1) & 1)) * int64_t(n);                                    // L(i0 + 15, .)
        // A block lies inside one document (documents begin at multiples of 256) and one training row: its keys start
        // at the document's first position, and its rows are hard or not together.
        const int begin = a.documents ? __ldg(a.documents + i0 / 256).x : 0;
        const bool active = a.hard[(a.documents ? i0 / (n / a.hard_rows) : b) * a.heads + h] != 0;
        if (!active) {  // rows that are not hard read as zero, like everywhere else on this path; nothing follows from them
            for (int e = threadIdx.x; e < DENSE_ROWS * (DV / 8); e += blockDim.x) {
                const int row = i0 + e / (DV / 8);
                reinterpret_cast<uint4*>(a.out + (vec0 + int64_t(row) * a.heads) * DV)[e % (DV / 8)] = make_uint4(0u, 0u, 0u, 0u);
                if (e % (DV / 8) == 0) a.lse2[int64_t(bh) * n + row] = 0.f;
            }
            continue;
        }
        const int low_step = begin / DENSE_COLUMNS;
        const int steps = (i0 + DENSE_ROWS + DENSE_COLUMNS - 1) / DENSE_COLUMNS;  // 32-column steps up to the causal edge

        unsigned query[KSTEPS][4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const unsigned* source = reinterpret_cast<const unsigned*>(a.sq + (vec0 + int64_t(i0 + g + 8 * s) * a.heads) * R);
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                query[k][s] = __ldg(source + k * 8 + t);
                query[k][s + 2] = __ldg(source + k * 8 + 4 + t);
            }
        }
        int query_label[DENSE_ROWS];  // the block's sixteen query labels, the same in every lane
#pragma unroll
        for (int r = 0; r < DENSE_ROWS; ++r) query_label[r] = __ldg(iq + i0 + r);

        float acc[VTILES][4], maximum[2] = {-INFINITY, -INFINITY}, denominator[2] = {0.f, 0.f};
#pragma unroll
        for (int c = 0; c < VTILES; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;

        // this warp's share of the block's columns: a contiguous run of 32-column steps
        const int first_step = low_step + warp * (steps - low_step) / DENSE_WARPS;
        const int last_step = low_step + (warp + 1) * (steps - low_step) / DENSE_WARPS;
        if (first_step < last_step) stage_columns(mine.stage[0], first_step * DENSE_COLUMNS);

        // Run lengths, one key column per lane: L(i0 + r, c) = pair ? L(i0 + r - 1, c - 1) + 1 : 0.  The cell up and to the
        // left is the lane below's previous row; lane 0 gets it from the last column of the step before (`edge`).
        int edge[DENSE_ROWS];  // edge[r] = L(i0 + r, c0 - 1), the same in every lane
        auto run_lengths = [&](int c0, bool keep) {
            const int column = c0 + lane;
            const int key_label = __ldg(ik + column);
            // L(i0 - 1, column - 1): none before the document's first key, none on the non-causal side
            int above = column >= begin + 1 && column <= i0 ? previous_row[column - 1] : 0;
            int run = 0, passed_on = 0;  // passed_on: the previous row's run of the last column, the next step's edge
#pragma unroll
            for (int r = 0; r < DENSE_ROWS; ++r) {
                if (r > 0) {
                    above = __shfl_up_sync(FULL, run, 1);
                    if (lane == 0) above = edge[r - 1];
                    edge[r - 1] = passed_on;  // the old value was just used
                }
                run = key_label == query_label[r] && column <= i0 + r ? above + 1 : 0;
                passed_on = __shfl_sync(FULL, run, 31);
                if (keep) mine.weight[r][lane] = __ldg(lut + run);  // entry 0 is the log of zero
            }
            edge[DENSE_ROWS - 1] = passed_on;
            if (keep) next_row[column] = run;
        };
#pragma unroll
        for (int r = 0; r < DENSE_ROWS; ++r) edge[r] = 0;
        // The first step's edge comes from the 32 columns before it, worked through without an edge of their own: a wrong
        // cell in their first column moves one column per row and cannot reach their last column within sixteen rows.
        if (first_step > low_step && first_step < last_step) run_lengths((first_step - 1) * DENSE_COLUMNS, false);

        int buffer = 0;
        for (int step = first_step; step < last_step; ++step, buffer ^= 1) {
            const int c0 = step * DENSE_COLUMNS;
            const bool more = step + 1 < last_step;
            if (more) stage_columns(mine.stage[buffer ^ 1], c0 + DENSE_COLUMNS);
            run_lengths(c0, true);
            if (more) cp_async_wait<1>();
            else cp_async_wait<0>();
            __syncwarp();

            // ---- two sixteen-key tiles: scores, weights, value product ------------------------------------------
            const DenseStage<R, DV>& keys = mine.stage[buffer];
#pragma unroll
            for (int tile = 0; tile < DENSE_COLUMNS / KT; ++tile) {
                if (c0 + tile * KT > i0 + DENSE_ROWS - 1) break;  // wholly on the non-causal side
                float x[8];  // log2 weight of element slot s * 4 + j * 2 + e: row g + 8 s, column tile * 16 + j * 8 + 2 t + e
                float top[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    const int s = slot >> 2, j = (slot >> 1) & 1, e = slot & 1;
                    x[slot] = mine.weight[g + 8 * s][tile * KT + j * 8 + 2 * t + e];
                    top[s] = fmaxf(top[s], x[slot]);
                }
                if (!__ballot_sync(FULL, fmaxf(top[0], top[1]) > .5f * LOG_ZERO)) continue;  // no pair in this tile
                float score[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    score[j][0] = score[j][1] = score[j][2] = score[j][3] = 0.f;
#pragma unroll
                    for (int k = 0; k < KSTEPS; ++k) {
                        const unsigned* source = reinterpret_cast<const unsigned*>(&keys.sk[tile * KT + j * 8 + g][k * 16]);
                        mma_bf16_16816(score[j], query[k], source[t], source[4 + t]);
                    }
                }
                float p[8];
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    top[s] = fmaxf(top[s], __shfl_xor_sync(FULL, top[s], 1));
                    top[s] = fmaxf(top[s], __shfl_xor_sync(FULL, top[s], 2));
                    if (top[s] > maximum[s] && top[s] > .5f * LOG_ZERO) {  // the row's running state follows its maximum
                        const float alpha = ex2(maximum[s] - top[s]);
                        denominator[s] *= alpha;
#pragma unroll
                        for (int c = 0; c < VTILES; ++c) { acc[c][2 * s] *= alpha; acc[c][2 * s + 1] *= alpha; }
                        maximum[s] = top[s];
                    }
                    float sum = 0.f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        p[s * 4 + q] = x[s * 4 + q] > .5f * LOG_ZERO ? ex2(x[s * 4 + q] - maximum[s]) : 0.f;
                        sum += p[s * 4 + q];
                    }
                    sum += __shfl_xor_sync(FULL, sum, 1);
                    sum += __shfl_xor_sync(FULL, sum, 2);
                    denominator[s] += sum;
                }
                unsigned weights[4];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int s = 0; s < 2; ++s)
                        weights[2 * j + s] = pack_bf16(p[s * 4 + j * 2] * score[j][2 * s], p[s * 4 + j * 2 + 1] * score[j][2 * s + 1]);
#pragma unroll
                for (int c = 0; c < VTILES; ++c) {
                    unsigned b0, b1;
                    ldmatrix_x2_trans(b0, b1, &keys.v[tile * KT + (lane & 15)][c * 8]);
                    mma_bf16_16816(acc[c], weights, b0, b1);
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();
        __syncwarp();

        // ---- the warp's share of the block's rows, then the merge over warps ---------------------------------------
#pragma unroll
        for (int s = 0; s < 2; ++s) {
#pragma unroll
            for (int c = 0; c < VTILES; ++c)
                *reinterpret_cast<float2*>(&mine.partial.acc[g + 8 * s][c * 8 + 2 * t]) = make_float2(acc[c][2 * s], acc[c][2 * s + 1]);
            if (t == 0) {
                mine.partial.maximum[g + 8 * s] = maximum[s];
                mine.partial.denominator[g + 8 * s] = denominator[s];
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < DENSE_ROWS / DENSE_WARPS; ++r) {
            const int row = warp * (DENSE_ROWS / DENSE_WARPS) + r;
            float top = 0.f;  // the reference's normalisation: the maximum starts at 0 and the denominator at 1
#pragma unroll
            for (int w = 0; w < DENSE_WARPS; ++w) top = fmaxf(top, shared[w].partial.maximum[row]);
            float scale[DENSE_WARPS], total = ex2(-top);
#pragma unroll
            for (int w = 0; w < DENSE_WARPS; ++w) {
                scale[w] = ex2(shared[w].partial.maximum[row] - top);  // a warp without pairs: ex2(-inf) = 0
                total = fmaf(shared[w].partial.denominator[row], scale[w], total);
            }
            const float inverse = __frcp_rn(total);
            __nv_bfloat16* out = a.out + (vec0 + int64_t(i0 + row) * a.heads) * DV;
#pragma unroll
            for (int column = 2 * lane; column < DV; column += 64) {
                float2 sum = make_float2(0.f, 0.f);
#pragma unroll
                for (int w = 0; w < DENSE_WARPS; ++w) {
                    const float2 part = *reinterpret_cast<const float2*>(&shared[w].partial.acc[row][column]);
                    sum.x = fmaf(part.x, scale[w], sum.x);
                    sum.y = fmaf(part.y, scale[w], sum.y);
                }
                *reinterpret_cast<__nv_bfloat162*>(out + column) = __floats2bfloat162_rn(sum.x * inverse, sum.y * inverse);
            }
            if (lane == 0) a.lse2[int64_t(bh) * n + i0 + row] = top + log2f(total);
        }
        __syncthreads();  // the partial rows lie in the stages the next block loads into; next_row is complete
    }
}

template <int R, int DV>
__global__ __launch_bounds__(DENSE_WARPS * 32, 1) void hard_forward_dense_kernel(const DenseArgs a) {
    const int batch_heads = a.batch * a.heads;
    if (!route_open(a.choice)) return;  // (the word holds still during a replay, so the whole grid agrees)
    if (!dense_any(a.route, batch_heads)) return;
    dense_walk_all(a.iq, a.ik, a.documents, a.route, a.rows, 1, batch_heads, a.chunks, a.n);
    __threadfence();
    cooperative_groups::this_grid().sync();
    for (int item = blockIdx.x; item < batch_heads * a.chunks; item += gridDim.x) {
        const int bh = item / a.chunks;
        if (a.route[bh] == DENSE_ROUTE) hard_forward_dense_chunk<R, DV>(a, bh, item % a.chunks);
    }
}

}  // namespace dism
