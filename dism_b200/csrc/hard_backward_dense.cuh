// Hard backward for dense labels: the consecutive-position tiles of hard_forward_dense.cuh, once
// owned by query rows (dSQ and the per-row tau terms) and once owned by key columns (dV, dSK).
//
// Both passes are the same sweep seen from either side of the diagonal.  The owners of a block are
// sixteen consecutive positions of one side; the partners are all positions of the other side on
// the causal side of the block, split among the warps of a CTA in contiguous runs of thirty-two.
// A lane owns one partner and steps through the block's sixteen owners: the run length of
// (owner r, partner p) is that of (owner r-1, partner p-1) plus one on a label match, which is the
// lane below's previous value; the first owner takes it from the vector the previous block left
// behind (for a chunk's first block, from the walk along whole diagonals that the grid does
// before the sweeps).  With the forward's
// log2 normaliser known the lane turns the run length straight into the pair's probability
// p = 2^(lut[L] - lse2[query]); the tiles then follow the label-block backward
// (hard_backward_blocks.cuh): S and E on tensor cores, coefficient tiles p o E and p o S as bf16
// value-and-remainder pairs, second products into the gradient rows, and the four centred moments
// of the tau derivative from row sums.  The warps' partial rows are added in a fixed order, so the
// results do not depend on timing; every output row is written once.
#pragma once
#include "hard_backward_blocks.cuh"
#include "hard_forward_dense.cuh"

namespace dism {

struct DenseBackwardArgs {
    const __nv_bfloat16 *sq, *sk, *v, *dout;
    const int *iq, *ik;
    const uint8_t* hard;
    const int2* documents;  // packed layouts: (first position, end) of the document of every 256-position block; else null
    int hard_rows;          // packed layouts: training rows the hard flags are given for
    const float *lut, *dlut, *lse2;
    const int* route;  // [BH]
    int* lines;        // [2 passes, BH, chunks, 3, N]: the vector before the chunk, then the two vectors the sweep alternates between
    float *dsq, *dtau_rows;
    __nv_bfloat16 *dsk, *dv;
    int batch, heads, n, lut_stride, chunks;
    const unsigned* choice;  // route word of a captured graph, or null
};

// Scratch of the dense backward: for each pass what the forward keeps for its one sweep.
__host__ __device__ inline size_t dense_backward_bytes(int batch_heads, int n) { return 2 * dense_bytes(batch_heads, n); }

template <int R, int DV>
struct alignas(16) DenseBackwardStage {
    __nv_bfloat16 a[DENSE_COLUMNS][R + 8];   // partners' R-vectors: sk (query-major) or sq
    __nv_bfloat16 b[DENSE_COLUMNS][DV + 8];  // partners' DV-vectors: v (query-major) or dO
};
template <int R, int DV>
struct alignas(16) DenseBackwardWarpShared {
    union {
        DenseBackwardStage<R, DV> stage[2];
        struct {
            float grad_a[DENSE_ROWS][R];
            float grad_b[DENSE_ROWS][DV];   // key-major only
            float moments[4][DENSE_ROWS];   // query-major only: u, z, v, w
        } partial;
    };
    float probability[DENSE_ROWS][DENSE_COLUMNS + 1];  // p of (owner, partner) for the current partners
    float weighted_gap[DENSE_ROWS][DENSE_COLUMNS + 1]; // query-major: p * (dlut[L] - centre of the row)
};

template <bool QUERY_MAJOR, int R, int DV>
__device__ __forceinline__ void hard_backward_dense_chunk(const DenseBackwardArgs& a, int bh, int chunk) {
    constexpr int KSTEPS = R / 16, VSTEPS = DV / 16, RTILES = R / 8, VTILES = DV / 8;
    extern __shared__ __align__(16) unsigned char storage[];
    auto* shared = reinterpret_cast<DenseBackwardWarpShared<R, DV>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    auto& mine = shared[warp];
    const int b = bh / a.heads, h = bh % a.heads, n = a.n;
    const int64_t vec0 = int64_t(b) * n * a.heads + h;
    const int* __restrict__ owner_labels = (QUERY_MAJOR ? a.iq : a.ik) + int64_t(bh) * n;
    const int* __restrict__ partner_labels = (QUERY_MAJOR ? a.ik : a.iq) + int64_t(bh) * n;
    const float* __restrict__ lut = a.lut + int64_t(h) * a.lut_stride;
    const float* __restrict__ dlut = a.dlut + int64_t(h) * a.lut_stride;
    const float* __restrict__ lse2 = a.lse2 + int64_t(bh) * n;
    int* lines = a.lines + ((int64_t(QUERY_MAJOR ? 0 : 1) * a.batch * a.heads + bh) * a.chunks + chunk) * 3 * n;
    const int first_block = dense_owner_start(QUERY_MAJOR, chunk, a.chunks, n), last_block = dense_owner_start(QUERY_MAJOR, chunk + 1, a.chunks, n);
    const __nv_bfloat16* own_a = QUERY_MAJOR ? a.sq : a.sk;    // R wide
    const __nv_bfloat16* own_b = QUERY_MAJOR ? a.dout : a.v;   // DV wide
    const __nv_bfloat16* other_a = QUERY_MAJOR ? a.sk : a.sq;
    const __nv_bfloat16* other_b = QUERY_MAJOR ? a.v : a.dout;
    const unsigned a_stride = unsigned(a.heads) * R * 2, b_stride = unsigned(a.heads) * DV * 2;
    const char* a_lane = reinterpret_cast<const char*>(other_a + vec0 * R) + (lane % (R / 8)) * 16;
    const char* b_lane = reinterpret_cast<const char*>(other_b + vec0 * DV) + (lane % (DV / 8)) * 16;

    auto stage_partners = [&](DenseBackwardStage<R, DV>& stage, int c0) {  // partners c0 .. c0 + 31 (all below n)
        constexpr int A_ROWS = 32 / (R / 8), B_ROWS = 32 / (DV / 8);
#pragma unroll
        for (int row = lane / (R / 8); row < DENSE_COLUMNS; row += A_ROWS)
            cp_async16_or_zeros(&stage.a[row][(lane % (R / 8)) * 8], a_lane + uint64_t(unsigned(c0 + row)) * a_stride, 16);
#pragma unroll
        for (int row = lane / (DV / 8); row < DENSE_COLUMNS; row += B_ROWS)
            cp_async16_or_zeros(&stage.b[row][(lane % (DV / 8)) * 8], b_lane + uint64_t(unsigned(c0 + row)) * b_stride, 16);
        cp_async_commit();
    };

    for (int block = first_block; block < last_block; ++block) {
        const int o0 = block * DENSE_ROWS;  // first owner of the block
        const int* previous_line = block == first_block ? lines : lines + (1 + (block & 1)) * int64_t(n);
        int* next_line = lines + (1 + ((block + 1) & 1)) * int64_t(n);
        // A block lies inside one document (documents begin at multiples of 256) and one training row.
        int begin = 0, end = n;
        if (a.documents) {
            const int2 document = __ldg(a.documents + o0 / 256);
            begin = document.x;
            end = document.y;
        }
        if (!a.hard[(a.documents ? o0 / (n / a.hard_rows) : b) * a.heads + h]) {  // rows that are not hard have zero gradients
            for (int e = threadIdx.x; e < DENSE_ROWS * 32; e += blockDim.x) {
                const int row = o0 + e / 32, piece = e % 32;
                const int64_t at = vec0 + int64_t(row) * a.heads;
                if (QUERY_MAJOR) {
                    if (piece < R / 4) reinterpret_cast<float4*>(a.dsq + at * R)[piece] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (piece == 31) a.dtau_rows[int64_t(bh) * n + row] = 0.f;
                } else {
                    if (piece < R / 8) reinterpret_cast<uint4*>(a.dsk + at * R)[piece] = make_uint4(0u, 0u, 0u, 0u);
                    if (piece >= 16 && piece - 16 < DV / 8) reinterpret_cast<uint4*>(a.dv + at * DV)[piece - 16] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            continue;
        }
        // 32-partner steps on the causal side inside the document: keys from its start up to the block's last query, or
        // queries from the block's first key to its end
        const int low_step = QUERY_MAJOR ? begin / DENSE_COLUMNS : o0 / DENSE_COLUMNS;
        const int high_step = QUERY_MAJOR ? (o0 + DENSE_ROWS + DENSE_COLUMNS - 1) / DENSE_COLUMNS : end / DENSE_COLUMNS;
        const int first_step = low_step + warp * (high_step - low_step) / DENSE_WARPS;
        const int last_step = low_step + (warp + 1) * (high_step - low_step) / DENSE_WARPS;

        unsigned frag_a[KSTEPS][4], frag_b[VSTEPS][4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int64_t at = vec0 + int64_t(o0 + g + 8 * s) * a.heads;
            const unsigned* source_a = reinterpret_cast<const unsigned*>(own_a + at * R);
            const unsigned* source_b = reinterpret_cast<const unsigned*>(own_b + at * DV);
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                frag_a[k][s] = __ldg(source_a + k * 8 + t);
                frag_a[k][s + 2] = __ldg(source_a + k * 8 + 4 + t);
            }
#pragma unroll
            for (int k = 0; k < VSTEPS; ++k) {
                frag_b[k][s] = __ldg(source_b + k * 8 + t);
                frag_b[k][s + 2] = __ldg(source_b + k * 8 + 4 + t);
            }
        }
        int owner_label[DENSE_ROWS];      // the same in every lane
        float owner_norm[DENSE_ROWS], owner_center[DENSE_ROWS];  // query-major: the rows' log2 normalisers and centres
#pragma unroll
        for (int r = 0; r < DENSE_ROWS; ++r) {
            owner_label[r] = __ldg(owner_labels + o0 + r);
            owner_norm[r] = QUERY_MAJOR ? __ldg(lse2 + o0 + r) : 0.f;
            owner_center[r] = QUERY_MAJOR ? __ldg(dlut + o0 + r - begin + 1) : 0.f;
        }

        float grad_a[RTILES][4], grad_b[QUERY_MAJOR ? 1 : VTILES][4];
#pragma unroll
        for (int c = 0; c < RTILES; ++c) grad_a[c][0] = grad_a[c][1] = grad_a[c][2] = grad_a[c][3] = 0.f;
#pragma unroll
        for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c) grad_b[c][0] = grad_b[c][1] = grad_b[c][2] = grad_b[c][3] = 0.f;
        float u[2] = {0.f, 0.f}, z[2] = {0.f, 0.f}, v[2] = {0.f, 0.f}, w[2] = {0.f, 0.f};

        if (first_step < last_step) stage_partners(mine.stage[0], first_step * DENSE_COLUMNS);

        // Run lengths, one partner per lane (see the forward's kernel); stored as probabilities.
        int edge[DENSE_ROWS];
        auto run_lengths = [&](int c0, bool keep) {
            const int partner = c0 + lane;
            const int partner_label = __ldg(partner_labels + partner);
            const float partner_norm = QUERY_MAJOR ? 0.f : __ldg(lse2 + partner);
            // the cell up and to the left exists inside the document and on the causal side
            const bool has_above = QUERY_MAJOR ? partner >= begin + 1 && partner <= o0 : o0 >= begin + 1 && partner >= o0;
            int above = has_above ? previous_line[partner - 1] : 0;
            int run = 0, passed_on = 0;
#pragma unroll
            for (int r = 0; r < DENSE_ROWS; ++r) {
                if (r > 0) {
                    above = __shfl_up_sync(FULL, run, 1);
                    if (lane == 0) above = edge[r - 1];
                    edge[r - 1] = passed_on;
                }
                const bool causal = QUERY_MAJOR ? partner <= o0 + r : partner >= o0 + r;
                run = partner_label == owner_label[r] && causal ? above + 1 : 0;
                passed_on = __shfl_sync(FULL, run, 31);
                if (keep) {
                    const float p = ex2(__ldg(lut + run) - (QUERY_MAJOR ? owner_norm[r] : partner_norm));  // entry 0 is the log of zero
                    mine.probability[r][lane] = p;
                    if (QUERY_MAJOR) mine.weighted_gap[r][lane] = p * (__ldg(dlut + run) - owner_center[r]);
                }
            }
            edge[DENSE_ROWS - 1] = passed_on;
            if (keep) next_line[partner] = run;
        };
#pragma unroll
        for (int r = 0; r < DENSE_ROWS; ++r) edge[r] = 0;
        if (first_step > low_step && first_step < last_step) run_lengths((first_step - 1) * DENSE_COLUMNS, false);

        int buffer = 0;
        for (int step = first_step; step < last_step; ++step, buffer ^= 1) {
            const int c0 = step * DENSE_COLUMNS;
            const bool more = step + 1 < last_step;
            if (more) stage_partners(mine.stage[buffer ^ 1], c0 + DENSE_COLUMNS);
            run_lengths(c0, true);
            if (more) cp_async_wait<1>();
            else cp_async_wait<0>();
            __syncwarp();
            const DenseBackwardStage<R, DV>& partners = mine.stage[buffer];
#pragma unroll
            for (int tile = 0; tile < DENSE_COLUMNS / KT; ++tile) {
                const int p0 = c0 + tile * KT;
                if (QUERY_MAJOR ? p0 > o0 + DENSE_ROWS - 1 : p0 + KT - 1 < o0) continue;  // wholly on the non-causal side
                float p[8], pg[8], largest = 0.f;  // element slot s * 4 + j * 2 + e: owner g + 8 s, partner p0 + j * 8 + 2 t + e
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    const int s = slot >> 2, j = (slot >> 1) & 1, e = slot & 1;
                    p[slot] = mine.probability[g + 8 * s][tile * KT + j * 8 + 2 * t + e];
                    pg[slot] = QUERY_MAJOR ? mine.weighted_gap[g + 8 * s][tile * KT + j * 8 + 2 * t + e] : 0.f;
                    largest = fmaxf(largest, p[slot]);
                }
                if (!__ballot_sync(FULL, largest > 0.f)) continue;  // no pair in this tile
                float s_tile[2][4], e_tile[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    s_tile[j][0] = s_tile[j][1] = s_tile[j][2] = s_tile[j][3] = 0.f;
                    e_tile[j][0] = e_tile[j][1] = e_tile[j][2] = e_tile[j][3] = 0.f;
#pragma unroll
                    for (int k = 0; k < KSTEPS; ++k) {
                        const unsigned* source = reinterpret_cast<const unsigned*>(&partners.a[tile * KT + j * 8 + g][k * 16]);
                        mma_bf16_16816(s_tile[j], frag_a[k], source[t], source[4 + t]);
                    }
#pragma unroll
                    for (int k = 0; k < VSTEPS; ++k) {
                        const unsigned* source = reinterpret_cast<const unsigned*>(&partners.b[tile * KT + j * 8 + g][k * 16]);
                        mma_bf16_16816(e_tile[j], frag_b[k], source[t], source[4 + t]);
                    }
                }
                unsigned coefficient_e[4], remainder_e[4], coefficient_s[4], remainder_s[4];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        float pe[2], ps[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int slot = s * 4 + j * 2 + e;
                            const float score = s_tile[j][2 * s + e], slope = e_tile[j][2 * s + e];
                            pe[e] = p[slot] * slope;
                            ps[e] = p[slot] * score;
                            if (QUERY_MAJOR) {
                                const float se = score * slope;
                                u[s] = fmaf(p[slot], se, u[s]);
                                z[s] += p[slot];
                                v[s] += pg[slot];
                                w[s] = fmaf(pg[slot], se, w[s]);
                            }
                        }
                        split_bf16(pe[0], pe[1], coefficient_e[2 * j + s], remainder_e[2 * j + s]);
                        if (!QUERY_MAJOR) split_bf16(ps[0], ps[1], coefficient_s[2 * j + s], remainder_s[2 * j + s]);
                    }
#pragma unroll
                for (int c = 0; c < RTILES; ++c) {  // (p o E) times the partners' R-vectors: dSQ or dSK
                    unsigned b0, b1;
                    ldmatrix_x2_trans(b0, b1, &partners.a[tile * KT + (lane & 15)][c * 8]);
                    mma_bf16_16816(grad_a[c], coefficient_e, b0, b1);
                    mma_bf16_16816(grad_a[c], remainder_e, b0, b1);
                }
                if (!QUERY_MAJOR) {  // (p o S) times the queries' dO rows: dV
#pragma unroll
                    for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c) {
                        unsigned b0, b1;
                        ldmatrix_x2_trans(b0, b1, &partners.b[tile * KT + (lane & 15)][c * 8]);
                        mma_bf16_16816(grad_b[c], coefficient_s, b0, b1);
                        mma_bf16_16816(grad_b[c], remainder_s, b0, b1);
                    }
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();
        __syncwarp();

        // ---- the warp's share of the block's rows, then the sum over warps in a fixed order ---------------------------
#pragma unroll
        for (int s = 0; s < 2; ++s) {
#pragma unroll
            for (int c = 0; c < RTILES; ++c)
                *reinterpret_cast<float2*>(&mine.partial.grad_a[g + 8 * s][c * 8 + 2 * t]) = make_float2(grad_a[c][2 * s], grad_a[c][2 * s + 1]);
            if (QUERY_MAJOR) {
                float moment[4] = {u[s], z[s], v[s], w[s]};
#pragma unroll
                for (int m = 0; m < 4; ++m) {  // the four lanes of a row summed different partners
                    moment[m] += __shfl_xor_sync(FULL, moment[m], 1);
                    moment[m] += __shfl_xor_sync(FULL, moment[m], 2);
                    if (t == 0) mine.partial.moments[m][g + 8 * s] = moment[m];
                }
            } else {
#pragma unroll
                for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c)
                    *reinterpret_cast<float2*>(&mine.partial.grad_b[g + 8 * s][c * 8 + 2 * t]) = make_float2(grad_b[c][2 * s], grad_b[c][2 * s + 1]);
            }
        }
        __syncthreads();
        for (int e = threadIdx.x; e < DENSE_ROWS * R / 2; e += blockDim.x) {
            const int row = e / (R / 2), column = 2 * (e % (R / 2));
            float2 sum = make_float2(0.f, 0.f);
#pragma unroll
            for (int wp = 0; wp < DENSE_WARPS; ++wp) {
                const float2 part = *reinterpret_cast<const float2*>(&shared[wp].partial.grad_a[row][column]);
                sum.x += part.x;
                sum.y += part.y;
            }
            const int64_t at = vec0 + int64_t(o0 + row) * a.heads;
            if (QUERY_MAJOR) *reinterpret_cast<float2*>(a.dsq + at * R + column) = sum;
            else *reinterpret_cast<__nv_bfloat162*>(a.dsk + at * R + column) = __floats2bfloat162_rn(sum.x, sum.y);
        }
        if (QUERY_MAJOR) {
            if (threadIdx.x < DENSE_ROWS) {
                const int row = threadIdx.x;
                float total[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int wp = 0; wp < DENSE_WARPS; ++wp)
#pragma unroll
                    for (int m = 0; m < 4; ++m) total[m] += shared[wp].partial.moments[m][row];
                // centred four-moment form: the fallback has unit weight and zero derivative
                const float norm = __ldg(lse2 + o0 + row), center = __ldg(dlut + o0 + row - begin + 1);
                const float fallback = ex2(-norm), inverse = __fdividef(1.f, total[1] + fallback);
                const float mean = fmaf(-fallback, center, total[2]) * inverse;
                a.dtau_rows[int64_t(bh) * n + o0 + row] = fmaf(-total[0], mean, total[3]) * inverse;
            }
        } else {
            for (int e = threadIdx.x; e < DENSE_ROWS * DV / 2; e += blockDim.x) {
                const int row = e / (DV / 2), column = 2 * (e % (DV / 2));
                float2 sum = make_float2(0.f, 0.f);
#pragma unroll
                for (int wp = 0; wp < DENSE_WARPS; ++wp) {
                    const float2 part = *reinterpret_cast<const float2*>(&shared[wp].partial.grad_b[row][column]);
                    sum.x += part.x;
                    sum.y += part.y;
                }
                *reinterpret_cast<__nv_bfloat162*>(a.dv + (vec0 + int64_t(o0 + row) * a.heads) * DV + column) = __floats2bfloat162_rn(sum.x, sum.y);
            }
        }
        __syncthreads();  // the partial rows lie in the stages the next block loads into; next_line is complete
    }
}

// Both sweeps of a backward in one launch: the work items are (pass, slice, chunk).
template <int R, int DV>
__global__ __launch_bounds__(DENSE_WARPS * 32, 1) void hard_backward_dense_kernel(const DenseBackwardArgs a) {
    const int batch_heads = a.batch * a.heads;
    if (!route_open(a.choice)) return;
    if (!dense_any(a.route, batch_heads)) return;
    dense_walk_all(a.iq, a.ik, a.documents, a.route, a.lines, 2, batch_heads, a.chunks, a.n);
    __threadfence();
    cooperative_groups::this_grid().sync();
    for (int item = blockIdx.x; item < 2 * batch_heads * a.chunks; item += gridDim.x) {
        const int slice = item / a.chunks, bh = slice % batch_heads;
        if (a.route[bh] != DENSE_ROUTE) continue;
        if (slice < batch_heads) hard_backward_dense_chunk<true, R, DV>(a, bh, item % a.chunks);
        else hard_backward_dense_chunk<false, R, DV>(a, bh, item % a.chunks);
    }
}

}  // namespace dism
