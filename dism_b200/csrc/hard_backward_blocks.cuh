// Hard backward as label-block tensor-core tiles (same decomposition as the forward).
//
// With the forward's log2 normaliser known, an ordinary pair (run length 1) has probability
// c_i = 2^(lut[1] - lse2_i): one constant per query.  Both passes therefore reduce to masked tile
// products on bf16 tensor cores:
//   query-major (dSQ, tau terms): S = SQ.SK^T, E = dO.V^T, dSQ += (c o mask o E).SK, and the four
//                                 moments from row sums of mask, mask o S o E;
//   key-major   (dV, dSK):        S^T = SK.SQ^T, E^T = V.dO^T, dV += (mask o S^T o c).dO,
//                                 dSK += (mask o E^T o c).SQ.
// The coefficient tiles are fed to the second product as a bf16 pair (value and rounding
// remainder), so they carry FP32-like accuracy.  Pairs with longer runs are rare; the whole warp
// adds them one by one in ascending partner order, walking the diagonal for the run length.
// Every output row belongs to one warp and is accumulated in a fixed order: no atomics, and the
// same bits for every grid size.
#pragma once
#include <type_traits>

#include "hard_forward_blocks.cuh"

namespace dism {

// Sixteen partner rows of one step: their two vectors (A: R wide, B: DV wide) and per-partner scalars.
template <int R, int DV>
struct alignas(16) PartnerStage {
    __nv_bfloat16 a[KT][R + 8];
    __nv_bfloat16 b[KT][DV + 8];
    int position[KT], label[KT], previous[KT];
    float common[KT], common_two[KT], norm[KT];  // key-major only: the query's weights of run lengths 1 and 2, and its log2 normaliser
};

template <int R, int DV>
struct alignas(16) BackwardWarpShared {
    PartnerStage<R, DV> stage[2];
    int position[QT], label[QT], previous[QT], begin[QT], end[QT], active[QT];
    float norm[QT], center[QT];
};

struct BackwardBlockArgs {
    const __nv_bfloat16 *sq, *sk, *v, *dout;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float *lut, *dlut, *lse2;
    SideIndex owners, partners;  // index of the side that owns the rows, and of the other side
    const int* tile_starts;
    const int4* tiles;
    int* next_tile;
    int tile_capacity;
    const int2* documents;
    float *dsq, *dtau_rows;
    __nv_bfloat16 *dsk, *dv;
    int batch, heads, n, lut_stride, hard_rows;
};

// value and rounding remainder of two floats, each packed as a bf16 pair
__device__ __forceinline__ void split_bf16(float x, float y, unsigned& high, unsigned& low) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 back = __bfloat1622float2(h);
    high = *reinterpret_cast<const unsigned*>(&h);
    low = pack_bf16(x - back.x, y - back.y);
}

// PACKED: rows carry document limits (a.documents is set); otherwise every row's document is the whole sequence
// and the limits are constants the compiler folds away.
template <bool QUERY_MAJOR, bool PACKED, int R, int DV>
__device__ __forceinline__ void hard_backward_blocks_pass(const BackwardBlockArgs& a) {
    constexpr int KSTEPS = R / 16, VSTEPS = DV / 16, RTILES = R / 8, VTILES = DV / 8;
    extern __shared__ __align__(16) unsigned char storage[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    auto& mine = reinterpret_cast<BackwardWarpShared<R, DV>*>(storage)[warp];
    const int bh = blockIdx.x, b = bh / a.heads, h = bh % a.heads;  // x: CTAs are handed out slice after slice, so every slice always has CTAs at work
    const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
    const int* iq = a.iq + int64_t(bh) * a.n;
    const int* ik = a.ik + int64_t(bh) * a.n;
    const int* boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
    const float* lut = a.lut + int64_t(h) * a.lut_stride;
    const float* dlut = a.dlut + int64_t(h) * a.lut_stride;
    const float* lse2 = a.lse2 + int64_t(bh) * a.n;
    const int2* owner_entries = a.owners.entries + int64_t(bh) * a.n;
    const int* owner_previous = a.owners.previous + int64_t(bh) * a.n;
    const int2* partner_entries = a.partners.entries + int64_t(bh) * a.n;
    const int* partner_previous = a.partners.previous + int64_t(bh) * a.n;
    const int4* tiles = a.tiles + int64_t(bh) * a.tile_capacity;
    const int tile_count = __ldg(a.tile_starts + int64_t(bh) * (BUCKETS + 1) + BUCKETS);
    const float weight_one = __ldg(lut + 1), derivative_one = __ldg(dlut + 1);
    const float weight_two = a.lut_stride > 2 ? __ldg(lut + 2) : 0.f, derivative_two = a.lut_stride > 2 ? __ldg(dlut + 2) : 0.f;
    // the owners' two vectors (rows of the first product) and the partners' (staged per step)
    const __nv_bfloat16* own_a = QUERY_MAJOR ? a.sq : a.sk;    // R wide
    const __nv_bfloat16* own_b = QUERY_MAJOR ? a.dout : a.v;   // DV wide
    const __nv_bfloat16* other_a = QUERY_MAJOR ? a.sk : a.sq;
    const __nv_bfloat16* other_b = QUERY_MAJOR ? a.v : a.dout;

    // gathered rows: a lane always copies the same 16-byte piece of a row, so its source is one pointer
    // plus position * stride (32-bit product: a (batch, head) slice spans less than 4 GB)
    const unsigned a_stride = unsigned(a.heads) * R * 2, b_stride = unsigned(a.heads) * DV * 2;
    const char* a_lane = reinterpret_cast<const char*>(other_a + vec0 * R) + (lane % (R / 8)) * 16;
    const char* b_lane = reinterpret_cast<const char*>(other_b + vec0 * DV) + (lane % (DV / 8)) * 16;

    for (;;) {
        int tile = 0;
        if (lane == 0) tile = atomicAdd(a.next_tile + bh, 1);
        tile = __shfl_sync(FULL, tile, 0);
        if (tile >= tile_count) break;
        const int4 plan = __ldg(tiles + tile);
        const int first_owner = plan.x, owners = plan.y;
        __syncwarp();
        if (lane < QT) {
            int2 entry = make_int2(-1, 0);
            int previous = 0, begin = 0, end = a.n, active = 0;
            float norm = 0.f, center = 0.f;
            if (lane < owners) {
                entry = __ldg(owner_entries + first_owner + lane);
                previous = __ldg(owner_previous + first_owner + lane);
                int hard_row = b;
                if (PACKED) {
                    const int2 document = __ldg(a.documents + entry.x / 256);
                    begin = document.x;
                    end = document.y;
                    hard_row = entry.x / (a.n / a.hard_rows);
                }
                active = a.hard[hard_row * a.heads + h];
                if (QUERY_MAJOR) {
                    norm = __ldg(lse2 + entry.x);
                    center = __ldg(dlut + entry.x - begin + 1);
                }
            }
            mine.position[lane] = entry.x;
            mine.label[lane] = entry.y;
            mine.previous[lane] = previous;
            mine.begin[lane] = begin;
            mine.end[lane] = end;
            mine.active[lane] = active;
            mine.norm[lane] = norm;
            mine.center[lane] = center;
        }
        __syncwarp();
        int position[2], label[2], previous[2], begin[2], end[2];
        bool active[2];
        float norm[2], center[2], common_row[2], common_two_row[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int r = g + 8 * s;
            position[s] = mine.position[r];
            label[s] = mine.label[r];
            previous[s] = mine.previous[r];
            begin[s] = PACKED ? mine.begin[r] : 0;
            end[s] = PACKED ? mine.end[r] : a.n;
            active[s] = mine.active[r] != 0;
            norm[s] = mine.norm[r];
            center[s] = mine.center[r];
            common_row[s] = active[s] ? ex2(weight_one - norm[s]) : 0.f;  // query-major: weight of an ordinary pair of the row
            common_two_row[s] = active[s] ? ex2(weight_two - norm[s]) : 0.f;  // and of a pair of run length 2
        }
        // partner range inside the bucket: keys from the earliest document start to the last query, or
        // queries from the first key to the latest document end
        int partner_begin = plan.z, partner_end = plan.w;
        if (QUERY_MAJOR) {
            if (PACKED) {
                int first = mine.begin[0];
                for (int r = 1; r < owners; ++r) first = min(first, mine.begin[r]);
                partner_begin = warp_lower_bound_position(partner_entries, partner_begin, partner_end, first, lane);
            }
        } else {
            // First query at or after the tile's first key.  The bucket's queries are probed 32 at a time by the
            // whole warp (one coalesced read each) before a binary search takes over: most buckets hold fewer.
            {
                const int bound = mine.position[0];
                int probed = 0;
                for (; probed < 64 && partner_begin < partner_end; probed += 32) {
                    const int at = partner_begin + lane;
                    const bool before = at < partner_end && __ldg(partner_entries + at).x < bound;
                    const unsigned mask = __ballot_sync(FULL, before);
                    partner_begin += __popc(mask);
                    if (mask != FULL) break;
                }
                if (probed >= 64) partner_begin = warp_lower_bound_position(partner_entries, partner_begin, partner_end, bound, lane);
            }
            if (PACKED) {
                int last = mine.end[0];
                for (int r = 1; r < owners; ++r) last = max(last, mine.end[r]);
                partner_end = warp_lower_bound_position(partner_entries, partner_begin, partner_end, last, lane);
            }
        }
        const int last_owner = mine.position[owners - 1];

        unsigned frag_a[KSTEPS][4], frag_b[VSTEPS][4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int64_t at = vec0 + int64_t(max(position[s], 0)) * a.heads;
            const unsigned* source_a = reinterpret_cast<const unsigned*>(own_a + at * R);
            const unsigned* source_b = reinterpret_cast<const unsigned*>(own_b + at * DV);
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                frag_a[k][s] = active[s] ? __ldg(source_a + k * 8 + t) : 0u;
                frag_a[k][s + 2] = active[s] ? __ldg(source_a + k * 8 + 4 + t) : 0u;
            }
#pragma unroll
            for (int k = 0; k < VSTEPS; ++k) {
                frag_b[k][s] = active[s] ? __ldg(source_b + k * 8 + t) : 0u;
                frag_b[k][s + 2] = active[s] ? __ldg(source_b + k * 8 + 4 + t) : 0u;
            }
        }
        // accumulators: query-major dSQ [R]; key-major dSK [R] and dV [DV]
        float grad_a[RTILES][4], grad_b[QUERY_MAJOR ? 1 : VTILES][4];
#pragma unroll
        for (int c = 0; c < RTILES; ++c) grad_a[c][0] = grad_a[c][1] = grad_a[c][2] = grad_a[c][3] = 0.f;
#pragma unroll
        for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c) grad_b[c][0] = grad_b[c][1] = grad_b[c][2] = grad_b[c][3] = 0.f;
        float sum_se[2] = {0.f, 0.f}, u[2] = {0.f, 0.f}, v[2] = {0.f, 0.f}, w[2] = {0.f, 0.f}, z[2] = {0.f, 0.f};
        int ordinary_total[2] = {0, 0};
        float sum_se_two[2] = {0.f, 0.f};  // the same two sums over the pairs of run length 2
        int two_total[2] = {0, 0};

        auto classify = [&](int s, int other, int other_label, int other_previous) {
            bool pair = active[s] && other_label == label[s];
            if (QUERY_MAJOR) pair = pair && other <= position[s] && other >= begin[s];
            else pair = pair && other >= position[s] && other < end[s];
            const bool longer = pair && other > begin[s] && position[s] > begin[s] && other_previous == previous[s];
            return pair ? (longer ? 2 : 1) : 0;
        };
        auto stage_partners = [&](PartnerStage<R, DV>& partners, int k0) {
            int other = 0x7fffffff;
            if (lane < KT) {
                int2 entry = make_int2(QUERY_MAJOR ? 0x7fffffff : -1, 0);
                int before = 0;
                if (k0 + lane < partner_end) {
                    entry = __ldg(partner_entries + k0 + lane);
                    before = __ldg(partner_previous + k0 + lane);
                    other = entry.x;
                }
                partners.position[lane] = entry.x;
                partners.label[lane] = entry.y;
                partners.previous[lane] = before;
            }
            float normaliser = 0.f;  // key-major: read now, stored after the rows are on their way
            if (!QUERY_MAJOR && other != 0x7fffffff) normaliser = __ldg(lse2 + other);
            constexpr int A_ROWS = 32 / (R / 8), B_ROWS = 32 / (DV / 8);  // rows a warp covers per round
#pragma unroll
            for (int row = lane / (R / 8); row < KT; row += A_ROWS) {
                const int at = __shfl_sync(FULL, other, row);
                const bool present = at != 0x7fffffff;
                cp_async16_or_zeros(&partners.a[row][(lane % (R / 8)) * 8], a_lane + (present ? uint64_t(unsigned(at)) * a_stride : 0), present ? 16 : 0);
            }
#pragma unroll
            for (int row = lane / (DV / 8); row < KT; row += B_ROWS) {
                const int at = __shfl_sync(FULL, other, row);
                const bool present = at != 0x7fffffff;
                cp_async16_or_zeros(&partners.b[row][(lane % (DV / 8)) * 8], b_lane + (present ? uint64_t(unsigned(at)) * b_stride : 0), present ? 16 : 0);
            }
            cp_async_commit();
            if (lane < KT) {
                partners.norm[lane] = normaliser;
                partners.common[lane] = ex2(weight_one - normaliser);
                partners.common_two[lane] = ex2(weight_two - normaliser);
            }
        };

        if (partner_begin < partner_end) stage_partners(mine.stage[0], partner_begin);
        int buffer = 0;
        for (int k0 = partner_begin; k0 < partner_end; k0 += KT, buffer ^= 1) {
            const bool more = k0 + KT < partner_end;
            if (more) stage_partners(mine.stage[buffer ^ 1], k0 + KT);
            if (more) cp_async_wait<1>();
            else cp_async_wait<0>();
            __syncwarp();
            const PartnerStage<R, DV>& partners = mine.stage[buffer];
            if (QUERY_MAJOR && partners.position[0] > last_owner) break;  // keys ascend: nothing causal follows

            // first products: S (owners' R-vectors against partners') and E (DV-vectors)
            float s_tile[2][4], e_tile[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                s_tile[j][0] = s_tile[j][1] = s_tile[j][2] = s_tile[j][3] = 0.f;
                e_tile[j][0] = e_tile[j][1] = e_tile[j][2] = e_tile[j][3] = 0.f;
#pragma unroll
                for (int k = 0; k < KSTEPS; ++k) {
                    const unsigned* source = reinterpret_cast<const unsigned*>(&partners.a[j * 8 + g][k * 16]);
                    mma_bf16_16816(s_tile[j], frag_a[k], source[t], source[4 + t]);
                }
#pragma unroll
                for (int k = 0; k < VSTEPS; ++k) {
                    const unsigned* source = reinterpret_cast<const unsigned*>(&partners.b[j * 8 + g][k * 16]);
                    mma_bf16_16816(e_tile[j], frag_b[k], source[t], source[4 + t]);
                }
            }
            unsigned ordinary_bits = 0, longer_bits = 0;  // one bit per element of this lane, at s * 4 + j * 2 + e
            int2 other_position[2], other_label[2], other_previous[2];  // this lane's four columns: j * 8 + 2 t + e
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                other_position[j] = *reinterpret_cast<const int2*>(&partners.position[j * 8 + 2 * t]);
                other_label[j] = *reinterpret_cast<const int2*>(&partners.label[j * 8 + 2 * t]);
                other_previous[j] = *reinterpret_cast<const int2*>(&partners.previous[j * 8 + 2 * t]);
            }
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (s == 1 && owners <= 8) continue;  // a tile of at most eight rows has no second half
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int kind = classify(s, e ? other_position[j].y : other_position[j].x, e ? other_label[j].y : other_label[j].x,
                                                  e ? other_previous[j].y : other_previous[j].x);
                        ordinary_bits |= unsigned(kind == 1) << (s * 4 + j * 2 + e);
                        longer_bits |= unsigned(kind == 2) << (s * 4 + j * 2 + e);
                    }
            }

            // A pair with a longer run is nearly always of length 2: the lane that holds it looks one cell further up
            // the diagonal, and such pairs join the ordinary ones on the tensor cores with the table's second entry.
            unsigned two_bits = 0;
            const bool any_longer = __ballot_sync(FULL, longer_bits != 0) != 0;
            if (any_longer) {
                unsigned unresolved = 0;
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    if ((longer_bits >> slot) & 1u) {
                        const int s = slot >> 2, j = (slot >> 1) & 1, e = slot & 1;
                        const int other = e ? other_position[j].y : other_position[j].x;
                        const int qi = QUERY_MAJOR ? position[s] : other, kj = QUERY_MAJOR ? other : position[s];
                        const bool ends = kj - 2 < begin[s] || __ldg(iq + qi - 2) != __ldg(ik + kj - 2);
                        if (ends) two_bits |= 1u << slot;
                        else unresolved |= 1u << slot;
                    }
                }
                longer_bits = unresolved;
            }
            // the rest: one at a time, partners ascending
            if (any_longer && __ballot_sync(FULL, longer_bits != 0)) {
#pragma unroll 1
                for (int column = 0; column < KT; ++column) {
                    const int j = column >> 3, e = column & 1;
                    const bool holder = t == ((column & 7) >> 1);
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        unsigned waiting = __ballot_sync(FULL, holder && ((longer_bits >> (s * 4 + j * 2 + e)) & 1u));
                        // the pair's two scalars are elements of the tiles just multiplied: the holder lane's registers
                        const float element_s = j ? (e ? s_tile[1][2 * s + 1] : s_tile[1][2 * s]) : (e ? s_tile[0][2 * s + 1] : s_tile[0][2 * s]);
                        const float element_e = j ? (e ? e_tile[1][2 * s + 1] : e_tile[1][2 * s]) : (e ? e_tile[0][2 * s + 1] : e_tile[0][2 * s]);
                        for (; waiting; waiting &= waiting - 1) {
                            const int source_lane = __ffs(waiting) - 1, row = (source_lane >> 2) + 8 * s;
                            const int owner_position = mine.position[row], other = partners.position[column];
                            const int qi = QUERY_MAJOR ? owner_position : other, kj = QUERY_MAJOR ? other : owner_position;
                            const int length = run_length(iq, ik, boundary, a.n, qi, kj, lane, PACKED ? mine.begin[row] : 0);
                            const float x = length == 2 ? weight_two : __ldg(lut + length);
                            const float p = ex2(x - (QUERY_MAJOR ? mine.norm[row] : partners.norm[column]));
                            const float score = __shfl_sync(FULL, element_s, source_lane), slope = __shfl_sync(FULL, element_e, source_lane);
                            if (g == (row & 7)) {  // the four lanes that hold this row
                                if (QUERY_MAJOR) {
                                    const float gap = (length == 2 ? derivative_two : __ldg(dlut + length)) - mine.center[row];
                                    const float pse = p * score * slope, pe = p * slope;
                                    u[s] += pse;
                                    v[s] = fmaf(p, gap, v[s]);
                                    w[s] = fmaf(pse, gap, w[s]);
                                    z[s] += p;
#pragma unroll
                                    for (int c = 0; c < RTILES; ++c) {
                                        const float2 key = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&partners.a[column][c * 8 + 2 * t]));
                                        grad_a[c][2 * s] = fmaf(pe, key.x, grad_a[c][2 * s]);
                                        grad_a[c][2 * s + 1] = fmaf(pe, key.y, grad_a[c][2 * s + 1]);
                                    }
                                } else {
                                    const float ps = p * score, pe = p * slope;
#pragma unroll
                                    for (int c = 0; c < RTILES; ++c) {
                                        const float2 query = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&partners.a[column][c * 8 + 2 * t]));
                                        grad_a[c][2 * s] = fmaf(pe, query.x, grad_a[c][2 * s]);
                                        grad_a[c][2 * s + 1] = fmaf(pe, query.y, grad_a[c][2 * s + 1]);
                                    }
#pragma unroll
                                    for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c) {
                                        const float2 derivative = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&partners.b[column][c * 8 + 2 * t]));
                                        grad_b[c][2 * s] = fmaf(ps, derivative.x, grad_b[c][2 * s]);
                                        grad_b[c][2 * s + 1] = fmaf(ps, derivative.y, grad_b[c][2 * s + 1]);
                                    }
                                }
                            }
                        }
                    }
                }
            }

            // ordinary pairs and pairs of run length 2 on tensor cores
            if (__ballot_sync(FULL, (ordinary_bits | two_bits) != 0)) {
                unsigned coefficient_e[4], remainder_e[4], coefficient_s[4], remainder_s[4];
                // two instances of the element loop: the common one knows that no pair of run length 2 is in the step
                auto coefficients = [&](auto with_two) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        float pe[2], ps[2];
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const bool on = (ordinary_bits >> (s * 4 + j * 2 + e)) & 1u;
                            const bool two = decltype(with_two)::value && ((two_bits >> (s * 4 + j * 2 + e)) & 1u);
                            float c = on ? (QUERY_MAJOR ? common_row[s] : partners.common[j * 8 + 2 * t + e]) : 0.f;
                            if (decltype(with_two)::value && two) c = QUERY_MAJOR ? common_two_row[s] : partners.common_two[j * 8 + 2 * t + e];
                            const float score = s_tile[j][2 * s + e], slope = e_tile[j][2 * s + e];
                            pe[e] = c * slope;
                            ps[e] = c * score;
                            if (QUERY_MAJOR && on) {
                                sum_se[s] = fmaf(score, slope, sum_se[s]);
                                ++ordinary_total[s];
                            }
                            if (QUERY_MAJOR && two) {
                                sum_se_two[s] = fmaf(score, slope, sum_se_two[s]);
                                ++two_total[s];
                            }
                        }
                        split_bf16(pe[0], pe[1], coefficient_e[2 * j + s], remainder_e[2 * j + s]);
                        if (!QUERY_MAJOR) split_bf16(ps[0], ps[1], coefficient_s[2 * j + s], remainder_s[2 * j + s]);
                    }
                };
                if (__ballot_sync(FULL, two_bits != 0)) coefficients(std::true_type{});
                else coefficients(std::false_type{});
                // (c o E) times the partners' R-vectors: dSQ (query-major) or dSK (key-major)
#pragma unroll
                for (int c = 0; c < RTILES; ++c) {
                    unsigned b0, b1;
                    ldmatrix_x2_trans(b0, b1, &partners.a[lane & 15][c * 8]);
                    mma_bf16_16816(grad_a[c], coefficient_e, b0, b1);
                    mma_bf16_16816(grad_a[c], remainder_e, b0, b1);
                }
                if (!QUERY_MAJOR) {  // (c o S) times the queries' dO rows: dV
#pragma unroll
                    for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c) {
                        unsigned b0, b1;
                        ldmatrix_x2_trans(b0, b1, &partners.b[lane & 15][c * 8]);
                        mma_bf16_16816(grad_b[c], coefficient_s, b0, b1);
                        mma_bf16_16816(grad_b[c], remainder_s, b0, b1);
                    }
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();

        // ---- write the tile's rows --------------------------------------------------------------------------
        if (QUERY_MAJOR) {
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                // the four lanes of a row summed different columns
                sum_se[s] += __shfl_xor_sync(FULL, sum_se[s], 1);
                sum_se[s] += __shfl_xor_sync(FULL, sum_se[s], 2);
                ordinary_total[s] += __shfl_xor_sync(FULL, ordinary_total[s], 1);
                ordinary_total[s] += __shfl_xor_sync(FULL, ordinary_total[s], 2);
                sum_se_two[s] += __shfl_xor_sync(FULL, sum_se_two[s], 1);
                sum_se_two[s] += __shfl_xor_sync(FULL, sum_se_two[s], 2);
                two_total[s] += __shfl_xor_sync(FULL, two_total[s], 1);
                two_total[s] += __shfl_xor_sync(FULL, two_total[s], 2);
            }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            if (g + 8 * s >= owners) continue;
            const int64_t at = vec0 + int64_t(position[s]) * a.heads;
            if (QUERY_MAJOR) {
                float term = 0.f;
                if (active[s]) {
                    // moments: ordinary pairs share weight c_i and the derivative of length 1
                    const float gap = derivative_one - center[s], mass = common_row[s] * float(ordinary_total[s]);
                    const float pse = common_row[s] * sum_se[s];
                    const float gap_two = derivative_two - center[s], mass_two = common_two_row[s] * float(two_total[s]);
                    const float pse_two = common_two_row[s] * sum_se_two[s];
                    const float total_u = u[s] + pse + pse_two, total_z = z[s] + mass + mass_two;
                    const float total_v = fmaf(mass_two, gap_two, fmaf(mass, gap, v[s]));
                    const float total_w = fmaf(pse_two, gap_two, fmaf(pse, gap, w[s]));
                    // centred four-moment form: the fallback has unit weight and zero derivative
                    const float fallback = ex2(-norm[s]), inverse = __fdividef(1.f, total_z + fallback);
                    const float mean = fmaf(-fallback, center[s], total_v) * inverse;
                    term = fmaf(-total_u, mean, total_w) * inverse;
                }
                float* out = a.dsq + at * R + 2 * t;
#pragma unroll
                for (int c = 0; c < RTILES; ++c) *reinterpret_cast<float2*>(out + c * 8) = make_float2(grad_a[c][2 * s], grad_a[c][2 * s + 1]);
                if (t == 0) a.dtau_rows[int64_t(bh) * a.n + position[s]] = term;
            } else {
                __nv_bfloat16* out_a = a.dsk + at * R + 2 * t;
                __nv_bfloat16* out_b = a.dv + at * DV + 2 * t;
#pragma unroll
                for (int c = 0; c < RTILES; ++c)
                    *reinterpret_cast<__nv_bfloat162*>(out_a + c * 8) = __floats2bfloat162_rn(grad_a[c][2 * s], grad_a[c][2 * s + 1]);
#pragma unroll
                for (int c = 0; c < (QUERY_MAJOR ? 1 : VTILES); ++c)
                    *reinterpret_cast<__nv_bfloat162*>(out_b + c * 8) = __floats2bfloat162_rn(grad_b[c][2 * s], grad_b[c][2 * s + 1]);
            }
        }
    }
}

// blockIdx.z + first_pass picks the pass (0 query-major, 1 key-major), so one launch can run either pass or both.  The
// passes do not depend on each other, and CTAs are handed out z last: in a launch of both, the key-major CTAs move into
// the SMs that the query-major pass frees as it runs out of tiles, and the launch has one ramp and one tail instead of
// two of each.  That pays when a GPU holds little work; with much work the passes are faster one after the other.
template <bool PACKED, int R, int DV>
__global__ __launch_bounds__(BLOCK_WARPS * 32, 2) void hard_backward_blocks_kernel(const BackwardBlockArgs by_query,
                                                                                  const BackwardBlockArgs by_key, int first_pass) {
    if (blockIdx.z + first_pass == 0) hard_backward_blocks_pass<true, PACKED, R, DV>(by_query);
    else hard_backward_blocks_pass<false, PACKED, R, DV>(by_key);
}

}  // namespace dism
