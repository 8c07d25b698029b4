// Hard forward as label-block tensor-core tiles.
//
// Two positions can only interact when their labels are equal, so after both sides are sorted by
// (label bucket, position) the whole causal pair set is a union of small dense blocks: the
// queries of a bucket against the keys of the same bucket.  A warp takes sixteen queries of one
// bucket (one m16 tile), walks the bucket's keys sixteen at a time, and does what a fused
// attention kernel does on such a tile with bf16 mma.sync: scores = SQ.SK^T, a mask (same label,
// same document, key not after the query), weights, then acc += P.V.  The rows of SQ are
// gathered once per tile and the rows of SK and V once per (tile, key step) instead of once per
// pair.
//
// Weights.  Almost every matching pair has run length 1 and therefore the same table entry
// lut[1]; its weight relative to the row's running maximum is one constant per row and key step
// and is folded into the score before the bf16 rounding.  A pair whose diagonal predecessor
// matches as well (run length >= 2) is rare in sparse data; those pairs are left out of the
// tiles and added one by one by the whole warp, in ascending key order, which walks the diagonal
// for the run length.  The running maximum and denominator follow the reference's online
// normalisation (maximum starts at 0, denominator at 1).  Each row is reduced by one warp in a
// fixed order: results do not depend on the grid.
#pragma once
#include "dense_route.cuh"

namespace dism {

constexpr int QT = 16;  // queries per tile (the m of m16n8k16)
constexpr int KT = 16;  // keys per step: two n8 score tiles, one k16 step of the value product
constexpr int BLOCK_WARPS = 8;
constexpr int WALK_CAP = 8;  // run lengths up to this are found by the lane that holds the pair

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x2_trans(unsigned& b0, unsigned& b1, const void* row) {
    const unsigned address = static_cast<unsigned>(__cvta_generic_to_shared(row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(address));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&pair);
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int s = 16; s; s >>= 1) x += __shfl_xor_sync(FULL, x, s);
    return x;
}

template <int R, int DV>
struct alignas(16) KeyStage {
    __nv_bfloat16 sk[KT][R + 8];  // padded rows: fragment loads and ldmatrix rows fall in distinct banks
    __nv_bfloat16 v[KT][DV + 8];
    int position[KT], label[KT], previous[KT];
};

template <int R, int DV>
struct alignas(16) BlockWarpShared {
    KeyStage<R, DV> stage[2];
    int position[QT], label[QT], previous[QT], begin[QT], active[QT];
};

struct BlockArgs {
    const __nv_bfloat16 *sq, *sk, *v;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float* lut;
    SideIndex keys, queries;
    const int* tile_starts;  // [BH, BUCKETS + 1]: first query tile of every bucket
    const int4* tiles;       // [BH, tile capacity]: (first query entry, queries, first key entry, end of key entries)
    int* next_tile;          // [BH]: the next tile to hand out (zeroed by the plan kernel)
    int tile_capacity;
    const int2* documents;
    __nv_bfloat16* out;
    float* lse2;
    int batch, heads, n, lut_stride, hard_rows;
    const unsigned* choice;  // route word of a captured graph, or null
};

// Number of 16-query tiles a (batch, head) can have at most: every bucket may end with a partial tile.
__host__ __device__ inline int tile_capacity_for(int n) { return n / QT + BUCKETS; }

// One descriptor per 16-query tile; tile_starts[b] = the first tile of bucket b, tile_starts[BUCKETS] = the number of tiles.
// With `route` set, a (batch, head) whose buckets hold at least dense_pairs label-matching pairs (causal or not) is
// marked for the dense kernel instead (route word 1) and gets no tiles here.
__device__ __forceinline__ void plan_query_tiles(const int* __restrict__ query_starts, const int* __restrict__ key_starts,
                                                 int* __restrict__ tile_starts, int4* __restrict__ tiles,
                                                 int* __restrict__ next_tile, int tile_capacity, int* __restrict__ route = nullptr,
                                                 unsigned long long dense_pairs = 0) {
    constexpr int PER = BUCKETS / 1024;
    constexpr int LONG_TILE = 4 * KT;  // a tile with more partners than this counts as long
    __shared__ unsigned long long warp_total[32];  // tiles before a warp: long ones in the high word, the others in the low word
    __shared__ unsigned long long warp_pairs[32];
    __shared__ int dense, long_tiles;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    query_starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    key_starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    tile_starts += int64_t(blockIdx.x) * (BUCKETS + 1);
    tiles += int64_t(blockIdx.x) * tile_capacity;
    // Tiles are handed out in the order of their descriptors.  The tiles of buckets with many partners take many times
    // longer than the others, so they come first: a long tile taken last would keep its slice, and the kernel, waiting.
    unsigned long long local[PER], sum = 0;
    unsigned long long pairs = 0;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        local[e] = sum;
        const int queries = query_starts[tid * PER + e + 1] - query_starts[tid * PER + e];
        const int partners = key_starts[tid * PER + e + 1] - key_starts[tid * PER + e];
        sum += (unsigned long long)((queries + QT - 1) / QT) << (partners > LONG_TILE ? 32 : 0);
        pairs += (unsigned long long)(queries) * (unsigned long long)(partners);
    }
    if (route) {
#pragma unroll
        for (int s = 16; s; s >>= 1) pairs += __shfl_xor_sync(FULL, pairs, s);
        if (lane == 0) warp_pairs[warp] = pairs;
    }
    unsigned long long prefix = sum;
#pragma unroll
    for (int s = 1; s < 32; s <<= 1) {
        const unsigned long long other = __shfl_up_sync(FULL, prefix, s);
        if (lane >= s) prefix += other;
    }
    if (lane == 31) warp_total[warp] = prefix;
    __syncthreads();
    if (route && tid == 0) {
        unsigned long long all = 0;
        for (int w = 0; w < 32; ++w) all += warp_pairs[w];
        dense = all >= dense_pairs;
        route[blockIdx.x] = dense;
    }
    if (warp == 0) {
        const unsigned long long mine = warp_total[lane];
        unsigned long long scan = mine;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const unsigned long long other = __shfl_up_sync(FULL, scan, s);
            if (lane >= s) scan += other;
        }
        warp_total[lane] = scan - mine;
        if (lane == 31) long_tiles = int(scan >> 32);
    }
    __syncthreads();
    const unsigned long long before = warp_total[warp] + prefix - sum;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int bucket = tid * PER + e;
        const int q0 = query_starts[bucket], q1 = query_starts[bucket + 1];
        const int k0 = key_starts[bucket], k1 = key_starts[bucket + 1];
        const unsigned long long at = before + local[e];
        const int first = k1 - k0 > LONG_TILE ? int(at >> 32) : long_tiles + int(at & 0xffffffffu);
        tile_starts[bucket] = first;
        for (int q = q0, tile = first; q < q1; q += QT, ++tile) tiles[tile] = make_int4(q, min(QT, q1 - q), k0, k1);
    }
    if (tid == 1023) {
        const unsigned long long all = before + sum;
        tile_starts[BUCKETS] = route && dense ? 0 : int(all >> 32) + int(all & 0xffffffffu);  // `dense` was written before the last barrier
        next_tile[blockIdx.x] = 0;
    }
}

static __global__ __launch_bounds__(1024) void plan_query_tiles_kernel(const int* query_starts, const int* key_starts,
                                                                       int* tile_starts, int4* tiles, int* next_tile,
                                                                       int tile_capacity, int* route, unsigned long long dense_pairs,
                                                                       const unsigned* choice) {
    if (!route_open(choice)) return;
    plan_query_tiles(query_starts, key_starts, tile_starts, tiles, next_tile, tile_capacity, route, dense_pairs);
}

// Two plans in one launch (the backward's query-major and key-major tiles): blockIdx.y picks the plan.
struct TilePlan {
    const int *owner_starts, *partner_starts;
    int* tile_starts;
    int4* tiles;
    int* next_tile;
};
// PACKED: rows carry document limits (a.documents is set); otherwise every row's document is the whole sequence
// and the limits are constants the compiler folds away.
template <bool PACKED, int R, int DV>
__global__ __launch_bounds__(BLOCK_WARPS * 32) void hard_forward_blocks_kernel(const BlockArgs a) {
    constexpr int KSTEPS = R / 16, VTILES = DV / 8;
    if (!route_open(a.choice)) return;
    extern __shared__ __align__(16) unsigned char storage[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    auto& mine = reinterpret_cast<BlockWarpShared<R, DV>*>(storage)[warp];
    const int bh = blockIdx.x, b = bh / a.heads, h = bh % a.heads;  // x: CTAs are handed out slice after slice, so every slice always has CTAs at work
    const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
    const int* iq = a.iq + int64_t(bh) * a.n;
    const int* ik = a.ik + int64_t(bh) * a.n;
    const int* boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
    const float* lut = a.lut + int64_t(h) * a.lut_stride;
    const int2* key_entries = a.keys.entries + int64_t(bh) * a.n;
    const int* key_previous = a.keys.previous + int64_t(bh) * a.n;
    const int2* query_entries = a.queries.entries + int64_t(bh) * a.n;
    const int* query_previous = a.queries.previous + int64_t(bh) * a.n;
    const int4* tiles = a.tiles + int64_t(bh) * a.tile_capacity;
    const int tile_count = __ldg(a.tile_starts + int64_t(bh) * (BUCKETS + 1) + BUCKETS);
    const float weight_one = __ldg(lut + 1), weight_two = a.lut_stride > 2 ? __ldg(lut + 2) : 0.f;
    // gathered rows: a lane always copies the same 16-byte piece of a row, so its source is one pointer
    // plus position * stride (32-bit product: a (batch, head) slice spans less than 4 GB)
    const unsigned sk_stride = unsigned(a.heads) * R * 2, v_stride = unsigned(a.heads) * DV * 2;
    const char* sk_lane = reinterpret_cast<const char*>(a.sk + vec0 * R) + (lane % (R / 8)) * 16;
    const char* v_lane = reinterpret_cast<const char*>(a.v + vec0 * DV) + (lane % (DV / 8)) * 16;

    // Tiles differ a lot in their number of key steps, so warps take them one at a time from a counter.
    // Getting to a tile's rows takes a chain of dependent reads (counter, descriptor, index entries), so the
    // chain runs ahead of the arithmetic: while tile i is worked on, the index entries of tile i+1, the
    // descriptor of tile i+2 and the number of tile i+3 are in flight.  A warp may claim up to three
    // numbers past the end; they are ignored.
    const int fixed_active = PACKED ? 0 : a.hard[b * a.heads + h];
    auto claim = [&]() { return lane == 0 ? atomicAdd(a.next_tile + bh, 1) : 0; };  // lane 0 holds the number
    auto descriptor = [&](int tile) { return tile < tile_count ? __ldg(tiles + tile) : make_int4(0, 0, 0, 0); };
    struct Entries {
        int2 owner, key;  // lane r < QT: query r of the tile; lane c < KT: key c of the first key step
        int owner_previous, key_previous;
    };
    auto entries_of = [&](const int4 plan) {
        Entries e{make_int2(-1, 0), make_int2(0x7fffffff, 0), 0, 0};
        if (lane < plan.y) {
            e.owner = __ldg(query_entries + plan.x + lane);
            e.owner_previous = __ldg(query_previous + plan.x + lane);
        }
        if (lane < KT && plan.z + lane < plan.w) {
            e.key = __ldg(key_entries + plan.z + lane);
            e.key_previous = __ldg(key_previous + plan.z + lane);
        }
        return e;
    };
    int tile = __shfl_sync(FULL, claim(), 0);
    int claimed = claim();
    int4 plan = descriptor(tile);
    int next_tile = __shfl_sync(FULL, claimed, 0);
    claimed = claim();
    int4 next_plan = descriptor(next_tile);
    Entries fetched = entries_of(plan);
    for (; tile < tile_count; ) {
        const int after_next = __shfl_sync(FULL, claimed, 0);
        claimed = claim();
        const int4 after_next_plan = descriptor(after_next);
        const Entries next_fetched = entries_of(next_plan);
        const int q0 = plan.x, queries = plan.y;
        (void)q0;
        __syncwarp();
        if (lane < QT) {
            const int2 entry = fetched.owner;
            const int previous = fetched.owner_previous;
            int begin = 0, active = 0;
            if (lane < queries) {
                active = fixed_active;
                if (PACKED) {
                    begin = __ldg(a.documents + entry.x / 256).x;
                    active = a.hard[entry.x / (a.n / a.hard_rows) * a.heads + h];
                }
            }
            mine.position[lane] = entry.x;
            mine.label[lane] = entry.y;
            mine.previous[lane] = previous;
            mine.begin[lane] = begin;
            mine.active[lane] = active;
        }
        __syncwarp();
        int position[2], label[2], previous[2], begin[2];
        bool active[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int r = g + 8 * s;
            position[s] = mine.position[r];
            label[s] = mine.label[r];
            previous[s] = mine.previous[r];
            begin[s] = PACKED ? mine.begin[r] : 0;
            active[s] = mine.active[r] != 0;
        }
        const int last_query = mine.position[queries - 1];
        int key_begin = plan.z;
        const int key_end = plan.w;
        if (PACKED) {  // the bucket also holds keys of earlier documents
            int first_begin = mine.begin[0];
            for (int r = 1; r < queries; ++r) first_begin = min(first_begin, mine.begin[r]);
            key_begin = warp_lower_bound_position(key_entries, key_begin, key_end, first_begin, lane);
        }

        unsigned query[KSTEPS][4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const unsigned* source = reinterpret_cast<const unsigned*>(a.sq + (vec0 + int64_t(max(position[s], 0)) * a.heads) * R);
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                query[k][s] = active[s] ? __ldg(source + k * 8 + t) : 0u;
                query[k][s + 2] = active[s] ? __ldg(source + k * 8 + 4 + t) : 0u;
            }
        }
        float acc[VTILES][4], maximum[2] = {0.f, 0.f}, denominator[2] = {1.f, 1.f};
#pragma unroll
        for (int c = 0; c < VTILES; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;

        // The kind of one score element: 1 = ordinary pair (run length 1), 2 = longer run, 0 = no pair.
        auto classify = [&](int s, int key_position, int key_label, int key_previous) {
            const bool pair = active[s] && key_label == label[s] && key_position <= position[s] && key_position >= begin[s];
            const bool longer = pair && key_position > begin[s] && position[s] > begin[s] && key_previous == previous[s];
            return pair ? (longer ? 2 : 1) : 0;
        };
        // Labels of a key step and its sk / v rows (cp.async); rows beyond the range are zero-filled.
        auto stage_entries = [&](KeyStage<R, DV>& keys, int2 entry, int before) {
            const int key_position = lane < KT ? entry.x : 0x7fffffff;
            if (lane < KT) {
                keys.position[lane] = entry.x;
                keys.label[lane] = entry.y;
                keys.previous[lane] = before;
            }
            constexpr int SK_ROWS = 32 / (R / 8), V_ROWS = 32 / (DV / 8);  // rows a warp covers per round
#pragma unroll
            for (int key = lane / (R / 8); key < KT; key += SK_ROWS) {
                const int at = __shfl_sync(FULL, key_position, key);
                const bool present = at != 0x7fffffff;
                cp_async16_or_zeros(&keys.sk[key][(lane % (R / 8)) * 8], sk_lane + (present ? uint64_t(unsigned(at)) * sk_stride : 0), present ? 16 : 0);
            }
#pragma unroll
            for (int key = lane / (DV / 8); key < KT; key += V_ROWS) {
                const int at = __shfl_sync(FULL, key_position, key);
                const bool present = at != 0x7fffffff;
                cp_async16_or_zeros(&keys.v[key][(lane % (DV / 8)) * 8], v_lane + (present ? uint64_t(unsigned(at)) * v_stride : 0), present ? 16 : 0);
            }
            cp_async_commit();
        };
        auto stage_keys = [&](KeyStage<R, DV>& keys, int k0) {
            int2 entry = make_int2(0x7fffffff, 0);
            int before = 0;
            if (lane < KT && k0 + lane < key_end) {
                entry = __ldg(key_entries + k0 + lane);
                before = __ldg(key_previous + k0 + lane);
            }
            stage_entries(keys, entry, before);
        };
        // Multiplies a row's running state when its maximum rises to x.
        auto raise = [&](int s, float x) {
            const float alpha = ex2(maximum[s] - x);
            denominator[s] *= alpha;
#pragma unroll
            for (int c = 0; c < VTILES; ++c) { acc[c][2 * s] *= alpha; acc[c][2 * s + 1] *= alpha; }
            maximum[s] = x;
        };

        if (key_begin < key_end) {
            if (PACKED) stage_keys(mine.stage[0], key_begin);  // the first step moved with the documents
            else stage_entries(mine.stage[0], fetched.key, fetched.key_previous);
        }
        int buffer = 0;
        for (int k0 = key_begin; k0 < key_end; k0 += KT, buffer ^= 1) {
            const bool more = k0 + KT < key_end;
            if (more) stage_keys(mine.stage[buffer ^ 1], k0 + KT);
            if (more) cp_async_wait<1>();
            else cp_async_wait<0>();
            __syncwarp();
            const KeyStage<R, DV>& keys = mine.stage[buffer];
            if (keys.position[0] > last_query) break;  // keys ascend: nothing causal from here on

            float score[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                score[j][0] = score[j][1] = score[j][2] = score[j][3] = 0.f;
#pragma unroll
                for (int k = 0; k < KSTEPS; ++k) {
                    const unsigned* source = reinterpret_cast<const unsigned*>(&keys.sk[j * 8 + g][k * 16]);
                    mma_bf16_16816(score[j], query[k], source[t], source[4 + t]);
                }
            }
            // one bit per score element of this lane, at s * 4 + j * 2 + e
            unsigned ordinary_bits = 0, longer_bits = 0;
            int2 key_position[2], key_label[2], key_previous[2];  // this lane's four columns: j * 8 + 2 t + e
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                key_position[j] = *reinterpret_cast<const int2*>(&keys.position[j * 8 + 2 * t]);
                key_label[j] = *reinterpret_cast<const int2*>(&keys.label[j * 8 + 2 * t]);
                key_previous[j] = *reinterpret_cast<const int2*>(&keys.previous[j * 8 + 2 * t]);
            }
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                if (s == 1 && queries <= 8) continue;  // a tile of at most eight rows has no second half
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int kind = classify(s, e ? key_position[j].y : key_position[j].x, e ? key_label[j].y : key_label[j].x,
                                                  e ? key_previous[j].y : key_previous[j].x);
                        ordinary_bits |= unsigned(kind == 1) << (s * 4 + j * 2 + e);
                        longer_bits |= unsigned(kind == 2) << (s * 4 + j * 2 + e);
                    }
            }
            int ordinary[2] = {__popc(ordinary_bits & 15u), __popc(ordinary_bits >> 4)};
            const bool any_longer = __ballot_sync(FULL, longer_bits != 0) != 0;
            if (any_longer) {
                // A lane walks the diagonals of its own pairs with longer runs, a few cells at most: nearly all such
                // runs are short, and all of them are then weighted and multiplied on the tensor cores together
                // with the ordinary pairs, each element with its own table entry.
                float x[8];  // log2 weight of element slot s * 4 + j * 2 + e
                unsigned tensor_bits = ordinary_bits, unresolved = 0;
#pragma unroll
                for (int slot = 0; slot < 8; ++slot) {
                    const int s = slot >> 2, j = (slot >> 1) & 1, e = slot & 1;
                    x[slot] = weight_one;
                    if ((longer_bits >> slot) & 1u) {
                        const int qi = position[s], kj = e ? key_position[j].y : key_position[j].x;
                        int length = 2;  // the pair and its diagonal predecessor match
                        while (length <= WALK_CAP && kj - length >= begin[s] && __ldg(iq + qi - length) == __ldg(ik + kj - length)) ++length;
                        if (length <= WALK_CAP) {
                            tensor_bits |= 1u << slot;
                            x[slot] = length == 2 ? weight_two : __ldg(lut + length);
                        } else {
                            unresolved |= 1u << slot;
                        }
                    }
                }
                float p[8], sum[2] = {0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    float top = -INFINITY;
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if ((tensor_bits >> (s * 4 + q)) & 1u) top = fmaxf(top, x[s * 4 + q]);
                    top = fmaxf(top, __shfl_xor_sync(FULL, top, 1));
                    top = fmaxf(top, __shfl_xor_sync(FULL, top, 2));
                    if (top > maximum[s]) raise(s, top);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        p[s * 4 + q] = (tensor_bits >> (s * 4 + q)) & 1u ? ex2(x[s * 4 + q] - maximum[s]) : 0.f;
                        sum[s] += p[s * 4 + q];
                    }
                    sum[s] += __shfl_xor_sync(FULL, sum[s], 1);
                    sum[s] += __shfl_xor_sync(FULL, sum[s], 2);
                    denominator[s] += sum[s];
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
                    ldmatrix_x2_trans(b0, b1, &keys.v[lane & 15][c * 8]);
                    mma_bf16_16816(acc[c], weights, b0, b1);
                }
                longer_bits = unresolved;
                ordinary[0] = ordinary[1] = 0;  // done above
            }
            // pairs whose run is longer than a lane walks: one at a time by the whole warp, keys ascending
            if (any_longer && __ballot_sync(FULL, longer_bits != 0)) {
#pragma unroll 1
                for (int column = 0; column < KT; ++column) {
                    const int j = column >> 3, e = column & 1;
                    const bool holder = t == ((column & 7) >> 1);
#pragma unroll
                    for (int s = 0; s < 2; ++s) {
                        unsigned waiting = __ballot_sync(FULL, holder && ((longer_bits >> (s * 4 + j * 2 + e)) & 1u));  // lanes = rows g + 8 s, ascending
                        // the pair's score is an element of the tile just multiplied: the holder lane's register
                        const float element = j ? (e ? score[1][2 * s + 1] : score[1][2 * s]) : (e ? score[0][2 * s + 1] : score[0][2 * s]);
                        for (; waiting; waiting &= waiting - 1) {
                            const int source_lane = __ffs(waiting) - 1, row = (source_lane >> 2) + 8 * s;
                            const int qi = mine.position[row], kj = keys.position[column];
                            const int length = run_length(iq, ik, boundary, a.n, qi, kj, lane, PACKED ? mine.begin[row] : 0);
                            const float x = length == 2 ? weight_two : __ldg(lut + length);
                            const float value_score = __shfl_sync(FULL, element, source_lane);
                            if (g == (row & 7)) {  // the four lanes that hold this row
                                if (x > maximum[s]) raise(s, x);
                                const float p = ex2(x - maximum[s]);
                                denominator[s] += p;
                                const float weight = p * value_score;
#pragma unroll
                                for (int c = 0; c < VTILES; ++c) {
                                    const float2 pair = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&keys.v[column][c * 8 + 2 * t]));
                                    acc[c][2 * s] = fmaf(weight, pair.x, acc[c][2 * s]);
                                    acc[c][2 * s + 1] = fmaf(weight, pair.y, acc[c][2 * s + 1]);
                                }
                            }
                        }
                    }
                }
            }
            // ordinary pairs: one weight per row, folded into the score, then the value product on tensor cores
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                ordinary[s] += __shfl_xor_sync(FULL, ordinary[s], 1);
                ordinary[s] += __shfl_xor_sync(FULL, ordinary[s], 2);
            }
            if (__ballot_sync(FULL, ordinary[0] + ordinary[1] > 0)) {
                float common[2];
#pragma unroll
                for (int s = 0; s < 2; ++s) {
                    if (ordinary[s] > 0 && weight_one > maximum[s]) raise(s, weight_one);
                    common[s] = ordinary[s] > 0 ? ex2(weight_one - maximum[s]) : 0.f;
                    denominator[s] = fmaf(common[s], float(ordinary[s]), denominator[s]);
                }
                unsigned weights[4];
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int s = 0; s < 2; ++s)
                        weights[2 * j + s] = pack_bf16(
                            (ordinary_bits >> (s * 4 + j * 2)) & 1u ? common[s] * score[j][2 * s] : 0.f,
                            (ordinary_bits >> (s * 4 + j * 2 + 1)) & 1u ? common[s] * score[j][2 * s + 1] : 0.f);
#pragma unroll
                for (int c = 0; c < VTILES; ++c) {
                    unsigned b0, b1;
                    ldmatrix_x2_trans(b0, b1, &keys.v[lane & 15][c * 8]);
                    mma_bf16_16816(acc[c], weights, b0, b1);
                }
            }
            __syncwarp();
        }
        cp_async_wait<0>();

        // ---- write the tile's rows --------------------------------------------------------------------------
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            if (g + 8 * s >= queries) continue;
            const float inverse = active[s] ? __frcp_rn(denominator[s]) : 0.f;
            __nv_bfloat16* out = a.out + (vec0 + int64_t(position[s]) * a.heads) * DV + 2 * t;
#pragma unroll
            for (int c = 0; c < VTILES; ++c)
                *reinterpret_cast<__nv_bfloat162*>(out + c * 8) = __floats2bfloat162_rn(acc[c][2 * s] * inverse, acc[c][2 * s + 1] * inverse);
            if (t == 0) a.lse2[int64_t(bh) * a.n + position[s]] = active[s] ? maximum[s] + log2f(denominator[s]) : 0.f;
        }
        tile = next_tile, plan = next_plan, fetched = next_fetched;
        next_tile = after_next, next_plan = after_next_plan;
    }
}

}  // namespace dism
