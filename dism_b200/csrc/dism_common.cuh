// Shared device helpers and launch-side declarations for the flash_dism hard path on sm_100a.
//
// How the hard kernels find their work.  A pair (query i, key j <= i) has non-zero weight only
// when its labels are equal, so the kernels never visit the N^2/2 pairs.  A small prepass sorts
// the positions of one side by (label bucket, position); the owner of a row then reads only the
// bucket of its own label (about N/256 entries), keeps the entries with the same label on the
// causal side, and gets its matching partners already in ascending order.  Eight lane groups of
// a warp each own one row and work through their queued partners together, so the per-pair
// arithmetic (run length, table lookup, two short dot products, one axpy) runs eight pairs wide.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dism {

constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG_ZERO = -1000000.f;  // LUT entry of length 0 (dism_v3/src/hard_forward.cu:15)
constexpr int BUCKETS = 256;            // label buckets of the position index
constexpr int OWN = 8;                  // rows per warp (one per group of four lanes)
constexpr int WARPS = 8;                // warps per CTA
constexpr int BLOCK_ROWS = WARPS * OWN;

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }

// COUNT consecutive bf16 values (a multiple of 4, 8 bytes aligned) as floats.
template <int COUNT>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float (&out)[COUNT]) {
    static_assert(COUNT % 4 == 0, "vector loads of 4 or 8 values");
    if constexpr (COUNT % 8 == 0) {
#pragma unroll
        for (int c = 0; c < COUNT / 8; ++c) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p) + c);
            const unsigned word[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                out[c * 8 + 2 * e] = __uint_as_float(word[e] << 16);
                out[c * 8 + 2 * e + 1] = __uint_as_float(word[e] & 0xffff0000u);
            }
        }
    } else {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
        out[0] = __uint_as_float(raw.x << 16); out[1] = __uint_as_float(raw.x & 0xffff0000u);
        out[2] = __uint_as_float(raw.y << 16); out[3] = __uint_as_float(raw.y & 0xffff0000u);
    }
}
template <int COUNT>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const float (&in)[COUNT]) {
    static_assert(COUNT % 4 == 0, "vector stores of 4 or 8 values");
    unsigned word[COUNT / 2];
#pragma unroll
    for (int e = 0; e < COUNT / 2; ++e) {
        __nv_bfloat162 pair = __floats2bfloat162_rn(in[2 * e], in[2 * e + 1]);
        word[e] = *reinterpret_cast<unsigned*>(&pair);
    }
    if constexpr (COUNT % 8 == 0) {
#pragma unroll
        for (int c = 0; c < COUNT / 8; ++c)
            reinterpret_cast<uint4*>(p)[c] = make_uint4(word[4 * c], word[4 * c + 1], word[4 * c + 2], word[4 * c + 3]);
    } else {
        *reinterpret_cast<uint2*>(p) = make_uint2(word[0], word[1]);
    }
}
// Sum over the four lanes of a group.
__device__ __forceinline__ float group_sum(float x) {
    x += __shfl_xor_sync(FULL, x, 1);
    x += __shfl_xor_sync(FULL, x, 2);
    return x;
}

__device__ __forceinline__ int bucket_of(int label) {
    unsigned x = unsigned(label);
    x ^= x >> 16;
    x ^= x >> 8;
    return int(x & (BUCKETS - 1));
}

// Number of consecutive label matches on the diagonal that ends at (i, j), given that (i, j)
// itself matches; one thread walks one diagonal.  With a boundary rectangle
// (int32 [(N-1)/32, N] of this batch/head, boundary[c][col] = col - L(32c+31, col)) the walk ends
// at the 32-row strip edge and reads the rest of the run from the rectangle.
__device__ __forceinline__ int run_length(const int* __restrict__ q, const int* __restrict__ k,
                                          const int* __restrict__ boundary, int n, int i, int j) {
    int s = 1;
    if (boundary) {
        const int inside = i & 31;  // rows i-1 .. i-inside share the strip of row i
        for (; s <= inside && j - s >= 0; ++s)
            if (__ldg(q + i - s) != __ldg(k + j - s)) return s;
        const int col = j - s;
        if (s == inside + 1 && col >= 0 && i >= 32) s += col - __ldg(boundary + int64_t((i >> 5) - 1) * n + col);
        return s;
    }
    while (j - s >= 0 && __ldg(q + i - s) == __ldg(k + j - s)) ++s;
    return s;
}

// Position index of one side of one (batch, head): `entries` holds (position, label) sorted by
// (bucket, position); bucket b occupies [starts[b], starts[b+1]).
struct SideIndex {
    const int2* entries;
    const int* starts;
};

// First entry of bucket range [lo, hi) whose position is >= bound (positions ascend).
__device__ __forceinline__ int lower_bound_position(const int2* __restrict__ entries, int lo, int hi, int bound) {
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(&entries[mid].x) < bound) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// Per-warp queue of the partners found in one round: up to 32 per owned row.
struct PairQueue {
    int position[OWN][32];
    int length[OWN][32];
};

// One round of partner search for the warp's OWN rows.  Lane r < OWN carries the label of row r
// and its cursor into the other side's index; each row reads its next 32 bucket entries, keeps
// those with the same label, computes their run lengths (one lane per partner) and queues them
// in ascending position.  Returns in lane r the number queued for row r.
// QUERY_MAJOR: owned rows are queries i = row0 + r and partners are keys; otherwise owned rows are
// keys j = row0 + r and partners are queries.
template <bool QUERY_MAJOR>
__device__ __forceinline__ int find_partners(PairQueue* queue, const int2* __restrict__ entries,
                                             const int* __restrict__ iq, const int* __restrict__ ik,
                                             const int* __restrict__ boundary, int n, int row0, int label,
                                             int& cursor, int end, int lane) {
    int queued = 0;
#pragma unroll 1
    for (int r = 0; r < OWN; ++r) {
        const int from = __shfl_sync(FULL, cursor, r), to = __shfl_sync(FULL, end, r);
        if (from >= to) continue;  // uniform
        const int wanted = __shfl_sync(FULL, label, r);
        const int at = from + lane;
        int2 entry = make_int2(0, 0);
        if (at < to) entry = __ldg(entries + at);
        const bool hit = at < to && entry.y == wanted;
        int length = 0;
        if (hit) length = QUERY_MAJOR ? run_length(iq, ik, boundary, n, row0 + r, entry.x)
                                      : run_length(iq, ik, boundary, n, entry.x, row0 + r);
        const unsigned mask = __ballot_sync(FULL, hit);
        if (hit) {
            const int slot = __popc(mask & ((1u << lane) - 1u));
            queue->position[r][slot] = entry.x;
            queue->length[r][slot] = length;
        }
        if (lane == r) {
            queued = __popc(mask);
            cursor = from + 32;
        }
    }
    return queued;
}

// Causal range of the bucket of `label` for owner position `row` (binary search on positions).
template <bool QUERY_MAJOR>
__device__ __forceinline__ void partner_range(const SideIndex& index, int label, int row, int& cursor, int& end) {
    const int bucket = bucket_of(label);
    const int lo = __ldg(index.starts + bucket), hi = __ldg(index.starts + bucket + 1);
    if (QUERY_MAJOR) {  // keys at positions <= row
        cursor = lo;
        end = lower_bound_position(index.entries, lo, hi, row + 1);
    } else {  // queries at positions >= row
        cursor = lower_bound_position(index.entries, lo, hi, row);
        end = hi;
    }
}

// ---- launch-side entry points (defined in the .cu files, called from the C ABI) -------------
struct HardShape {
    int batch, heads, n, r, dv;
};

int device_sm_count();
cudaError_t launch_labels(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int batch, int n, int heads,
                          int d, int vocab, int* labels, cudaStream_t stream);
cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream);
cudaError_t launch_hard_chunk(const int* summary, int* boundary, int batch_heads, int n, cudaStream_t stream);

// Index workspace: per (batch, head) N entries of int2 plus BUCKETS+1 starts, for `sides` sides.
size_t index_bytes(int batch_heads, int n, int sides);
// Builds the index of `labels` ([BH, N]) into `workspace` (side 0 at the front, side 1 after it).
cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream);
SideIndex side_index(void* workspace, int batch_heads, int n, int side, int sides);

size_t longest_match_workspace_bytes(int batch, int n);
cudaError_t launch_longest_match(const int* streams, int batch, int n, int* end, int* length, int* next,
                                 void* workspace, cudaStream_t stream);
cudaError_t launch_log_weights(const float* tau, int heads, int n, float* lut, cudaStream_t stream);
size_t hard_forward_workspace_bytes(int batch, int heads, int n);
cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const float* lut, int lut_stride, int ctas,
                                __nv_bfloat16* out, float* lse2, void* workspace, cudaStream_t stream);
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride);
cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const float* lut, int lut_stride,
                                 const float* lse2, int ctas, float* dsq, __nv_bfloat16* dsk, __nv_bfloat16* dv,
                                 float* dtau, void* workspace, cudaStream_t stream);

}  // namespace dism
