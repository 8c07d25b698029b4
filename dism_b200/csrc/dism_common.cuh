// Shared device helpers and launch-side declarations for the flash_dism hard path on sm_100a.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dism {

constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG_ZERO = -1000000.f;  // LUT entry of length 0 (dism_v3/src/hard_forward.cu:15)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
// PER consecutive bf16 values (PER = 1, 2 or 4) as floats, with one vector load.
template <int PER>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float (&out)[PER]) {
    if constexpr (PER == 1) out[0] = bf2f(*p);
    else if constexpr (PER == 2) {
        float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
        out[0] = f.x; out[1] = f.y;
    } else {
        static_assert(PER == 4, "1, 2 or 4 values per lane");
        uint2 raw = *reinterpret_cast<const uint2*>(p);
        float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        out[0] = lo.x; out[1] = lo.y; out[2] = hi.x; out[3] = hi.y;
    }
}
template <int PER>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const float (&in)[PER]) {
    if constexpr (PER == 1) *p = __float2bfloat16_rn(in[0]);
    else if constexpr (PER == 2) *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(in[0], in[1]);
    else {
        static_assert(PER == 4, "1, 2 or 4 values per lane");
        __nv_bfloat162 lo = __floats2bfloat162_rn(in[0], in[1]), hi = __floats2bfloat162_rn(in[2], in[3]);
        uint2 raw{*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi)};
        *reinterpret_cast<uint2*>(p) = raw;
    }
}
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
    for (int s = 16; s; s >>= 1) x += __shfl_xor_sync(FULL, x, s);
    return x;
}

// Number of consecutive label matches on the diagonal that ends at (i, j), given that (i, j)
// itself matches.  The whole warp calls this with the same (i, j).  With a boundary rectangle
// (int32 [(N-1)/32, N] of this batch/head, boundary[c][col] = col - L(32c+31, col)) the walk
// stops at the 32-row strip edge and reads the rest; without one it walks 32 cells per step.
__device__ __forceinline__ int match_length(const int* __restrict__ q, const int* __restrict__ k,
                                            const int* __restrict__ boundary, int n, int i, int j, int lane) {
    int length = 1, bi = i - 1, bj = j - 1;
    if (boundary) {
        const int inside = i & 31;  // rows i-1 .. i-inside share the strip of row i
        bool ok = lane < inside && bj - lane >= 0 && __ldg(q + bi - lane) == __ldg(k + bj - lane);
        unsigned mask = __ballot_sync(FULL, ok);
        int run = __ffs(~mask) - 1;
        length += run;
        int col = bj - inside;
        if (run == inside && col >= 0 && i >= 32)
            length += col - __ldg(boundary + int64_t((i >> 5) - 1) * n + col);
        return length;
    }
    while (bj >= 0) {
        bool ok = bj - lane >= 0 && __ldg(q + bi - lane) == __ldg(k + bj - lane);
        unsigned mask = __ballot_sync(FULL, ok);
        if (mask != FULL) return length + __ffs(~mask) - 1;
        length += 32;
        bi -= 32;
        bj -= 32;
    }
    return length;
}

// One warp owns OWN consecutive positions of one (batch, head) and streams the other side's
// labels in slabs of 1024 (32 per lane, kept in registers), comparing with a ballot per
// (owned position, 32 streamed positions).  Proc::hits handles the set bits in ascending order,
// so every owned position sees its matches in ascending streamed order whatever the grid size.
// QUERY_MAJOR: owned = queries, streamed = keys s <= owner.  Otherwise owned = keys and
// streamed = queries s >= owner.
constexpr int OWN = 8;
constexpr int SLAB = 1024;

template <bool QUERY_MAJOR, class Proc, class State>
__device__ __forceinline__ void stream_matches(State* st, const int* __restrict__ own_labels,
                                               const int* __restrict__ stream_labels, int n, int row0,
                                               int lane) {
    const int own = __ldg(own_labels + row0 + (lane & (OWN - 1)));
    const int first = QUERY_MAJOR ? 0 : (row0 & ~(SLAB - 1));
    const int last = QUERY_MAJOR ? row0 + OWN - 1 : n - 1;  // last streamed position of interest
    for (int s0 = first; s0 <= last; s0 += SLAB) {
        int reg[32];
#pragma unroll
        for (int t = 0; t < 32; ++t) {
            int s = s0 + t * 32 + lane;
            reg[t] = s < n ? __ldg(stream_labels + s) : 0;
        }
        const bool interior = QUERY_MAJOR ? (s0 + SLAB - 1 <= row0) : (s0 >= row0 + OWN - 1 && s0 + SLAB <= n);
        if (interior) {
            for (int r = 0; r < OWN; ++r) {
                const int label = __shfl_sync(FULL, own, r);
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    unsigned m = __ballot_sync(FULL, reg[t] == label);
                    if (m) Proc::hits(st, r, s0 + t * 32, m);
                }
            }
        } else {
            for (int r = 0; r < OWN; ++r) {
                const int label = __shfl_sync(FULL, own, r);
                const int rel = row0 + r - s0;  // owner position relative to the slab
#pragma unroll
                for (int t = 0; t < 32; ++t) {
                    if (s0 + t * 32 >= n || (QUERY_MAJOR && t * 32 > rel + OWN - 1 - r)) break;
                    const int d = rel - t * 32;  // owner relative to this 32-wide tile
                    unsigned valid;
                    if (QUERY_MAJOR) valid = d >= 31 ? FULL : (d < 0 ? 0u : (2u << d) - 1u);
                    else valid = d <= 0 ? FULL : (d > 31 ? 0u : FULL << d);
                    unsigned m = __ballot_sync(FULL, reg[t] == label) & valid;
                    if (m) Proc::hits(st, r, s0 + t * 32, m);
                }
            }
        }
    }
}

// ---- launch-side entry points (defined in the .cu files, called from the C ABI) -------------
struct HardShape {
    int batch, heads, n, r, dv;
};

cudaError_t launch_labels(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int batch, int n, int heads,
                          int d, int vocab, int* labels, cudaStream_t stream);
cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream);
cudaError_t launch_hard_chunk(const int* summary, int* boundary, int batch_heads, int n, cudaStream_t stream);
cudaError_t launch_longest_match(const int* streams, int batch, int n, int* end, int* length, int* next,
                                 cudaStream_t stream);
cudaError_t launch_log_weights(const float* tau, int heads, int n, float* lut, cudaStream_t stream);
cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const float* lut, int lut_stride, int ctas,
                                __nv_bfloat16* out, float* lse2, cudaStream_t stream);
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride);
cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const float* lut, int lut_stride,
                                 const float* lse2, int ctas, float* dsq, __nv_bfloat16* dsk, __nv_bfloat16* dv,
                                 float* dtau, void* workspace, cudaStream_t stream);
int device_sm_count();

}  // namespace dism
