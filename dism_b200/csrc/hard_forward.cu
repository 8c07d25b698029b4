// Hard forward: log-weight table and the fused match / normalise / signed-readout kernel.
//
// Replaces, behind the C ABI, the reference's hard_log_weights_kernel and hard_forward_kernel
// (dism_v3/src/hard_forward.cu:9-118, dism_v3/include/forward/readout.cuh:16-100).  The design is
// not a translation: the table entry of length 0 is -1e6, whose weight flushes to exactly 0, so
// only pairs with equal labels contribute.  Each group of four lanes owns one query row, finds
// its matching keys through the key-side position index, and accumulates them in ascending key
// order with the online max / unit-fallback normalisation of the reference (maximum starts at 0,
// denominator at 1).  A row is reduced by one group in a fixed order, so outputs do not depend on
// the grid size.
#include "hard_rows.cuh"

namespace dism {

__global__ void log_weights_kernel(const float* __restrict__ tau, float* __restrict__ out, int stride) {
    int length = blockIdx.x * blockDim.x + threadIdx.x;
    if (length >= stride) return;
    float t = tau[blockIdx.y], result = LOG_ZERO;
    if (length > 0) {
        if (t == 0.f) result = log2f(float(length));
        else {
            float a = fabsf(t);
            result = (t > 0.f ? float(length) * t : t) * 1.4426950408889634f +
                     log2f(-expm1f(-float(length) * a)) - log2f(-expm1f(-a));
        }
    }
    out[int64_t(blockIdx.y) * stride + length] = result;
}

cudaError_t launch_log_weights(const float* tau, int heads, int n, float* lut, cudaStream_t stream) {
    KernelTimer timer("log_weights", stream);
    log_weights_kernel<<<dim3((n + 256) / 256, heads), 256, 0, stream>>>(tau, lut, n + 1);
    return cudaGetLastError();
}

template <int R_, int DV>
struct ForwardPolicy {
    static constexpr bool QUERY_MAJOR = true, EXTRA = false;
    static constexpr int R = R_, VPL = DV / 4, MIN_CTAS = DV <= 64 ? 3 : 2;
    using Args = RowsArgs;
    static const char* name() { return "hard_forward"; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_a(const Args& a) { return a.sk; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_b(const Args& a) { return a.v; }

    float query[8], acc[VPL], maximum, denominator;

    // `leading` is false for the lane groups that reduce a later part of a shared row: the unit
    // fallback of the normaliser is counted once, by the leading group.
    __device__ __forceinline__ void begin(const Args& a, const RowContext& ctx, int row, int part, bool has_r, bool active,
                                          bool leading) {
        maximum = 0.f;
        denominator = leading ? 1.f : 0.f;
#pragma unroll
        for (int c = 0; c < VPL; ++c) acc[c] = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) query[c] = 0.f;
        if (active && has_r) load_bf16<8>(a.sq + (ctx.vec0 + int64_t(row) * ctx.heads) * R + part * 8, query);
    }
    __device__ __forceinline__ void pair(bool live, float x, float, const float (&key)[8], const float (&value)[VPL]) {
        float partial = 0.f;
        if (live) {
#pragma unroll
            for (int c = 0; c < 8; ++c) partial = fmaf(query[c], key[c], partial);
        }
        const float s = group_sum(partial);
        if (live) {
            if (x > maximum) {
                const float alpha = ex2(maximum - x);
                denominator *= alpha;
#pragma unroll
                for (int c = 0; c < VPL; ++c) acc[c] *= alpha;
                maximum = x;
            }
            const float p = ex2(x - maximum);
            denominator += p;
            const float weight = p * s;
#pragma unroll
            for (int c = 0; c < VPL; ++c) acc[c] = fmaf(weight, value[c], acc[c]);
        }
    }
    // Combines the eight lane groups' partial results of one row (same tree on every lane).
    __device__ __forceinline__ void merge_groups() {
#pragma unroll
        for (int step = 4; step < 32; step <<= 1) {
            const float other_maximum = __shfl_xor_sync(FULL, maximum, step);
            const float other_denominator = __shfl_xor_sync(FULL, denominator, step);
            const float merged = fmaxf(maximum, other_maximum);
            const float mine = ex2(maximum - merged), theirs = ex2(other_maximum - merged);
            denominator = denominator * mine + other_denominator * theirs;
#pragma unroll
            for (int c = 0; c < VPL; ++c) acc[c] = acc[c] * mine + __shfl_xor_sync(FULL, acc[c], step) * theirs;
            maximum = merged;
        }
    }
    __device__ __forceinline__ void finish(const Args& a, const RowContext& ctx, int row, int part, bool, bool active) {
        float normalizer = 0.f;
        if (active) {
            const float inverse = 1.f / denominator;
#pragma unroll
            for (int c = 0; c < VPL; ++c) acc[c] *= inverse;
            normalizer = maximum + log2f(denominator);
        }
        store_bf16<VPL>(a.out + (ctx.vec0 + int64_t(row) * ctx.heads) * DV + part * VPL, acc);
        if (part == 0) a.lse2_out[int64_t(ctx.bh) * ctx.n + row] = normalizer;
    }
};

int device_sm_count() {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

size_t hard_forward_workspace_bytes(int batch, int heads, int n) { return index_bytes(batch * heads, n, 1); }

cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const int2* documents, int hard_rows, const float* lut,
                                int lut_stride, int ctas, __nv_bfloat16* out, float* lse2, void* workspace,
                                cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = launch_build_index(ik, batch_heads, shape.n, workspace, 0, 1, stream);
    if (status != cudaSuccess) return status;
    RowsArgs args{};
    args.sq = sq; args.sk = sk; args.v = v;
    args.iq = iq; args.ik = ik; args.boundary = boundary; args.hard = hard;
    args.documents = documents; args.hard_rows = hard_rows;
    args.lut = lut;
    args.index = side_index(workspace, batch_heads, shape.n, 0, 1);
    args.out = out; args.lse2_out = lse2;
    args.batch = shape.batch; args.heads = shape.heads; args.n = shape.n; args.lut_stride = lut_stride;
    args.tasks = batch_heads * (shape.n / TASK_ROWS);
#define DISM_CASE(RR, VV) \
    if (shape.r == RR && shape.dv == VV) return launch_rows_kernel<ForwardPolicy<RR, VV>>(args, ctas, stream);
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    return cudaErrorInvalidValue;
}

}  // namespace dism
