// Hard forward: log-weight table and the fused match / normalise / signed-readout kernel.
//
// Replaces, behind the C ABI, the reference's hard_log_weights_kernel and hard_forward_kernel
// (dism_v3/src/hard_forward.cu:9-118, dism_v3/include/forward/readout.cuh:16-100).  The design is
// not a translation: a pair (query i, key j) contributes only when its labels match (the table
// entry of length 0 is -1e6, whose weight flushes to exactly 0), so a warp that owns eight query
// rows finds its matching keys with register-resident label compares and warp ballots, and only
// those pairs pay for the run length, the table lookup, the sq.sk dot product and the value
// accumulation.  Each row is reduced by one warp in ascending key order, so outputs do not
// depend on the grid size.
#include "dism_common.cuh"

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
    log_weights_kernel<<<dim3((n + 256) / 256, heads), 256, 0, stream>>>(tau, lut, n + 1);
    return cudaGetLastError();
}

template <int DV>
struct ForwardWarp {
    float acc[OWN][DV];
    float sq[OWN][32];
    float maximum[OWN], denominator[OWN];
    const int *iq, *ik, *boundary;
    const float* lut;
    const __nv_bfloat16 *sk, *v;  // row 0 of this (batch, head); rows are `stride` elements apart
    int n, row0, stride_r, stride_v;
};

template <int R, int DV>
struct ForwardProc {
    static __device__ __noinline__ void hits(ForwardWarp<DV>* w, int r, int base, unsigned mask) {
        constexpr int PER = DV / 32;
        const int lane = threadIdx.x & 31, i = w->row0 + r;
        float maximum = w->maximum[r], denominator = w->denominator[r], acc[PER];
#pragma unroll
        for (int c = 0; c < PER; ++c) acc[c] = w->acc[r][lane * PER + c];
        const float a = w->sq[r][lane];
        do {
            const int j = base + __ffs(mask) - 1;
            mask &= mask - 1;
            const int length = match_length(w->iq, w->ik, w->boundary, w->n, i, j, lane);
            const float x = __ldg(w->lut + length);
            float b = lane < R ? bf2f(w->sk[int64_t(j) * w->stride_r + lane]) : 0.f;
            const float s = warp_sum(a * b);
            if (x > maximum) {
                const float alpha = ex2(maximum - x);
                denominator *= alpha;
#pragma unroll
                for (int c = 0; c < PER; ++c) acc[c] *= alpha;
                maximum = x;
            }
            const float p = ex2(x - maximum);
            denominator += p;
            const float weight = p * s;
            float value[PER];
            load_bf16<PER>(w->v + int64_t(j) * w->stride_v + lane * PER, value);
#pragma unroll
            for (int c = 0; c < PER; ++c) acc[c] = fmaf(weight, value[c], acc[c]);
        } while (mask);
#pragma unroll
        for (int c = 0; c < PER; ++c) w->acc[r][lane * PER + c] = acc[c];
        w->maximum[r] = maximum;
        w->denominator[r] = denominator;
    }
};

struct ForwardArgs {
    const __nv_bfloat16 *sq, *sk, *v;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float* lut;
    __nv_bfloat16* out;
    float* lse2;
    int batch, heads, n, lut_stride, tasks;
};

constexpr int FORWARD_WARPS = 8;
constexpr int BLOCK_ROWS = FORWARD_WARPS * OWN;  // 64 query rows per CTA pass

template <int R, int DV>
__global__ __launch_bounds__(FORWARD_WARPS * 32) void hard_forward_kernel(const ForwardArgs a) {
    constexpr int PER = DV / 32;
    extern __shared__ __align__(16) unsigned char storage[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto* w = reinterpret_cast<ForwardWarp<DV>*>(storage) + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half;
        const int b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = (int64_t(b) * a.n * a.heads + h);  // (b, 0, h) in units of one vector
        // A light and a heavy row block per task keep causal work per task constant.
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            if (active) {
                __syncwarp();
                if (lane == 0) {
                    w->iq = a.iq + int64_t(bh) * a.n;
                    w->ik = a.ik + int64_t(bh) * a.n;
                    w->boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
                    w->lut = a.lut + int64_t(h) * a.lut_stride;
                    w->sk = a.sk + vec0 * R;
                    w->v = a.v + vec0 * DV;
                    w->n = a.n;
                    w->row0 = row0;
                    w->stride_r = a.heads * R;
                    w->stride_v = a.heads * DV;
                }
                for (int r = 0; r < OWN; ++r) {
#pragma unroll
                    for (int c = 0; c < PER; ++c) w->acc[r][lane * PER + c] = 0.f;
                    w->sq[r][lane] = lane < R ? bf2f(a.sq[(vec0 + int64_t(row0 + r) * a.heads) * R + lane]) : 0.f;
                    if (lane == 0) { w->maximum[r] = 0.f; w->denominator[r] = 1.f; }
                }
                __syncwarp();
                stream_matches<true, ForwardProc<R, DV>>(w, a.iq + int64_t(bh) * a.n, a.ik + int64_t(bh) * a.n,
                                                         a.n, row0, lane);
                __syncwarp();
            }
            for (int r = 0; r < OWN; ++r) {
                const int i = row0 + r;
                __nv_bfloat16* o = a.out + (vec0 + int64_t(i) * a.heads) * DV + lane * PER;
                float result[PER];
                float normalizer = 0.f;
#pragma unroll
                for (int c = 0; c < PER; ++c) result[c] = 0.f;
                if (active) {
                    const float denominator = w->denominator[r], inverse = 1.f / denominator;
#pragma unroll
                    for (int c = 0; c < PER; ++c) result[c] = w->acc[r][lane * PER + c] * inverse;
                    normalizer = w->maximum[r] + log2f(denominator);
                }
                store_bf16<PER>(o, result);
                if (lane == 0) a.lse2[int64_t(bh) * a.n + i] = normalizer;
            }
        }
    }
}

int device_sm_count() {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

template <int R, int DV>
static cudaError_t launch_forward_variant(const ForwardArgs& args, int ctas, cudaStream_t stream) {
    auto kernel = hard_forward_kernel<R, DV>;
    const int shared = sizeof(ForwardWarp<DV>) * FORWARD_WARPS;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    int resident = 1;
    status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, FORWARD_WARPS * 32, shared);
    if (status != cudaSuccess) return status;
    int grid = ctas ? ctas : device_sm_count() * (resident > 0 ? resident : 1);
    if (grid > args.tasks) grid = args.tasks;
    kernel<<<grid, FORWARD_WARPS * 32, shared, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const float* lut, int lut_stride, int ctas,
                                __nv_bfloat16* out, float* lse2, cudaStream_t stream) {
    ForwardArgs args{sq, sk, v, iq, ik, boundary, hard, lut, out, lse2,
                     shape.batch, shape.heads, shape.n, lut_stride,
                     shape.batch * shape.heads * (shape.n / BLOCK_ROWS / 2)};
#define DISM_CASE(RR, VV) \
    if (shape.r == RR && shape.dv == VV) return launch_forward_variant<RR, VV>(args, ctas, stream);
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    return cudaErrorInvalidValue;
}

}  // namespace dism
