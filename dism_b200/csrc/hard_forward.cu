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

struct ForwardArgs {
    const __nv_bfloat16 *sq, *sk, *v;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float* lut;
    SideIndex keys;
    __nv_bfloat16* out;
    float* lse2;
    int batch, heads, n, lut_stride, tasks;
};

template <int R, int DV>
struct ForwardShared {
    PairQueue<false> queue[WARPS];
    GatherRing<8, DV / 4> ring[WARPS];
};

template <int R, int DV>
__global__ __launch_bounds__(WARPS * 32) void hard_forward_kernel(const ForwardArgs a) {
    constexpr int RPL = 8, VPL = DV / 4;  // elements per lane of a four-lane group (R=16: two lanes hold sq/sk)
    extern __shared__ __align__(16) unsigned char storage[];
    auto& shared = *reinterpret_cast<ForwardShared<R, DV>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group = lane >> 2, part = lane & 3;
    const bool has_r = part * RPL < R;  // this lane holds a slice of the R-wide vectors
    PairQueue<false>* queue = shared.queue + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half, b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = int64_t(b) * a.n * a.heads + h;  // (b, 0, h) in units of one vector
        const int* iq = a.iq + int64_t(bh) * a.n;
        const int* ik = a.ik + int64_t(bh) * a.n;
        const int* boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
        const float* lut = a.lut + int64_t(h) * a.lut_stride;
        const SideIndex keys{a.keys.entries + int64_t(bh) * a.n, a.keys.starts + int64_t(bh) * (BUCKETS + 1)};
        // A light and a heavy row block per task keep the causal work per task constant.
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            const int row = row0 + group;
            float acc[VPL], maximum = 0.f, denominator = 1.f;
#pragma unroll
            for (int c = 0; c < VPL; ++c) acc[c] = 0.f;
            if (active) {
                float query[RPL];
#pragma unroll
                for (int c = 0; c < RPL; ++c) query[c] = 0.f;
                if (has_r) load_bf16<RPL>(a.sq + (vec0 + int64_t(row) * a.heads) * R + part * RPL, query);
                const int searched = row0 + (lane & (OWN - 1));
                SearchRow search;
                search.label = __ldg(iq + searched);
                search.previous = searched ? __ldg(iq + searched - 1) : 0;
                partner_range<true>(keys, search.label, searched, search.cursor, search.end);
                while (__ballot_sync(FULL, lane < OWN && search.cursor < search.end)) {
                    __syncwarp();
                    const int queued = find_partners<true, false>(queue, keys.entries, iq, ik, boundary, lut, nullptr,
                                                                  nullptr, a.n, row0, search, lane);
                    __syncwarp();
                    const int mine = __shfl_sync(FULL, queued, group);
                    const int rounds = __reduce_max_sync(FULL, mine);
                    drain_partners<RPL, VPL>(
                        queue->position[group], mine, rounds, shared.ring + warp,
                        a.sk + vec0 * R + part * RPL, int64_t(a.heads) * R, has_r, a.v + vec0 * DV + part * VPL,
                        int64_t(a.heads) * DV, lane, [&](bool live, int slot, const float(&key)[RPL], const float(&value)[VPL]) {
                            float partial = 0.f;
                            if (live) {
#pragma unroll
                                for (int c = 0; c < RPL; ++c) partial = fmaf(query[c], key[c], partial);
                            }
                            const float s = group_sum(partial);
                            if (live) {
                                const float x = queue->weight[group][slot];
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
                        });
                }
            }
            float normalizer = 0.f;
            if (active) {
                const float inverse = 1.f / denominator;
#pragma unroll
                for (int c = 0; c < VPL; ++c) acc[c] *= inverse;
                normalizer = maximum + log2f(denominator);
            }
            store_bf16<VPL>(a.out + (vec0 + int64_t(row) * a.heads) * DV + part * VPL, acc);
            if (part == 0) a.lse2[int64_t(bh) * a.n + row] = normalizer;
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
    const int shared = sizeof(ForwardShared<R, DV>);
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    int resident = 1;
    status = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, WARPS * 32, shared);
    if (status != cudaSuccess) return status;
    int grid = ctas ? ctas : device_sm_count() * (resident > 0 ? resident : 1);
    if (grid > args.tasks) grid = args.tasks;
    kernel<<<grid, WARPS * 32, shared, stream>>>(args);
    return cudaGetLastError();
}

size_t hard_forward_workspace_bytes(int batch, int heads, int n) { return index_bytes(batch * heads, n, 1); }

cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const float* lut, int lut_stride, int ctas,
                                __nv_bfloat16* out, float* lse2, void* workspace, cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = launch_build_index(ik, batch_heads, shape.n, workspace, 0, 1, stream);
    if (status != cudaSuccess) return status;
    ForwardArgs args{sq, sk, v, iq, ik, boundary, hard, lut, side_index(workspace, batch_heads, shape.n, 0, 1),
                     out, lse2, shape.batch, shape.heads, shape.n, lut_stride,
                     batch_heads * (shape.n / BLOCK_ROWS / 2)};
#define DISM_CASE(RR, VV) \
    if (shape.r == RR && shape.dv == VV) return launch_forward_variant<RR, VV>(args, ctas, stream);
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    return cudaErrorInvalidValue;
}

}  // namespace dism
