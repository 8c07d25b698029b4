// Hard backward: dlog-weight table, the query-major pass (dSQ and the per-row tau terms), the
// key-major pass (dV, dSK) and the per-head tau reduction.
//
// Replaces, behind the C ABI, the reference's hard_dlog_weights_kernel, hard_backward_kernel and
// hard_tau_reduce_kernel (dism_v3/src/hard_backward.cu:7-197; formulas in
// dism_v3/docs/HARD_BACKWARD_QUADRATIC.md:60-97).  Where the reference runs one key-major kernel
// and adds dSQ and four per-query moments across CTAs with FP32 atomics, this design walks the
// matched pairs twice, once owned by queries and once owned by keys: every gradient row is then
// accumulated by exactly one lane group in ascending partner order, with no atomics, no
// zero-filled accumulators and bit-identical results for any grid size.  Pair coefficients stay
// in FP32 (the reference rounds them to BF16 to feed its tensor-core tiles).
#include "dism_common.cuh"

namespace dism {

// g[h,l] = d ln W_l / d tau with tau recovered from the log2 table (lut[h,1] = tau * log2 e).
__global__ void dlog_weights_kernel(const float* __restrict__ lut, float* __restrict__ out, int stride) {
    int l = blockIdx.x * blockDim.x + threadIdx.x, head = blockIdx.y;
    if (l >= stride) return;
    float t = lut[int64_t(head) * stride + 1] * 0.6931471805599453f;
    float a = fabsf(t), length = float(l), x = length * t, g = 0.f;
    if (l && fabsf(x) < .1f) {
        g = (length + 1.f) * .5f + (length * length - 1.f) * t * (1.f / 12.f - (x * x + t * t) * (1.f / 720.f));
    } else if (l) {
        float tail = length * a > 80.f ? 0.f : __fdividef(length, expm1f(length * a));
        float negative = __fdividef(1.f, -expm1f(-a)) - tail;
        g = t > 0 ? length + 1.f - negative : negative;
    }
    out[int64_t(head) * stride + l] = g;
}

struct BackwardArgs {
    const __nv_bfloat16 *sq, *sk, *v, *dout;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float *lut, *dlut, *lse2;
    SideIndex keys, queries;
    float *dsq, *dtau_rows;
    __nv_bfloat16 *dsk, *dv;
    int batch, heads, n, lut_stride, tasks;
};

// ---- query-major pass: dSQ and the per-row tau term ----------------------------------------------
template <int R, int DV, bool EXTRA>
struct BackwardShared {
    PairQueue<EXTRA> queue[WARPS];
    GatherRing<8, DV / 4> ring[WARPS];
};

template <int R, int DV>
__global__ __launch_bounds__(WARPS * 32) void hard_backward_query_kernel(const BackwardArgs a) {
    constexpr int RPL = 8, VPL = DV / 4;
    extern __shared__ __align__(16) unsigned char storage[];
    auto& shared = *reinterpret_cast<BackwardShared<R, DV, true>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group = lane >> 2, part = lane & 3;
    const bool has_r = part * RPL < R;  // this lane holds a slice of the R-wide vectors
    PairQueue<true>* queue = shared.queue + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half, b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
        const int* iq = a.iq + int64_t(bh) * a.n;
        const int* ik = a.ik + int64_t(bh) * a.n;
        const int* boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
        const float* lut = a.lut + int64_t(h) * a.lut_stride;
        const float* dlut = a.dlut + int64_t(h) * a.lut_stride;
        const SideIndex keys{a.keys.entries + int64_t(bh) * a.n, a.keys.starts + int64_t(bh) * (BUCKETS + 1)};
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            const int row = row0 + group;
            float dsq[RPL], term = 0.f;
#pragma unroll
            for (int c = 0; c < RPL; ++c) dsq[c] = 0.f;
            if (active) {
                float query[RPL], derivative[VPL];
#pragma unroll
                for (int c = 0; c < RPL; ++c) query[c] = 0.f;
                if (has_r) load_bf16<RPL>(a.sq + (vec0 + int64_t(row) * a.heads) * R + part * RPL, query);
                load_bf16<VPL>(a.dout + (vec0 + int64_t(row) * a.heads) * DV + part * VPL, derivative);
                const float norm = __ldg(a.lse2 + int64_t(bh) * a.n + row), center = __ldg(dlut + row + 1);
                float u = 0.f, v = 0.f, w = 0.f, z = 0.f;
                const int searched = row0 + (lane & (OWN - 1));
                SearchRow search;
                search.label = __ldg(iq + searched);
                search.previous = searched ? __ldg(iq + searched - 1) : 0;
                partner_range<true>(keys, search.label, searched, search.cursor, search.end);
                while (__ballot_sync(FULL, lane < OWN && search.cursor < search.end)) {
                    __syncwarp();
                    const int queued = find_partners<true, true>(queue, keys.entries, iq, ik, boundary, lut, dlut, nullptr,
                                                                 a.n, row0, search, lane);
                    __syncwarp();
                    const int mine = __shfl_sync(FULL, queued, group);
                    const int rounds = __reduce_max_sync(FULL, mine);
                    drain_partners<RPL, VPL>(
                        queue->position[group], mine, rounds, shared.ring + warp,
                        a.sk + vec0 * R + part * RPL, int64_t(a.heads) * R, has_r, a.v + vec0 * DV + part * VPL,
                        int64_t(a.heads) * DV, lane, [&](bool live, int slot, const float(&key)[RPL], const float(&value)[VPL]) {
                            float partial_s = 0.f, partial_e = 0.f;
                            if (live) {
#pragma unroll
                                for (int c = 0; c < RPL; ++c) partial_s = fmaf(query[c], key[c], partial_s);
#pragma unroll
                                for (int c = 0; c < VPL; ++c) partial_e = fmaf(derivative[c], value[c], partial_e);
                            }
                            const float s = group_sum(partial_s), e = group_sum(partial_e);
                            if (live) {
                                const float p = ex2(queue->weight[group][slot] - norm);
                                const float g = queue->extra[group][slot] - center;
                                const float pse = p * s * e, pe = p * e;
                                u += pse;
                                v = fmaf(p, g, v);
                                w = fmaf(pse, g, w);
                                z += p;
#pragma unroll
                                for (int c = 0; c < RPL; ++c) dsq[c] = fmaf(pe, key[c], dsq[c]);
                            }
                        });
                }
                // Centred four-moment form: the fallback has unit weight and zero derivative.
                const float fallback = ex2(-norm), inverse = __fdividef(1.f, z + fallback);
                const float mean = fmaf(-fallback, center, v) * inverse;
                term = fmaf(-u, mean, w) * inverse;
            }
            float* out = a.dsq + (vec0 + int64_t(row) * a.heads) * R + part * RPL;
            if (has_r) {
#pragma unroll
                for (int c = 0; c < RPL; c += 4)
                    *reinterpret_cast<float4*>(out + c) = make_float4(dsq[c], dsq[c + 1], dsq[c + 2], dsq[c + 3]);
            }
            if (part == 0) a.dtau_rows[int64_t(bh) * a.n + row] = term;
        }
    }
}

// ---- key-major pass: dV and dSK ---------------------------------------------------------------------
template <int R, int DV>
__global__ __launch_bounds__(WARPS * 32) void hard_backward_key_kernel(const BackwardArgs a) {
    constexpr int RPL = 8, VPL = DV / 4;
    extern __shared__ __align__(16) unsigned char storage[];
    auto& shared = *reinterpret_cast<BackwardShared<R, DV, false>*>(storage);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, group = lane >> 2, part = lane & 3;
    const bool has_r = part * RPL < R;  // this lane holds a slice of the R-wide vectors
    PairQueue<false>* queue = shared.queue + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half, b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
        const int* iq = a.iq + int64_t(bh) * a.n;
        const int* ik = a.ik + int64_t(bh) * a.n;
        const int* boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
        const float* lut = a.lut + int64_t(h) * a.lut_stride;
        const float* lse2 = a.lse2 + int64_t(bh) * a.n;
        const SideIndex queries{a.queries.entries + int64_t(bh) * a.n, a.queries.starts + int64_t(bh) * (BUCKETS + 1)};
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            const int row = row0 + group;
            float dv[VPL], dsk[RPL];
#pragma unroll
            for (int c = 0; c < VPL; ++c) dv[c] = 0.f;
#pragma unroll
            for (int c = 0; c < RPL; ++c) dsk[c] = 0.f;
            if (active) {
                float key[RPL], value[VPL];
#pragma unroll
                for (int c = 0; c < RPL; ++c) key[c] = 0.f;
                if (has_r) load_bf16<RPL>(a.sk + (vec0 + int64_t(row) * a.heads) * R + part * RPL, key);
                load_bf16<VPL>(a.v + (vec0 + int64_t(row) * a.heads) * DV + part * VPL, value);
                const int searched = row0 + (lane & (OWN - 1));
                SearchRow search;
                search.label = __ldg(ik + searched);
                search.previous = searched ? __ldg(ik + searched - 1) : 0;
                partner_range<false>(queries, search.label, searched, search.cursor, search.end);
                while (__ballot_sync(FULL, lane < OWN && search.cursor < search.end)) {
                    __syncwarp();
                    const int queued = find_partners<false, false>(queue, queries.entries, iq, ik, boundary, lut, nullptr,
                                                                   lse2, a.n, row0, search, lane);
                    __syncwarp();
                    const int mine = __shfl_sync(FULL, queued, group);
                    const int rounds = __reduce_max_sync(FULL, mine);
                    drain_partners<RPL, VPL>(
                        queue->position[group], mine, rounds, shared.ring + warp,
                        a.sq + vec0 * R + part * RPL, int64_t(a.heads) * R, has_r, a.dout + vec0 * DV + part * VPL,
                        int64_t(a.heads) * DV, lane,
                        [&](bool live, int slot, const float(&query)[RPL], const float(&derivative)[VPL]) {
                            float partial_s = 0.f, partial_e = 0.f;
                            if (live) {
#pragma unroll
                                for (int c = 0; c < RPL; ++c) partial_s = fmaf(query[c], key[c], partial_s);
#pragma unroll
                                for (int c = 0; c < VPL; ++c) partial_e = fmaf(derivative[c], value[c], partial_e);
                            }
                            const float s = group_sum(partial_s), e = group_sum(partial_e);
                            if (live) {
                                const float p = ex2(queue->weight[group][slot]);  // table entry minus the query's normaliser
                                const float ps = p * s, pe = p * e;
#pragma unroll
                                for (int c = 0; c < VPL; ++c) dv[c] = fmaf(ps, derivative[c], dv[c]);
#pragma unroll
                                for (int c = 0; c < RPL; ++c) dsk[c] = fmaf(pe, query[c], dsk[c]);
                            }
                        });
                }
            }
            store_bf16<VPL>(a.dv + (vec0 + int64_t(row) * a.heads) * DV + part * VPL, dv);
            if (has_r) store_bf16<RPL>(a.dsk + (vec0 + int64_t(row) * a.heads) * R + part * RPL, dsk);
        }
    }
}

// dtau[h] = sum over batch and rows of the per-row terms, in a fixed order (thread-strided partial
// sums, then a tree), so the result is the same for every launch.
__global__ __launch_bounds__(1024) void tau_reduce_kernel(const float* __restrict__ rows, float* __restrict__ dtau,
                                                          int batch, int heads, int n) {
    const int head = blockIdx.x;
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
    for (int b = 0; b < batch; ++b) {
        const float4* source = reinterpret_cast<const float4*>(rows + (int64_t(b) * heads + head) * n);
        for (int e = threadIdx.x; e < n / 4; e += blockDim.x) {
            const float4 x = __ldg(source + e);
            sum[0] += x.x; sum[1] += x.y; sum[2] += x.z; sum[3] += x.w;
        }
    }
    __shared__ float partial[1024];
    partial[threadIdx.x] = (sum[0] + sum[1]) + (sum[2] + sum[3]);
    __syncthreads();
    for (int s = 512; s; s >>= 1) {
        if (threadIdx.x < s) partial[threadIdx.x] += partial[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) dtau[head] = partial[0];
}

// Workspace: both position indices, then the per-row tau terms [B, H, N] (read back as float4, so
// they come first and stay 16-byte aligned) and the dlog table [H, lut_stride], all FP32.
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride) {
    return index_bytes(batch * heads, n, 2) + sizeof(float) * (size_t(heads) * lut_stride + size_t(batch) * heads * n);
}

template <int R, int DV>
static cudaError_t launch_backward_variant(const BackwardArgs& args, int ctas, cudaStream_t stream) {
    auto query = hard_backward_query_kernel<R, DV>;
    auto key = hard_backward_key_kernel<R, DV>;
    const int shared_q = sizeof(BackwardShared<R, DV, true>), shared_k = sizeof(BackwardShared<R, DV, false>);
    cudaError_t status = cudaFuncSetAttribute(query, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_q);
    if (status != cudaSuccess) return status;
    status = cudaFuncSetAttribute(key, cudaFuncAttributeMaxDynamicSharedMemorySize, shared_k);
    if (status != cudaSuccess) return status;
    int resident_q = 1, resident_k = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_q, query, WARPS * 32, shared_q);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_k, key, WARPS * 32, shared_k);
    const int sms = device_sm_count();
    int grid_q = ctas ? ctas : sms * (resident_q > 0 ? resident_q : 1);
    int grid_k = ctas ? ctas : sms * (resident_k > 0 ? resident_k : 1);
    if (grid_q > args.tasks) grid_q = args.tasks;
    if (grid_k > args.tasks) grid_k = args.tasks;
    query<<<grid_q, WARPS * 32, shared_q, stream>>>(args);
    key<<<grid_k, WARPS * 32, shared_k, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const float* lut, int lut_stride,
                                 const float* lse2, int ctas, float* dsq, __nv_bfloat16* dsk, __nv_bfloat16* dv,
                                 float* dtau, void* workspace, cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = launch_build_index(ik, batch_heads, shape.n, workspace, 0, 2, stream);
    if (status != cudaSuccess) return status;
    status = launch_build_index(iq, batch_heads, shape.n, workspace, 1, 2, stream);
    if (status != cudaSuccess) return status;
    float* rows = reinterpret_cast<float*>(static_cast<char*>(workspace) + index_bytes(batch_heads, shape.n, 2));
    float* dlut = rows + size_t(batch_heads) * shape.n;
    dlog_weights_kernel<<<dim3((lut_stride + 255) / 256, shape.heads), 256, 0, stream>>>(lut, dlut, lut_stride);
    BackwardArgs args{sq, sk, v, dout, iq, ik, boundary, hard, lut, dlut, lse2,
                      side_index(workspace, batch_heads, shape.n, 0, 2), side_index(workspace, batch_heads, shape.n, 1, 2),
                      dsq, rows, dsk, dv, shape.batch, shape.heads, shape.n, lut_stride,
                      batch_heads * (shape.n / BLOCK_ROWS / 2)};
    status = cudaErrorInvalidValue;
#define DISM_CASE(RR, VV) \
    if (shape.r == RR && shape.dv == VV) status = launch_backward_variant<RR, VV>(args, ctas, stream);
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    if (status != cudaSuccess) return status;
    tau_reduce_kernel<<<shape.heads, 1024, 0, stream>>>(rows, dtau, shape.batch, shape.heads, shape.n);
    return cudaGetLastError();
}

}  // namespace dism
