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
#include "hard_rows.cuh"

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

// ---- query-major pass: dSQ and the per-row tau term ----------------------------------------------
template <int R_, int DV>
struct QueryBackwardPolicy {
    static constexpr bool QUERY_MAJOR = true, EXTRA = true;
    static constexpr int R = R_, VPL = DV / 4, MIN_CTAS = 2;
    using Args = RowsArgs;
    static const char* name() { return "hard_backward_query"; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_a(const Args& a) { return a.sk; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_b(const Args& a) { return a.v; }

    float query[8], derivative[VPL], dsq[8], u, v, w, z, norm, center;

    __device__ __forceinline__ void begin(const Args& a, const RowContext& ctx, int row, int part, bool has_r, bool active,
                                          bool) {
        u = v = w = z = norm = center = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) { query[c] = 0.f; dsq[c] = 0.f; }
#pragma unroll
        for (int c = 0; c < VPL; ++c) derivative[c] = 0.f;
        if (active) {
            const int64_t at = ctx.vec0 + int64_t(row) * ctx.heads;
            if (has_r) load_bf16<8>(a.sq + at * R + part * 8, query);
            load_bf16<VPL>(a.dout + at * DV + part * VPL, derivative);
            norm = __ldg(ctx.lse2 + row);
            center = __ldg(ctx.dlut + row - ctx.begin + 1);  // document-local position
        }
    }
    __device__ __forceinline__ void pair(bool live, float x, float extra, const float (&key)[8], const float (&value)[VPL]) {
        float partial_s = 0.f, partial_e = 0.f;
        if (live) {
#pragma unroll
            for (int c = 0; c < 8; ++c) partial_s = fmaf(query[c], key[c], partial_s);
#pragma unroll
            for (int c = 0; c < VPL; ++c) partial_e = fmaf(derivative[c], value[c], partial_e);
        }
        const float s = group_sum(partial_s), e = group_sum(partial_e);
        if (live) {
            const float p = ex2(x - norm), g = extra - center;
            const float pse = p * s * e, pe = p * e;
            u += pse;
            v = fmaf(p, g, v);
            w = fmaf(pse, g, w);
            z += p;
#pragma unroll
            for (int c = 0; c < 8; ++c) dsq[c] = fmaf(pe, key[c], dsq[c]);
        }
    }
    // Adds up the eight lane groups' partial sums of one row (same tree on every lane).
    __device__ __forceinline__ void merge_groups() {
#pragma unroll
        for (int step = 4; step < 32; step <<= 1) {
            u += __shfl_xor_sync(FULL, u, step);
            v += __shfl_xor_sync(FULL, v, step);
            w += __shfl_xor_sync(FULL, w, step);
            z += __shfl_xor_sync(FULL, z, step);
#pragma unroll
            for (int c = 0; c < 8; ++c) dsq[c] += __shfl_xor_sync(FULL, dsq[c], step);
        }
    }
    __device__ __forceinline__ void finish(const Args& a, const RowContext& ctx, int row, int part, bool has_r, bool active) {
        float term = 0.f;
        if (active) {
            // Centred four-moment form: the fallback has unit weight and zero derivative.
            const float fallback = ex2(-norm), inverse = __fdividef(1.f, z + fallback);
            const float mean = fmaf(-fallback, center, v) * inverse;
            term = fmaf(-u, mean, w) * inverse;
        }
        if (has_r) {
            float* out = a.dsq + (ctx.vec0 + int64_t(row) * ctx.heads) * R + part * 8;
            *reinterpret_cast<float4*>(out) = make_float4(dsq[0], dsq[1], dsq[2], dsq[3]);
            *reinterpret_cast<float4*>(out + 4) = make_float4(dsq[4], dsq[5], dsq[6], dsq[7]);
        }
        if (part == 0) a.dtau_rows[int64_t(ctx.bh) * ctx.n + row] = term;
    }
};

// ---- key-major pass: dV and dSK ---------------------------------------------------------------------
template <int R_, int DV>
struct KeyBackwardPolicy {
    static constexpr bool QUERY_MAJOR = false, EXTRA = false;
    static constexpr int R = R_, VPL = DV / 4, MIN_CTAS = 2;
    using Args = RowsArgs;
    static const char* name() { return "hard_backward_key"; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_a(const Args& a) { return a.sq; }
    static __device__ __forceinline__ const __nv_bfloat16* gather_b(const Args& a) { return a.dout; }

    float key[8], value[VPL], dv[VPL], dsk[8];

    __device__ __forceinline__ void begin(const Args& a, const RowContext& ctx, int row, int part, bool has_r, bool active,
                                          bool) {
#pragma unroll
        for (int c = 0; c < 8; ++c) { key[c] = 0.f; dsk[c] = 0.f; }
#pragma unroll
        for (int c = 0; c < VPL; ++c) { value[c] = 0.f; dv[c] = 0.f; }
        if (active) {
            const int64_t at = ctx.vec0 + int64_t(row) * ctx.heads;
            if (has_r) load_bf16<8>(a.sk + at * R + part * 8, key);
            load_bf16<VPL>(a.v + at * DV + part * VPL, value);
        }
    }
    // x is the table entry minus the partner query's log2 normaliser
    __device__ __forceinline__ void pair(bool live, float x, float, const float (&query)[8], const float (&derivative)[VPL]) {
        float partial_s = 0.f, partial_e = 0.f;
        if (live) {
#pragma unroll
            for (int c = 0; c < 8; ++c) partial_s = fmaf(query[c], key[c], partial_s);
#pragma unroll
            for (int c = 0; c < VPL; ++c) partial_e = fmaf(derivative[c], value[c], partial_e);
        }
        const float s = group_sum(partial_s), e = group_sum(partial_e);
        if (live) {
            const float p = ex2(x), ps = p * s, pe = p * e;
#pragma unroll
            for (int c = 0; c < VPL; ++c) dv[c] = fmaf(ps, derivative[c], dv[c]);
#pragma unroll
            for (int c = 0; c < 8; ++c) dsk[c] = fmaf(pe, query[c], dsk[c]);
        }
    }
    __device__ __forceinline__ void merge_groups() {
#pragma unroll
        for (int step = 4; step < 32; step <<= 1) {
#pragma unroll
            for (int c = 0; c < VPL; ++c) dv[c] += __shfl_xor_sync(FULL, dv[c], step);
#pragma unroll
            for (int c = 0; c < 8; ++c) dsk[c] += __shfl_xor_sync(FULL, dsk[c], step);
        }
    }
    __device__ __forceinline__ void finish(const Args& a, const RowContext& ctx, int row, int part, bool has_r, bool) {
        const int64_t at = ctx.vec0 + int64_t(row) * ctx.heads;
        store_bf16<VPL>(a.dv + at * DV + part * VPL, dv);
        if (has_r) store_bf16<8>(a.dsk + at * R + part * 8, dsk);
    }
};

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

cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const int2* documents, int hard_rows,
                                 const float* lut, int lut_stride, const float* lse2, int ctas, float* dsq,
                                 __nv_bfloat16* dsk, __nv_bfloat16* dv, float* dtau, void* workspace,
                                 cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = launch_build_index(ik, batch_heads, shape.n, workspace, 0, 2, stream);
    if (status != cudaSuccess) return status;
    status = launch_build_index(iq, batch_heads, shape.n, workspace, 1, 2, stream);
    if (status != cudaSuccess) return status;
    float* rows = reinterpret_cast<float*>(static_cast<char*>(workspace) + index_bytes(batch_heads, shape.n, 2));
    float* dlut = rows + size_t(batch_heads) * shape.n;
    {
        KernelTimer timer("dlog_weights", stream);
        dlog_weights_kernel<<<dim3((lut_stride + 255) / 256, shape.heads), 256, 0, stream>>>(lut, dlut, lut_stride);
    }
    RowsArgs args{};
    args.sq = sq; args.sk = sk; args.v = v; args.dout = dout;
    args.iq = iq; args.ik = ik; args.boundary = boundary; args.hard = hard;
    args.documents = documents; args.hard_rows = hard_rows;
    args.lut = lut; args.dlut = dlut; args.lse2 = lse2;
    args.dsq = dsq; args.dtau_rows = rows; args.dsk = dsk; args.dv = dv;
    args.batch = shape.batch; args.heads = shape.heads; args.n = shape.n; args.lut_stride = lut_stride;
    args.tasks = batch_heads * (shape.n / TASK_ROWS);
    RowsArgs by_query = args, by_key = args;
    by_query.index = side_index(workspace, batch_heads, shape.n, 0, 2);  // queries look up keys
    by_key.index = side_index(workspace, batch_heads, shape.n, 1, 2);    // keys look up queries
    status = cudaErrorInvalidValue;
#define DISM_CASE(RR, VV)                                                                         \
    if (shape.r == RR && shape.dv == VV) {                                                        \
        status = launch_rows_kernel<QueryBackwardPolicy<RR, VV>>(by_query, ctas, stream);         \
        if (status == cudaSuccess) status = launch_rows_kernel<KeyBackwardPolicy<RR, VV>>(by_key, ctas, stream); \
    }
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    if (status != cudaSuccess) return status;
    KernelTimer timer("tau_reduce", stream);
    tau_reduce_kernel<<<shape.heads, 1024, 0, stream>>>(rows, dtau, shape.batch, shape.heads, shape.n);
    return cudaGetLastError();
}

}  // namespace dism
