// Hard backward: dlog-weight table, the query-major pass (dSQ and the per-row tau terms), the
// key-major pass (dV, dSK) and the per-head tau reduction.
//
// Replaces, behind the C ABI, the reference's hard_dlog_weights_kernel, hard_backward_kernel and
// hard_tau_reduce_kernel (dism_v3/src/hard_backward.cu:7-197; formulas in
// dism_v3/docs/HARD_BACKWARD_QUADRATIC.md:60-97).  Where the reference runs one key-major kernel
// and adds dSQ and four per-query moments across CTAs with FP32 atomics, this design runs the
// matched-pair stream twice, once owned by queries and once owned by keys: every gradient row is
// then accumulated by exactly one warp in a fixed order, with no atomics, no zero-filled
// accumulators and bit-identical results for any grid size.
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

// ---- query-major pass ------------------------------------------------------------------------
template <int DV>
struct QueryWarp {
    float dsq[OWN][32], sq[OWN][32], dout[OWN][DV];
    float u[OWN], v[OWN], w[OWN], z[OWN], norm[OWN], center[OWN];
    const int *iq, *ik, *boundary;
    const float *lut, *dlut;
    const __nv_bfloat16 *sk, *value;
    int n, row0, stride_r, stride_v;
};

template <int R, int DV>
struct QueryProc {
    static __device__ __noinline__ void hits(QueryWarp<DV>* w, int r, int base, unsigned mask) {
        constexpr int PER = DV / 32;
        const int lane = threadIdx.x & 31, i = w->row0 + r;
        float dsq = w->dsq[r][lane], u = w->u[r], v = w->v[r], ww = w->w[r], z = w->z[r];
        const float a = w->sq[r][lane], norm = w->norm[r], center = w->center[r];
        float d[PER];
#pragma unroll
        for (int c = 0; c < PER; ++c) d[c] = w->dout[r][lane * PER + c];
        do {
            const int j = base + __ffs(mask) - 1;
            mask &= mask - 1;
            const int length = match_length(w->iq, w->ik, w->boundary, w->n, i, j, lane);
            const float p = ex2(__ldg(w->lut + length) - norm);
            const float g = __ldg(w->dlut + length) - center;
            const float b = lane < R ? bf2f(w->sk[int64_t(j) * w->stride_r + lane]) : 0.f;
            float value[PER], partial = 0.f;
            load_bf16<PER>(w->value + int64_t(j) * w->stride_v + lane * PER, value);
#pragma unroll
            for (int c = 0; c < PER; ++c) partial = fmaf(d[c], value[c], partial);
            const float s = warp_sum(a * b), e = warp_sum(partial);
            const float pse = p * s * e;
            u += pse;
            v = fmaf(p, g, v);
            ww = fmaf(pse, g, ww);
            z += p;
            dsq = fmaf(p * e, b, dsq);
        } while (mask);
        w->dsq[r][lane] = dsq;
        w->u[r] = u; w->v[r] = v; w->w[r] = ww; w->z[r] = z;
    }
};

struct BackwardArgs {
    const __nv_bfloat16 *sq, *sk, *v, *dout;
    const int *iq, *ik, *boundary;
    const uint8_t* hard;
    const float *lut, *dlut, *lse2;
    float *dsq, *dtau_rows;
    __nv_bfloat16 *dsk, *dv;
    int batch, heads, n, lut_stride, tasks;
};

constexpr int BACKWARD_WARPS = 8;
constexpr int BLOCK_ROWS = BACKWARD_WARPS * OWN;

template <int R, int DV>
__global__ __launch_bounds__(BACKWARD_WARPS * 32) void hard_backward_query_kernel(const BackwardArgs a) {
    constexpr int PER = DV / 32;
    extern __shared__ __align__(16) unsigned char storage[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto* w = reinterpret_cast<QueryWarp<DV>*>(storage) + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half, b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
        const float* dlut = a.dlut + int64_t(h) * a.lut_stride;
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            if (active) {
                __syncwarp();
                if (lane == 0) {
                    w->iq = a.iq + int64_t(bh) * a.n;
                    w->ik = a.ik + int64_t(bh) * a.n;
                    w->boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
                    w->lut = a.lut + int64_t(h) * a.lut_stride;
                    w->dlut = dlut;
                    w->sk = a.sk + vec0 * R;
                    w->value = a.v + vec0 * DV;
                    w->n = a.n; w->row0 = row0; w->stride_r = a.heads * R; w->stride_v = a.heads * DV;
                }
                for (int r = 0; r < OWN; ++r) {
                    const int64_t row = vec0 + int64_t(row0 + r) * a.heads;
                    float d[PER];
                    load_bf16<PER>(a.dout + row * DV + lane * PER, d);
#pragma unroll
                    for (int c = 0; c < PER; ++c) w->dout[r][lane * PER + c] = d[c];
                    w->sq[r][lane] = lane < R ? bf2f(a.sq[row * R + lane]) : 0.f;
                    w->dsq[r][lane] = 0.f;
                    if (lane == 0) {
                        w->u[r] = w->v[r] = w->w[r] = w->z[r] = 0.f;
                        w->norm[r] = a.lse2[int64_t(bh) * a.n + row0 + r];
                        w->center[r] = dlut[row0 + r + 1];
                    }
                }
                __syncwarp();
                stream_matches<true, QueryProc<R, DV>>(w, a.iq + int64_t(bh) * a.n, a.ik + int64_t(bh) * a.n,
                                                       a.n, row0, lane);
                __syncwarp();
            }
            for (int r = 0; r < OWN; ++r) {
                const int i = row0 + r;
                if (lane < R) a.dsq[(vec0 + int64_t(i) * a.heads) * R + lane] = active ? w->dsq[r][lane] : 0.f;
                if (lane == 0) {
                    float term = 0.f;
                    if (active) {
                        // Centred four-moment form: the fallback has unit weight and zero derivative.
                        const float fallback = ex2(-w->norm[r]);
                        const float inverse = __fdividef(1.f, w->z[r] + fallback);
                        const float mean = fmaf(-fallback, w->center[r], w->v[r]) * inverse;
                        term = fmaf(-w->u[r], mean, w->w[r]) * inverse;
                    }
                    a.dtau_rows[int64_t(bh) * a.n + i] = term;
                }
            }
        }
    }
}

// ---- key-major pass ----------------------------------------------------------------------------
template <int DV>
struct KeyWarp {
    float dv[OWN][DV], value[OWN][DV], dsk[OWN][32], sk[OWN][32];
    const int *iq, *ik, *boundary;
    const float *lut, *lse2;
    const __nv_bfloat16 *sq, *dout;
    int n, row0, stride_r, stride_v;
};

template <int R, int DV>
struct KeyProc {
    static __device__ __noinline__ void hits(KeyWarp<DV>* w, int r, int base, unsigned mask) {
        constexpr int PER = DV / 32;
        const int lane = threadIdx.x & 31, j = w->row0 + r;
        float dsk = w->dsk[r][lane], dv[PER], value[PER];
        const float b = w->sk[r][lane];
#pragma unroll
        for (int c = 0; c < PER; ++c) { dv[c] = w->dv[r][lane * PER + c]; value[c] = w->value[r][lane * PER + c]; }
        do {
            const int i = base + __ffs(mask) - 1;
            mask &= mask - 1;
            const int length = match_length(w->iq, w->ik, w->boundary, w->n, i, j, lane);
            const float p = ex2(__ldg(w->lut + length) - __ldg(w->lse2 + i));
            const float a = lane < R ? bf2f(w->sq[int64_t(i) * w->stride_r + lane]) : 0.f;
            float d[PER], partial = 0.f;
            load_bf16<PER>(w->dout + int64_t(i) * w->stride_v + lane * PER, d);
#pragma unroll
            for (int c = 0; c < PER; ++c) partial = fmaf(d[c], value[c], partial);
            const float s = warp_sum(a * b), e = warp_sum(partial);
            const float ps = p * s, pe = p * e;
#pragma unroll
            for (int c = 0; c < PER; ++c) dv[c] = fmaf(ps, d[c], dv[c]);
            dsk = fmaf(pe, a, dsk);
        } while (mask);
        w->dsk[r][lane] = dsk;
#pragma unroll
        for (int c = 0; c < PER; ++c) w->dv[r][lane * PER + c] = dv[c];
    }
};

template <int R, int DV>
__global__ __launch_bounds__(BACKWARD_WARPS * 32) void hard_backward_key_kernel(const BackwardArgs a) {
    constexpr int PER = DV / 32;
    extern __shared__ __align__(16) unsigned char storage[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto* w = reinterpret_cast<KeyWarp<DV>*>(storage) + warp;
    const int blocks = a.n / BLOCK_ROWS, half = blocks / 2;
    for (int task = blockIdx.x; task < a.tasks; task += gridDim.x) {
        const int bh = task / half, pair = task % half, b = bh / a.heads, h = bh % a.heads;
        const bool active = a.hard[bh];
        const int64_t vec0 = int64_t(b) * a.n * a.heads + h;
        for (int side = 0; side < 2; ++side) {
            const int row0 = (side ? blocks - 1 - pair : pair) * BLOCK_ROWS + warp * OWN;
            if (active) {
                __syncwarp();
                if (lane == 0) {
                    w->iq = a.iq + int64_t(bh) * a.n;
                    w->ik = a.ik + int64_t(bh) * a.n;
                    w->boundary = a.boundary ? a.boundary + int64_t(bh) * ((a.n - 1) / 32) * a.n : nullptr;
                    w->lut = a.lut + int64_t(h) * a.lut_stride;
                    w->lse2 = a.lse2 + int64_t(bh) * a.n;
                    w->sq = a.sq + vec0 * R;
                    w->dout = a.dout + vec0 * DV;
                    w->n = a.n; w->row0 = row0; w->stride_r = a.heads * R; w->stride_v = a.heads * DV;
                }
                for (int r = 0; r < OWN; ++r) {
                    const int64_t row = vec0 + int64_t(row0 + r) * a.heads;
                    float value[PER];
                    load_bf16<PER>(a.v + row * DV + lane * PER, value);
#pragma unroll
                    for (int c = 0; c < PER; ++c) { w->value[r][lane * PER + c] = value[c]; w->dv[r][lane * PER + c] = 0.f; }
                    w->sk[r][lane] = lane < R ? bf2f(a.sk[row * R + lane]) : 0.f;
                    w->dsk[r][lane] = 0.f;
                }
                __syncwarp();
                stream_matches<false, KeyProc<R, DV>>(w, a.ik + int64_t(bh) * a.n, a.iq + int64_t(bh) * a.n,
                                                      a.n, row0, lane);
                __syncwarp();
            }
            for (int r = 0; r < OWN; ++r) {
                const int64_t row = vec0 + int64_t(row0 + r) * a.heads;
                float result[PER];
#pragma unroll
                for (int c = 0; c < PER; ++c) result[c] = active ? w->dv[r][lane * PER + c] : 0.f;
                store_bf16<PER>(a.dv + row * DV + lane * PER, result);
                if (lane < R) a.dsk[row * R + lane] = __float2bfloat16_rn(active ? w->dsk[r][lane] : 0.f);
            }
        }
    }
}

// dtau[h] = sum over batch and rows of the per-row terms, in a fixed order.
__global__ void tau_reduce_kernel(const float* __restrict__ rows, float* __restrict__ dtau, int batch, int heads,
                                  int n) {
    const int head = blockIdx.x;
    float sum = 0.f;
    for (int64_t e = threadIdx.x; e < int64_t(batch) * n; e += blockDim.x)
        sum += rows[(e / n * heads + head) * n + e % n];
    __shared__ float partial[256];
    partial[threadIdx.x] = sum;
    __syncthreads();
    for (int s = 128; s; s >>= 1) {
        if (threadIdx.x < s) partial[threadIdx.x] += partial[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) dtau[head] = partial[0];
}

// Workspace: the dlog table [H, lut_stride] followed by the per-row tau terms [B, H, N], FP32.
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride) {
    return sizeof(float) * (size_t(heads) * lut_stride + size_t(batch) * heads * n);
}

template <int R, int DV>
static cudaError_t launch_backward_variant(const BackwardArgs& args, int ctas, cudaStream_t stream) {
    auto query = hard_backward_query_kernel<R, DV>;
    auto key = hard_backward_key_kernel<R, DV>;
    const int query_shared = sizeof(QueryWarp<DV>) * BACKWARD_WARPS, key_shared = sizeof(KeyWarp<DV>) * BACKWARD_WARPS;
    cudaError_t status = cudaFuncSetAttribute(query, cudaFuncAttributeMaxDynamicSharedMemorySize, query_shared);
    if (status != cudaSuccess) return status;
    status = cudaFuncSetAttribute(key, cudaFuncAttributeMaxDynamicSharedMemorySize, key_shared);
    if (status != cudaSuccess) return status;
    int resident_q = 1, resident_k = 1;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_q, query, BACKWARD_WARPS * 32, query_shared);
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident_k, key, BACKWARD_WARPS * 32, key_shared);
    const int sms = device_sm_count();
    int grid_q = ctas ? ctas : sms * (resident_q > 0 ? resident_q : 1);
    int grid_k = ctas ? ctas : sms * (resident_k > 0 ? resident_k : 1);
    if (grid_q > args.tasks) grid_q = args.tasks;
    if (grid_k > args.tasks) grid_k = args.tasks;
    query<<<grid_q, BACKWARD_WARPS * 32, query_shared, stream>>>(args);
    key<<<grid_k, BACKWARD_WARPS * 32, key_shared, stream>>>(args);
    return cudaGetLastError();
}

cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const float* lut, int lut_stride,
                                 const float* lse2, int ctas, float* dsq, __nv_bfloat16* dsk, __nv_bfloat16* dv,
                                 float* dtau, void* workspace, cudaStream_t stream) {
    float* dlut = static_cast<float*>(workspace);
    float* rows = dlut + size_t(shape.heads) * lut_stride;
    dlog_weights_kernel<<<dim3((lut_stride + 255) / 256, shape.heads), 256, 0, stream>>>(lut, dlut, lut_stride);
    BackwardArgs args{sq, sk, v, dout, iq, ik, boundary, hard, lut, dlut, lse2, dsq, rows, dsk, dv,
                      shape.batch, shape.heads, shape.n, lut_stride,
                      shape.batch * shape.heads * (shape.n / BLOCK_ROWS / 2)};
    cudaError_t status = cudaErrorInvalidValue;
#define DISM_CASE(RR, VV) \
    if (shape.r == RR && shape.dv == VV) status = launch_backward_variant<RR, VV>(args, ctas, stream);
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    if (status != cudaSuccess) return status;
    tau_reduce_kernel<<<shape.heads, 256, 0, stream>>>(rows, dtau, shape.batch, shape.heads, shape.n);
    return cudaGetLastError();
}

}  // namespace dism
