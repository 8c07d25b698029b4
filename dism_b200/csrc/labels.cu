// Discretiser: per-head arg-max symbol of x . E^T.
//
// Replaces the label part of the reference's vocabulary kernels
// (dism_v3/python/flash_dism/emb_kernel.py:88-108, kernels/interp_true.py:25-33): bf16 rows against
// bf16 codebooks, FP32 accumulation, lowest index on ties.  The accumulation order is pinned
// (d ascending, one rounding per add; bf16 products are exact in FP32) so the labels can be
// reproduced bit for bit on a CPU.
#include "dism_common.cuh"

namespace dism {

constexpr int LABEL_ROWS = 128;   // rows (threads) per CTA
constexpr int LABEL_CODES = 64;   // codebook rows staged per pass

template <int D>
__global__ __launch_bounds__(LABEL_ROWS) void labels_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ codebook, int n,
                                                            int heads, int vocab, int* __restrict__ labels) {
    __shared__ __align__(16) float codes[LABEL_CODES][D];
    const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
    const int row = blockIdx.x * LABEL_ROWS + threadIdx.x;
    float value[D];
    if (row < n) {
        const uint4* source = reinterpret_cast<const uint4*>(x + ((int64_t(b) * n + row) * heads + h) * D);
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            uint4 raw = source[c];
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float2 f = __bfloat1622float2(pairs[e]);
                value[c * 8 + 2 * e] = f.x;
                value[c * 8 + 2 * e + 1] = f.y;
            }
        }
    }
    float best = 0.f;
    int arg = 0;
    for (int v0 = 0; v0 < vocab; v0 += LABEL_CODES) {
        __syncthreads();
        for (int e = threadIdx.x; e < LABEL_CODES * D; e += LABEL_ROWS) {
            const int v = v0 + e / D;
            codes[e / D][e % D] = v < vocab ? bf2f(codebook[(int64_t(h) * vocab + v) * D + e % D]) : 0.f;
        }
        __syncthreads();
        if (row < n) {
            const int count = min(LABEL_CODES, vocab - v0);
            for (int v = 0; v < count; ++v) {
                float acc = 0.f;
#pragma unroll
                for (int d = 0; d < D; d += 4) {
                    const float4 e = *reinterpret_cast<const float4*>(&codes[v][d]);
                    acc = __fadd_rn(acc, __fmul_rn(value[d], e.x));
                    acc = __fadd_rn(acc, __fmul_rn(value[d + 1], e.y));
                    acc = __fadd_rn(acc, __fmul_rn(value[d + 2], e.z));
                    acc = __fadd_rn(acc, __fmul_rn(value[d + 3], e.w));
                }
                if ((v0 == 0 && v == 0) || acc > best) { best = acc; arg = v0 + v; }
            }
        }
    }
    if (row < n) labels[int64_t(bh) * n + row] = arg;
}

cudaError_t launch_labels(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int batch, int n, int heads,
                          int d, int vocab, int* labels, cudaStream_t stream) {
    dim3 grid((n + LABEL_ROWS - 1) / LABEL_ROWS, batch * heads);
    if (d == 32) labels_kernel<32><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else if (d == 64) labels_kernel<64><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else if (d == 128) labels_kernel<128><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

}  // namespace dism
