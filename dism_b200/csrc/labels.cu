// Discretiser: per-head arg-max symbol of x . E^T.
//
// Replaces the label part of the reference's vocabulary kernels
// (dism_v3/python/flash_dism/emb_kernel.py:88-108, kernels/interp_true.py:25-33): bf16 rows against
// bf16 codebooks, FP32 accumulation, lowest index on ties.
//
// The labels are defined by a pinned accumulation order (d ascending, one FP32 rounding per add;
// bf16 products are exact in FP32), so a CPU can reproduce them bit for bit.  The kernel gets there
// in two steps: the logits come from bf16 tensor-core tiles, whose summation order differs, and
// every row whose best and second-best tensor-core logits are closer than a rigorous bound on
// that difference is recomputed in the pinned order.  For all other rows the two orders provably
// agree on the arg-max.
#include "dism_common.cuh"

namespace dism {

constexpr int LABEL_WARPS = 4;
constexpr int LABEL_ROWS = LABEL_WARPS * 32;  // rows per CTA: two m16 tiles per warp
constexpr int LABEL_CODES = 64;               // codebook rows per staged tile (eight n8 tiles)

__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct Best {
    float first, second;
    int arg;
    // branch-free: the old maximum or the newcomer, whichever is smaller, competes for second place
    __device__ __forceinline__ void offer(float x, int index) {
        second = fmaxf(second, fminf(first, x));
        arg = x > first ? index : arg;
        first = fmaxf(first, x);
    }
    __device__ __forceinline__ void merge(float other_first, float other_second, int other_arg) {
        if (other_first > first || (other_first == first && other_arg < arg)) {
            second = fmaxf(first, other_second);
            first = other_first;
            arg = other_arg;
        } else {
            second = fmaxf(second, other_first);
        }
    }
};

template <int D>
__global__ __launch_bounds__(LABEL_ROWS) void labels_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ codebook, int n,
                                                            int heads, int vocab, int* __restrict__ labels) {
    constexpr int KSTEPS = D / 16, PITCH = D + 8;  // padded rows keep fragment loads bank-conflict free
    __shared__ __align__(16) __nv_bfloat16 codes[LABEL_CODES][PITCH];
    __shared__ int flagged[LABEL_ROWS], flagged_count;
    __shared__ float scale_shared[LABEL_WARPS];
    __shared__ float exact_value[LABEL_WARPS];
    __shared__ int exact_arg[LABEL_WARPS];
    const int bh = blockIdx.y, b = bh / heads, h = bh % heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row_base = blockIdx.x * LABEL_ROWS + warp * 32;
    const __nv_bfloat16* head_codes = codebook + int64_t(h) * vocab * D;
    if (threadIdx.x == 0) flagged_count = 0;

    // A fragments of the warp's 32 rows: two m16 tiles, KSTEPS k16 steps, four registers each.
    unsigned a[2][KSTEPS][4];
    float norm2[2][2] = {{0.f, 0.f}, {0.f, 0.f}};  // sum x^2 of rows (tile, g) and (tile, g+8): this lane's share
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = row_base + m * 16 + half * 8 + g;
            const unsigned* source = reinterpret_cast<const unsigned*>(x + ((int64_t(b) * n + min(row, n - 1)) * heads + h) * D);
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k)
#pragma unroll
                for (int hi = 0; hi < 2; ++hi) {
                    const unsigned word = __ldg(source + k * 8 + hi * 4 + t);
                    a[m][k][half + 2 * hi] = word;
                    const float lo = __uint_as_float(word << 16), hi_value = __uint_as_float(word & 0xffff0000u);
                    norm2[m][half] = fmaf(lo, lo, fmaf(hi_value, hi_value, norm2[m][half]));
                }
        }
    Best best[2][2];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) best[m][half] = Best{-INFINITY, -INFINITY, 0};
    float code_max = 0.f;  // largest squared code norm seen while staging

    // The next codebook tile is fetched into registers while the current one is multiplied.
    constexpr int PIECES = LABEL_CODES * (D / 8) / LABEL_ROWS;  // 16-byte pieces per thread and tile
    uint4 staged[PIECES];
    auto fetch = [&](int v0) {
#pragma unroll
        for (int piece = 0; piece < PIECES; ++piece) {
            const int e = threadIdx.x + piece * LABEL_ROWS, v = e / (D / 8), c = e % (D / 8);
            staged[piece] = make_uint4(0, 0, 0, 0);
            if (v0 + v < vocab) staged[piece] = __ldg(reinterpret_cast<const uint4*>(head_codes + int64_t(v0 + v) * D) + c);
        }
    };
    fetch(0);
    for (int v0 = 0; v0 < vocab; v0 += LABEL_CODES) {
        __syncthreads();
#pragma unroll
        for (int piece = 0; piece < PIECES; ++piece) {
            const int e = threadIdx.x + piece * LABEL_ROWS, v = e / (D / 8), c = e % (D / 8);
            const uint4 raw = staged[piece];
            *reinterpret_cast<uint4*>(&codes[v][c * 8]) = raw;
            const unsigned word[4] = {raw.x, raw.y, raw.z, raw.w};
            float squares = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float lo = __uint_as_float(word[w] << 16), hi = __uint_as_float(word[w] & 0xffff0000u);
                squares = fmaf(lo, lo, fmaf(hi, hi, squares));
            }
            // the D/8 consecutive threads that staged one code row add up its squared norm
#pragma unroll
            for (int s = 1; s < D / 8; s <<= 1) squares += __shfl_xor_sync(FULL, squares, s);
            code_max = fmaxf(code_max, squares);
        }
        if (v0 + LABEL_CODES < vocab) fetch(v0 + LABEL_CODES);
        __syncthreads();
#pragma unroll
        for (int tile = 0; tile < LABEL_CODES / 8; ++tile) {
            float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int k = 0; k < KSTEPS; ++k) {
                const unsigned* source = reinterpret_cast<const unsigned*>(&codes[tile * 8 + g][k * 16]);
                const unsigned b0 = source[t], b1 = source[4 + t];
                mma_bf16(c[0], a[0][k], b0, b1);
                mma_bf16(c[1], a[1][k], b0, b1);
            }
            const int column = v0 + tile * 8 + 2 * t;
            if (v0 + LABEL_CODES <= vocab) {  // whole tile inside the codebook: no bound checks
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        best[m][half].offer(c[m][2 * half], column);
                        best[m][half].offer(c[m][2 * half + 1], column + 1);
                    }
            } else {
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (column < vocab) best[m][half].offer(c[m][2 * half], column);
                        if (column + 1 < vocab) best[m][half].offer(c[m][2 * half + 1], column + 1);
                    }
            }
        }
    }
    // Largest squared code norm of this head (every thread staged a share of every tile).
#pragma unroll
    for (int s = 16; s; s >>= 1) code_max = fmaxf(code_max, __shfl_xor_sync(FULL, code_max, s));
    if (lane == 0) scale_shared[warp] = code_max;
    __syncthreads();
    code_max = fmaxf(fmaxf(scale_shared[0], scale_shared[1]), fmaxf(scale_shared[2], scale_shared[3]));

    // Combine the four lanes that share a row; flag rows whose margin is inside the error bound.
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            Best& mine = best[m][half];
            float l2 = norm2[m][half];
#pragma unroll
            for (int s = 1; s <= 2; s <<= 1) {
                const float f = __shfl_xor_sync(FULL, mine.first, s), sec = __shfl_xor_sync(FULL, mine.second, s);
                const int arg = __shfl_xor_sync(FULL, mine.arg, s);
                mine.merge(f, sec, arg);
                l2 += __shfl_xor_sync(FULL, l2, s);
            }
            const int row = row_base + m * 16 + half * 8 + g;
            if (t == 0 && row < n) {
                // Both orders are within D u sum|x e| of the exact logit (u = 2^-24; twice that is allowed for
                // the tensor core in case it truncates), and sum|x e| <= |x|_2 |e|_2.  A margin above twice
                // the summed bound makes the two arg-maxes equal.
                const float tolerance = float(3 * D) * 5.9604645e-8f * sqrtf(l2 * code_max) * 1.01f;
                if (mine.first - mine.second <= 2.f * tolerance) flagged[atomicAdd(&flagged_count, 1)] = row;
                else labels[int64_t(bh) * n + row] = mine.arg;
            }
        }
    __syncthreads();

    // Pinned-order recomputation of the flagged rows: 128 threads share the codes of one row.
    const int count = flagged_count;
    for (int f = 0; f < count; ++f) {
        const int row = flagged[f];
        const __nv_bfloat16* source = x + ((int64_t(b) * n + row) * heads + h) * D;
        float top = -INFINITY;
        int arg = 0x7fffffff;
        for (int v = threadIdx.x; v < vocab; v += LABEL_ROWS) {
            const __nv_bfloat16* code = head_codes + int64_t(v) * D;
            float acc = 0.f;
#pragma unroll 8
            for (int d = 0; d < D; ++d) acc = __fadd_rn(acc, __fmul_rn(bf2f(source[d]), bf2f(code[d])));
            if (acc > top) { top = acc; arg = v; }  // ascending v per thread: first maximum kept
        }
#pragma unroll
        for (int s = 16; s; s >>= 1) {
            const float other = __shfl_xor_sync(FULL, top, s);
            const int other_arg = __shfl_xor_sync(FULL, arg, s);
            if (other > top || (other == top && other_arg < arg)) { top = other; arg = other_arg; }
        }
        __syncthreads();
        if (lane == 0) { exact_value[warp] = top; exact_arg[warp] = arg; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < LABEL_WARPS; ++w)
                if (exact_value[w] > top || (exact_value[w] == top && exact_arg[w] < arg)) { top = exact_value[w]; arg = exact_arg[w]; }
            labels[int64_t(bh) * n + row] = arg;
        }
    }
}

cudaError_t launch_labels(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int batch, int n, int heads,
                          int d, int vocab, int* labels, cudaStream_t stream) {
    if (labels_tcgen05_covers(x, codebook, batch, n, heads, d, vocab))
        return launch_labels_tcgen05(x, codebook, labels, nullptr, nullptr, nullptr, batch, n, heads, d, vocab, stream);
    dim3 grid((n + LABEL_ROWS - 1) / LABEL_ROWS, batch * heads);
    KernelTimer timer("labels", stream);
    if (d == 32) labels_kernel<32><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else if (d == 64) labels_kernel<64><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else if (d == 128) labels_kernel<128><<<grid, LABEL_ROWS, 0, stream>>>(x, codebook, n, heads, vocab, labels);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

// Two tensors of the same shape (the q and the k side of a step), in one launch where the tensor-memory pipeline covers both.
cudaError_t launch_labels_pair(const __nv_bfloat16* x0, const __nv_bfloat16* codebook0, int* labels0, const __nv_bfloat16* x1,
                               const __nv_bfloat16* codebook1, int* labels1, int batch, int n, int heads, int d, int vocab,
                               cudaStream_t stream) {
    if (2 * int64_t(batch) * heads <= 65535 && labels_tcgen05_covers(x0, codebook0, batch, n, heads, d, vocab) &&
        labels_tcgen05_covers(x1, codebook1, batch, n, heads, d, vocab))
        return launch_labels_tcgen05(x0, codebook0, labels0, x1, codebook1, labels1, batch, n, heads, d, vocab, stream);
    const cudaError_t status = launch_labels(x0, codebook0, batch, n, heads, d, vocab, labels0, stream);
    return status != cudaSuccess ? status : launch_labels(x1, codebook1, batch, n, heads, d, vocab, labels1, stream);
}

}  // namespace dism
