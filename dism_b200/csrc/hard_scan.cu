// Integer stages of the hard path: strip summaries, boundary composition, and the single
// longest earlier match of a symbol stream.
//
// hard_summary / hard_chunk keep the reference's checkpoint rectangle
// (dism_v3/src/hard_summary.cu:6-104, dism_v3/src/hard_chunk.cu:19-69) for callers that ask for
// the saved state; the fused forward and backward never need it.
#include "dism_common.cuh"

namespace dism {

// summary[bh][c][j] = largest mismatching key coordinate on the diagonal segment that ends at
// (32c+31, j) inside strip c, or -1.  One thread per entry walks up the diagonal and stops at the
// first mismatch, which is the largest coordinate because columns fall as the walk rises.
__global__ void hard_summary_kernel(const int* __restrict__ iq, const int* __restrict__ ik,
                                    const uint8_t* __restrict__ hard, int batch_heads, int n,
                                    int* __restrict__ out) {
    const int checkpoints = (n - 1) / 32;
    const int64_t total = int64_t(batch_heads) * checkpoints * n;
    for (int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; e < total; e += int64_t(gridDim.x) * blockDim.x) {
        const int j = int(e % n);
        const int64_t t = e / n;
        const int c = int(t % checkpoints), bh = int(t / checkpoints);
        int result = -1;
        if (hard[bh] && j <= 32 * c + 31) {
            const int* q = iq + int64_t(bh) * n + 32 * c + 31;
            const int* k = ik + int64_t(bh) * n + j;
            const int steps = min(32, j + 1);
            for (int s = 0; s < steps; ++s)
                if (__ldg(q - s) != __ldg(k - s)) { result = j - s; break; }
        }
        out[e] = result;
    }
}

cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream) {
    const int64_t total = int64_t(batch) * heads * ((n - 1) / 32) * n;
    if (!total) return cudaSuccess;
    int64_t blocks = (total + 255) / 256;
    const int64_t cap = ctas ? ctas : int64_t(device_sm_count()) * 32;
    if (blocks > cap) blocks = cap;
    hard_summary_kernel<<<int(blocks), 256, 0, stream>>>(iq, ik, hard, batch * heads, n, summary);
    return cudaGetLastError();
}

// boundary[c][j] = max(summary[c][j], boundary[c-1][j-32]).  A thread owns one chain
// (c, e+32c), c ascending, so in-place operation is safe; entries right of a strip's last row are
// written -1 and never read.
__global__ void hard_chunk_kernel(const int* __restrict__ summary, int* __restrict__ out, int batch_heads, int n) {
    const int checkpoints = (n - 1) / 32, chains = 32 * checkpoints;
    const int64_t plane = int64_t(checkpoints) * n;
    const int64_t threads = int64_t(gridDim.x) * blockDim.x, self = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t id = self; id < int64_t(batch_heads) * chains; id += threads) {
        const int bh = int(id / chains), e = 31 - int(id % chains);
        const int64_t base = bh * plane;
        int state = -1;
        for (int c = e >= 0 ? 0 : (31 - e) / 32; c < checkpoints; ++c) {
            const int64_t at = base + int64_t(c) * n + e + 32 * c;
            state = max(state, summary[at]);
            out[at] = state;
        }
    }
    for (int64_t id = self; id < int64_t(batch_heads) * plane; id += threads) {
        const int j = int(id % n), c = int(id / n % checkpoints);
        if (j > 32 * c + 31) out[id] = -1;
    }
}

cudaError_t launch_hard_chunk(const int* summary, int* boundary, int batch_heads, int n, cudaStream_t stream) {
    const int checkpoints = (n - 1) / 32;
    if (!checkpoints || !batch_heads) return cudaSuccess;
    int64_t blocks = (int64_t(batch_heads) * checkpoints * 32 + 127) / 128;
    const int64_t cap = int64_t(device_sm_count()) * 64;
    if (blocks > cap) blocks = cap;
    hard_chunk_kernel<<<int(blocks), 128, 0, stream>>>(summary, boundary, batch_heads, n);
    return cudaGetLastError();
}

// ---- single longest earlier match (symbol streams, iq = ik = s) ---------------------------------
struct LongestWarp {
    int best[OWN], arg[OWN];
    const int* s;
    int n, row0;
};

struct LongestProc {
    static __device__ __noinline__ void hits(LongestWarp* w, int r, int base, unsigned mask) {
        const int lane = threadIdx.x & 31, i = w->row0 + r;
        int best = w->best[r], arg = w->arg[r];
        do {
            const int j = base + __ffs(mask) - 1;
            mask &= mask - 1;
            if (j == i) continue;  // the diagonal always matches itself
            const int length = match_length(w->s, w->s, nullptr, w->n, i, j, lane);
            if (length >= best) { best = length; arg = j; }
        } while (mask);
        w->best[r] = best;
        w->arg[r] = arg;
    }
};

__global__ __launch_bounds__(256) void longest_match_kernel(const int* __restrict__ streams, int batch, int n,
                                                             int* __restrict__ end, int* __restrict__ length,
                                                             int* __restrict__ next) {
    __shared__ LongestWarp state[8];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    LongestWarp* w = state + warp;
    const int groups = n / OWN;
    for (int64_t task = int64_t(blockIdx.x) * 8 + warp; task < int64_t(batch) * groups; task += int64_t(gridDim.x) * 8) {
        const int b = int(task / groups), row0 = int(task % groups) * OWN;
        const int* s = streams + int64_t(b) * n;
        __syncwarp();
        if (lane < OWN) { w->best[lane] = 0; w->arg[lane] = -1; }
        if (lane == 0) { w->s = s; w->n = n; w->row0 = row0; }
        __syncwarp();
        stream_matches<true, LongestProc>(w, s, s, n, row0, lane);
        __syncwarp();
        if (lane < OWN) {
            const int i = row0 + lane, arg = w->arg[lane];
            end[int64_t(b) * n + i] = arg;
            length[int64_t(b) * n + i] = w->best[lane];
            next[int64_t(b) * n + i] = arg >= 0 ? s[arg + 1] : -1;
        }
    }
}

cudaError_t launch_longest_match(const int* streams, int batch, int n, int* end, int* length, int* next,
                                 cudaStream_t stream) {
    int64_t blocks = (int64_t(batch) * (n / OWN) + 7) / 8;
    const int64_t cap = int64_t(device_sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (!blocks) return cudaSuccess;
    longest_match_kernel<<<int(blocks), 256, 0, stream>>>(streams, batch, n, end, length, next);
    return cudaGetLastError();
}

}  // namespace dism
