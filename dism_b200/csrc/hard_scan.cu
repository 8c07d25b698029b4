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
                                    int* __restrict__ out, const unsigned* choice) {
    if (!route_open(choice)) return;
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
    KernelTimer timer("hard_summary", stream);
    hard_summary_kernel<<<int(blocks), 256, 0, stream>>>(iq, ik, hard, batch * heads, n, summary, route_word());
    return cudaGetLastError();
}

// boundary[c][j] = max(summary[c][j], boundary[c-1][j-32]).  A thread owns one chain
// (c, e+32c), c ascending, so in-place operation is safe; entries right of a strip's last row are
// written -1 and never read.
__global__ void hard_chunk_kernel(const int* __restrict__ summary, int* __restrict__ out, int batch_heads, int n,
                                  const unsigned* choice) {
    if (!route_open(choice)) return;
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
    KernelTimer timer("hard_chunk", stream);
    hard_chunk_kernel<<<int(blocks), 128, 0, stream>>>(summary, boundary, batch_heads, n, route_word());
    return cudaGetLastError();
}

// ---- single longest earlier match (symbol streams, iq = ik = s) ---------------------------------
// Each lane group is not needed here: lane r < OWN carries row r, the warp reads the row's bucket
// of the stream's own position index and keeps the longest run, the most recent one on ties.
__global__ __launch_bounds__(WARPS * 32) void longest_match_kernel(const int* __restrict__ streams, SideIndex index,
                                                                    int batch, int n, int* __restrict__ end,
                                                                    int* __restrict__ length, int* __restrict__ next) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = n / OWN;
    for (int64_t task = int64_t(blockIdx.x) * WARPS + warp; task < int64_t(batch) * groups;
         task += int64_t(gridDim.x) * WARPS) {
        const int b = int(task / groups), row0 = int(task % groups) * OWN;
        const int* s = streams + int64_t(b) * n;
        const SideIndex mine{index.entries + int64_t(b) * n, index.starts + int64_t(b) * (BUCKETS + 1), nullptr};
        for (int r = 0; r < OWN; ++r) {
            const int i = row0 + r, label = __ldg(s + i);
            int from, to;
            partner_range<true>(mine, label, i, from, to);
            long long best = -1;  // (run length << 32) | position: larger run first, then later position
            for (int base = from; base < to; base += 32) {  // positions ascend: stop at the first one >= i
                const int at = base + lane;
                int2 entry = make_int2(0x7fffffff, 0);
                if (at < to) entry = __ldg(mine.entries + at);
                const bool hit = entry.x < i && entry.y == label;
                // a run longer than one needs the diagonal predecessor to match as well
                const bool longer = hit && entry.x > 0 && i > 0 && __ldg(s + entry.x - 1) == __ldg(s + i - 1);
                if (hit && !longer) best = max(best, (1ll << 32) | entry.x);
                for (unsigned waiting = __ballot_sync(FULL, longer); waiting; waiting &= waiting - 1) {
                    const int owner = __ffs(waiting) - 1, j = __shfl_sync(FULL, entry.x, owner);
                    const int length = run_length(s, s, nullptr, n, i, j, lane);
                    best = max(best, (static_cast<long long>(length) << 32) | j);
                }
                if (__ballot_sync(FULL, entry.x >= i)) break;
            }
#pragma unroll
            for (int step = 16; step; step >>= 1) best = max(best, __shfl_xor_sync(FULL, best, step));
            if (lane == 0) {
                const int arg = best < 0 ? -1 : int(best & 0xffffffff);
                end[int64_t(b) * n + i] = arg;
                length[int64_t(b) * n + i] = best < 0 ? 0 : int(best >> 32);
                next[int64_t(b) * n + i] = arg >= 0 ? s[arg + 1] : -1;
            }
        }
    }
}

size_t longest_match_workspace_bytes(int batch, int n) { return index_bytes(batch, n, 1); }

cudaError_t launch_longest_match(const int* streams, int batch, int n, int* end, int* length, int* next,
                                 void* workspace, cudaStream_t stream) {
    cudaError_t status = launch_build_index(streams, batch, n, workspace, 0, 1, stream);
    if (status != cudaSuccess) return status;
    int64_t blocks = (int64_t(batch) * (n / OWN) + WARPS - 1) / WARPS;
    const int64_t cap = int64_t(device_sm_count()) * 8;
    if (blocks > cap) blocks = cap;
    if (!blocks) return cudaSuccess;
    KernelTimer timer("longest_match", stream);
    longest_match_kernel<<<int(blocks), WARPS * 32, 0, stream>>>(streams, side_index(workspace, batch, n, 0, 1), batch,
                                                                 n, end, length, next);
    return cudaGetLastError();
}

}  // namespace dism
