// Integer stages of the hard path: strip summaries, boundary composition, and the single
// longest earlier match of a symbol stream.
//
// hard_summary / hard_chunk keep the reference's checkpoint rectangle
// (dism_v3/src/hard_summary.cu:6-104, dism_v3/src/hard_chunk.cu:19-69) for callers that ask for
// the saved state; the fused forward and backward never need it.
#include "dism_common.cuh"

namespace dism {

// summary[bh][c][j] = largest mismatching key coordinate on the diagonal segment that ends at
// (32c+31, j) inside strip c, or -1.  An entry walks up its diagonal and stops at the first
// mismatch, which is the largest coordinate because columns fall as the walk rises.  The stage is
// bound by the 4 bytes it writes per entry: a CTA takes whole (slice, strip) rows of the rectangle
// (row and column come from the loop counters, not from a division per entry), a thread fills four
// adjacent entries and writes them with one 16-byte streaming store; entries right of the strip's
// last row are -1 without a look at the labels.
__global__ __launch_bounds__(256) void hard_summary_kernel(const int* __restrict__ iq, const int* __restrict__ ik,
                                                           const uint8_t* __restrict__ hard, int batch_heads, int n,
                                                           int* __restrict__ out, const unsigned* choice) {
    if (!route_open(choice)) return;
    const int checkpoints = (n - 1) / 32;
    const int64_t rows = int64_t(batch_heads) * checkpoints;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int bh = int(row / checkpoints), c = int(row - int64_t(bh) * checkpoints);
        const int last = 32 * c + 31;  // the strip's last query row
        const bool walk = hard[bh] != 0;
        const int* q = iq + int64_t(bh) * n + last;
        const int* k = ik + int64_t(bh) * n;
        int4* target = reinterpret_cast<int4*>(out + row * n);
        for (int j4 = threadIdx.x * 4; j4 < n; j4 += blockDim.x * 4) {
            int result[4] = {-1, -1, -1, -1};
            if (walk && j4 <= last) {  // (then j4 + 3 <= last too: last + 1 is a multiple of 32)
                // the four walks go up together: step s compares query label last - s with keys j4 - s .. j4 - s + 3,
                // three of which the step before already held
                const int4 head = __ldg(reinterpret_cast<const int4*>(k + j4));
                int window[4] = {head.x, head.y, head.z, head.w};
                unsigned pending = 0xf;
                for (int s = 0; s < 32 && pending; ++s) {
                    const int mine = __ldg(q - s);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        if (j4 + u - s < 0) pending &= ~(1u << u);  // the diagonal left the rectangle
                        else if ((pending >> u & 1) && window[u] != mine) {
                            result[u] = j4 + u - s;
                            pending &= ~(1u << u);
                        }
                    }
                    window[3] = window[2]; window[2] = window[1]; window[1] = window[0];
                    window[0] = j4 - s - 1 >= 0 ? __ldg(k + j4 - s - 1) : 0;
                }
            }
            __stcs(target + j4 / 4, make_int4(result[0], result[1], result[2], result[3]));
        }
    }
}

cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream) {
    const int64_t rows = int64_t(batch) * heads * ((n - 1) / 32);
    if (!rows) return cudaSuccess;
    int64_t blocks = rows;
    const int64_t cap = ctas ? ctas : int64_t(device_sm_count()) * 16;
    if (blocks > cap) blocks = cap;
    KernelTimer timer("hard_summary", stream);
    hard_summary_kernel<<<int(blocks), 256, 0, stream>>>(iq, ik, hard, batch * heads, n, summary, route_word());
    return cudaGetLastError();
}

// boundary[c][j] = max(summary[c][j], boundary[c-1][j-32]).  A thread owns one chain
// (c, e+32c), c ascending, so in-place operation is safe (no __restrict__: the two may be one
// buffer); the 32 chains of a warp read and write one aligned 128-byte line per strip.  Entries
// right of a strip's last row are written -1, row by row with 16-byte stores, and never read.
__global__ __launch_bounds__(128) void hard_chunk_kernel(const int* summary, int* out, int batch_heads, int n,
                                                         const unsigned* choice) {
    if (!route_open(choice)) return;
    const int checkpoints = (n - 1) / 32, chains = 32 * checkpoints;
    const int64_t plane = int64_t(checkpoints) * n;
    const int64_t threads = int64_t(gridDim.x) * blockDim.x, self = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t id = self; id < int64_t(batch_heads) * chains; id += threads) {
        const int bh = int(id / chains), e = 31 - int(id - int64_t(bh) * chains);
        const int first = e >= 0 ? 0 : (31 - e) / 32;
        const int* source = summary + bh * plane + e;
        int* target = out + bh * plane + e;
        int state = -1;
        int c = first;
        for (; c + 8 <= checkpoints; c += 8) {  // eight independent loads in flight, then the dependent maxima
            int value[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) value[u] = __ldcs(source + int64_t(c + u) * (n + 32));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                state = max(state, value[u]);
                __stcs(target + int64_t(c + u) * (n + 32), state);
            }
        }
        for (; c < checkpoints; ++c) {
            state = max(state, __ldcs(source + int64_t(c) * (n + 32)));
            __stcs(target + int64_t(c) * (n + 32), state);
        }
    }
    const int64_t rows = int64_t(batch_heads) * checkpoints;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int c = int(row % checkpoints);
        int4* target = reinterpret_cast<int4*>(out + row * n);
        for (int j4 = 32 * c + 32 + threadIdx.x * 4; j4 < n; j4 += blockDim.x * 4) __stcs(target + j4 / 4, make_int4(-1, -1, -1, -1));
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
