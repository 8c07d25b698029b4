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
//
// One row: strip c of a sequence of n positions whose labels start at q and k.
__device__ __forceinline__ void summary_row(const int* __restrict__ q, const int* __restrict__ k, bool walk, int c, int n,
                                            int* __restrict__ out) {
    const int last = 32 * c + 31;  // the strip's last query row
    q += last;
    int4* target = reinterpret_cast<int4*>(out);
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

__global__ __launch_bounds__(256) void hard_summary_kernel(const int* __restrict__ iq, const int* __restrict__ ik,
                                                           const uint8_t* __restrict__ hard, int batch_heads, int n,
                                                           int* __restrict__ out, const unsigned* choice) {
    if (!route_open(choice)) return;
    const int checkpoints = (n - 1) / 32;
    const int64_t rows = int64_t(batch_heads) * checkpoints;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const int bh = int(row / checkpoints), c = int(row - int64_t(bh) * checkpoints);
        summary_row(iq + int64_t(bh) * n, ik + int64_t(bh) * n, hard[bh] != 0, c, n, out + row * n);
    }
}

// A pack of documents (one batch row of n tokens, flags per training row of row_tokens).  `table` holds, per
// non-empty document, (first position, length, rows before it, rectangle elements before it): the rectangle is the
// documents' [H, strips, length] regions one after the other, a row is one (head, strip) of one document.
struct PackedDocument {
    int begin, length, strips;
    int64_t local;  // row (or chain) number inside the document
    int64_t first_element;
};
__device__ __forceinline__ PackedDocument packed_document(const long long* __restrict__ table, int documents, int64_t row) {
    int lo = 0, hi = documents;  // the last document whose first row is <= row
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(table + 4 * mid + 2) <= row) lo = mid;
        else hi = mid;
    }
    PackedDocument d;
    d.begin = int(__ldg(table + 4 * lo));
    d.length = int(__ldg(table + 4 * lo + 1));
    d.strips = (d.length - 1) / 32;
    d.local = row - __ldg(table + 4 * lo + 2);
    d.first_element = __ldg(table + 4 * lo + 3);
    return d;
}

__global__ __launch_bounds__(256) void hard_summary_packed_kernel(const int* __restrict__ iq, const int* __restrict__ ik,
                                                                  const uint8_t* __restrict__ hard,
                                                                  const long long* __restrict__ table, int documents,
                                                                  int64_t rows, int heads, int n, int row_tokens,
                                                                  int* __restrict__ out, const unsigned* choice) {
    if (!route_open(choice)) return;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const PackedDocument d = packed_document(table, documents, row);
        const int h = int(d.local / d.strips), c = int(d.local - int64_t(h) * d.strips);
        const bool walk = hard[(d.begin / row_tokens) * heads + h] != 0;
        summary_row(iq + int64_t(h) * n + d.begin, ik + int64_t(h) * n + d.begin, walk, c, d.length,
                    out + d.first_element + d.local * d.length);
    }
}

static int scan_grid(int64_t items, int64_t cap) { return int(items < cap ? items : cap); }

cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream) {
    const int64_t rows = int64_t(batch) * heads * ((n - 1) / 32);
    if (!rows) return cudaSuccess;
    KernelTimer timer("hard_summary", stream);
    hard_summary_kernel<<<scan_grid(rows, ctas ? ctas : int64_t(device_sm_count()) * 16), 256, 0, stream>>>(
        iq, ik, hard, batch * heads, n, summary, route_word());
    return cudaGetLastError();
}

cudaError_t launch_hard_summary_packed(const int* iq, const int* ik, const uint8_t* hard, const long long* table,
                                       int documents, int64_t rows, int heads, int n, int hard_rows, int ctas, int* summary,
                                       cudaStream_t stream) {
    if (!rows || !documents) return cudaSuccess;
    KernelTimer timer("hard_summary", stream);
    hard_summary_packed_kernel<<<scan_grid(rows, ctas ? ctas : int64_t(device_sm_count()) * 16), 256, 0, stream>>>(
        iq, ik, hard, table, documents, rows, heads, n, n / hard_rows, summary, route_word());
    return cudaGetLastError();
}

// boundary[c][j] = max(summary[c][j], boundary[c-1][j-32]).  A thread owns one chain
// (c, e+32c), c ascending, so in-place operation is safe (no __restrict__: the two may be one
// buffer); the 32 chains of a warp read and write one aligned 128-byte line per strip.  Entries
// right of a strip's last row are written -1, row by row with 16-byte stores, and never read.
//
// Chain e of one [checkpoints, n] plane.
__device__ __forceinline__ void compose_chain(const int* source, int* target, int e, int checkpoints, int n) {
    source += e;
    target += e;
    int state = -1;
    int c = e >= 0 ? 0 : (31 - e) / 32;
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
// The entries of strip row c right of its last query row.
__device__ __forceinline__ void fill_row(int* out, int c, int n) {
    int4* target = reinterpret_cast<int4*>(out);
    for (int j4 = 32 * c + 32 + threadIdx.x * 4; j4 < n; j4 += blockDim.x * 4) __stcs(target + j4 / 4, make_int4(-1, -1, -1, -1));
}

__global__ __launch_bounds__(128) void hard_chunk_kernel(const int* summary, int* out, int batch_heads, int n,
                                                         const unsigned* choice) {
    if (!route_open(choice)) return;
    const int checkpoints = (n - 1) / 32, chains = 32 * checkpoints;
    const int64_t plane = int64_t(checkpoints) * n;
    const int64_t threads = int64_t(gridDim.x) * blockDim.x, self = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t id = self; id < int64_t(batch_heads) * chains; id += threads) {
        const int bh = int(id / chains), e = 31 - int(id - int64_t(bh) * chains);
        compose_chain(summary + bh * plane, out + bh * plane, e, checkpoints, n);
    }
    const int64_t rows = int64_t(batch_heads) * checkpoints;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) fill_row(out + row * n, int(row % checkpoints), n);
}

// The same over a pack: a document's 32 * strips chains per head follow one another, 32 to a row number.
__global__ __launch_bounds__(128) void hard_chunk_packed_kernel(const int* summary, int* out, const long long* __restrict__ table,
                                                                int documents, int64_t rows, const unsigned* choice) {
    if (!route_open(choice)) return;
    const int64_t threads = int64_t(gridDim.x) * blockDim.x, self = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t id = self; id < rows * 32; id += threads) {
        const PackedDocument d = packed_document(table, documents, id >> 5);
        const int64_t chain = d.local * 32 + (id & 31);  // chain number inside the document: [head][32 * strips]
        const int per_head = 32 * d.strips;
        const int h = int(chain / per_head), e = 31 - int(chain - int64_t(h) * per_head);
        const int64_t plane = d.first_element + int64_t(h) * d.strips * d.length;
        compose_chain(summary + plane, out + plane, e, d.strips, d.length);
    }
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const PackedDocument d = packed_document(table, documents, row);
        fill_row(out + d.first_element + d.local * d.length, int(d.local % d.strips), d.length);
    }
}

cudaError_t launch_hard_chunk(const int* summary, int* boundary, int batch_heads, int n, cudaStream_t stream) {
    const int checkpoints = (n - 1) / 32;
    if (!checkpoints || !batch_heads) return cudaSuccess;
    KernelTimer timer("hard_chunk", stream);
    hard_chunk_kernel<<<scan_grid((int64_t(batch_heads) * checkpoints * 32 + 127) / 128, int64_t(device_sm_count()) * 64), 128, 0, stream>>>(
        summary, boundary, batch_heads, n, route_word());
    return cudaGetLastError();
}

cudaError_t launch_hard_chunk_packed(const int* summary, int* boundary, const long long* table, int documents, int64_t rows,
                                     cudaStream_t stream) {
    if (!rows || !documents) return cudaSuccess;
    KernelTimer timer("hard_chunk", stream);
    hard_chunk_packed_kernel<<<scan_grid((rows * 32 + 127) / 128, int64_t(device_sm_count()) * 64), 128, 0, stream>>>(
        summary, boundary, table, documents, rows, route_word());
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
