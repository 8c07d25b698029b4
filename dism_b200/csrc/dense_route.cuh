// What the consecutive-position (dense) kernels of the forward and the backward share: the route word,
// how the positions of a (batch, head) are cut into chunks, and the walk along whole diagonals that
// gives every chunk the run lengths of the line before its first block.
//
// A dense kernel is one cooperative launch of one CTA per SM.  With no dense slice (the usual case)
// every CTA reads the route words and returns.  Otherwise the whole grid first walks the diagonals of
// the dense slices, meets at a grid barrier, and then takes the (slice, chunk) work items in turn.
#pragma once
#include "dism_common.cuh"

namespace dism {

constexpr int DENSE_ROWS = 16;     // owners (query rows or key columns) per block
constexpr int DENSE_COLUMNS = 32;  // partners per warp step: two tiles
constexpr int DENSE_WARPS = 8;
constexpr int DENSE_ROUTE = 1;     // route word of a (batch, head) that takes the dense route
constexpr int DENSE_SHARE = 10;    // it does when at least N^2 / DENSE_SHARE pairs (causal or not) have equal labels

// Chunks per (batch, head): enough CTAs for about two per SM of a 148-SM part, at least 128 positions each.
__host__ __device__ inline int dense_chunks(int batch_heads, int n) {
    int chunks = (296 + batch_heads - 1) / batch_heads;
    if (chunks > n / 128) chunks = n / 128;
    if (chunks > 64) chunks = 64;
    return chunks < 1 ? 1 : chunks;
}
// First row block of chunk c: chunks have about equal numbers of causal pairs (rows weigh as their index).
__host__ __device__ inline int dense_chunk_start(int chunk, int chunks, int n) {
    const int blocks = n / DENSE_ROWS;
    if (chunk <= 0) return 0;
    if (chunk >= chunks) return blocks;
    int start = int(float(blocks) * sqrtf(float(chunk) / float(chunks)));
    return start > blocks ? blocks : start;
}
// First owner block of chunk c.  Query-major chunks are as above; key-major chunks mirror them, because a key
// column's pairs are the rows below it.
__host__ __device__ inline int dense_owner_start(bool query_major, int chunk, int chunks, int n) {
    return query_major ? dense_chunk_start(chunk, chunks, n) : n / DENSE_ROWS - dense_chunk_start(chunks - chunk, chunks, n);
}
// Scratch of one dense sweep: per (batch, head) and chunk one walked line and two sweep lines of N run lengths.
__host__ __device__ inline size_t dense_bytes(int batch_heads, int n) {
    return size_t(batch_heads) * dense_chunks(batch_heads, n) * 3 * size_t(n) * sizeof(int);
}

// line[c][0][.] of one (batch, head) and pass, for chunks c >= 1: the run lengths of the line before the chunk's
// first owner o0: query-major L(o0 - 1, key) over keys, key-major L(query, o0 - 1) over queries.  The thread walks
// diagonal query - key = d from its start, so one walk serves the lines of all chunks.
// With packed documents a run ends where the key would lie before the query's document, and begins at its first key.
static __device__ __forceinline__ void dense_walk_diagonal(const int* __restrict__ iq, const int* __restrict__ ik,
                                                           const int2* __restrict__ documents, int* lines, int chunks, int n,
                                                           bool query_major, int d) {
    int i = d, j = 0, run = 0;
    for (int chunk = 1; chunk < chunks; ++chunk) {
        const int line = dense_owner_start(query_major, chunk, chunks, n) * DENSE_ROWS - 1;
        const int steps = query_major ? line - i + 1 : line - j + 1;  // to this diagonal's cell in that line
        if (steps <= 0) continue;    // query-major: the diagonal starts below that row
        if (i + steps > n) break;    // key-major: the diagonal ends before that column
#pragma unroll 8
        for (int s = 0; s < steps; ++s) {
            // a document's first key starts a run afresh: on the main diagonal the cell before it belongs to the
            // previous document, elsewhere it lies outside the query's document and has ended the run already
            const int first_key = documents ? __ldg(documents + ((i + s) >> 8)).x : 0;
            if (j + s <= first_key) run = 0;
            run = j + s >= first_key && __ldg(iq + i + s) == __ldg(ik + j + s) ? run + 1 : 0;
        }
        i += steps;
        j += steps;
        lines[int64_t(chunk) * 3 * n + (query_major ? j - 1 : i - 1)] = run;
    }
}
// All diagonals of all dense slices, spread over the grid.  lines: [passes, BH, chunks, 3, N]; pass 0 is query-major.
static __device__ __forceinline__ void dense_walk_all(const int* __restrict__ iq, const int* __restrict__ ik,
                                                      const int2* __restrict__ documents, const int* __restrict__ route, int* lines,
                                                      int passes, int batch_heads, int chunks, int n) {
    if (chunks < 2) return;
    const int64_t total = int64_t(passes) * batch_heads * n;
    for (int64_t work = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; work < total; work += int64_t(gridDim.x) * blockDim.x) {
        const int slice = int(work / n), bh = slice % batch_heads;
        if (route[bh] != DENSE_ROUTE) continue;
        dense_walk_diagonal(iq + int64_t(bh) * n, ik + int64_t(bh) * n, documents, lines + int64_t(slice) * chunks * 3 * n, chunks, n,
                            slice < batch_heads, int(work % n));
    }
}

// Whether any (batch, head) takes the dense route (the same answer in every thread of the CTA).
static __device__ __forceinline__ bool dense_any(const int* __restrict__ route, int batch_heads) {
    int mine = 0;
    for (int bh = threadIdx.x; bh < batch_heads; bh += blockDim.x) mine |= route[bh] == DENSE_ROUTE;
    return __syncthreads_or(mine) != 0;
}

}  // namespace dism
