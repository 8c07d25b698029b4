// Shared device helpers and launch-side declarations for the flash_dism hard path on sm_100a.
//
// How the hard kernels find their work.  A pair (query i, key j <= i) has non-zero weight only
// when its labels are equal, so the kernels never visit the N^2/2 pairs.  A small prepass sorts
// the positions of one side by (label bucket, position); the owner of a row then reads only the
// bucket of its own label (with 4096 buckets, almost always exactly the positions with that label), keeps the entries with the same label on the
// causal side, and gets its matching partners already in ascending order.  Because both sides are
// sorted the same way, the causal pair set is a union of small dense blocks (the queries of a
// bucket against the keys of the same bucket); a warp works through one such block sixteen rows
// by sixteen partners at a time on the tensor cores (hard_forward_blocks.cuh, hard_backward_blocks.cuh).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dism {

constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG_ZERO = -1000000.f;  // LUT entry of length 0 (dism_v3/src/hard_forward.cu:15)
constexpr int BUCKETS = 4096;           // label buckets of the position index
constexpr int OWN = 8;                  // rows per warp of the longest-match kernel
constexpr int WARPS = 8;                // its warps per CTA

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float bf2f(__nv_bfloat16 x) { return __bfloat162float(x); }

__device__ __forceinline__ int bucket_of(int label) {
    unsigned x = unsigned(label);  // labels below 4096 keep a bucket each
    x ^= (x >> 12) ^ (x >> 24);
    return int(x & (BUCKETS - 1));
}

// Number of consecutive label matches on the diagonal that ends at (i, j), given that (i, j)
// itself matches.  The whole warp calls this with the same (i, j) and checks 32 cells per step.
// With a boundary rectangle (int32 [(N-1)/32, N] of this batch/head,
// boundary[c][col] = col - L(32c+31, col)) the walk ends at the 32-row strip edge and reads the
// rest of the run from the rectangle.
__device__ __forceinline__ int run_length(const int* __restrict__ q, const int* __restrict__ k,
                                          const int* __restrict__ boundary, int n, int i, int j, int lane,
                                          int begin = 0) {  // positions below `begin` belong to another document
    int length = 1, bi = i - 1, bj = j - 1;
    if (boundary) {
        const int inside = i & 31;  // rows i-1 .. i-inside share the strip of row i
        const bool ok = lane < inside && bj - lane >= begin && __ldg(q + bi - lane) == __ldg(k + bj - lane);
        const int run = __ffs(~__ballot_sync(FULL, ok)) - 1;
        length += run;
        const int col = bj - inside;
        if (run == inside && col >= 0 && i >= 32)
            length += col - __ldg(boundary + int64_t((i >> 5) - 1) * n + col);
        return length;
    }
    while (bj >= begin) {
        const bool ok = bj - lane >= begin && __ldg(q + bi - lane) == __ldg(k + bj - lane);
        const unsigned mask = __ballot_sync(FULL, ok);
        if (mask != FULL) return length + __ffs(~mask) - 1;
        length += 32;
        bi -= 32;
        bj -= 32;
    }
    return length;
}

// Position index of one side of one (batch, head): `entries` holds (position, label) sorted by
// (bucket, position); bucket b occupies [starts[b], starts[b+1]).
struct SideIndex {
    const int2* entries;
    const int* starts;
    const int* previous;  // parallel to entries: the same side's label one position earlier (0 at position 0)
};

// First entry of bucket range [lo, hi) whose position is >= bound (positions ascend).
__device__ __forceinline__ int lower_bound_position(const int2* __restrict__ entries, int lo, int hi, int bound) {
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(&entries[mid].x) < bound) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

// The same by a whole warp (every lane calls it with the same arguments): 32 evenly spaced probes per round, so one
// dependent load per factor of 32 of the range instead of one per factor of 2.
__device__ __forceinline__ int warp_lower_bound_position(const int2* __restrict__ entries, int lo, int hi, int bound, int lane) {
    while (lo < hi) {
        const int stride = (hi - lo + 31) >> 5;
        const int at = lo + lane * stride;
        const unsigned mask = __ballot_sync(FULL, at < hi && __ldg(&entries[at].x) < bound);
        const int count = __popc(mask);  // positions ascend, so the probes below the bound are the first `count`
        if (stride == 1) return lo + count;
        if (count == 0) return lo;
        hi = min(hi, lo + count * stride);  // the first probe at or above the bound, if there is one
        lo += (count - 1) * stride + 1;     // one past the last probe below it
    }
    return lo;
}

// Range of the bucket of `label` that can hold causal partners of owner position `row`.
template <bool QUERY_MAJOR>
__device__ __forceinline__ void partner_range(const SideIndex& index, int label, int row, int& cursor, int& end,
                                              int begin = 0, int limit = 0x7fffffff) {
    const int bucket = bucket_of(label);
    const int lo = __ldg(index.starts + bucket), hi = __ldg(index.starts + bucket + 1);
    // positions ascend inside a bucket: keys from the document start up to the row, queries from
    // the row to the document end
    if (QUERY_MAJOR) {
        cursor = begin > 0 ? lower_bound_position(index.entries, lo, hi, begin) : lo;
        end = lower_bound_position(index.entries, cursor, hi, row + 1);
    } else {
        cursor = lower_bound_position(index.entries, lo, hi, row);
        end = limit < 0x7fffffff ? lower_bound_position(index.entries, cursor, hi, limit) : hi;
    }
}

// ---- asynchronous 16-byte copies into shared memory ------------------------------------------
__device__ __forceinline__ void cp_async16(void* shared, const void* global) {
    const unsigned target = static_cast<unsigned>(__cvta_generic_to_shared(shared));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(target), "l"(global));
}
// The same, but `bytes` (16 or 0) are read and the rest of the 16 is filled with zeros: a missing row
// costs no branch.  `global` must be a mapped address even when nothing is read.
__device__ __forceinline__ void cp_async16_or_zeros(void* shared, const void* global, int bytes) {
    const unsigned target = static_cast<unsigned>(__cvta_generic_to_shared(shared));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(target), "l"(global), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// ---- route word of a captured graph (dism_v3/include/common/graph_route.cuh:8-13) --------------
// A graph that holds both the quadratic hard path and another route reads one device word per
// replay: 0 runs this path, anything else makes every kernel of it return before it reads or
// writes anything.  A null pointer (eager calls) always runs.
__device__ __forceinline__ bool route_open(const unsigned* choice) {
    if (!choice) return true;
    unsigned value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(choice) : "memory");
    return value == 0;
}
// The word the calling thread's launches pass to their kernels (set through dism_route_word).
const unsigned* route_word();

struct KernelTimer {
    KernelTimer(const char* name, cudaStream_t stream);
    ~KernelTimer();
    int slot;
    cudaStream_t stream;
};

// ---- launch-side entry points (defined in the .cu files, called from the C ABI) -------------
struct HardShape {
    int batch, heads, n, r, dv;
};

int device_sm_count();
cudaError_t launch_labels(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int batch, int n, int heads,
                          int d, int vocab, int* labels, cudaStream_t stream);
// Tensor-memory pipeline for the shapes it covers (labels_tcgen05.cu); launch_labels picks it when it can.
bool labels_tcgen05_covers(const void* x, const void* codebook, int batch, int n, int heads, int d, int vocab);
cudaError_t launch_labels_tcgen05(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int* labels, const __nv_bfloat16* x1,
                                  const __nv_bfloat16* codebook1, int* labels1, int batch, int n, int heads, int d, int vocab,
                                  cudaStream_t stream);
cudaError_t launch_labels_pair(const __nv_bfloat16* x0, const __nv_bfloat16* codebook0, int* labels0, const __nv_bfloat16* x1,
                               const __nv_bfloat16* codebook1, int* labels1, int batch, int n, int heads, int d, int vocab,
                               cudaStream_t stream);
cudaError_t read_labels_fault(int* code);
cudaError_t run_wait_selftest(int code, int* outcome, cudaStream_t stream);
cudaError_t launch_hard_summary(const int* iq, const int* ik, const uint8_t* hard, int batch, int heads, int n,
                                int ctas, int* summary, cudaStream_t stream);
cudaError_t launch_hard_chunk(const int* summary, int* boundary, int batch_heads, int n, cudaStream_t stream);
cudaError_t launch_hard_summary_packed(const int* iq, const int* ik, const uint8_t* hard, const long long* table,
                                       int documents, int64_t rows, int heads, int n, int hard_rows, int ctas, int* summary,
                                       cudaStream_t stream);
cudaError_t launch_hard_chunk_packed(const int* summary, int* boundary, const long long* table, int documents, int64_t rows,
                                     cudaStream_t stream);

// Index workspace: per (batch, head) N entries of int2 plus BUCKETS+1 starts, for `sides` sides.
size_t index_bytes(int batch_heads, int n, int sides);
// Builds the index of `labels` ([BH, N]) into `workspace` (side 0 at the front, side 1 after it).
cudaError_t launch_build_index(const int* labels, int batch_heads, int n, void* workspace, int side, int sides,
                               cudaStream_t stream);
// Both sides of a readout (labels0 -> side 0, labels1 -> side 1) in one launch.
cudaError_t launch_build_index_pair(const int* labels0, const int* labels1, int batch_heads, int n, void* workspace,
                                    cudaStream_t stream);
SideIndex side_index(void* workspace, int batch_heads, int n, int side, int sides);

size_t longest_match_workspace_bytes(int batch, int n);
cudaError_t launch_longest_match(const int* streams, int batch, int n, int* end, int* length, int* next,
                                 void* workspace, cudaStream_t stream);
cudaError_t launch_log_weights(const float* tau, int heads, int n, float* lut, cudaStream_t stream);
// g[h, l] = d ln W_l / d tau from the log2 table lut [heads, lut_stride]; out has the same shape.
cudaError_t launch_dlog_weights(const float* lut, int heads, int lut_stride, float* out, cudaStream_t stream);
size_t hard_forward_workspace_bytes(int batch, int heads, int n);
cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const int2* documents, int hard_rows, const float* lut,
                                int lut_stride, int ctas, __nv_bfloat16* out, float* lse2, void* workspace,
                                cudaStream_t stream);
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride);
cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const int2* documents, int hard_rows,
                                 const float* lut, int lut_stride, const float* lse2, int ctas, float* dsq,
                                 __nv_bfloat16* dsk, __nv_bfloat16* dv, float* dtau, void* workspace, const void* readout_workspace,
                                 cudaStream_t stream);

}  // namespace dism
