// Hard backward: dlog-weight table, the query-major pass (dSQ and the per-row tau terms), the
// key-major pass (dV, dSK) and the per-head tau reduction.
//
// Replaces, behind the C ABI, the reference's hard_dlog_weights_kernel, hard_backward_kernel and
// hard_tau_reduce_kernel (dism_v3/src/hard_backward.cu:7-197; formulas in
// dism_v3/docs/HARD_BACKWARD_QUADRATIC.md:60-97).  Where the reference runs one key-major kernel
// and adds dSQ and four per-query moments across CTAs with FP32 atomics, this design walks the
// matched pairs twice, once owned by queries and once owned by keys: every gradient row is then
// accumulated by exactly one warp, tile by tile in ascending partner order, with no atomics, no
// zero-filled accumulators and bit-identical results for any grid size.  Pair coefficients enter
// the second tensor-core product as a bf16 value plus its rounding remainder, i.e. with FP32-like
// accuracy (the reference rounds them to BF16 once).  Slices with dense labels take the
// consecutive-position sweeps of hard_backward_dense.cuh instead.
#include "hard_backward_dense.cuh"

namespace dism {

// g[h,l] = d ln W_l / d tau with tau recovered from the log2 table (lut[h,1] = tau * log2 e).
__device__ __forceinline__ float dlog_weight(float table_one, int l) {
    float t = table_one * 0.6931471805599453f;
    float a = fabsf(t), length = float(l), x = length * t, g = 0.f;
    if (l && fabsf(x) < .1f) {
        g = (length + 1.f) * .5f + (length * length - 1.f) * t * (1.f / 12.f - (x * x + t * t) * (1.f / 720.f));
    } else if (l) {
        float tail = length * a > 80.f ? 0.f : __fdividef(length, expm1f(length * a));
        float negative = __fdividef(1.f, -expm1f(-a)) - tail;
        g = t > 0 ? length + 1.f - negative : negative;
    }
    return g;
}
__global__ void dlog_weights_kernel(const float* __restrict__ lut, float* __restrict__ out, int stride, const unsigned* choice) {
    if (!route_open(choice)) return;
    int l = blockIdx.x * blockDim.x + threadIdx.x, head = blockIdx.y;
    if (l >= stride) return;
    out[int64_t(head) * stride + l] = dlog_weight(lut[int64_t(head) * stride + 1], l);
}

// What the backward prepares in one launch: blockIdx.y 0 and 1 plan the query-major and key-major tiles of
// (batch, head) blockIdx.x (and choose its route); blockIdx.y 2 fills the dlog table, all CTAs of that row together.
static __global__ __launch_bounds__(1024) void prepare_backward_kernel(const TilePlan first, const TilePlan second, int tile_capacity,
                                                                       int* route, unsigned long long dense_pairs,
                                                                       const float* __restrict__ lut, float* __restrict__ dlut,
                                                                       int heads, int lut_stride, const unsigned* choice) {
    if (!route_open(choice)) {
        // The backward tile kernels take no route word (they sit at their register limit): a closed route leaves them no tiles
        // and marks no slice dense, so they read their tile count and return.
        if (blockIdx.y < 2 && threadIdx.x == 0) {
            const TilePlan& plan = blockIdx.y ? second : first;
            plan.tile_starts[int64_t(blockIdx.x) * (BUCKETS + 1) + BUCKETS] = 0;
            plan.next_tile[blockIdx.x] = 0;
            route[blockIdx.x] = 0;
        }
        return;
    }
    if (blockIdx.y == 2) {
        for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < heads * lut_stride; e += gridDim.x * blockDim.x)
            dlut[e] = dlog_weight(lut[int64_t(e / lut_stride) * lut_stride + 1], e % lut_stride);
        return;
    }
    const TilePlan& plan = blockIdx.y ? second : first;
    plan_query_tiles(plan.owner_starts, plan.partner_starts, plan.tile_starts, plan.tiles, plan.next_tile, tile_capacity, route, dense_pairs);
}

cudaError_t launch_dlog_weights(const float* lut, int heads, int lut_stride, float* out, cudaStream_t stream) {
    KernelTimer timer("dlog_weights", stream);
    dlog_weights_kernel<<<dim3((lut_stride + 255) / 256, heads), 256, 0, stream>>>(lut, out, lut_stride, route_word());
    return cudaGetLastError();
}

// dtau[h] = sum over batch and rows of the per-row terms, in a fixed order (thread-strided partial
// sums with all of a thread's loads in flight together, then a shuffle tree per warp and one over the
// warps), so the result is the same for every launch.
__global__ __launch_bounds__(1024) void tau_reduce_kernel(const float* __restrict__ rows, float* __restrict__ dtau,
                                                          int batch, int heads, int n, const unsigned* choice) {
    if (!route_open(choice)) return;
    const int head = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int per_row = n / 4, total = batch * per_row;  // float4 pieces of this head: [batch][n / 4]
    float sum = 0.f;
    for (int first = threadIdx.x; first < total; first += 8 * blockDim.x) {
        float4 piece[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int e = first + u * blockDim.x;
            piece[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (e < total) piece[u] = __ldg(reinterpret_cast<const float4*>(rows + (int64_t(e / per_row) * heads + head) * n) + e % per_row);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) sum += (piece[u].x + piece[u].y) + (piece[u].z + piece[u].w);
    }
#pragma unroll
    for (int s = 16; s; s >>= 1) sum += __shfl_xor_sync(FULL, sum, s);
    __shared__ float partial[32];
    if (lane == 0) partial[warp] = sum;
    __syncthreads();
    if (warp == 0) {
        float all = lane < blockDim.x / 32 ? partial[lane] : 0.f;
#pragma unroll
        for (int s = 16; s; s >>= 1) all += __shfl_xor_sync(FULL, all, s);
        if (lane == 0) dtau[head] = all;
    }
}

// Workspace: both position indices, a tile plan (descriptors, first-tile table, counter) for each of
// the two passes, then the per-row tau terms [B, H, N] (read back as float4, so 16-byte aligned) and the
// dlog table [H, lut_stride], FP32.
static size_t plan_bytes(int batch_heads, int n) {
    size_t bytes = size_t(batch_heads) * tile_capacity_for(n) * sizeof(int4) + size_t(batch_heads) * (BUCKETS + 2) * sizeof(int);
    return (bytes + 255) & ~size_t(255);
}

static size_t tables_bytes(int batch, int heads, int n, int lut_stride) {  // tau rows, dlog table, route words
    const size_t bytes = sizeof(float) * (size_t(heads) * lut_stride + size_t(batch) * heads * n) + sizeof(int) * size_t(batch) * heads;
    return (bytes + 15) & ~size_t(15);
}
size_t hard_backward_workspace_bytes(int batch, int heads, int n, int lut_stride) {
    return index_bytes(batch * heads, n, 2) + 2 * plan_bytes(batch * heads, n) + tables_bytes(batch, heads, n, lut_stride) +
           dense_backward_bytes(batch * heads, n);
}

// One cooperative launch of one CTA per SM for both passes: see dense_route.cuh.
template <int R, int DV>
static cudaError_t launch_dense_backward(const DenseBackwardArgs& args, cudaStream_t stream) {
    auto kernel = hard_backward_dense_kernel<R, DV>;
    const int shared = sizeof(DenseBackwardWarpShared<R, DV>) * DENSE_WARPS;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    KernelTimer timer("hard_backward_dense", stream);
    void* parameters[] = {const_cast<DenseBackwardArgs*>(&args)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(device_sm_count()), dim3(DENSE_WARPS * 32), parameters,
                                       shared, stream);
}

template <bool PACKED, int R, int DV>
static cudaError_t launch_backward_variant(const BackwardBlockArgs& by_query, const BackwardBlockArgs& by_key, int ctas, cudaStream_t stream) {
    auto kernel = hard_backward_blocks_kernel<PACKED, R, DV>;
    const int shared = sizeof(BackwardWarpShared<R, DV>) * BLOCK_WARPS;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    const int batch_heads = by_query.batch * by_query.heads, n = by_query.n;
    // about eight full tiles per warp (partial tiles of small buckets come on top), and with few (batch, head) slices at
    // least four CTAs per SM over each pass: warps take tiles from a counter, so any grid covers the work;
    // `ctas` caps the grid of a pass
    int per_head = n / (QT * BLOCK_WARPS * 8);
    const int fill = (4 * device_sm_count() + batch_heads - 1) / batch_heads;
    if (per_head < fill) per_head = fill;
    if (per_head > (n + QT * BLOCK_WARPS - 1) / (QT * BLOCK_WARPS)) per_head = (n + QT * BLOCK_WARPS - 1) / (QT * BLOCK_WARPS);
    if (per_head < 1) per_head = 1;
    if (ctas) per_head = ctas / batch_heads > 0 ? ctas / batch_heads : 1;
    if (int64_t(batch_heads) * n <= 262144) {  // little work on this GPU: both passes in one launch
        KernelTimer timer("hard_backward", stream);
        kernel<<<dim3(batch_heads, per_head, 2), BLOCK_WARPS * 32, shared, stream>>>(by_query, by_key, 0);
        return cudaGetLastError();
    }
    {
        KernelTimer timer("hard_backward_query", stream);
        kernel<<<dim3(batch_heads, per_head), BLOCK_WARPS * 32, shared, stream>>>(by_query, by_key, 0);
    }
    KernelTimer timer("hard_backward_key", stream);
    kernel<<<dim3(batch_heads, per_head), BLOCK_WARPS * 32, shared, stream>>>(by_query, by_key, 1);
    return cudaGetLastError();
}

template <int R, int DV>
static cudaError_t launch_backward_blocks(const BackwardBlockArgs& by_query, const BackwardBlockArgs& by_key, int ctas, cudaStream_t stream) {
    return by_query.documents ? launch_backward_variant<true, R, DV>(by_query, by_key, ctas, stream)
                              : launch_backward_variant<false, R, DV>(by_query, by_key, ctas, stream);
}

cudaError_t launch_hard_backward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                 const __nv_bfloat16* v, const __nv_bfloat16* dout, const int* iq, const int* ik,
                                 const uint8_t* hard, const int* boundary, const int2* documents, int hard_rows,
                                 const float* lut, int lut_stride, const float* lse2, int ctas, float* dsq,
                                 __nv_bfloat16* dsk, __nv_bfloat16* dv, float* dtau, void* workspace,
                                 const void* readout_workspace, cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = cudaSuccess;
    // the forward's workspace starts with the same two-sided index (keys first): reuse it when the caller kept it
    void* index = const_cast<void*>(readout_workspace);
    if (!index) {
        index = workspace;
        status = launch_build_index_pair(ik, iq, batch_heads, shape.n, workspace, stream);
        if (status != cudaSuccess) return status;
    }
    const SideIndex keys = side_index(index, batch_heads, shape.n, 0, 2), queries = side_index(index, batch_heads, shape.n, 1, 2);
    char* cursor = static_cast<char*>(workspace) + index_bytes(batch_heads, shape.n, 2);
    const int capacity = tile_capacity_for(shape.n);
    int4* tiles[2];
    int* tile_starts[2];
    for (int pass = 0; pass < 2; ++pass) {
        tiles[pass] = reinterpret_cast<int4*>(cursor);
        tile_starts[pass] = reinterpret_cast<int*>(tiles[pass] + size_t(batch_heads) * capacity);
        cursor += plan_bytes(batch_heads, shape.n);
    }
    float* rows = reinterpret_cast<float*>(cursor);
    float* dlut = rows + size_t(batch_heads) * shape.n;
    int* route = reinterpret_cast<int*>(dlut + size_t(shape.heads) * lut_stride);
    int* lines = reinterpret_cast<int*>(cursor + tables_bytes(shape.batch, shape.heads, shape.n, lut_stride));
    // dense labels: the same rule as the forward (a tenth of all pairs matching)
    const bool dense_allowed = shape.n % DENSE_COLUMNS == 0 && (documents || lut_stride > shape.n);  // (a pack's table length is checked by the caller)
    {
        KernelTimer timer("plan_tiles", stream);
        const TilePlan by_query{queries.starts, keys.starts, tile_starts[0], tiles[0], tile_starts[0] + size_t(batch_heads) * (BUCKETS + 1)};
        const TilePlan by_key{keys.starts, queries.starts, tile_starts[1], tiles[1], tile_starts[1] + size_t(batch_heads) * (BUCKETS + 1)};
        prepare_backward_kernel<<<dim3(batch_heads, 3), 1024, 0, stream>>>(by_query, by_key, capacity, route,
                                                                           dense_allowed ? (unsigned long long)(shape.n) * shape.n / DENSE_SHARE : ~0ull,
                                                                           lut, dlut, shape.heads, lut_stride, route_word());
    }
    BackwardBlockArgs args{};
    args.sq = sq; args.sk = sk; args.v = v; args.dout = dout;
    args.iq = iq; args.ik = ik; args.boundary = boundary; args.hard = hard;
    args.documents = documents; args.hard_rows = hard_rows;
    args.lut = lut; args.dlut = dlut; args.lse2 = lse2;
    args.dsq = dsq; args.dtau_rows = rows; args.dsk = dsk; args.dv = dv;
    args.batch = shape.batch; args.heads = shape.heads; args.n = shape.n; args.lut_stride = lut_stride;
    args.tile_capacity = capacity;
    BackwardBlockArgs by_query = args, by_key = args;
    by_query.owners = queries; by_query.partners = keys;
    by_query.tiles = tiles[0]; by_query.tile_starts = tile_starts[0];
    by_query.next_tile = tile_starts[0] + size_t(batch_heads) * (BUCKETS + 1);
    by_key.owners = keys; by_key.partners = queries;
    by_key.tiles = tiles[1]; by_key.tile_starts = tile_starts[1];
    by_key.next_tile = tile_starts[1] + size_t(batch_heads) * (BUCKETS + 1);
    DenseBackwardArgs dense{};
    dense.sq = sq; dense.sk = sk; dense.v = v; dense.dout = dout; dense.iq = iq; dense.ik = ik; dense.hard = hard; dense.documents = documents; dense.hard_rows = hard_rows;
    dense.lut = lut; dense.dlut = dlut; dense.lse2 = lse2; dense.route = route; dense.lines = lines;
    dense.dsq = dsq; dense.dtau_rows = rows; dense.dsk = dsk; dense.dv = dv;
    dense.batch = shape.batch; dense.heads = shape.heads; dense.n = shape.n; dense.lut_stride = lut_stride;
    dense.chunks = dense_chunks(batch_heads, shape.n);
    dense.choice = route_word();
    status = cudaErrorInvalidValue;
#define DISM_CASE(RR, VV)                                                                         \
    if (shape.r == RR && shape.dv == VV) {                                                        \
        status = launch_backward_blocks<RR, VV>(by_query, by_key, ctas, stream);                  \
        if (status == cudaSuccess && dense_allowed) status = launch_dense_backward<RR, VV>(dense, stream); \
    }
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    if (status != cudaSuccess) return status;
    KernelTimer timer("tau_reduce", stream);
    tau_reduce_kernel<<<shape.heads, 1024, 0, stream>>>(rows, dtau, shape.batch, shape.heads, shape.n, route_word());
    return cudaGetLastError();
}

}  // namespace dism
