// Hard forward: log-weight table and the fused match / normalise / signed-readout kernel.
//
// Replaces, behind the C ABI, the reference's hard_log_weights_kernel and hard_forward_kernel
// (dism_v3/src/hard_forward.cu:9-118, dism_v3/include/forward/readout.cuh:16-100).  The design is
// not a translation: the table entry of length 0 is -1e6, whose weight flushes to exactly 0, so
// only pairs with equal labels contribute.  Both sides are sorted by (label bucket, position); a
// warp takes sixteen queries of one bucket, walks the bucket's keys sixteen at a time and
// accumulates them in ascending key order with the online max / unit-fallback normalisation of
// the reference (maximum starts at 0, denominator at 1).  A row is reduced by one warp in a fixed
// order, so outputs do not depend on the grid size.  This file holds the table kernel, the
// workspace layout and the launches; the tile kernel is in hard_forward_blocks.cuh, the kernel
// that takes the slices with dense labels in hard_forward_dense.cuh.
#include "hard_forward_dense.cuh"

namespace dism {

__global__ void log_weights_kernel(const float* __restrict__ tau, float* __restrict__ out, int stride, const unsigned* choice) {
    if (!route_open(choice)) return;
    int length = blockIdx.x * blockDim.x + threadIdx.x;
    if (length >= stride) return;
    float t = tau[blockIdx.y], result = LOG_ZERO;
    if (length > 0) {
        if (t == 0.f) result = log2f(float(length));
        else {
            float a = fabsf(t);
            result = (t > 0.f ? float(length) * t : t) * 1.4426950408889634f +
                     log2f(-expm1f(-float(length) * a)) - log2f(-expm1f(-a));
        }
    }
    out[int64_t(blockIdx.y) * stride + length] = result;
}

cudaError_t launch_log_weights(const float* tau, int heads, int n, float* lut, cudaStream_t stream) {
    KernelTimer timer("log_weights", stream);
    log_weights_kernel<<<dim3((n + 256) / 256, heads), 256, 0, stream>>>(tau, lut, n + 1, route_word());
    return cudaGetLastError();
}

int device_sm_count() {
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    return sms;
}

// Workspace: both position indices, the tile descriptors [BH, N/16 + BUCKETS] (16-byte records), the
// first-tile table [BH, BUCKETS + 1], one tile counter and one route word per (batch, head), and the
// run-length rows of the dense route.
static size_t plan_words_bytes(size_t batch_heads) { return (batch_heads * (BUCKETS + 3) * sizeof(int) + 15) & ~size_t(15); }
size_t hard_forward_workspace_bytes(int batch, int heads, int n) {
    const size_t batch_heads = size_t(batch) * heads;
    return index_bytes(batch * heads, n, 2) + batch_heads * tile_capacity_for(n) * sizeof(int4) +
           plan_words_bytes(batch_heads) + dense_bytes(batch * heads, n);
}

// One cooperative launch of one CTA per SM (the kernel's shared memory allows no second one): see dense_route.cuh.
template <int R, int DV>
static cudaError_t launch_dense(const DenseArgs& args, cudaStream_t stream) {
    auto kernel = hard_forward_dense_kernel<R, DV>;
    const int shared = sizeof(DenseWarpShared<R, DV>) * DENSE_WARPS;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    KernelTimer timer("hard_forward_dense", stream);
    void* parameters[] = {const_cast<DenseArgs*>(&args)};
    return cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(kernel), dim3(device_sm_count()), dim3(DENSE_WARPS * 32), parameters,
                                       shared, stream);
}

template <bool PACKED, int R, int DV>
static cudaError_t launch_blocks_layout(const BlockArgs& args, int ctas, cudaStream_t stream) {
    auto kernel = hard_forward_blocks_kernel<PACKED, R, DV>;
    const int shared = sizeof(BlockWarpShared<R, DV>) * BLOCK_WARPS;
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (status != cudaSuccess) return status;
    const int batch_heads = args.batch * args.heads;
    // about eight full tiles per warp (partial tiles of small buckets come on top), and with few (batch, head) slices at
    // least four CTAs per SM over the whole grid: warps take tiles from a counter, so any grid covers the work;
    // `ctas` caps the whole grid
    int per_head = args.n / (QT * BLOCK_WARPS * 8);
    const int fill = (4 * device_sm_count() + batch_heads - 1) / batch_heads;
    if (per_head < fill) per_head = fill;
    if (per_head > (args.n + QT * BLOCK_WARPS - 1) / (QT * BLOCK_WARPS)) per_head = (args.n + QT * BLOCK_WARPS - 1) / (QT * BLOCK_WARPS);
    if (per_head < 1) per_head = 1;
    if (ctas) per_head = ctas / batch_heads > 0 ? ctas / batch_heads : 1;
    KernelTimer timer("hard_forward", stream);
    kernel<<<dim3(batch_heads, per_head), BLOCK_WARPS * 32, shared, stream>>>(args);
    return cudaGetLastError();
}

template <int R, int DV>
static cudaError_t launch_blocks_variant(const BlockArgs& args, int ctas, cudaStream_t stream) {
    return args.documents ? launch_blocks_layout<true, R, DV>(args, ctas, stream) : launch_blocks_layout<false, R, DV>(args, ctas, stream);
}

cudaError_t launch_hard_forward(HardShape shape, const __nv_bfloat16* sq, const __nv_bfloat16* sk,
                                const __nv_bfloat16* v, const int* iq, const int* ik, const uint8_t* hard,
                                const int* boundary, const int2* documents, int hard_rows, const float* lut,
                                int lut_stride, int ctas, __nv_bfloat16* out, float* lse2, void* workspace,
                                cudaStream_t stream) {
    const int batch_heads = shape.batch * shape.heads;
    cudaError_t status = launch_build_index_pair(ik, iq, batch_heads, shape.n, workspace, stream);
    if (status != cudaSuccess) return status;
    BlockArgs args{};
    args.sq = sq; args.sk = sk; args.v = v;
    args.iq = iq; args.ik = ik; args.boundary = boundary; args.hard = hard;
    args.documents = documents; args.hard_rows = hard_rows;
    args.lut = lut;
    args.keys = side_index(workspace, batch_heads, shape.n, 0, 2);
    args.queries = side_index(workspace, batch_heads, shape.n, 1, 2);
    int4* tiles = reinterpret_cast<int4*>(static_cast<char*>(workspace) + index_bytes(batch_heads, shape.n, 2));
    args.tile_capacity = tile_capacity_for(shape.n);
    int* tile_starts = reinterpret_cast<int*>(tiles + size_t(batch_heads) * args.tile_capacity);
    args.tiles = tiles;
    args.tile_starts = tile_starts;
    args.next_tile = tile_starts + size_t(batch_heads) * (BUCKETS + 1);
    args.out = out; args.lse2 = lse2;
    args.batch = shape.batch; args.heads = shape.heads; args.n = shape.n; args.lut_stride = lut_stride;
    args.choice = route_word();
    // The dense route takes sequences whose length its 32-column steps divide (packed or not); a (batch, head) goes
    // there when at least a tenth of all N^2 pairs have equal labels.
    int* route = args.next_tile + batch_heads;
    const bool dense_allowed = shape.n % DENSE_COLUMNS == 0 && (documents || lut_stride > shape.n);  // (a pack's table length is checked by the caller)
    {
        KernelTimer timer("plan_query_tiles", stream);
        plan_query_tiles_kernel<<<batch_heads, 1024, 0, stream>>>(args.queries.starts, args.keys.starts, tile_starts, tiles,
                                                                  args.next_tile, args.tile_capacity, route,
                                                                  dense_allowed ? (unsigned long long)(shape.n) * shape.n / DENSE_SHARE : ~0ull,
                                                                  route_word());
    }
    DenseArgs dense{};
    dense.sq = sq; dense.sk = sk; dense.v = v; dense.iq = iq; dense.ik = ik; dense.hard = hard; dense.documents = documents; dense.hard_rows = hard_rows; dense.lut = lut;
    dense.route = route;
    dense.rows = reinterpret_cast<int*>(reinterpret_cast<char*>(tile_starts) + plan_words_bytes(batch_heads));
    dense.out = out; dense.lse2 = lse2;
    dense.batch = shape.batch; dense.heads = shape.heads; dense.n = shape.n; dense.lut_stride = lut_stride;
    dense.chunks = dense_chunks(batch_heads, shape.n);
    dense.choice = route_word();
    cudaError_t status_blocks = cudaErrorInvalidValue;
#define DISM_CASE(RR, VV)                                                                   \
    if (shape.r == RR && shape.dv == VV) {                                                  \
        status_blocks = launch_blocks_variant<RR, VV>(args, ctas, stream);                  \
        if (status_blocks == cudaSuccess && dense_allowed) status_blocks = launch_dense<RR, VV>(dense, stream); \
    }
    DISM_CASE(16, 32) DISM_CASE(16, 64) DISM_CASE(16, 128)
    DISM_CASE(32, 32) DISM_CASE(32, 64) DISM_CASE(32, 128)
#undef DISM_CASE
    return status_blocks;
}

}  // namespace dism
