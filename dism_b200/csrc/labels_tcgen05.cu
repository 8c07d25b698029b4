// Discretiser on the fifth-generation tensor cores: arg-max symbol of x . E^T per head.
//
// Same contract as the general kernel in labels.cu (reference: dism_v3/python/flash_dism/emb_kernel.py:88-108,
// kernels/interp_true.py:25-33) for the shapes the tensor-memory pipeline covers: D of 64 or 128,
// a codebook of a multiple of 256 codes that fits in 128 KiB, N a multiple of 128.
//
// One persistent CTA per SM walks a contiguous range of (head, 128-row tile) pairs:
//   producer warp   TMA: the head's whole codebook once (128-byte swizzled, K-major), then one
//                   128 x D tile of x per step into a ring;
//   MMA warp        one elected lane issues tcgen05.mma (M=128, N=256, K=16) for each 256-code slice of
//                   the codebook into one of two FP32 accumulators: all of tensor memory;
//   norm warp       largest squared code norm of the head (the margin below scales with it);
//   two finishing   put the column ranges of a row together: label, pair list or crowded list;
//   warps
//   sixteen         read the accumulators with tcgen05.ld (row = tensor-memory lane = thread; a warp
//   epilogue warps  owns 32 rows and a quarter of the columns of every accumulator) and keep, per row,
//                   the largest logit and the columns of all logits within a safety margin of it; a tile
//                   ahead, each of their threads also sums a quarter of a row's squares (the margin
//                   scales with the row norm too).
//
// The epilogue is the instruction bound of the kernel, and min/max/logic instructions issue at half
// the FMA rate.  So the half-rate pipe only finds the maximum of each 32-column chunk (three-input
// max: half an instruction per logit); the full-rate pipe marks the logits above the threshold with
// a saturating FMA, g = sat((s - t) * gain), and a packed FMA shifts two g at a time into bit masks.
// gain is a power of two chosen from the exponent of t so that g is exactly 0 or 1 for every float s.
// The masks are folded into the row's candidates once per 64 columns.
//
// Labels are defined by the pinned FP32 order (d ascending, one rounding per add).  delta is a
// rigorous bound on how far the tensor-core order can move the difference of two logits, so only
// columns within delta of the row's largest logit can win in the pinned order.  One such column:
// it is the label.  Two (a near tie): the two pinned logits are computed by one thread after the
// CTA's last tile.  More: a whole warp recomputes the row in the pinned order.
//
// Every wait on an mbarrier is bounded: when one runs out the CTA records a fault code, all roles
// leave their loops, tensor memory is freed and the kernel returns.
#include <cuda.h>

#include "dism_common.cuh"

namespace dism {
namespace {

constexpr int TILE_ROWS = 128;   // rows of x per tile: the 128 lanes of tensor memory
constexpr int TILE_CODES = 256;  // codes per accumulator: 256 FP32 columns, the widest single instruction
constexpr int KBLOCK = 64;       // elements in one 128-byte swizzled row
constexpr int BLOCK_BYTES = TILE_ROWS * 128;        // 128 rows of x, 64 elements each
constexpr int CODE_BLOCK_BYTES = TILE_CODES * 128;  // 256 codes, 64 elements each
constexpr int ACC_STAGES = 2;    // two accumulators: all 512 columns of tensor memory
constexpr int MAX_A_STAGES = 4;
constexpr int NORM_RING = 4;     // norms are prepared one tile ahead; warps are never more than one tile apart
constexpr int EPILOGUE_WARPS = 16, EPILOGUE_GROUPS = 4, PRODUCER_WARP = 16, MMA_WARP = 17, NORM_WARP = 18;
constexpr int FINISH_WARP = 19, FINISH_WARPS = 2, THREADS = (FINISH_WARP + FINISH_WARPS) * 32;
constexpr int LIST_CAPACITY = 128;  // per quarter of the rows and list
constexpr unsigned WAIT_LIMIT = 1u << 16, SETTLE_LIMIT = 1u << 14, PARK_NANOSECONDS = 20000;  // a wait gives up after about a second at most
constexpr int MAX_CODE_BYTES = 128 * 1024;

// Columns that can still win a row: none yet (count 0), a, a and b, or too many to list (count 3).
struct Candidates {
    float first;  // largest logit seen
    int a, b, count;
};

struct Control {
    uint64_t code_full, code_empty, drain, list_ready;
    uint64_t a_full[MAX_A_STAGES], a_empty[MAX_A_STAGES], norm_done[NORM_RING];
    uint64_t acc_full[ACC_STAGES], acc_empty[ACC_STAGES];
    uint64_t exchange_full[2], exchange_empty[2];
    Candidates exchange[2][EPILOGUE_GROUPS][TILE_ROWS];
    float norm2[NORM_RING][TILE_ROWS];  // squared row norms of the tile of a step, ring over steps
    float code_max[2 * NORM_RING];      // largest squared code norm of that tile's head; the norm warp may be five steps ahead
    int pairs[4][LIST_CAPACITY][3];  // near ties: row id and the two columns
    int crowded[4][LIST_CAPACITY];   // rows with more than two columns in reach
    int pair_count[4], crowded_count[4];
    uint32_t tensor_memory;
    int abort;
};

__device__ int labels_fault_code;  // first bounded wait that ran out (0: none)

__device__ __forceinline__ uint32_t shared_address(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void barrier_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(bar)), "r"(count));
}
__device__ __forceinline__ void barrier_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(shared_address(bar)) : "memory");
}
__device__ __forceinline__ void barrier_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool barrier_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
                 : "=r"(done) : "r"(shared_address(bar)), "r"(parity) : "memory");
    return done != 0;
}
// The same test, but the hardware may park the thread for up to `nanoseconds` while the phase is open.
__device__ __forceinline__ bool barrier_test_parked(uint64_t* bar, uint32_t parity, uint32_t nanoseconds) {
    uint32_t done;
    asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p;}"
                 : "=r"(done) : "r"(shared_address(bar)), "r"(parity), "r"(nanoseconds) : "memory");
    return done != 0;
}
// Bounded wait.  False: this wait ran out (fault `code` recorded) or another role already gave up.
__device__ __noinline__ bool barrier_wait_slow(uint64_t* bar, uint32_t parity, Control& control, int code) {
    for (unsigned tries = 0; tries < WAIT_LIMIT; ++tries) {
        if (barrier_test_parked(bar, parity, PARK_NANOSECONDS)) return true;
        if (*reinterpret_cast<volatile int*>(&control.abort)) return false;
        if (tries >= 4) __nanosleep(tries < 64 ? 40 : 200);  // a waiting warp must not eat the issue slots of working ones
    }
    *reinterpret_cast<volatile int*>(&control.abort) = 1;
    atomicCAS(&labels_fault_code, 0, code);
    return false;
}
__device__ __forceinline__ bool barrier_wait(uint64_t* bar, uint32_t parity, Control& control, int code) {
    return barrier_test(bar, parity) || barrier_wait_slow(bar, parity, control, code);
}
// The same for the warp that feeds the tensor core: it is on the critical path of every accumulator and
// polls without sleeping.
__device__ __noinline__ bool barrier_wait_eager(uint64_t* bar, uint32_t parity, Control& control, int code) {
    for (unsigned tries = 0; tries < WAIT_LIMIT * 64; ++tries) {
        if (barrier_test(bar, parity)) return true;
        if ((tries & 255) == 255 && *reinterpret_cast<volatile int*>(&control.abort)) return false;
    }
    *reinterpret_cast<volatile int*>(&control.abort) = 1;
    atomicCAS(&labels_fault_code, 0, code);
    return false;
}
// One lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t elected;
    asm volatile("{.reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p;}" : "=r"(elected));
    return elected != 0;
}
// After a fault: give copies or products in flight a bounded time to land before the CTA leaves.
__device__ __noinline__ void barrier_settle(uint64_t* bar, uint32_t parity) {
    for (unsigned tries = 0; tries < SETTLE_LIMIT; ++tries)
        if (barrier_test(bar, parity)) return;
}

__device__ __forceinline__ void tma_load(void* destination, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(shared_address(destination)), "l"(map), "r"(x), "r"(y), "r"(shared_address(bar)) : "memory");
}

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, eight-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t address) {
    return uint64_t((address & 0x3ffff) >> 4) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) | (uint64_t(1) << 46) |
           (uint64_t(2) << 61);
}
// bf16 x bf16 -> f32, both operands K-major, M = 128, N = 256
constexpr uint32_t INSTRUCTION = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(TILE_CODES >> 3) << 17) | (uint32_t(TILE_ROWS >> 4) << 24);

__device__ __forceinline__ void mma(uint32_t accumulator, uint64_t a, uint64_t b, uint32_t accumulate) {
    asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;}"
                 ::"r"(accumulator), "l"(a), "l"(b), "r"(INSTRUCTION), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(shared_address(bar)) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive FP32 columns of this thread's tensor-memory lane.  The destinations are float registers:
// a bit-cast from integer registers after an asynchronous load costs a move per value.
__device__ __forceinline__ void load_columns(float (&r)[32], uint32_t address) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
                 : "r"(address));
}
__device__ __forceinline__ void wait_columns() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float fma_saturate(float a, float b, float c) {
    float d;
    asm("fma.rn.sat.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Largest of 32 logits: sixteen three-input max instructions.
__device__ __forceinline__ float chunk_max(const float (&r)[32]) {
    float m0 = max3(r[0], r[1], r[2]);
    float m1 = max3(r[3], r[4], r[5]);
#pragma unroll
    for (int i = 6; i < 30; i += 4) {
        m0 = max3(m0, r[i], r[i + 1]);
        m1 = max3(m1, r[i + 2], r[i + 3]);
    }
    return fmaxf(max3(m0, r[30], r[31]), m1);
}

// Bit i set: logit i of the chunk is above the threshold.  (s - t) * gain saturates to exactly 1
// or 0 (see make_threshold), so the two sums are exact 16-bit integers.  They are built high bit
// first, acc = 2 acc + g, for columns i and 16 + i at once with the packed FP32 FMA: half the
// instructions of two scalar chains.
__device__ __forceinline__ unsigned chunk_mask(const float (&r)[32], float gain, float offset) {
    unsigned long long acc, two;
    asm("mov.b64 %0, {%1, %1};" : "=l"(two) : "f"(2.f));
    asm("mov.b64 %0, {%1, %1};" : "=l"(acc) : "f"(0.f));
#pragma unroll
    for (int i = 15; i >= 0; --i) {
        unsigned long long g;
        asm("mov.b64 %0, {%1, %2};" : "=l"(g) : "f"(fma_saturate(r[i], gain, offset)), "f"(fma_saturate(r[16 + i], gain, offset)));
        asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc) : "l"(two), "l"(g));
    }
    float low, high;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(low), "=f"(high) : "l"(acc));
    return unsigned(low) | (unsigned(high) << 16);
}

// Threshold for a chunk: t = best - delta, where best is the largest logit of the row so far; a logit
// at or below t cannot win the row.  gain = 2^(27 - exponent of t), so (s - t) * gain is at least 8
// for every float s > t (two distinct floats near t differ by at least 2^-24 |t|) and at most 0 for
// s <= t; the product with a power of two is exact.  Not valid: |t| below 2^-100 or not finite.
struct Threshold {
    float gain, offset;
    bool valid;
};
__device__ __forceinline__ Threshold make_threshold(float best, float delta) {
    const float threshold = best - delta;
    const unsigned exponent = __float_as_uint(threshold) & 0x7f800000u;
    Threshold t;
    t.valid = exponent - (27u << 23) < (228u << 23);  // biased exponent in [27, 255)
    t.gain = __uint_as_float((281u << 23) - exponent);
    t.offset = -threshold * t.gain;
    return t;
}

// Folds one accumulator half (columns base .. base+63: chunk maxima and masks) into the row's
// candidates.  Each mask was taken against the best logit known at the time, which is at most the
// best now, so it holds every column of its chunk within delta of the best now, and possibly more.
// A chunk whose threshold was not valid carries a full mask and makes the row crowded if it matters.
__device__ __forceinline__ void fold_product(Candidates& row, float top0, unsigned mask0, float top1, unsigned mask1, float best,
                                             int base, float delta) {
    const float reach = best - delta;
    const unsigned m0 = top0 >= reach ? mask0 : 0u, m1 = top1 >= reach ? mask1 : 0u;
    const int kept = row.first >= reach ? row.count : 0;  // a leader out of reach takes its columns with it
    const int inside = __popc(m0) + __popc(m1);
    const int lowest = base + (m0 ? __ffs(m0) - 1 : 31 + __ffs(m1));
    const int highest = base + (m1 ? 63 - __clz(m1) : 31 - __clz(m0));
    row.b = (inside >= 1 && kept == 1) ? lowest : ((inside == 2 && kept == 0) ? highest : row.b);
    row.a = (inside >= 1 && kept == 0) ? lowest : row.a;
    row.count = min(kept + inside, 3);
    row.first = best;
}

// |tensor-core logit - exact| <= 4 D u sum|x e| (sixteen-term blocks whose addends may be truncated),
// |pinned logit - exact| <= D u sum|x e|, u = 2^-24, and sum|x e| <= |x|_2 |e|_2.  Two logits
// further apart than delta = 2 * 5 D u |x|_2 |e|_2 (with a little slack) keep their order.
template <int D>
__device__ __forceinline__ float margin(float row_norm2, float code_norm2) {
    return 2.f * float(5 * D) * 5.9604645e-8f * sqrtf(row_norm2 * code_norm2) * 1.02f + 1e-37f;
}

// Adds the candidates of another column range of the same row.
__device__ __forceinline__ void merge_candidates(Candidates& row, const Candidates other, float best, float delta) {
    if (!(other.first >= best - delta) || other.count == 0) return;  // everything there is out of reach
    if (other.count == 3 || row.count + other.count > 2) { row.count = 3; return; }
    if (row.count == 0) row.a = other.a; else row.b = other.a;
    if (other.count == 2) row.b = other.b;
    row.count += other.count;
}

__device__ __forceinline__ float squares(uint4 raw, float sum) {
    const unsigned word[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const float low = __uint_as_float(word[w] << 16), high = __uint_as_float(word[w] & 0xffff0000u);
        sum = fmaf(low, low, fmaf(high, high, sum));
    }
    return sum;
}

// Squared norm of one 128-byte-swizzled operand row in shared memory (the swizzle permutes the
// 16-byte pieces inside the row, which a sum of squares does not see).  Lanes start at different
// pieces so that a warp reading 32 consecutive rows meets no bank conflict.
template <int D, int KBLOCK_BYTES>
__device__ __forceinline__ float shared_row_squares(const unsigned char* tile, int row, int lane) {
    float sum = 0.f;
#pragma unroll
    for (int kb = 0; kb < D / KBLOCK; ++kb)
#pragma unroll
        for (int c = 0; c < 8; ++c)
            sum = squares(*reinterpret_cast<const uint4*>(tile + kb * KBLOCK_BYTES + row * 128 + ((c + lane) & 7) * 16), sum);
    return sum;
}

// Pinned-order arg-max of one row by a whole warp; every lane returns the label.  A lane works on
// four codes at a time, because the additions of one code form a serial chain.
template <int D>
__device__ __noinline__ int pinned_label(const __nv_bfloat16* __restrict__ row, const __nv_bfloat16* __restrict__ codes, int vocab, int lane) {
    float top = -INFINITY;
    int arg = 0x7fffffff;
    for (int v0 = lane; v0 < vocab; v0 += 128) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < D / 8; ++c) {
            const uint4 packed = __ldg(reinterpret_cast<const uint4*>(row) + c);
            const unsigned xs[4] = {packed.x, packed.y, packed.z, packed.w};
            unsigned es[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const uint4 e = __ldg(reinterpret_cast<const uint4*>(codes + int64_t(min(v0 + 32 * u, vocab - 1)) * D) + c);
                es[u][0] = e.x, es[u][1] = e.y, es[u][2] = e.z, es[u][3] = e.w;
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    acc[u] = __fadd_rn(acc[u], __fmul_rn(__uint_as_float(xs[w] << 16), __uint_as_float(es[u][w] << 16)));
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    acc[u] = __fadd_rn(acc[u], __fmul_rn(__uint_as_float(xs[w] & 0xffff0000u), __uint_as_float(es[u][w] & 0xffff0000u)));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u)  // ascending v per lane: the first maximum is kept
            if (v0 + 32 * u < vocab && acc[u] > top) { top = acc[u]; arg = v0 + 32 * u; }
    }
#pragma unroll
    for (int s = 16; s; s >>= 1) {
        const float other = __shfl_xor_sync(FULL, top, s);
        const int other_arg = __shfl_xor_sync(FULL, arg, s);
        if (other > top || (other == top && other_arg < arg)) { top = other; arg = other_arg; }
    }
    return arg;
}

// Pinned-order logit of one row against one code, by one thread.
template <int D>
__device__ __noinline__ float pinned_logit(const __nv_bfloat16* __restrict__ row, const __nv_bfloat16* __restrict__ code) {
    float acc = 0.f;
#pragma unroll
    for (int c = 0; c < D / 8; ++c) {
        const uint4 xs = __ldg(reinterpret_cast<const uint4*>(row) + c), es = __ldg(reinterpret_cast<const uint4*>(code) + c);
        const unsigned xw[4] = {xs.x, xs.y, xs.z, xs.w}, ew[4] = {es.x, es.y, es.z, es.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            acc = __fadd_rn(acc, __fmul_rn(__uint_as_float(xw[w] << 16), __uint_as_float(ew[w] << 16)));
            acc = __fadd_rn(acc, __fmul_rn(__uint_as_float(xw[w] & 0xffff0000u), __uint_as_float(ew[w] & 0xffff0000u)));
        }
    }
    return acc;
}

// The tensors of one launch: one (x, codebook, labels) triple, or two of the same shape (the q and the k side of a
// step), which then share one pipeline fill and drain.  Tiles are numbered side by side: `heads` heads of the first
// triple, then those of the second; a "virtual head" below is that running number.
struct LabelSides {
    const __nv_bfloat16* x[2];
    const __nv_bfloat16* codebook[2];
    int* labels[2];
};

template <int D>
__global__ __launch_bounds__(THREADS, 1) void labels_tcgen05_kernel(const __grid_constant__ CUtensorMap x_map0,
                                                                    const __grid_constant__ CUtensorMap code_map0,
                                                                    const __grid_constant__ CUtensorMap x_map1,
                                                                    const __grid_constant__ CUtensorMap code_map1,
                                                                    const LabelSides sides, int n, int heads,
                                                                    int vocab, int tiles_per_head, int total_tiles) {
    constexpr int KBLOCKS = D / KBLOCK, A_BYTES = KBLOCKS * BLOCK_BYTES, A_STAGES = D == 64 ? 4 : 2;
    extern __shared__ unsigned char raw[];
    unsigned char* base = raw + ((1024u - (shared_address(raw) & 1023u)) & 1023u);  // swizzled tiles: 1024-byte aligned
    const int code_tiles = vocab / TILE_CODES;
    unsigned char* codes = base;
    unsigned char* a_ring = codes + code_tiles * KBLOCKS * CODE_BLOCK_BYTES;
    Control& control = *reinterpret_cast<Control*>(a_ring + A_STAGES * A_BYTES);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first_tile = int(int64_t(blockIdx.x) * total_tiles / gridDim.x);
    const int last_tile = int(int64_t(blockIdx.x + 1) * total_tiles / gridDim.x);

    if (threadIdx.x == 0) {
        barrier_init(&control.code_full, 1);
        barrier_init(&control.code_empty, 2);  // the tensor core and the norm warp
        barrier_init(&control.drain, 1);
        barrier_init(&control.list_ready, FINISH_WARPS);
        for (int s = 0; s < A_STAGES; ++s) {
            barrier_init(&control.a_full[s], 1);
            barrier_init(&control.a_empty[s], 2 + EPILOGUE_WARPS);  // tensor core, norm warp, the warps that measure the rows
        }
        for (int s = 0; s < NORM_RING; ++s) barrier_init(&control.norm_done[s], 1 + EPILOGUE_WARPS);
        for (int s = 0; s < ACC_STAGES; ++s) {
            barrier_init(&control.acc_full[s], 1);
            barrier_init(&control.acc_empty[s], EPILOGUE_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            barrier_init(&control.exchange_full[s], EPILOGUE_WARPS);
            barrier_init(&control.exchange_empty[s], FINISH_WARPS);
        }
        for (int s = 0; s < 4; ++s) control.pair_count[s] = control.crowded_count[s] = 0;
        control.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(shared_address(&control.tensor_memory)),
                     "r"(ACC_STAGES * TILE_CODES) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tensor_memory = *reinterpret_cast<volatile uint32_t*>(&control.tensor_memory);

    if (warp == PRODUCER_WARP) {
        if (lane == 0) {
            int loaded_head = -1, code_loads = 0, step = 0;
            for (int tile = first_tile; tile < last_tile; ++tile, ++step) {
                const int head = tile / tiles_per_head, row = (tile % tiles_per_head) * TILE_ROWS;  // virtual head
                const bool second = head >= heads;
                const int real_head = second ? head - heads : head;
                const CUtensorMap* x_map = second ? &x_map1 : &x_map0;
                const CUtensorMap* code_map = second ? &code_map1 : &code_map0;
                if (head != loaded_head) {
                    // the tensor core must have finished with the previous head's codes
                    if (code_loads > 0 && !barrier_wait(&control.code_empty, (code_loads - 1) & 1, control, 1)) break;
                    barrier_expect(&control.code_full, uint32_t(code_tiles * KBLOCKS * CODE_BLOCK_BYTES));
                    for (int j = 0; j < code_tiles; ++j)
                        for (int kb = 0; kb < KBLOCKS; ++kb)
                            tma_load(codes + (j * KBLOCKS + kb) * CODE_BLOCK_BYTES, code_map, kb * KBLOCK, real_head * vocab + j * TILE_CODES,
                                     &control.code_full);
                    loaded_head = head;
                    ++code_loads;
                }
                const int stage = step % A_STAGES;
                if (!barrier_wait(&control.a_empty[stage], ((step / A_STAGES) & 1) ^ 1, control, 2)) break;
                barrier_expect(&control.a_full[stage], uint32_t(A_BYTES));
                for (int kb = 0; kb < KBLOCKS; ++kb)
                    tma_load(a_ring + stage * A_BYTES + kb * BLOCK_BYTES, x_map, real_head * D + kb * KBLOCK, row, &control.a_full[stage]);
            }
            if (*reinterpret_cast<volatile int*>(&control.abort)) {  // let the copies in flight land
                if (code_loads > 0) barrier_settle(&control.code_full, (code_loads - 1) & 1);
                for (int back = 1; back <= A_STAGES && back <= step; ++back)
                    barrier_settle(&control.a_full[(step - back) % A_STAGES], ((step - back) / A_STAGES) & 1);
            }
        }
    } else if (warp == MMA_WARP) {
        // The whole warp walks the loop, so that addresses and descriptors live in uniform registers; one
        // elected lane issues the products and their commits.  Descriptors are built once, and a K step
        // only adds its byte offset (in 16-byte units).
        const uint64_t a_base = operand_descriptor(shared_address(a_ring)), b_base = operand_descriptor(shared_address(codes));
        int head = first_tile / tiles_per_head, tile_in_head = first_tile % tiles_per_head;
        int loaded_head = -1, code_uses = 0, step = 0, product = 0;
        bool ok = true;
        for (int tile = first_tile; tile < last_tile && ok; ++tile, ++step) {
            if (head != loaded_head) {
                ok = __all_sync(FULL, barrier_wait_eager(&control.code_full, code_uses & 1, control, 3));
                if (!ok) break;
                ++code_uses;
                loaded_head = head;
            }
            const int stage = step % A_STAGES;
            ok = __all_sync(FULL, barrier_wait_eager(&control.a_full[stage], (step / A_STAGES) & 1, control, 4));
            if (!ok) break;
            fence_after_sync();
            const uint64_t a_tile = a_base + uint64_t(stage * (A_BYTES >> 4));
            for (int j = 0; j < code_tiles; ++j, ++product) {
                const int slot = product % ACC_STAGES;
                ok = __all_sync(FULL, barrier_wait_eager(&control.acc_empty[slot], ((product / ACC_STAGES) & 1) ^ 1, control, 5));
                if (!ok) break;
                fence_after_sync();
                const uint64_t b_tile = b_base + uint64_t(j * (KBLOCKS * CODE_BLOCK_BYTES >> 4));
                if (elect_one()) {
#pragma unroll
                    for (int kb = 0; kb < KBLOCKS; ++kb)
#pragma unroll
                        for (int ks = 0; ks < KBLOCK / 16; ++ks)
                            mma(tensor_memory + slot * TILE_CODES, a_tile + uint64_t((kb * BLOCK_BYTES + ks * 32) >> 4),
                                b_tile + uint64_t((kb * CODE_BLOCK_BYTES + ks * 32) >> 4), (kb | ks) != 0);
                    mma_commit(&control.acc_full[slot]);
                }
                __syncwarp();
            }
            if (!ok) break;
            const bool last_of_head = tile_in_head + 1 == tiles_per_head;
            if (elect_one()) {
                mma_commit(&control.a_empty[stage]);
                if (tile + 1 < last_tile && last_of_head) mma_commit(&control.code_empty);
            }
            __syncwarp();
            if (last_of_head) { tile_in_head = 0; ++head; } else ++tile_in_head;
        }
        // every product issued above has completed once this commit arrives
        if (elect_one()) mma_commit(&control.drain);
        __syncwarp();
        barrier_settle(&control.drain, 0);
    } else if (warp == NORM_WARP) {
        int step = 0, loaded_head = -1, code_uses = 0;
        float code_max = 0.f;
        for (int tile = first_tile; tile < last_tile; ++tile, ++step) {
            const int stage = step % A_STAGES, head = tile / tiles_per_head;
            if (head != loaded_head) {  // largest squared code norm of the head
                if (!barrier_wait(&control.code_full, code_uses & 1, control, 11)) break;
                ++code_uses;
                code_max = 0.f;
                for (int v = lane; v < vocab; v += 32)
                    code_max = fmaxf(code_max, shared_row_squares<D, CODE_BLOCK_BYTES>(codes + (v / TILE_CODES) * KBLOCKS * CODE_BLOCK_BYTES, v % TILE_CODES, lane));
#pragma unroll
                for (int s = 16; s; s >>= 1) code_max = fmaxf(code_max, __shfl_xor_sync(FULL, code_max, s));
                __syncwarp();
                if (lane == 0) barrier_arrive(&control.code_empty);
                loaded_head = head;
            }
            // The landing of this step's tile paces this warp: by then every epilogue warp has read the slot's
            // previous value.  The stage may not be refilled before this warp has seen the landing (a waiter
            // that misses a whole phase of an mbarrier waits for the wrong one), hence the arrival below.
            if (!barrier_wait(&control.a_full[stage], (step / A_STAGES) & 1, control, 12)) break;
            if (lane == 0) {
                barrier_arrive(&control.a_empty[stage]);
                control.code_max[step % (2 * NORM_RING)] = code_max;
                barrier_arrive(&control.norm_done[step % NORM_RING]);
            }
        }
    } else if (warp >= FINISH_WARP) {
        // Two warps put the four column ranges of a row together, off the path that paces the accumulators:
        // one column in reach is the label; two go to the pair list; more, or no valid threshold, to the
        // crowded list.  Each warp owns two quarters of the rows and their lists.
        const int tiles_per_batch = n / TILE_ROWS;
        int head = first_tile / tiles_per_head, tile_in_batch = first_tile % tiles_per_head % tiles_per_batch;
        int batch = first_tile % tiles_per_head / tiles_per_batch, step = 0;
        bool ok = true;
        for (int tile = first_tile; tile < last_tile && ok; ++tile, ++step) {
            const int side = step & 1;
            ok = barrier_wait(&control.exchange_full[side], (step >> 1) & 1, control, 8);
            if (!ok) break;
            const float code_max = control.code_max[step % (2 * NORM_RING)];
            const int which = head >= heads, real_head = head - which * heads;
            const __nv_bfloat16* x = sides.x[which];
            int* labels = sides.labels[which];
            const __nv_bfloat16* head_codes = sides.codebook[which] + int64_t(real_head) * vocab * D;
#pragma unroll 1
            for (int quarter = (warp - FINISH_WARP) * 2; quarter < (warp - FINISH_WARP) * 2 + 2; ++quarter) {
                const int row_in_tile = quarter * 32 + lane, position = tile_in_batch * TILE_ROWS + row_in_tile;
                const float delta = margin<D>(control.norm2[step % NORM_RING][row_in_tile], code_max);
                const Candidates part[EPILOGUE_GROUPS] = {control.exchange[side][0][row_in_tile], control.exchange[side][1][row_in_tile],
                                                          control.exchange[side][2][row_in_tile], control.exchange[side][3][row_in_tile]};
                const float best = fmaxf(fmaxf(part[0].first, part[1].first), fmaxf(part[2].first, part[3].first));
                Candidates all{best, 0, 0, 0};
#pragma unroll
                for (int g = 0; g < EPILOGUE_GROUPS; ++g) merge_candidates(all, part[g], best, delta);
                if (all.count == 1) labels[(int64_t(batch) * heads + real_head) * n + position] = all.a;
                const int id = tile * TILE_ROWS + row_in_tile;
                // near ties go to the pair list while it has room, everything else to the crowded list
                unsigned pair_mask = __ballot_sync(FULL, all.count == 2);
                if (pair_mask) {
                    const int count = control.pair_count[quarter], more = __popc(pair_mask);
                    if (count + more <= LIST_CAPACITY) {
                        if (all.count == 2) {
                            int* entry = control.pairs[quarter][count + __popc(pair_mask & ((1u << lane) - 1))];
                            entry[0] = id, entry[1] = all.a, entry[2] = all.b;
                        }
                        __syncwarp();
                        if (lane == 0) control.pair_count[quarter] = count + more;
                        __syncwarp();
                        pair_mask = 0;
                    }
                }
                const bool crowded = all.count != 1 && (all.count != 2 || pair_mask != 0);
                const unsigned crowded_mask = __ballot_sync(FULL, crowded);
                if (crowded_mask) {
                    const int count = control.crowded_count[quarter], more = __popc(crowded_mask);
                    if (count + more <= LIST_CAPACITY) {
                        if (crowded) control.crowded[quarter][count + __popc(crowded_mask & ((1u << lane) - 1))] = id;
                        __syncwarp();
                        if (lane == 0) control.crowded_count[quarter] = count + more;
                        __syncwarp();
                    } else {  // list full: recompute here
                        for (unsigned rest = crowded_mask; rest; rest &= rest - 1) {
                            const int p = tile_in_batch * TILE_ROWS + quarter * 32 + __ffs(rest) - 1;
                            const int label = pinned_label<D>(x + ((int64_t(batch) * n + p) * heads + real_head) * D, head_codes, vocab, lane);
                            if (lane == 0) labels[(int64_t(batch) * heads + real_head) * n + p] = label;
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) barrier_arrive(&control.exchange_empty[side]);
            if (++tile_in_batch == tiles_per_batch) {
                tile_in_batch = 0;
                if (++batch == tiles_per_head / tiles_per_batch) { batch = 0; ++head; }
            }
        }
        if (ok) {
            __syncwarp();
            if (lane == 0) barrier_arrive(&control.list_ready);
        }
    } else {
        // Rows quarter*32 .. +31 of every tile; columns group*64 .. +63 of every accumulator.
        const int quarter = warp & 3, group = warp >> 2, row_in_tile = quarter * 32 + lane;
        const uint32_t lanes = tensor_memory + (uint32_t(quarter * 32) << 16) + group * (TILE_CODES / EPILOGUE_GROUPS);
        int step = 0, product = 0;
        bool ok = true;
        // Squared row norms of the tile of step t, shared by all epilogue threads: four threads per row,
        // each sums a quarter of the row's 16-byte pieces (which ones does not matter, so the swizzle is
        // ignored; the rotation by row keeps the warp's reads off each other's banks).
        auto measure_rows = [&](int t) -> bool {
            const int stage = t % A_STAGES;
            if (!barrier_wait(&control.a_full[stage], (t / A_STAGES) & 1, control, 10)) return false;
            const int r = (warp * 32 + lane) >> 2, part = lane & 3;
            const unsigned char* tile_rows = a_ring + stage * A_BYTES + r * 128;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int kb = 0; kb < KBLOCKS; ++kb) {
                sum0 = squares(*reinterpret_cast<const uint4*>(tile_rows + kb * BLOCK_BYTES + ((part * 2 + r) & 7) * 16), sum0);
                sum1 = squares(*reinterpret_cast<const uint4*>(tile_rows + kb * BLOCK_BYTES + ((part * 2 + 1 + r) & 7) * 16), sum1);
            }
            float sum = sum0 + sum1;
            sum += __shfl_xor_sync(FULL, sum, 1);
            sum += __shfl_xor_sync(FULL, sum, 2);
            if (part == 0) control.norm2[t % NORM_RING][r] = sum;
            __syncwarp();
            if (lane == 0) {
                barrier_arrive(&control.a_empty[stage]);
                barrier_arrive(&control.norm_done[t % NORM_RING]);
            }
            return true;
        };
        if (first_tile < last_tile) ok = measure_rows(0);
        for (int tile = first_tile; tile < last_tile && ok; ++tile, ++step) {
            if (tile + 1 < last_tile) {
                ok = measure_rows(step + 1);
                if (!ok) break;
            }
            ok = barrier_wait(&control.norm_done[step % NORM_RING], (step / NORM_RING) & 1, control, 13);
            if (!ok) break;
            const float norm2 = control.norm2[step % NORM_RING][row_in_tile], code_max = control.code_max[step % (2 * NORM_RING)];
            const float delta = margin<D>(norm2, code_max);
            Candidates mine{-INFINITY, 0, 0, 0};
            for (int j = 0; j < code_tiles; ++j, ++product) {
                const int slot = product % ACC_STAGES;
                ok = barrier_wait(&control.acc_full[slot], (product / ACC_STAGES) & 1, control, 6);
                if (!ok) break;
                fence_after_sync();
                const uint32_t address = lanes + slot * TILE_CODES;
                float r[32];
                load_columns(r, address);
                wait_columns();
                const float top0 = chunk_max(r), best0 = fmaxf(mine.first, top0);
                const Threshold t0 = make_threshold(best0, delta);
                const unsigned mask0 = t0.valid ? chunk_mask(r, t0.gain, t0.offset) : ~0u;
                load_columns(r, address + 32);
                wait_columns();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(&control.acc_empty[slot]);  // the logits are in registers
                const float top1 = chunk_max(r), best1 = fmaxf(best0, top1);
                const Threshold t1 = make_threshold(best1, delta);
                const unsigned mask1 = t1.valid ? chunk_mask(r, t1.gain, t1.offset) : ~0u;
                fold_product(mine, top0, mask0, top1, mask1, best1, j * TILE_CODES + group * (TILE_CODES / EPILOGUE_GROUPS), delta);
            }
            if (!ok) break;
            const int side = step & 1;
            ok = barrier_wait(&control.exchange_empty[side], ((step >> 1) & 1) ^ 1, control, 7);
            if (!ok) break;
            control.exchange[side][group][row_in_tile] = mine;
            __syncwarp();
            if (lane == 0) barrier_arrive(&control.exchange_full[side]);
        }
        // The lists: near ties one thread per row, crowded rows one warp per row, all epilogue warps.
        if (ok && barrier_wait(&control.list_ready, 0, control, 9)) {
            for (int list = 0; list < 4; ++list) {
                const int count = *reinterpret_cast<volatile int*>(&control.pair_count[list]);
                for (int entry = threadIdx.x; entry < count; entry += EPILOGUE_WARPS * 32) {
                    const int id = control.pairs[list][entry][0], a = control.pairs[list][entry][1], b = control.pairs[list][entry][2];
                    const int tile = id / TILE_ROWS, which = tile / tiles_per_head >= heads, head = tile / tiles_per_head - which * heads;
                    const int r = (tile % tiles_per_head) * TILE_ROWS + id % TILE_ROWS;
                    const __nv_bfloat16* source = sides.x[which] + (int64_t(r) * heads + head) * D;
                    const __nv_bfloat16* head_codes = sides.codebook[which] + int64_t(head) * vocab * D;
                    int* labels = sides.labels[which];
                    const float logit_a = pinned_logit<D>(source, head_codes + int64_t(a) * D);
                    const float logit_b = pinned_logit<D>(source, head_codes + int64_t(b) * D);
                    const bool first_wins = logit_a > logit_b || (logit_a == logit_b && a < b);
                    labels[(int64_t(r / n) * heads + head) * n + r % n] = first_wins ? a : b;
                }
            }
            int turn = 0;
            for (int list = 0; list < 4; ++list) {
                const int count = *reinterpret_cast<volatile int*>(&control.crowded_count[list]);
                for (int entry = 0; entry < count; ++entry, ++turn) {
                    if (turn % EPILOGUE_WARPS != warp) continue;
                    const int id = control.crowded[list][entry], tile = id / TILE_ROWS;
                    const int which = tile / tiles_per_head >= heads, head = tile / tiles_per_head - which * heads;
                    const int r = (tile % tiles_per_head) * TILE_ROWS + id % TILE_ROWS;
                    const int label = pinned_label<D>(sides.x[which] + (int64_t(r) * heads + head) * D,
                                                      sides.codebook[which] + int64_t(head) * vocab * D, vocab, lane);
                    if (lane == 0) sides.labels[which][(int64_t(r / n) * heads + head) * n + r % n] = label;
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tensor_memory), "r"(ACC_STAGES * TILE_CODES) : "memory");
    }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled entry = [] {
        void* address = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &address, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            address = nullptr;
        return reinterpret_cast<EncodeTiled>(address);
    }();
    return entry;
}

// bf16 matrix [rows, columns] (row stride in elements) read in boxes of 64 columns by box_rows rows, 128-byte swizzle
bool make_map(CUtensorMap* map, const void* data, uint64_t rows, uint64_t columns, uint64_t row_stride, int box_rows) {
    const EncodeTiled encode = encode_tiled();
    if (!encode) return false;
    const cuuint64_t dims[2] = {columns, rows}, strides[1] = {row_stride * 2};
    const cuuint32_t box[2] = {KBLOCK, cuuint32_t(box_rows)}, element_strides[2] = {1, 1};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(data), dims, strides, box, element_strides,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Dynamic shared memory of a CTA: the codebook, the ring of row tiles, the control block, alignment slack.
int shared_bytes(int d, int vocab) { return vocab * d * 2 + (d == 64 ? 4 : 2) * (d / KBLOCK) * BLOCK_BYTES + int(sizeof(Control)) + 1024; }
constexpr int SHARED_LIMIT = 227 * 1024;

template <int D>
cudaError_t launch(const CUtensorMap (&x_map)[2], const CUtensorMap (&code_map)[2], const LabelSides& sides, int n, int heads, int vocab,
                   int tiles_per_head, int total_tiles, cudaStream_t stream) {
    const int bytes = shared_bytes(D, vocab);
    const cudaError_t status = cudaFuncSetAttribute(labels_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (status != cudaSuccess) return status;
    const int grid = total_tiles < device_sm_count() ? total_tiles : device_sm_count();
    labels_tcgen05_kernel<D><<<grid, THREADS, bytes, stream>>>(x_map[0], code_map[0], x_map[1], code_map[1], sides, n, heads, vocab,
                                                               tiles_per_head, total_tiles);
    return cudaGetLastError();
}

}  // namespace

bool labels_tcgen05_covers(const void* x, const void* codebook, int batch, int n, int heads, int d, int vocab) {
    return (d == 64 || d == 128) && vocab % TILE_CODES == 0 && int64_t(vocab) * d * 2 <= MAX_CODE_BYTES && shared_bytes(d, vocab) <= SHARED_LIMIT && n % TILE_ROWS == 0 &&
           int64_t(batch) * n * heads < (int64_t(1) << 31) && reinterpret_cast<uintptr_t>(x) % 16 == 0 &&
           reinterpret_cast<uintptr_t>(codebook) % 16 == 0 && encode_tiled() != nullptr;
}

// One triple (x1 == nullptr) or two triples of the same shape in one launch.
cudaError_t launch_labels_tcgen05(const __nv_bfloat16* x, const __nv_bfloat16* codebook, int* labels, const __nv_bfloat16* x1,
                                  const __nv_bfloat16* codebook1, int* labels1, int batch, int n, int heads, int d, int vocab,
                                  cudaStream_t stream) {
    const int count = x1 ? 2 : 1;
    const LabelSides sides{{x, x1 ? x1 : x}, {codebook, x1 ? codebook1 : codebook}, {labels, x1 ? labels1 : labels}};
    CUtensorMap x_map[2], code_map[2];
    for (int side = 0; side < 2; ++side)
        if (!make_map(&x_map[side], sides.x[side], uint64_t(batch) * n, uint64_t(heads) * d, uint64_t(heads) * d, TILE_ROWS) ||
            !make_map(&code_map[side], sides.codebook[side], uint64_t(heads) * vocab, uint64_t(d), uint64_t(d), TILE_CODES))
            return cudaErrorInvalidValue;
    const int tiles_per_head = int(int64_t(batch) * n / TILE_ROWS), total_tiles = tiles_per_head * heads * count;
    KernelTimer timer(count == 2 ? "labels_pair" : "labels", stream);
    if (d == 64) return launch<64>(x_map, code_map, sides, n, heads, vocab, tiles_per_head, total_tiles, stream);
    return launch<128>(x_map, code_map, sides, n, heads, vocab, tiles_per_head, total_tiles, stream);
}

// First bounded wait that ran out in any earlier launch on this device (0: none).  Synchronises the device.
cudaError_t read_labels_fault(int* code) {
    const cudaError_t status = cudaMemcpyFromSymbol(code, labels_fault_code, sizeof(int));
    if (status != cudaSuccess) return status;
    const int none = 0;
    return cudaMemcpyToSymbol(labels_fault_code, &none, sizeof(int));  // read and clear
}

namespace {
// A wait that nothing ever satisfies, through the same bounded-wait code as the pipeline: two warps wait on
// one barrier; the first to run out records `code` and raises the flag that releases the other.
__global__ void wait_selftest_kernel(int code, int* outcome) {
    __shared__ Control control;
    if (threadIdx.x == 0) {
        barrier_init(&control.drain, 1);
        control.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool passed = barrier_wait(&control.drain, 0, control, code);
    if ((threadIdx.x & 31) == 0) outcome[threadIdx.x >> 5] = passed ? 1 : 0;
}
}  // namespace

// Runs the self-test on `stream` and waits for it.  outcome[0..1]: 1 if the wait of warp 0 / warp 1 came
// back satisfied (it must not).  The recorded fault code is read with read_labels_fault.
cudaError_t run_wait_selftest(int code, int* outcome, cudaStream_t stream) {
    int* device = nullptr;
    cudaError_t status = cudaMalloc(&device, 2 * sizeof(int));
    if (status != cudaSuccess) return status;
    const int unset[2] = {-1, -1};
    status = cudaMemcpyAsync(device, unset, sizeof(unset), cudaMemcpyHostToDevice, stream);
    if (status == cudaSuccess) {
        wait_selftest_kernel<<<1, 64, 0, stream>>>(code, device);
        status = cudaGetLastError();
    }
    if (status == cudaSuccess) status = cudaMemcpyAsync(outcome, device, 2 * sizeof(int), cudaMemcpyDeviceToHost, stream);
    if (status == cudaSuccess) status = cudaStreamSynchronize(stream);
    cudaFree(device);
    return status;
}

}  // namespace dism
