// Multi-sequence Q4_K dequant-GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
//     Y[m][row] = sum_e dequant(W)[row][e] * X[m][e],   m < M  (M <= 64 per launch)
// the batched contract of the reference's Linear::forward_batched (Y = X . W^T,
// crates/modgrad-device/src/backend/tensor.rs:1839-1853) for Q4_K weights; the reference has no
// kernel for it, so results are compared with M independent matvecs of its CPU path on the
// same f32 activations.
//
// Numerics.  Each sequence is scaled by the power of two that brings its largest magnitude into
// [2^9, 2^10) and split into TWO half-precision limbs, x ~= hi + 2^-11 * lo (22 significant
// bits; the error left is below 2^-22 of the sequence's largest magnitude per element).  tcgen05
// kind::f16 needs A and B in the same 16-bit format on this part, hence half for both.  The
// weight operand is not a rounded dequantised weight: per super-block
//     y = d * sum_sub sc_sub * sum_l q_l x_l  -  dmin * sum_sub m_sub * sum_l x_l ,
// so the tensor cores multiply the small integers sc*q (<= 945, exact in f16) by the half limbs
// (every product exact in f32) and accumulate in f32 in TMEM over one super-block; the per-row
// f16 factors d and dmin are applied on the CUDA cores when the accumulator is drained (once per
// 256 weights), where hi and lo columns are joined.  The second term is a 24-deep product of the
// integers m with three-limb half sums of x, on the tensor cores as well.
//
// One CTA per SM walks work items (128 output rows x a range of super-blocks); the pipeline runs
// across item boundaries.  Warps:
//   0      MMA issuer.  The whole warp walks the loop and waits on the barriers (the index
//          arithmetic then stays in the uniform datapath); one elected lane issues tcgen05.mma (A, B
//          from shared memory through matrix descriptors, D in TMEM, two accumulator sets so that
//          block b+1 multiplies while b drains) and tcgen05.commit onto mbarriers.  A 16-deep step
//          of 128 rows takes the tensor pipe ~55 cycles whatever N <= 128 is, so the pipe's own
//          floor is ~1000 cycles per super-block.  One issuer only: with a second issuing warp
//          (one per accumulator set) results were corrupted at N = 128.
//   1      one thread issues the raw-weight TMA loads: ONE 2-D tensor-map box (128 rows x 144
//          bytes) per super-block into a ring of raw stages, started before the kernel waits for
//          its predecessor in the stream (weights are never produced by the activation kernels).
//   2      one thread brings the prepared activation slabs in with 1-D bulk copies.
//   3-10   drain warps, thread = (row, half of the sequences): tcgen05.ld of the block's
//          accumulators, acc += d * (hi + 2^-11 lo) - dmin * D2, store at the end of the item.
//   11-26  producers, thread = (row, 32-byte group of the super-block): read the row's header and
//          group from the raw stage, unpack nibbles and 6-bit scales in registers, form sc*q as
//          f16 pairs (one HFMA2 per two weights; high nibbles are used in place as 16 q with the
//          scale divided by 16) and write one 64-deep slab row of the 128-byte-swizzled K-major A
//          ring.  One producer group per block also writes the block's eight mins (A2) and its
//          d/dmin pair for the drain.
// A/B stages are quarter super-blocks handed over in pairs.  A parity wait is only sound for a
// waiter that cannot be two phases away from the barrier: most waiters see every phase of their
// barriers in order; where the producers do not (`empty` with three pairs, `d_full`), the ring
// order bounds the distance (comments at those waits).  Every wait is bounded: on expiry an error word is set, the CTA stops
// issuing, waits (bounded) for the copies it has in flight, frees its TMEM and returns; the host
// reports cudaErrorLaunchTimeout.
#include <cuda_fp16.h>

#include "launch_common.cuh"
#include "q4k_device.cuh"
#include "tensor_map.hpp"

namespace {

constexpr int kRows = 128;                // rows per tile = TMEM lanes = MMA M
constexpr int kSlabBytes = kRows * 128;   // one 64-deep f16 slab of A: 16 KiB
constexpr int kRawBytes = kRows * q4k::kBlockBytes;  // one super-block column of a tile, as stored: 18 KiB
constexpr int kParts = 4;                 // producer groups: one per 32-byte group (64 weights) of a super-block
constexpr int kProducerWarps = kParts * (kRows / 32);   // 16
constexpr int kDrainWarps = 8;
// Warp roles by index.
constexpr int kMmaWarp = 0, kRawWarp = 1, kActWarp = 2;
constexpr int kDrainWarp0 = 3;                          // 3..10; warp index mod 4 = TMEM lane quadrant
constexpr int kProducerWarp0 = kDrainWarp0 + kDrainWarps;  // 11..26
constexpr int kThreads = (kProducerWarp0 + kProducerWarps) * 32;  // 864
constexpr int kDdDepth = 4;               // blocks whose d/dmin pairs are kept for the drain
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr size_t kTailBytes = 1024;  // scratch tail: error word, row maxima, flags, row scales (256 B each)

// Pipeline depths per padded sequence count M (N = 2M accumulator columns): A/B ring stages of a
// quarter super-block each, raw stages of a whole super-block each.
template <int M> struct Depth;
template <> struct Depth<16> { static constexpr int kStages = 6, kRaw = 4; };
template <> struct Depth<32> { static constexpr int kStages = 6, kRaw = 3; };
template <> struct Depth<64> { static constexpr int kStages = 4, kRaw = 3; };

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on phase parity; false on expiry or when another thread already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try(b, parity)) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// The same for a whole converged warp: every lane polls, the verdict is made uniform.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* b, uint32_t parity, volatile int* abort_flag) {
    return __all_sync(0xFFFFFFFFu, mbar_wait(b, parity, abort_flag));
}
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xFFFFFFFF;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// One 2-D tiled TMA load (no multicast): box at element coordinates (x, y) of the tensor map.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols));
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols));
}
// D[tmem_d] (+)= A . B^T, one 16-deep step.  The descriptors arrive as their low words (start
// address, leading offset); the high word is the same for every operand of this kernel.
template <bool kAccumulate>
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint32_t desc_a_lo, uint32_t desc_b_lo, uint32_t desc_hi,
                                         uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(tmem_d),
        "r"(desc_a_lo), "r"(desc_b_lo), "r"(desc_hi), "r"(idesc), "n"(kAccumulate ? 1 : 0)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t addr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(addr));
}
// tcgen05.wait::ld with the loaded registers as in/out operands: without that tie the compiler is
// free to schedule arithmetic on the registers above the wait (it only orders volatile asm
// statements among themselves), and the values would be read before the asynchronous load lands.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&a)[8], uint32_t (&b)[8], uint32_t (&c)[8]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(a[0]), "+r"(a[1]), "+r"(a[2]), "+r"(a[3]), "+r"(a[4]), "+r"(a[5]), "+r"(a[6]), "+r"(a[7]),
                   "+r"(b[0]), "+r"(b[1]), "+r"(b[2]), "+r"(b[3]), "+r"(b[4]), "+r"(b[5]), "+r"(b[6]), "+r"(b[7]),
                   "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7])
                 :
                 : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Shared-memory matrix descriptor of a K-major operand with 128-byte swizzle, 8-row groups 1024 B
// apart.  Low word: start address >> 4 and the (unused) leading byte offset; high word: stride
// byte offset, the descriptor version of this architecture (bit 46), SWIZZLE_128B (bits 61-63).
// Advancing the operand by 16 k (32 bytes along the swizzled row) adds 2 to the low word.
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16); }
constexpr uint32_t kDescHi = (uint32_t)(1024 >> 4) | (1u << 14) | (2u << 29);
// Instruction descriptor: D f32, A and B f16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t idesc_f16(int n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
}
// Byte offset of 16-byte chunk `chunk` (0..7) of row `r` inside a 64-deep K-major slab.
__host__ __device__ __forceinline__ uint32_t sw128_off(int r, int chunk) {
    return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((chunk ^ (r & 7)) << 4));
}

// K order inside every group of four consecutive weights: (0, 2, 1, 3) — the order in which
// two masks per 32-bit word yield f16 pairs.  The activation slabs use the same order.
__host__ __device__ constexpr int kperm(int k) { return (k & ~3) | (((k & 1) << 1) | ((k >> 1) & 1)); }

// ---- activation slabs ----------------------------------------------------------------------------
// Step 1: per-sequence maximum magnitude (bit pattern of a non-negative float, so an integer
// atomicMax orders it) and a non-finite flag; row_bits[n] / row_bad[n] start at zero.
__global__ void __launch_bounds__(256) mm_row_max_kernel(const float* __restrict__ x, int m_rows, int k_dim,
                                                         unsigned* __restrict__ row_bits, int* __restrict__ row_bad) {
    const int n = blockIdx.x;
    if (n >= m_rows) return;
    const float* xr = x + (size_t)n * k_dim;
    float amax = 0.0f;
    int bad = 0;
    for (int k = blockIdx.y * blockDim.x + threadIdx.x; k < k_dim; k += gridDim.y * blockDim.x) {
        const float a = fabsf(xr[k]);
        bad |= !(a <= 3.0e38f);
        amax = fmaxf(amax, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(row_bits + n, __float_as_uint(amax));
        if (bad) atomicOr(row_bad + n, 1);
    }
}

// Step 2: one warp per (sequence, sub-block).  B image: for every quarter super-block (64 k) one
// slab [2M rows][64 k] of halves in the swizzled K-major layout (M*256 bytes): row n holds the hi
// limbs of sequence n, row M+n the lo limbs.  B2 image: per super-block one slab [M rows][64 k]:
// k = 3*sub + limb holds limb `limb` of sum(x) over sub-block `sub`, k = 24..31 zero, the rest is
// never read.  row_scale[n]: the power of two that undoes the scaling.  Launched with
// programmatic dependent launch behind step 1: row_bits / row_bad are not `__restrict__`.
template <int M>
__global__ void __launch_bounds__(256) mm_prepare_x_kernel(const float* __restrict__ x, int m_rows, int k_dim,
                                                           const unsigned* row_bits, const int* row_bad,
                                                           uint8_t* __restrict__ b_img, uint8_t* __restrict__ b2_img,
                                                           float* __restrict__ row_scale) {
    mg::pdl_prologue();
    const int n = blockIdx.x, lane = threadIdx.x & 31;
    const int n_sub = k_dim / 32;
    const int sub = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (sub >= n_sub) return;
    const bool live = n < m_rows;
    const float amax = live ? __uint_as_float(row_bits[n]) : 0.0f;
    const bool bad = live && row_bad[n] != 0;
    int E = (int)(__float_as_uint(amax) >> 23) - 127;  // floor(log2(amax))
    E = max(E, -100);
    if (amax == 0.0f) E = 9;
    const float to_half = __uint_as_float((uint32_t)(9 - E + 127) << 23);  // 2^(9-E): max lands in [2^9, 2^10)
    if (sub == 0 && lane == 0) {
        // a non-finite activation makes its whole output row NaN
        row_scale[n] = bad ? __uint_as_float(0x7FC00000u) : __uint_as_float((uint32_t)(E - 9 + 127) << 23);
    }
    const float xv = (live && !bad) ? x[(size_t)n * k_dim + sub * 32 + lane] * to_half : 0.0f;
    const __half xh = __float2half_rn(xv);
    const float rem = xv - __half2float(xh);             // exact
    const __half xl = __float2half_rn(rem * 2048.0f);    // |rem * 2^11| <= |xh|
    const int quarter = sub >> 1;
    const int kk = kperm((sub & 1) * 32 + lane);
    uint8_t* slab = b_img + (size_t)quarter * (M * 256);
    *reinterpret_cast<__half*>(slab + sw128_off(n, kk >> 3) + (kk & 7) * 2) = xh;
    *reinterpret_cast<__half*>(slab + sw128_off(M + n, kk >> 3) + (kk & 7) * 2) = xl;
    // sum of the values the tensor cores will see, |s| <= 32 * 2^10
    const float s = q4k::warp_sum(fmaf(__half2float(xl), 1.0f / 2048.0f, __half2float(xh)));
    const int blk = sub >> 3, sb = sub & 7;
    uint8_t* t2 = b2_img + (size_t)blk * (M * 128);
    if (lane < 3) {
        const __half h = __float2half_rn(s);
        const float r1 = s - __half2float(h);
        const __half m = __float2half_rn(r1);
        const __half l = __float2half_rn(r1 - __half2float(m));
        const __half v = lane == 0 ? h : (lane == 1 ? m : l);
        const int k2 = sb * 3 + lane;
        *reinterpret_cast<__half*>(t2 + sw128_off(n, k2 >> 3) + (k2 & 7) * 2) = v;
    } else if (lane == 3 && sb == 7) {
        *reinterpret_cast<uint4*>(t2 + sw128_off(n, 3)) = make_uint4(0, 0, 0, 0);  // k = 24 .. 31
    }
}

// ---- the GEMM ---------------------------------------------------------------------------------------
struct Params {
    const uint8_t* b_img;
    const uint8_t* b2_img;
    const float* row_scale;
    float* y;
    int* error_word;
    int m_rows, out_dim, bpr;
    int splits, blocks_per_split, n_items;
};

template <int M>
struct Ctl {
    uint64_t raw_full[Depth<M>::kRaw], raw_empty[Depth<M>::kRaw];
    // A/B stages are handed over in PAIRS of quarter stages (half a super-block): every barrier
    // round trip costs the issuing warp instructions, and it is the pipeline's narrowest point.
    uint64_t full[Depth<M>::kStages / 2];   // pair filled: eight producer warps + the activation slabs
    uint64_t empty[Depth<M>::kStages / 2];  // pair released by one tcgen05.commit
    uint64_t full2[2];                      // A2/B2 of accumulator set t filled
    uint64_t d_full[2], d_free[2];          // accumulator set t: MMAs done (A2/B2 free again) / drained
    uint32_t tmem_base;
    int abort_flag;
};

template <int M>
struct Layout {
    static constexpr int N = 2 * M;
    static constexpr int S = Depth<M>::kStages, R = Depth<M>::kRaw;
    static_assert(S % 2 == 0, "stages are released in pairs");
    static constexpr int kBStage = N * 128;       // hi and lo rows of a quarter super-block
    static constexpr int kB2Bytes = M * 128;
    static constexpr int oA = 0;
    static constexpr int oA2 = oA + S * kSlabBytes;           // one slab: set t in chunks 4t .. 4t+3
    static constexpr int oB = oA2 + kSlabBytes;
    static constexpr int oB2 = oB + S * kBStage;
    static constexpr int oRaw = oB2 + 2 * kB2Bytes;
    static constexpr int oDd = oRaw + R * kRawBytes;          // [kDdDepth][128] raw (d, dmin) half pairs
    static constexpr int oCtl = oDd + kDdDepth * kRows * 4;
    static constexpr int kBytes = oCtl + (int)sizeof(Ctl<M>) + 1024;  // + alignment slack
    static constexpr uint32_t kTmemCols = 6 * M <= 128 ? 128 : (6 * M <= 256 ? 256 : 512);
};

// Blocks [blk0, blk0 + n_blk) of work item `item`.
__device__ __forceinline__ void item_range(const Params& p, int item, int& tile, int& blk0, int& n_blk) {
    tile = item / p.splits;
    const int split = item - tile * p.splits;
    blk0 = split * p.blocks_per_split;
    n_blk = min(p.bpr, blk0 + p.blocks_per_split) - blk0;
}

template <int M>
__global__ void __launch_bounds__(kThreads, 1)
matmul_q4k_tc_kernel(const Params p, const __grid_constant__ CUtensorMap wmap) {
    using L = Layout<M>;
    constexpr int N = L::N, S = L::S, R = L::R, P = S / 2;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* sA = base + L::oA;
    uint8_t* sA2 = base + L::oA2;
    uint8_t* sB = base + L::oB;
    uint8_t* sB2 = base + L::oB2;
    uint8_t* sRaw = base + L::oRaw;
    uint32_t* sDd = reinterpret_cast<uint32_t*>(base + L::oDd);
    Ctl<M>* ctl = reinterpret_cast<Ctl<M>*>(base + L::oCtl);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < R; ++i) {
            mbar_init(&ctl->raw_full[i], 1);
            mbar_init(&ctl->raw_empty[i], kProducerWarps);
        }
        for (int i = 0; i < P; ++i) {
            mbar_init(&ctl->full[i], 2 * (kRows / 32) + 1);  // the warps of two producer groups + the bulk copies' arrive
            mbar_init(&ctl->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&ctl->full2[i], kRows / 32 + 1);
            mbar_init(&ctl->d_full[i], 1);
            mbar_init(&ctl->d_free[i], kDrainWarps);
        }
        ctl->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        tmem_alloc(&ctl->tmem_base, L::kTmemCols);
        tmem_relinquish();
    }
    // k = 24..31 of both A2 sets stay zero for the whole kernel
    if (threadIdx.x < kRows) {
        *reinterpret_cast<uint4*>(sA2 + sw128_off(threadIdx.x, 3)) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(sA2 + sw128_off(threadIdx.x, 7)) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctl->tmem_base;
    volatile int* abort_flag = &ctl->abort_flag;
    const int grid = (int)gridDim.x;

    if (warp >= kProducerWarp0) {
        // ================= producers: thread = (row of the tile, 32-byte group) =========================
        const int part = (warp - kProducerWarp0) >> 2;
        const int r = ((warp - kProducerWarp0) & 3) * 32 + lane;
        // byte offsets of this row's eight 16-byte chunks inside a slab (128-byte swizzle)
        const uint32_t row_off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128), rx = (uint32_t)(r & 7) << 4;
        const uint32_t sA_addr = smem_u32(sA) + row_off;
        const uint32_t raw_addr = smem_u32(sRaw) + (uint32_t)r * q4k::kBlockBytes;
        uint32_t gb = 0;  // super-blocks processed so far, over all items
        bool ok = true;
        for (int item = blockIdx.x; item < p.n_items && ok; item += grid) {
            int tile, blk0, n_blk;
            item_range(p, item, tile, blk0, n_blk);
            for (int b = 0; b < n_blk; ++b, ++gb) {
                const uint32_t rs = gb % R;
                ok = mbar_wait(&ctl->raw_full[rs], (gb / R) & 1u, abort_flag);
                if (!ok) break;
                const uint32_t src = raw_addr + rs * kRawBytes;
                const uint4 hdr = lds128(src), qa = lds128(src + 16 + 32 * part), qb = lds128(src + 32 + 32 * part);
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->raw_empty[rs]);
                const q4k::ScaleMin sm = q4k::unpack_scales(hdr.y, hdr.z, hdr.w);
                // ---- A: sc*q as f16 for this thread's 64 weights: one slab row -----------------------
                const uint32_t it = 4u * gb + (uint32_t)part, s = it % S;
                // Pair use u = it / 2 waits for the release of use u - P.  With three pairs a group meets a
                // pair only every second use; use u - 2P cannot still be pending then, because the group's
                // previous fill (use u - 2) waited for the release of u - 2 - P >= u - 2P, and one issuer
                // releases in order.
                const uint32_t pr = (it >> 1) % P;
                ok = mbar_wait(&ctl->empty[pr], (((it >> 1) / P) & 1u) ^ 1u, abort_flag);
                if (!ok) break;
                {
                    // low nibbles: (1024 + q) * sc - 1024 sc; high nibbles in place: (1024 + 16 q) * (sc / 16)
                    // - 64 sc.  Both are q * sc exactly (one rounding of an exact value).
                    const float sc_lo_f = (float)q4k::scale_of(sm, 2 * part), sc_hi_f = (float)q4k::scale_of(sm, 2 * part + 1);
                    const __half2 sc_lo = __float2half2_rn(sc_lo_f), sc_hi = __float2half2_rn(sc_hi_f * 0.0625f);
                    const __half2 off_lo = __float2half2_rn(-1024.0f * sc_lo_f);
                    const __half2 off_hi = __float2half2_rn(-64.0f * sc_hi_f);
                    const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                    const uint32_t slab = sA_addr + s * kSlabBytes;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {  // chunk c: low nibbles of words 2c, 2c+1; chunk c+4: high
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            const uint32_t v = qw[2 * c + t], w = v >> 8;
                            const uint32_t p0 = (v & 0x000F000Fu) | 0x64006400u;  // bytes 0,2 low
                            const uint32_t p1 = (w & 0x000F000Fu) | 0x64006400u;  // bytes 1,3 low
                            const uint32_t p2 = (v & 0x00F000F0u) | 0x64006400u;  // bytes 0,2 high, as 16 q
                            const uint32_t p3 = (w & 0x00F000F0u) | 0x64006400u;  // bytes 1,3 high, as 16 q
                            const __half2 a0 = __hfma2(*reinterpret_cast<const __half2*>(&p0), sc_lo, off_lo);
                            const __half2 a1 = __hfma2(*reinterpret_cast<const __half2*>(&p1), sc_lo, off_lo);
                            const __half2 a2 = __hfma2(*reinterpret_cast<const __half2*>(&p2), sc_hi, off_hi);
                            const __half2 a3 = __hfma2(*reinterpret_cast<const __half2*>(&p3), sc_hi, off_hi);
                            lo[2 * t] = *reinterpret_cast<const uint32_t*>(&a0);
                            lo[2 * t + 1] = *reinterpret_cast<const uint32_t*>(&a1);
                            hi[2 * t] = *reinterpret_cast<const uint32_t*>(&a2);
                            hi[2 * t + 1] = *reinterpret_cast<const uint32_t*>(&a3);
                        }
                        sts128(slab + (((uint32_t)c << 4) ^ rx), lo[0], lo[1], lo[2], lo[3]);
                        sts128(slab + (((uint32_t)(c + 4) << 4) ^ rx), hi[0], hi[1], hi[2], hi[3]);
                    }
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->full[pr]);
                }
                // ---- A2 (the eight 6-bit mins, each three times: one per limb of sum(x)) and the block's
                //      d/dmin pair, by the producer group whose turn it is ------------------------------------
                if ((uint32_t)part == (gb & 3u)) {
                    const uint32_t t2 = gb & 1u;
                    // Set t2 is free again when the MMAs of block gb - 2 have completed.  This group last looked
                    // at d_full[t2] four blocks ago; block gb - 4 is certainly complete, because the A stage
                    // this group has just been granted was released by MMAs issued after block gb - 2's
                    // first pair, and those were issued only after the drain of block gb - 4.
                    ok = mbar_wait(&ctl->d_full[t2], ((gb >> 1) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    uint32_t h[8];  // half bits of the mins: 0x6400 | m is 1024 + m
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const __half v = __hsub(__ushort_as_half((unsigned short)(0x6400u | q4k::min_of(sm, j))),
                                                __ushort_as_half((unsigned short)0x6400u));
                        h[j] = (uint32_t)__half_as_ushort(v);
                    }
                    auto pair = [&](int a, int b2) { return h[a] | (h[b2] << 16); };
                    const uint32_t a2 = smem_u32(sA2) + row_off;
                    sts128(a2 + (((4 * t2 + 0) << 4) ^ rx), pair(0, 0), pair(0, 1), pair(1, 1), pair(2, 2));
                    sts128(a2 + (((4 * t2 + 1) << 4) ^ rx), pair(2, 3), pair(3, 3), pair(4, 4), pair(4, 5));
                    sts128(a2 + (((4 * t2 + 2) << 4) ^ rx), pair(5, 5), pair(6, 6), pair(6, 7), pair(7, 7));
                    sDd[(gb % kDdDepth) * kRows + r] = hdr.x;
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ctl->full2[t2]);
                }
            }
        }
    } else if (warp >= kDrainWarp0) {
        // ================= drain: thread = (row, half of the sequences) ====================================
        constexpr int MH = M / 2;
        const int dw = warp - kDrainWarp0;
        const int quad = warp & 3;       // TMEM lanes 32*quad .. (a warp reaches the quadrant warp_id % 4)
        const int half_id = dw >> 2;
        const int r = quad * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        float acc[MH];
#pragma unroll
        for (int i = 0; i < MH; ++i) acc[i] = 0.0f;
        uint32_t gb = 0;
        bool ok = true;
        bool waited = false;
        for (int item = blockIdx.x; item < p.n_items && ok; item += grid) {
            int tile, blk0, n_blk;
            item_range(p, item, tile, blk0, n_blk);
            for (int b = 0; b < n_blk; ++b, ++gb) {
                const uint32_t t = gb & 1u;
                ok = mbar_wait(&ctl->d_full[t], (gb >> 1) & 1u, abort_flag);
                if (!ok) break;
                tc_fence_after();
                const uint32_t dd = sDd[(gb % kDdDepth) * kRows + r];
                const float d = q4k::half_bits_finite_or_zero(dd), ndmin = -q4k::half_bits_finite_or_zero(dd >> 16);
#pragma unroll
                for (int c = 0; c < MH / 8; ++c) {
                    uint32_t vh[8], vl[8], v2[8];
                    const uint32_t col = (uint32_t)(half_id * MH + 8 * c);
                    tmem_ld8(lane_base + t * N + col, vh);
                    tmem_ld8(lane_base + t * N + M + col, vl);
                    tmem_ld8(lane_base + 2 * N + t * M + col, v2);
                    tmem_ld_wait(vh, vl, v2);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float v = fmaf(__uint_as_float(vl[i]), 1.0f / 2048.0f, __uint_as_float(vh[i]));
                        acc[8 * c + i] = fmaf(d, v, acc[8 * c + i]);
                        acc[8 * c + i] = fmaf(ndmin, __uint_as_float(v2[i]), acc[8 * c + i]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&ctl->d_free[t]);
            }
            if (!ok) break;
            if (!waited) {  // row_scale comes from the activation kernel launched just before
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
            }
            const int orow = tile * kRows + r;
#pragma unroll
            for (int i = 0; i < MH; ++i) {
                const int n = half_id * MH + i;
                if (orow < p.out_dim && n < p.m_rows) {
                    const float v = acc[i] * p.row_scale[n];  // undo the sequence's power-of-two scaling
                    if (p.splits > 1) atomicAdd(&p.y[(size_t)n * p.out_dim + orow], v);
                    else p.y[(size_t)n * p.out_dim + orow] = v;
                }
                acc[i] = 0.0f;
            }
        }
    } else if (warp == kMmaWarp) {
        // ================= MMA issuer ========================================================================
        // The whole warp walks the loop and waits on the barriers, so that the index arithmetic stays in
        // the uniform datapath; one elected lane issues the tensor-core instructions.  (Issuing from two
        // warps, one per accumulator set, corrupted results at N = 128: one issuer only.)
        {
            constexpr uint32_t idesc = idesc_f16(N), idesc2 = idesc_f16(M);
            const uint32_t a_lo0 = smem_desc_lo(smem_u32(sA)), b_lo0 = smem_desc_lo(smem_u32(sB));
            const uint32_t a2_lo0 = smem_desc_lo(smem_u32(sA2)), b2_lo0 = smem_desc_lo(smem_u32(sB2));
            uint32_t gb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.n_items && ok; item += grid) {
                int tile, blk0, n_blk;
                item_range(p, item, tile, blk0, n_blk);
                for (int b = 0; b < n_blk && ok; ++b, ++gb) {
                    const uint32_t t = gb & 1u;
                    const uint32_t d1 = tmem + t * N, d2 = tmem + 2 * N + t * M;
                    ok = mbar_wait_warp(&ctl->d_free[t], ((gb >> 1) & 1u) ^ 1u, abort_flag);  // accumulators drained
                    if (!ok) break;
#pragma unroll
                    for (uint32_t h = 0; h < 2; ++h) {
                        const uint32_t u = 2u * gb + h, pr = u % P;
                        ok = mbar_wait_warp(&ctl->full[pr], (u / P) & 1u, abort_flag);
                        if (!ok) break;
                        tc_fence_after();
                        // the pair's two slabs lie back to back: eight 16-deep steps
                        const uint32_t a_lo = a_lo0 + pr * (2 * kSlabBytes >> 4), b_lo = b_lo0 + pr * (2 * L::kBStage >> 4);
                        if (elect_one()) {
#pragma unroll
                            for (uint32_t j = 0; j < 2; ++j) {
                                const uint32_t aj = a_lo + j * (kSlabBytes >> 4), bj = b_lo + j * (L::kBStage >> 4);
                                if (h == 0 && j == 0) umma_f16<false>(d1, aj, bj, kDescHi, idesc);
                                else umma_f16<true>(d1, aj, bj, kDescHi, idesc);
                                umma_f16<true>(d1, aj + 2, bj + 2, kDescHi, idesc);  // 16 weights = 32 bytes along the swizzled row
                                umma_f16<true>(d1, aj + 4, bj + 4, kDescHi, idesc);
                                umma_f16<true>(d1, aj + 6, bj + 6, kDescHi, idesc);
                            }
                            umma_commit(&ctl->empty[pr]);
                        }
                        __syncwarp();
                    }
                    if (!ok) break;
                    ok = mbar_wait_warp(&ctl->full2[t], (gb >> 1) & 1u, abort_flag);
                    if (!ok) break;
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t a2_lo = a2_lo0 + t * (64 >> 4), b2_lo = b2_lo0 + t * (L::kB2Bytes >> 4);
                        umma_f16<false>(d2, a2_lo, b2_lo, kDescHi, idesc2);  // 24 live k values: two 16-deep steps
                        umma_f16<true>(d2, a2_lo + 2, b2_lo + 2, kDescHi, idesc2);
                        umma_commit(&ctl->d_full[t]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == kRawWarp) {
        // ================= raw-weight loader: one TMA box (128 rows x 144 bytes) per super-block ============
        if (lane == 0) {
            uint32_t gb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.n_items && ok; item += grid) {
                int tile, blk0, n_blk;
                item_range(p, item, tile, blk0, n_blk);
                for (int b = 0; b < n_blk; ++b, ++gb) {
                    const uint32_t rs = gb % R;
                    ok = mbar_wait(&ctl->raw_empty[rs], ((gb / R) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&ctl->raw_full[rs], kRawBytes);
                    tma_load_2d(sRaw + rs * kRawBytes, &wmap, (blk0 + b) * q4k::kBlockBytes, tile * kRows, &ctl->raw_full[rs]);
                }
            }
            if (*abort_flag) {  // let the copies in flight land before the CTA's shared memory goes away
                for (uint32_t j = 0; j < (uint32_t)R && j < gb; ++j) {
                    const uint32_t i = gb - 1 - j;
                    for (uint32_t n = 0; n < (1u << 16) && !mbar_try(&ctl->raw_full[i % R], (i / R) & 1u); ++n) {}
                }
            }
        }
    } else if (warp == kActWarp) {
        // ================= activation-slab loader =========================================================
        if (lane == 0) {
            asm volatile("griddepcontrol.wait;" ::: "memory");  // the slabs come from the kernel launched just before
            uint32_t gb = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < p.n_items && ok; item += grid) {
                int tile, blk0, n_blk;
                item_range(p, item, tile, blk0, n_blk);
                for (int b = 0; b < n_blk && ok; ++b, ++gb) {
                    for (uint32_t h = 0; h < 2; ++h) {
                        const uint32_t u = 2u * gb + h, pr = u % P;
                        ok = mbar_wait(&ctl->empty[pr], ((u / P) & 1u) ^ 1u, abort_flag);
                        if (!ok) break;
                        // the two quarter slabs of a half block are contiguous in the image and in the ring
                        mbar_arrive_expect_tx(&ctl->full[pr], 2 * L::kBStage);
                        bulk_copy_g2s(sB + pr * (2 * L::kBStage), p.b_img + ((size_t)(blk0 + b) * 2 + h) * (2 * L::kBStage),
                                      2 * L::kBStage, &ctl->full[pr]);
                    }
                    if (!ok) break;
                    const uint32_t t = gb & 1u;
                    ok = mbar_wait(&ctl->d_full[t], ((gb >> 1) & 1u) ^ 1u, abort_flag);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&ctl->full2[t], L::kB2Bytes);
                    bulk_copy_g2s(sB2 + t * L::kB2Bytes, p.b2_img + (size_t)(blk0 + b) * L::kB2Bytes, L::kB2Bytes, &ctl->full2[t]);
                }
            }
            if (*abort_flag) {
                // Copies in flight complete on barriers that the producers may never complete; give them
                // time to land (bounded) instead of waiting on a phase.
                for (uint32_t n = 0; n < (1u << 16); ++n) __nanosleep(32);
            }
        }
    }
    // ---- teardown: everything this CTA started has been consumed or abandoned ----------------------
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ctl->abort_flag && p.error_word) atomicExch(p.error_word, 1);
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, L::kTmemCols);
    }
}

template <int M>
cudaError_t launch_mm(const uint8_t* w, const float* x, float* y, int m_rows, int out_dim, int bpr, void* scratch,
                      int* error_word, int sms, cudaStream_t s) {
    using L = Layout<M>;
    static_assert(L::kBytes <= 227 * 1024, "shared-memory plan exceeds the per-CTA limit");
    const mg::EncodeTiledFn encode = mg::encode_tiled();
    if (encode == nullptr) return cudaErrorNotSupported;
    const int k_dim = bpr * 256;
    uint8_t* b_img = static_cast<uint8_t*>(scratch);
    uint8_t* b2_img = b_img + (size_t)(4 * bpr) * L::kBStage;
    // scratch tail: error word +0, row maxima (bits) +256, non-finite flags +512, row scales +768
    uint8_t* tail = reinterpret_cast<uint8_t*>(error_word);
    unsigned* row_bits = reinterpret_cast<unsigned*>(tail + 256);
    int* row_bad = reinterpret_cast<int*>(tail + 512);
    float* row_scale = reinterpret_cast<float*>(tail + 768);
    cudaError_t e = cudaMemsetAsync(tail, 0, 768, s);
    if (e != cudaSuccess) return e;
    const int tiles = (out_dim + kRows - 1) / kRows;
    int splits = 1;
    if (tiles < sms) {
        splits = sms / tiles;
        if (splits > bpr) splits = bpr;
        if (splits < 1) splits = 1;
    }
    const int blocks_per_split = (bpr + splits - 1) / splits;
    splits = (bpr + blocks_per_split - 1) / blocks_per_split;
    if (splits > 1) {
        e = cudaMemsetAsync(y, 0, (size_t)m_rows * out_dim * sizeof(float), s);
        if (e != cudaSuccess) return e;
    }
    // The weight matrix as a 2-D byte tensor [out_dim][bpr * 144]; box = 128 rows x one super-block.
    // Rows past out_dim read as zero (d = 0: they contribute nothing and are not stored).
    CUtensorMap wmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)bpr * q4k::kBlockBytes, (cuuint64_t)out_dim};
    const cuuint64_t gstride[1] = {(cuuint64_t)bpr * q4k::kBlockBytes};
    const cuuint32_t box[2] = {(cuuint32_t)q4k::kBlockBytes, (cuuint32_t)kRows};
    const cuuint32_t estride[2] = {1u, 1u};
    if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(w), gdim, gstride, box, estride,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        e = cudaFuncSetAttribute(matmul_q4k_tc_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    mm_row_max_kernel<<<dim3((unsigned)m_rows, 8), 256, 0, s>>>(x, m_rows, k_dim, row_bits, row_bad);
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    e = mg::launch_pdl(mm_prepare_x_kernel<M>, dim3((unsigned)M, (unsigned)((k_dim / 32 + 7) / 8)), dim3(256), 0, s, x,
                       m_rows, k_dim, (const unsigned*)row_bits, (const int*)row_bad, b_img, b2_img, row_scale);
    if (e != cudaSuccess) return e;
    Params p = {};
    p.b_img = b_img; p.b2_img = b2_img; p.row_scale = row_scale; p.y = y; p.error_word = error_word;
    p.m_rows = m_rows; p.out_dim = out_dim; p.bpr = bpr;
    p.splits = splits; p.blocks_per_split = blocks_per_split; p.n_items = tiles * splits;
    const int grid = p.n_items < sms ? p.n_items : sms;
    return mg::launch_pdl(matmul_q4k_tc_kernel<M>, dim3((unsigned)grid), dim3(kThreads), (size_t)L::kBytes, s, p, wmap);
}

constexpr int padded_m(int m_rows) { return m_rows <= 16 ? 16 : (m_rows <= 32 ? 32 : 64); }

}  // namespace

extern "C" {

// Device scratch the launcher needs: the prepared activation slabs, one error word, the
// per-sequence scales.
size_t mg_matmul_q4k_scratch_bytes(int m_rows, int blocks_per_row) {
    if (m_rows <= 0 || blocks_per_row <= 0) return 0;
    const size_t m = (size_t)padded_m(m_rows);
    return (size_t)blocks_per_row * (4 * m * 256 + m * 128) + kTailBytes;
}

// Y[m_rows][out_dim] (row-major; exactly m_rows * out_dim floats are written) = X[m_rows][K] .
// dequant(W)^T.  m_rows <= 64 per call.  `scratch`: mg_matmul_q4k_scratch_bytes(...) bytes,
// 1024-byte aligned.
int launch_matmul_q4k_on_stream(const uint8_t* w_q4, const float* x, float* y, int m_rows, int out_dim,
                                int blocks_per_row, void* scratch, void* stream) {
    if (m_rows <= 0 || m_rows > 64 || out_dim <= 0 || blocks_per_row <= 0) return (int)cudaErrorInvalidValue;
    if (!w_q4 || !x || !y || !scratch) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(w_q4) || (reinterpret_cast<uintptr_t>(scratch) & 1023u)) return (int)cudaErrorInvalidValue;
    const mg::DeviceProps& dp = mg::device_props();
    const int sms = dp.ok ? dp.sm_count : 148;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t total = mg_matmul_q4k_scratch_bytes(m_rows, blocks_per_row);
    int* error_word = reinterpret_cast<int*>(static_cast<uint8_t*>(scratch) + total - kTailBytes);
    if (m_rows <= 16) return (int)launch_mm<16>(w_q4, x, y, m_rows, out_dim, blocks_per_row, scratch, error_word, sms, s);
    if (m_rows <= 32) return (int)launch_mm<32>(w_q4, x, y, m_rows, out_dim, blocks_per_row, scratch, error_word, sms, s);
    return (int)launch_mm<64>(w_q4, x, y, m_rows, out_dim, blocks_per_row, scratch, error_word, sms, s);
}

// After synchronising: 0 when the last launch that used `scratch` completed normally,
// cudaErrorLaunchTimeout (702) when a bounded wait inside the kernel expired.
int mg_matmul_q4k_status(const void* scratch, int m_rows, int blocks_per_row) {
    if (!scratch) return (int)cudaErrorInvalidValue;
    const size_t total = mg_matmul_q4k_scratch_bytes(m_rows, blocks_per_row);
    int word = 0;
    cudaError_t e = cudaMemcpy(&word, static_cast<const uint8_t*>(scratch) + total - kTailBytes, sizeof(int),
                               cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return (int)e;
    return word ? (int)cudaErrorLaunchTimeout : 0;
}

}  // extern "C"
