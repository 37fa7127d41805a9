// Batch-1 Q4_K matvec on the integer tensor-core path: y[row] = sum_e dequant(W)[row][e] * x[e] (+ addend).
//
// The GEMV is HBM-bound (0.5625 bytes per weight) but its instruction count decides whether a
// launch reaches the memory rate: with dp4a every weight costs about two lane-operations.  Here
// the dot products go to `mma.sync.m16n8k32` (u8 x s8 -> s32) and the lanes only mask nibbles and
// apply the 6-bit scales, a little over one lane-operation per weight, so eight warps keep up
// with the memory system and a CTA needs half an SM.  Two CTAs of consecutive launches are then
// resident together: under programmatic dependent launch the successor's weight stream is
// already in shared memory when its predecessor retires.
//
// Arithmetic (per 256-weight super-block b and row r; the format is q4k_device.cuh):
//   x is rewritten once per CTA as 23-bit integers a_e with ONE power-of-two scale s_b per
//   super-block, x_e ~= s_b * a_e, |a_e| <= 2^22, and each a_e as three balanced signed byte limbs
//   a = a2*65536 + a1*256 + a0 (a1, a0 in [-128, 127]).  The rounding error per element is at most
//   2^-22 of the largest magnitude of its super-block.  For a 16-row tile and a 64-byte pair of
//   quant groups two chained MMAs give, per row, the exact integer sums  S[sub][limb] = sum q*a_limb
//   of two sub-blocks at once (the k = 32 slots of an MMA are 16 bytes of either group, the
//   activation operand holds the limbs of one group in columns 0..2 and of the other in 3..5,
//   zero elsewhere).  Lanes fold the 6-bit scales in integer arithmetic, acc[limb] += sc * S, and
//   once per super-block  y += d * s_b * (65536*acc2 + 256*acc1 + acc0).  High nibbles are used
//   in place as 16*q.  The min term  -dmin * s_b * sum_sub m[sub] * sum(a)[sub]  is one more MMA
//   whose weight operand is the unpacked 6-bit mins and whose activation operand holds four byte
//   limbs of the eight sub-block sums.
//
// Pipeline: a CTA owns 16-row tiles (tile = blockIdx.x + i * gridDim.x).  A manager warp streams
// them into a ring of shared-memory stages with ONE 2-D tensor-map TMA load per stage (box = 16
// rows x up to 14 super-blocks; issuing a bulk copy per row instead costs ~40 ns of TMA issue time
// each and caps the stream), completion on an mbarrier per stage.  Rows lie dense in a stage; the
// MMA rows are a permutation of the tile rows chosen so that the two rows a quarter-warp reads
// together are 64 bytes apart modulo 128 (conflict-free 16-byte reads), which needs a window
// width that is not a multiple of 8 super-blocks.  The eight consumer warps split the
// super-blocks of a stage round-robin, keep per-row partial sums in registers, and after the last
// window of a tile leave them in shared memory; their arrival on the stage's second mbarrier
// tells the manager that the stage can be refilled and that the partials can be summed (fixed
// order: results are deterministic) and stored.  Every wait is bounded; a wait that runs out is
// counted and the CTA drains and returns.
//
// The first copies are issued BEFORE the kernel waits for its predecessor in the stream
// (griddepcontrol.wait): weights must not be produced by the kernel launched just before a
// matvec on the same stream.
#include "gemv_q4k_mma.hpp"

#include <cuda.h>

#include <float.h>

#include "gemv_q4k_device.cuh"
#include "launch_common.cuh"
#include "q4k_device.cuh"
#include "tensor_map.hpp"

namespace gemvmma {

using gemvdev::bulk_copy_g2s;
using gemvdev::griddep_launch_dependents;
using gemvdev::griddep_wait;
using gemvdev::mbar_arrive_expect_tx;
using gemvdev::mbar_init;
using gemvdev::mbar_try_wait;
using gemvdev::smem_u32;

constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 2) * 32;  // consumers, manager, sentinel
constexpr int kTileRows = 16;
constexpr int kMaxDepth = 6;
constexpr int kXBlockBytes = 816;  // per super-block: 768 B limb fragments, 32 B sum fragments, scale, pad
constexpr uint32_t kSpinLimit = 1u << 22;

struct Params {
    const uint8_t* w;
    const float* x;
    const float* addend;  // may be null; may alias y
    float* y;
    int rows, bpr;
    int n_win, kb;      // windows per tile, super-blocks per window (the last may be shorter)
    int depth;          // stages in the ring
    int row_stride;     // bytes between the rows of a stage (kb * 144, dense)
    int row_swap;       // MMA row m reads tile row "m with bits 0 and row_swap exchanged"
    int x_aligned, hold_trigger;
    int speculate;      // convert x and start computing before the previous kernel has completed
    // 0xFFFFFFFF, passed at run time so that "w - (w & 0xF0F0F0F0)" stays a multiply-add: the
    // integer multiply-add runs on the FMA pipe, which has room, the logic pipe does not
    uint32_t neg_one;
    unsigned* timeouts;
};

__host__ __device__ inline int round128(int v) { return (v + 127) & ~127; }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One 2-D tiled TMA load (no multicast): box at element coordinates (x, y) of the tensor map.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void mma_u8s8(int& c0, int& c1, int& c2, int& c3, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c0), "+r"(c1), "+r"(c2), "+r"(c3)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------------
// x -> per-super-block operand table.  One warp converts one super-block; lane l owns elements
// 8l .. 8l+7 (a quarter of sub-block l/4).
//
// Table of one super-block (816 bytes):
//   [ (p*2+h)*12 + idx ] x 16 bytes, p = pair of quant groups (0,1), h = nibble plane (0 low, 1 high):
//       the activation fragments of the two chained MMAs of (p, h) for the lane that holds column
//       n of slot group t:  idx = n*2 + t for n < 3, t < 2 (limbs of group 2p) and
//       6 + (n-3)*2 + (t-2) for 3 <= n < 6, t >= 2 (limbs of group 2p+1); bytes 0..7 = registers
//       b0, b1 of the first MMA, 8..15 of the second.  Slot (t, half, i) of MMA j is quant byte
//       16t + 8j + 4*half + i of the 64-byte pair.
//   768 + (n*2 + t)*4 + i : limb n (most significant first) of the integer sum of sub-block 4t + i
//   800 : f32 scale s_b / 16 (NaN when the super-block holds a non-finite activation)
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void load8(float (&v)[8], const float* p, int aligned) {
    if (aligned) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = p[i];
    }
}

// verify = false: writes the table of one super-block.  verify = true: writes nothing and returns
// (to every lane) whether the table differs from what these activations convert to.  (One body
// for both, and rolled loops around it: the kernel's instruction footprint matters.)
__device__ __forceinline__ bool convert_block(const float (&v)[8], uint8_t* xb, int lane, bool verify) {
    float amax = 0.f;
    int bad = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float a = fabsf(v[i]);
        bad |= !(a <= FLT_MAX);  // inf or NaN
        amax = fmaxf(amax, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    }
    int E = (int)(__float_as_uint(amax) >> 23) - 127;  // floor(log2(amax)); -127 for 0 / sub-normal
    E = max(E, -100);
    const float inv = __uint_as_float((uint32_t)(21 - E + 127) << 23);  // 2^(21-E)
    uint32_t lo[3] = {0, 0, 0}, hi[3] = {0, 0, 0};
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int a = bad ? 0 : __float2int_rn(v[i] * inv);  // |a| <= 2^22
        sum += a;
        const int l0 = (a << 24) >> 24;  // balanced digits
        const int r1 = (a - l0) >> 8;
        const int l1 = (r1 << 24) >> 24;
        const int l2 = (r1 - l1) >> 8;
        const int sh = 8 * (i & 3);
        uint32_t* dst = i < 4 ? lo : hi;
        dst[0] |= ((uint32_t)l2 & 0xFFu) << sh;
        dst[1] |= ((uint32_t)l1 & 0xFFu) << sh;
        dst[2] |= ((uint32_t)l0 & 0xFFu) << sh;
    }
    const int sub = lane >> 2, G = sub >> 1, h = sub & 1, p = G >> 1;
    const int tlow = (lane & 3) >> 1, j = lane & 1;
    // A non-finite activation poisons its super-block: every row's sum becomes NaN, as it does in
    // the reference (w * NaN).
    const uint32_t s16 = bad ? 0x7FC00000u : (uint32_t)(E - 25 + 127) << 23;  // 2^(E-21) / 16
    if (verify) {
        // The sub-block sums are a function of the limbs: limbs and scale equal => table equal.
        bool diff = false;
#pragma unroll
        for (int n = 0; n < 3; ++n) {
            const int idx = (G & 1) * 6 + n * 2 + tlow;
            const uint2 t = *reinterpret_cast<const uint2*>(xb + ((p * 2 + h) * 12 + idx) * 16 + j * 8);
            diff |= (t.x != lo[n]) | (t.y != hi[n]);
        }
        if (lane == 0) diff |= *reinterpret_cast<const uint32_t*>(xb + 800) != s16;
        return __any_sync(0xFFFFFFFFu, diff);
    }
#pragma unroll
    for (int n = 0; n < 3; ++n) {
        const int idx = (G & 1) * 6 + n * 2 + tlow;
        *reinterpret_cast<uint2*>(xb + ((p * 2 + h) * 12 + idx) * 16 + j * 8) = make_uint2(lo[n], hi[n]);
    }
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
    sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
    if ((lane & 3) == 0) {  // |sum| <= 2^27: four balanced limbs
        const int l3 = (sum << 24) >> 24;
        const int r1 = (sum - l3) >> 8;
        const int l2 = (r1 << 24) >> 24;
        const int r2 = (r1 - l2) >> 8;
        const int l1 = (r2 << 24) >> 24;
        const int l0 = (r2 - l1) >> 8;
        uint8_t* s = xb + 768 + (sub >> 2) * 4 + (sub & 3);
        s[0] = (uint8_t)l0;
        s[8] = (uint8_t)l1;
        s[16] = (uint8_t)l2;
        s[24] = (uint8_t)l3;
    }
    if (lane == 0) *reinterpret_cast<uint32_t*>(xb + 800) = s16;
    return false;
}

// Super-blocks warp, warp + 9, ... of x are converted (or verified) by warp `warp` of the nine
// working warps, two at a time so that their loads overlap.  Returns (verify) whether any of the
// warp's super-blocks no longer matches the table.
__device__ __noinline__ bool convert_mine(const float* x, int bpr, int x_aligned, uint8_t* xtab, int warp, int lane,
                                          bool verify) {
    constexpr int kWarps = kConsumerWarps + 1;
    bool diff = false;
#pragma unroll 1
    for (int b = warp; b < bpr; b += 2 * kWarps) {
        float v0[8], v1[8];
        const bool two = b + kWarps < bpr;
        load8(v0, x + (size_t)b * 256 + lane * 8, x_aligned);
        if (two) load8(v1, x + (size_t)(b + kWarps) * 256 + lane * 8, x_aligned);
        diff |= convert_block(v0, xtab + (size_t)b * kXBlockBytes, lane, verify);
        if (two) diff |= convert_block(v1, xtab + (size_t)(b + kWarps) * kXBlockBytes, lane, verify);
    }
    return diff;
}

// Per-lane constants of the MMA fragment layout (g = lane / 4 is the row / column group,
// t = lane % 4 the slot group).
struct LaneConst {
    int g, t;
    int row_a, row_b;     // tile rows behind MMA rows g and g + 8
    int b_active, b_off;  // activation fragment of the limb MMAs: byte offset inside a (p, h) group
    int s_active, s_off;  // activation fragment of the min-term MMA
    uint32_t sel0, sel1;  // byte_perm selectors of the scale for accumulator columns 2t and 2t+1
    float w0, w1;         // limb weights of those columns
    float v0, v1;         // limb weights of the sum columns
    uint32_t neg_one;
};

__device__ __forceinline__ int swap_bits(int m, int k) {  // exchange bits 0 and k of m
    const int d = ((m >> k) ^ m) & 1;
    return m ^ (d | (d << k));
}
__device__ __forceinline__ LaneConst lane_const(int lane, uint32_t neg_one, int row_swap) {
    LaneConst c;
    c.neg_one = neg_one;
    c.g = lane >> 2;
    c.t = lane & 3;
    c.row_a = swap_bits(c.g, row_swap);
    c.row_b = swap_bits(c.g + 8, row_swap);
    const int n = c.g;
    c.b_active = (n < 3 && c.t < 2) || (n >= 3 && n < 6 && c.t >= 2);
    c.b_off = (n < 3 ? n * 2 + c.t : 6 + (n - 3) * 2 + (c.t - 2)) * 16;
    c.s_active = n < 4 && c.t < 2;
    c.s_off = 768 + (n * 2 + c.t) * 4;
    // columns 0..2: limbs of the pair's first group, 3..5: of its second group
    c.sel0 = 0x4440u + (c.t >= 2 ? 2u : 0u);
    c.sel1 = 0x4440u + (c.t >= 1 ? 2u : 0u);
    c.w0 = c.t == 0 ? 65536.f : (c.t == 1 ? 1.f : (c.t == 2 ? 256.f : 0.f));
    c.w1 = c.t == 0 ? 256.f : (c.t == 1 ? 65536.f : (c.t == 2 ? 1.f : 0.f));
    c.v0 = c.t == 0 ? 16777216.f : (c.t == 1 ? 256.f : 0.f);
    c.v1 = c.t == 0 ? 65536.f : (c.t == 1 ? 1.f : 0.f);
    return c;
}

// One super-block of a 16-row tile: blk = the block's bytes of row 0 inside the stage, xb = the
// block's operand table.  racc0 / racc1 accumulate rows g and g + 8 (partial over this lane's columns).
__device__ __forceinline__ void process_block(const uint8_t* blk, int row_stride, const uint8_t* xb,
                                              const LaneConst& lc, float& racc0, float& racc1) {
    const uint8_t* r0p = blk + lc.row_a * row_stride;
    const uint8_t* r1p = blk + lc.row_b * row_stride;
    const uint4 h0 = *reinterpret_cast<const uint4*>(r0p);
    const uint4 h1 = *reinterpret_cast<const uint4*>(r1p);
    const float2 dd0 = __half22float2(*reinterpret_cast<const __half2*>(&h0.x));
    const float2 dd1 = __half22float2(*reinterpret_cast<const __half2*>(&h1.x));
    const float d0 = fabsf(dd0.x) <= 65504.0f ? dd0.x : 0.0f;  // inf / NaN -> 0
    const float m0 = fabsf(dd0.y) <= 65504.0f ? dd0.y : 0.0f;
    const float d1 = fabsf(dd1.x) <= 65504.0f ? dd1.x : 0.0f;
    const float m1 = fabsf(dd1.y) <= 65504.0f ? dd1.y : 0.0f;
    const q4k::ScaleMin s0 = q4k::unpack_scales(h0.y, h0.z, h0.w);
    const q4k::ScaleMin s1 = q4k::unpack_scales(h1.y, h1.z, h1.w);
    const float s_b = *reinterpret_cast<const float*>(xb + 800);

    // min term: sum_sub m[sub] * sum(a)[sub], limbs of the sums in columns 0..3
    int cm0 = 0, cm1 = 0, cm2 = 0, cm3 = 0;
    {
        const uint32_t am0 = lc.t == 0 ? s0.m_lo : (lc.t == 1 ? s0.m_hi : 0u);
        const uint32_t am1 = lc.t == 0 ? s1.m_lo : (lc.t == 1 ? s1.m_hi : 0u);
        uint32_t bm = 0;
        if (lc.s_active) bm = *reinterpret_cast<const uint32_t*>(xb + lc.s_off);
        mma_u8s8(cm0, cm1, cm2, cm3, am0, am1, 0u, 0u, bm, 0u);
    }
    int lo00 = 0, lo01 = 0, lo10 = 0, lo11 = 0, hi00 = 0, hi01 = 0, hi10 = 0, hi11 = 0;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const uint4 q0 = *reinterpret_cast<const uint4*>(r0p + 16 + p * 64 + lc.t * 16);
        const uint4 q1 = *reinterpret_cast<const uint4*>(r1p + 16 + p * 64 + lc.t * 16);
        const uint32_t scw0 = p ? s0.sc_hi : s0.sc_lo;
        const uint32_t scw1 = p ? s1.sc_hi : s1.sc_lo;
        // high nibbles in place (16 * q) with one logic op, low nibbles as w - 16 * q on the FMA pipe
        const uint32_t w0[4] = {q0.x, q0.y, q0.z, q0.w}, w1[4] = {q1.x, q1.y, q1.z, q1.w};
        uint32_t hq0[4], hq1[4], lq0[4], lq1[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            hq0[k] = w0[k] & 0xF0F0F0F0u;
            hq1[k] = w1[k] & 0xF0F0F0F0u;
            lq0[k] = hq0[k] * lc.neg_one + w0[k];
            lq1[k] = hq1[k] * lc.neg_one + w1[k];
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint4 bf = make_uint4(0u, 0u, 0u, 0u);
            if (lc.b_active) bf = *reinterpret_cast<const uint4*>(xb + (p * 2 + h) * 192 + lc.b_off);
            int c0 = 0, c1 = 0, c2 = 0, c3 = 0;
            mma_u8s8(c0, c1, c2, c3, h ? hq0[0] : lq0[0], h ? hq1[0] : lq1[0], h ? hq0[1] : lq0[1],
                     h ? hq1[1] : lq1[1], bf.x, bf.y);
            mma_u8s8(c0, c1, c2, c3, h ? hq0[2] : lq0[2], h ? hq1[2] : lq1[2], h ? hq0[3] : lq0[3],
                     h ? hq1[3] : lq1[3], bf.z, bf.w);
            const int sc00 = (int)__byte_perm(scw0, 0u, lc.sel0 + h), sc01 = (int)__byte_perm(scw0, 0u, lc.sel1 + h);
            const int sc10 = (int)__byte_perm(scw1, 0u, lc.sel0 + h), sc11 = (int)__byte_perm(scw1, 0u, lc.sel1 + h);
            if (h == 0) {
                lo00 += sc00 * c0; lo01 += sc01 * c1; lo10 += sc10 * c2; lo11 += sc11 * c3;
            } else {
                hi00 += sc00 * c0; hi01 += sc01 * c1; hi10 += sc10 * c2; hi11 += sc11 * c3;
            }
        }
    }
    // |lo| <= 4*63*15*128*32 < 2^24, |hi| <= 16 times that: lo*16 + hi < 2^29, exact
    const float k00 = (float)(lo00 * 16 + hi00), k01 = (float)(lo01 * 16 + hi01);
    const float k10 = (float)(lo10 * 16 + hi10), k11 = (float)(lo11 * 16 + hi11);
    const float v0 = fmaf(lc.w0, k00, lc.w1 * k01);
    const float v1 = fmaf(lc.w0, k10, lc.w1 * k11);
    const float n0 = fmaf(lc.v0, (float)cm0, lc.v1 * (float)cm1);
    const float n1 = fmaf(lc.v0, (float)cm2, lc.v1 * (float)cm3);
    racc0 = fmaf(d0 * s_b, v0, racc0);
    racc0 = fmaf(-(m0 * s_b) * 16.0f, n0, racc0);
    racc1 = fmaf(d1 * s_b, v1, racc1);
    racc1 = fmaf(-(m1 * s_b) * 16.0f, n1, racc1);
}

// Control words of a CTA (shared memory).
struct Control {
    uint64_t full_bar[kMaxDepth];  // stage filled (transaction bytes)
    uint64_t done_bar[kMaxDepth];  // stage consumed (eight consumer warps)
    uint64_t verified_bar;         // the nine working warps have re-checked their part of x
    int abort;                     // a bounded wait ran out somewhere in the CTA
    int released;                  // the previous kernel of the stream has completed (set by the sentinel warp)
    int mismatch;                  // x changed after it was converted speculatively
    int verdict;                   // 0 unknown, 1 the speculative operand table is valid, 2 it is not
};
constexpr int kVerdictOk = 1, kVerdictRedo = 2;

__device__ __forceinline__ int ld_volatile(const int* p) { return *reinterpret_cast<const volatile int*>(p); }

// One pass over this CTA's tiles.
//   SPEC = true : x was converted BEFORE the previous kernel of the stream is known to have completed.
//                 Results are kept in shared memory until the sentinel warp reports the table valid
//                 (verdict 1: flush and continue storing directly) or stale (verdict 2: give up, the
//                 caller runs the pass again with SPEC = false).  Every working warp re-checks its
//                 share of x as soon as `released` is set, whatever it is doing.
//   SPEC = false: x is final; results are stored directly.
// Returns false when a bounded wait ran out.
__device__ __forceinline__ void run_pass(const bool SPEC, const Params& p, const CUtensorMap* wmap, Control* c,
                                         uint8_t* xtab, float* partials, float* results, uint8_t* stages, int warp,
                                         int lane) {
    const int depth = p.depth;
    const int stage_bytes = kTileRows * p.row_stride;
    const int n_tiles = (p.rows + kTileRows - 1) / kTileRows;
    const int my_tiles = (int)blockIdx.x < n_tiles ? (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int total = my_tiles * p.n_win;  // stage uses of this CTA
    volatile int* abort_flag = &c->abort;
    bool verified = !SPEC;  // this warp has re-checked its share of x

    // Re-check of this warp's share of x once the previous kernel has completed; called from every
    // loop and every wait so that the verdict never waits for a warp that is busy or blocked.
    auto poll_verify = [&]() {
        if (verified || !ld_volatile(&c->released)) return;
        const bool diff = convert_mine(p.x, p.bpr, p.x_aligned, xtab, warp, lane, true);
        if (lane == 0) {
            if (diff) atomicOr(&c->mismatch, 1);
            mbar_arrive(&c->verified_bar);
        }
        verified = true;
    };
    // Bounded wait for an mbarrier phase that keeps the verification going; false: give up / abort.
    auto wait_bar = [&](uint64_t* bar, uint32_t parity) {
        uint32_t spins = 0;
        while (!mbar_try_wait(bar, parity)) {
            if (SPEC) {
                poll_verify();
                if (ld_volatile(&c->verdict) == kVerdictRedo) return false;
            }
            if (++spins > kSpinLimit || *abort_flag) {
                if (lane == 0 && !*abort_flag) {
                    atomicAdd(p.timeouts, 1u);
                    *abort_flag = 1;
                }
                return false;
            }
        }
        return true;
    };

    // Fills the stage of use `u` (tile u / n_win, window u % n_win) with one TMA load: the box is
    // always whole (rows past the matrix and super-blocks past the row arrive as zeros).
    auto issue = [&](int u) {
        if (lane != 0) return;
        const int ti = u / p.n_win, win = u - ti * p.n_win;
        const int row0 = ((int)blockIdx.x + ti * (int)gridDim.x) * kTileRows;
        const int s = u % depth;
        mbar_arrive_expect_tx(c->full_bar + s, (uint32_t)stage_bytes);
        tma_load_2d(stages + (size_t)s * stage_bytes, wmap, win * p.kb * (q4k::kBlockBytes / 8), row0, c->full_bar + s);
    };

    // Which warp takes super-block b of a tile: (b + phase) % 8, phase = (tile counter * bpr) % 8,
    // so that over consecutive tiles every warp gets the same number of super-blocks.  A warp's
    // partial sum of a tile therefore holds the blocks b = j (mod 8) for j = (warp - phase) % 8, and
    // the manager adds the partials in the order j = 0..7: the summation order of a row does not
    // depend on where the row sits in the matrix.
    if (warp == kConsumerWarps) {
        // ---- manager: fill stages, refill them as they are released, finish tiles -----------------
        int issued = 0;
        for (; issued < depth && issued < total; ++issued) issue(issued);
        int ti = 0, win = 0, u = 0, s = 0, pidx = 0, phase = 0, flushed = 0;
        uint32_t par = 0;
        bool direct = !SPEC;  // results go straight to y
        // y[row] of local tile `t` from its sum
        auto store_row = [&](int t, float sum) {
            const int row = ((int)blockIdx.x + t * (int)gridDim.x) * kTileRows + lane;
            if (lane < kTileRows && row < p.rows) p.y[row] = p.addend != nullptr ? sum + p.addend[row] : sum;
        };
        auto maybe_flush = [&]() {  // the table turned out valid: write what was held back
            if (direct || ld_volatile(&c->verdict) != kVerdictOk) return;
            for (; flushed < ti; ++flushed) store_row(flushed, lane < kTileRows ? results[flushed * kTileRows + lane] : 0.0f);
            direct = true;
        };
        bool alive = true;
#pragma unroll 1
        for (; u < total; ++u) {
            if (!wait_bar(c->done_bar + s, par)) {
                alive = false;
                break;
            }
            if (issued < total) issue(issued++);
            if (win == p.n_win - 1) {
                float sum = 0.0f;
                if (lane < kTileRows) {
                    const float* pp = partials + (size_t)pidx * kConsumerWarps * kTileRows + lane;
#pragma unroll
                    for (int j = 0; j < kConsumerWarps; ++j) sum += pp[((phase + j) & 7) * kTileRows];
                }
                if (SPEC) maybe_flush();
                if (direct) store_row(ti, sum);
                else if (lane < kTileRows) results[ti * kTileRows + lane] = sum;
                win = 0;
                ++ti;
                phase = (phase + p.bpr) & 7;
                if (++pidx > depth) pidx = 0;
            } else {
                ++win;
            }
            if (++s == depth) {
                s = 0;
                par ^= 1u;
            }
        }
        if (SPEC && alive) {  // everything computed: wait for the verdict, then publish
            uint32_t spins = 0;
            while (!ld_volatile(&c->verdict)) {
                poll_verify();
                __nanosleep(100);
                if (++spins > kSpinLimit || *abort_flag) {
                    if (lane == 0 && !*abort_flag) {
                        atomicAdd(p.timeouts, 1u);
                        *abort_flag = 1;
                    }
                    break;
                }
            }
            maybe_flush();
        }
        if (!alive) {
            // Gave up (stale table, or a wait that ran out): let the copies still in flight land before
            // the stages are reused or the CTA goes away.
            for (int v = max(0, issued - depth); v < issued; ++v) {
                uint32_t spins = 0;
                while (!mbar_try_wait(c->full_bar + v % depth, (uint32_t)(v / depth) & 1u) && ++spins < kSpinLimit) {
                }
            }
        }
        if (SPEC) {  // the verification needs every working warp, also after a stale verdict or an abort
            uint32_t spins = 0;
            while (!verified && ++spins < kSpinLimit && !*abort_flag) {
                poll_verify();
                if (!verified) __nanosleep(100);
            }
        }
    } else {
        // ---- consumers ---------------------------------------------------------------------------
        const LaneConst lc = lane_const(lane, p.neg_one, p.row_swap);
        float racc0 = 0.0f, racc1 = 0.0f;
        int win = 0, s = 0, pidx = 0, phase = 0;
        uint32_t par = 0;
#pragma unroll 1
        for (int u = 0; u < total; ++u) {
            if (SPEC) {
                poll_verify();
                if (ld_volatile(&c->verdict) == kVerdictRedo) break;
            }
            if (!wait_bar(c->full_bar + s, par)) break;
            const int b0 = win * p.kb;
            const int nb = min(p.kb, p.bpr - b0);
            const uint8_t* stage = stages + (size_t)s * stage_bytes;
#pragma unroll 1
            for (int i = (warp - phase - b0) & 7; i < nb; i += kConsumerWarps)
                process_block(stage + i * q4k::kBlockBytes, p.row_stride, xtab + (size_t)(b0 + i) * kXBlockBytes, lc,
                              racc0, racc1);
            if (win == p.n_win - 1) {
                racc0 += __shfl_xor_sync(0xFFFFFFFFu, racc0, 1);
                racc0 += __shfl_xor_sync(0xFFFFFFFFu, racc0, 2);
                racc1 += __shfl_xor_sync(0xFFFFFFFFu, racc1, 1);
                racc1 += __shfl_xor_sync(0xFFFFFFFFu, racc1, 2);
                if (lc.t == 0) {
                    float* pp = partials + ((size_t)pidx * kConsumerWarps + warp) * kTileRows;
                    pp[lc.row_a] = racc0;
                    pp[lc.row_b] = racc1;
                }
                racc0 = racc1 = 0.0f;
                win = 0;
                phase = (phase + p.bpr) & 7;
                if (++pidx > depth) pidx = 0;
            } else {
                ++win;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(c->done_bar + s);
            if (++s == depth) {
                s = 0;
                par ^= 1u;
            }
        }
        if (SPEC) {
            uint32_t spins = 0;
            while (!verified && ++spins < kSpinLimit && !*abort_flag) {
                poll_verify();
                if (!verified) __nanosleep(100);
            }
        }
    }
}

__device__ __forceinline__ void init_barriers(Control* c, int depth) {
    for (int s = 0; s < depth; ++s) {
        mbar_init(c->full_bar + s, 1);
        mbar_init(c->done_bar + s, kConsumerWarps);
    }
    mbar_init(&c->verified_bar, kConsumerWarps + 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Warps 0..7 consume, warp 8 manages the ring and the results, warp 9 (the sentinel) does nothing
// but wait for the previous kernel of the stream and judge the speculation.
__global__ void __launch_bounds__(kThreads, 2)
matvec_q4k_mma_kernel(const Params p, const __grid_constant__ CUtensorMap wmap) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ __align__(8) Control ctl;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (p.rows + kTileRows - 1) / kTileRows;
    const int max_tiles = (n_tiles + (int)gridDim.x - 1) / (int)gridDim.x;
    uint8_t* xtab = smem;
    float* partials = reinterpret_cast<float*>(smem + round128(p.bpr * kXBlockBytes));  // [depth+1][8][16]
    float* results = partials + (p.depth + 1) * kConsumerWarps * kTileRows;              // [max_tiles][16]
    uint8_t* stages = smem + round128(p.bpr * kXBlockBytes) +
                      round128(((p.depth + 1) * kConsumerWarps + max_tiles) * kTileRows * 4);
    const bool working = warp <= kConsumerWarps;

    if (!p.hold_trigger) griddep_launch_dependents();
    if (threadIdx.x == 0) {
        init_barriers(&ctl, p.depth);
        ctl.abort = 0;
        ctl.released = 0;
        ctl.mismatch = 0;
        ctl.verdict = 0;
    }
    __syncthreads();

    // Pass 0 (only with p.speculate): on x as it is NOW, while the kernel before this one may still
    // run.  Pass 1: on the final x, when there was no speculation or it turned out stale.
    bool spec = p.speculate != 0;
#pragma unroll 1
    for (int pass = 0; pass < 2; ++pass) {
        if (!spec) griddep_wait();  // x may be produced by the kernel launched just before this one
        if (working) {
            convert_mine(p.x, p.bpr, p.x_aligned, xtab, warp, lane, false);
            asm volatile("bar.sync 1, %0;" ::"n"((kConsumerWarps + 1) * 32) : "memory");
            run_pass(spec, p, &wmap, &ctl, xtab, partials, results, stages, warp, lane);
        } else if (spec) {
            griddep_wait();  // the kernel launched just before this one has completed
            if (lane == 0) {
                __threadfence_block();
                *reinterpret_cast<volatile int*>(&ctl.released) = 1;
                uint32_t spins = 0;
                bool ok = true;
                while (!mbar_try_wait(&ctl.verified_bar, 0u)) {
                    if (++spins > kSpinLimit || ld_volatile(&ctl.abort)) {
                        ok = false;
                        break;
                    }
                }
                if (!ok && !ld_volatile(&ctl.abort)) {
                    atomicAdd(p.timeouts, 1u);
                    *reinterpret_cast<volatile int*>(&ctl.abort) = 1;
                }
                __threadfence_block();
                *reinterpret_cast<volatile int*>(&ctl.verdict) = (ok && !ld_volatile(&ctl.mismatch)) ? kVerdictOk : kVerdictRedo;
            }
        }
        if (!spec) break;
        __syncthreads();
        if (ctl.verdict == kVerdictOk || ctl.abort) break;
        // x changed under the speculation: start over on the final x
        if (threadIdx.x == 0) {
            for (int s = 0; s < p.depth; ++s) {
                asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(ctl.full_bar + s)) : "memory");
                asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(ctl.done_bar + s)) : "memory");
            }
            asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(&ctl.verified_bar)) : "memory");
            init_barriers(&ctl, p.depth);
        }
        __syncthreads();
        spec = false;
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int kSmemTwoPerSm = 115456;  // two CTAs per SM: 2 x (this + static + 1 KiB reserved) <= 228 KiB
constexpr int kSmemOnePerSm = 226 * 1024;
constexpr int kMaxWindow = 14;  // super-blocks per stage row: 14 * 18 eight-byte elements <= 256 (TMA box limit)

struct Config {
    int n_win = 0, kb = 0, depth = 0, row_swap = 0, smem = 0;
};

// Rows lie dense in a stage (kb * 144 bytes apart).  The two tile rows a quarter-warp reads together
// must be 64 bytes apart modulo 128: rows r and r + 2^k with 2^k * kb = 4 (mod 8); none exists when
// kb is a multiple of 8.
int row_swap_for(int kb) {
    for (int k = 0; k < 3; ++k)
        if ((((1 << k) * kb) & 7) == 4) return k;
    return -1;
}

// The ring for rows of `bpr` super-blocks inside `budget` bytes of shared memory: the fewest windows
// per tile (every stage use costs a round of barrier traffic), then the deepest ring that fits.
bool pick_config(int bpr, int budget, int max_tiles, Config& best) {
    const int xtab = round128(bpr * kXBlockBytes);
    for (int n_win = (bpr + kMaxWindow - 1) / kMaxWindow; n_win <= bpr; ++n_win) {
        int kb = (bpr + n_win - 1) / n_win;
        if ((kb & 7) == 0) {  // widen the window by one if the split stays valid
            if (kb + 1 > kMaxWindow || (n_win - 1) * (kb + 1) >= bpr) continue;
            ++kb;
        }
        if ((n_win - 1) * kb >= bpr) continue;
        const int swap = row_swap_for(kb);
        if (swap < 0) continue;
        const int stage = kTileRows * kb * q4k::kBlockBytes;
        for (int depth = kMaxDepth; depth >= 3; --depth) {
            const int smem = xtab + round128(((depth + 1) * kConsumerWarps + max_tiles) * kTileRows * 4) + depth * stage;
            if (smem > budget) continue;
            best = Config{n_win, kb, depth, swap, smem};
            return true;
        }
    }
    return false;
}

using mg::encode_tiled;
using mg::EncodeTiledFn;

}  // namespace

bool supported(int blocks_per_row) {
    Config c;
    return blocks_per_row > 0 && encode_tiled() != nullptr && pick_config(blocks_per_row, kSmemOnePerSm, 64, c);
}

bool fits_half_sm(int blocks_per_row) {
    Config c;
    // ... with whole rows in a stage: windows of longer rows cost a round of barrier traffic each
    return blocks_per_row > 0 && encode_tiled() != nullptr && pick_config(blocks_per_row, kSmemTwoPerSm, 16, c) &&
           c.n_win == 1;
}

cudaError_t launch(const uint8_t* w, const float* x, const float* addend, float* y, int rows, int bpr,
                   int hold_trigger, int speculate, unsigned* timeouts, int sms, cudaStream_t stream) {
    Config c;
    const int n_tiles = (rows + kTileRows - 1) / kTileRows;
    const int grid = n_tiles < sms ? n_tiles : sms;
    const int max_tiles = (n_tiles + grid - 1) / grid;
    // Half an SM when a useful ring fits beside the operand table (the successor kernel can then be
    // resident early); the whole SM for long rows.
    if (!pick_config(bpr, kSmemTwoPerSm, max_tiles, c) && !pick_config(bpr, kSmemOnePerSm, max_tiles, c))
        return cudaErrorInvalidValue;
    const EncodeTiledFn encode = encode_tiled();
    if (encode == nullptr) return cudaErrorNotSupported;
    // The weight matrix as a 2-D tensor of 8-byte elements: [rows][bpr * 18]; box = 16 rows x kb * 18.
    CUtensorMap wmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)bpr * 18u, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)bpr * q4k::kBlockBytes};
    const cuuint32_t box[2] = {(cuuint32_t)c.kb * 18u, (cuuint32_t)kTileRows};
    const cuuint32_t estride[2] = {1u, 1u};
    if (encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(w), gdim, gstride, box, estride,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return cudaErrorInvalidValue;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(matvec_q4k_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             kSmemOnePerSm);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(matvec_q4k_mma_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 (int)cudaSharedmemCarveoutMaxShared);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    Params p = {};
    p.w = w; p.x = x; p.addend = addend; p.y = y;
    p.rows = rows; p.bpr = bpr;
    p.n_win = c.n_win; p.kb = c.kb; p.depth = c.depth; p.row_stride = c.kb * q4k::kBlockBytes; p.row_swap = c.row_swap;
    p.x_aligned = mg::aligned16(x) ? 1 : 0;
    p.hold_trigger = hold_trigger;
    p.speculate = speculate;
    p.timeouts = timeouts;
    p.neg_one = 0xFFFFFFFFu;
    return mg::launch_pdl(matvec_q4k_mma_kernel, dim3((unsigned)grid), dim3(kThreads), (size_t)c.smem, stream, p, wmap);
}

}  // namespace gemvmma
