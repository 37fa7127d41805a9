// Q5_K and Q6_K: the other two K-quant formats real GGUF checkpoints mix with Q4_K (LM head and
// token embedding are Q6_K, attn_v / ffn_down often Q5_K: crates/modgrad-gemma/src/rocm_gemma.rs:295-297, :338).
//
//   launch_matvec_q5k       replaces crates/modgrad-device/kernels/matvec_q5k.hip:55-121
//   launch_matvec_q6k       replaces crates/modgrad-device/kernels/matvec_q6k.hip:32-94
//   mg_matvec_kquant_on_stream: either of them with the residual add of the decode loop folded in, from f32
//                           activations or from limb records
//   mg_embed_kquant_on_stream: one row of a Q4_K / Q5_K / Q6_K embedding table, the token in device memory
//   launch_matvec_q6k_dp4a  replaces crates/modgrad-device/kernels/matvec_q6k_dp4a.hip:56-150 (int8 activations
//                           from launch_quantize_q8_1; lossy like its Q4_K sibling)
//   mg_dequant_q5k / mg_dequant_q6k_on_stream: bulk dequantisation, bit-exact against the host
//                           dequantisers (crates/modgrad-device/src/kfd/gguf.rs:421-455, :458-484);
//                           no device counterpart in the reference (it dequantises these on the host).
//
// Block formats (256 weights each):
//   Q5_K, 176 bytes: d half, dmin half, scales[12] (as Q4_K), qh[32], ql[128]; element 64g + 32hi + l =
//        nibble hi of ql[32g + l] + 16 * bit (2g + hi) of qh[l];  w = fl(fl(d*sc) * q) - fl(dmin*m).
//   Q6_K, 210 bytes: ql[128], qh[64], sc[16] signed bytes, d half at +208; element 128G + 32k + l =
//        (nibble (k >= 2) of ql[64G + 32(k&1) + l] | bits 2k,2k+1 of qh[32G + l] << 4) - 32, scale
//        sc[8G + 2k + l/16];  w = fl(fl(d*sc) * q).  Rows are only 2-byte aligned (210 = 2 * 105).
//
// Matvecs: the limb kernels further down (integer dot products with dp4a on the activation records of
// xlimbs.cuh) whenever the weight is 4-byte aligned and the records of a row fit one CTA's shared memory;
// otherwise the float kernel: a CTA owns a few consecutive rows and its warps split the rows'
// super-blocks, one block per warp and step; a lane owns adjacent columns of every quant group (packed
// 32-bit loads for Q5_K, 16-bit for the 2-byte-aligned Q6_K), eight weights per lane and block, f32
// accumulate, warp-shuffle then fixed-order cross-warp reduction.  The dequantisers keep one warp per
// block with byte loads.
#include <float.h>

#include "gemv_q4k_device.cuh"
#include "launch_common.cuh"
#include "q4k_device.cuh"
#include "xlimbs.cuh"

namespace {

constexpr int kQ5Bytes = 176, kQ6Bytes = 210;
constexpr int kThreads = 256, kWarps = kThreads / 32;

struct Q5Header {
    float dsc[8], dm[8];  // fl(d * sc[s]), fl(dmin * m[s])
};
// b is 16-byte aligned (176 = 11 * 16 and the tensor base is).
__device__ __forceinline__ Q5Header q5_header(const uint8_t* b) {
    const uint4 h = *reinterpret_cast<const uint4*>(b);
    const float d = q4k::half_bits_finite_or_zero(h.x);
    const float dmin = q4k::half_bits_finite_or_zero(h.x >> 16);
    const q4k::ScaleMin sm = q4k::unpack_scales(h.y, h.z, h.w);
    Q5Header r;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        r.dsc[s] = __fmul_rn(d, (float)q4k::scale_of(sm, s));
        r.dm[s] = __fmul_rn(dmin, (float)q4k::min_of(sm, s));
    }
    return r;
}

__global__ void __launch_bounds__(kThreads) dequant_q5k_kernel(const uint8_t* __restrict__ q, float* __restrict__ out,
                                                               int n_blocks) {
    const int lane = threadIdx.x & 31;
    for (int blk = blockIdx.x * kWarps + (threadIdx.x >> 5); blk < n_blocks; blk += gridDim.x * kWarps) {
        const uint8_t* b = q + (size_t)blk * kQ5Bytes;
        const Q5Header h = q5_header(b);
        const uint32_t qh = b[16 + lane];
        float* o = out + (size_t)blk * 256;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t v = b[48 + 32 * g + lane];
            const float q_lo = (float)((v & 0xFu) + (((qh >> (2 * g)) & 1u) << 4));
            const float q_hi = (float)((v >> 4) + (((qh >> (2 * g + 1)) & 1u) << 4));
            o[64 * g + lane] = __fsub_rn(__fmul_rn(h.dsc[2 * g], q_lo), h.dm[2 * g]);
            o[64 * g + 32 + lane] = __fsub_rn(__fmul_rn(h.dsc[2 * g + 1], q_hi), h.dm[2 * g + 1]);
        }
    }
}

// The four 6-bit quants of lane l in group G of a Q6_K block, as signed ints in [-32, 31].
__device__ __forceinline__ void q6_quants(const uint8_t* b, int G, int lane, int (&q)[4]) {
    const uint32_t a = b[64 * G + lane], c = b[64 * G + 32 + lane], h = b[128 + 32 * G + lane];
    q[0] = (int)((a & 0xFu) | ((h & 3u) << 4)) - 32;
    q[1] = (int)((c & 0xFu) | (((h >> 2) & 3u) << 4)) - 32;
    q[2] = (int)((a >> 4) | (((h >> 4) & 3u) << 4)) - 32;
    q[3] = (int)((c >> 4) | (((h >> 6) & 3u) << 4)) - 32;
}
__device__ __forceinline__ float q6_d(const uint8_t* b) {
    return q4k::half_bits_finite_or_zero((uint32_t)b[208] | ((uint32_t)b[209] << 8));
}

__global__ void __launch_bounds__(kThreads) dequant_q6k_kernel(const uint8_t* __restrict__ q, float* __restrict__ out,
                                                               int n_blocks) {
    const int lane = threadIdx.x & 31;
    for (int blk = blockIdx.x * kWarps + (threadIdx.x >> 5); blk < n_blocks; blk += gridDim.x * kWarps) {
        const uint8_t* b = q + (size_t)blk * kQ6Bytes;
        const float d = q6_d(b);
        const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
        float* o = out + (size_t)blk * 256;
#pragma unroll
        for (int G = 0; G < 2; ++G) {
            int qv[4];
            q6_quants(b, G, lane, qv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float ds = __fmul_rn(d, (float)sc[8 * G + 2 * k + (lane >> 4)]);
                o[128 * G + 32 * k + lane] = __fmul_rn(ds, (float)qv[k]);
            }
        }
    }
}

// One row of a quantised token-embedding table, dequantised exactly as the bulk dequantisers do
// (the reference dequantises the row on the host and uploads it: crates/modgrad-gemma/src/rocm_gemma.rs:316-323).
// The token is a device-side integer, so the launch can sit in a replayed graph.  One warp per super-block.
template <int KIND>
__global__ void __launch_bounds__(kThreads) embed_kquant_kernel(const uint8_t* __restrict__ table, const int* token_dev,
                                                                int token_arg, float* __restrict__ out, int bpr,
                                                                int vocab) {
    mg::pdl_prologue();
    int tok = token_dev ? *token_dev : token_arg;
    tok = min(max(tok, 0), vocab - 1);
    const int lane = threadIdx.x & 31;
    const int blk = blockIdx.x * kWarps + (threadIdx.x >> 5);
    if (blk >= bpr) return;
    constexpr int kBytes = KIND == 4 ? 144 : KIND == 5 ? kQ5Bytes : kQ6Bytes;
    const uint8_t* b = table + ((size_t)tok * bpr + blk) * kBytes;
    float* o = out + (size_t)blk * 256;
    if (KIND == 4) {
        const uint4 h = *reinterpret_cast<const uint4*>(b);
        const float d = q4k::half_bits_finite_or_zero(h.x);
        const float dmin = q4k::half_bits_finite_or_zero(h.x >> 16);
        const q4k::ScaleMin sm = q4k::unpack_scales(h.y, h.z, h.w);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t v = b[16 + 32 * g + lane];
            const float d_lo = __fmul_rn(d, (float)q4k::scale_of(sm, 2 * g)), m_lo = __fmul_rn(dmin, (float)q4k::min_of(sm, 2 * g));
            const float d_hi = __fmul_rn(d, (float)q4k::scale_of(sm, 2 * g + 1)),
                        m_hi = __fmul_rn(dmin, (float)q4k::min_of(sm, 2 * g + 1));
            o[64 * g + lane] = __fsub_rn(__fmul_rn(d_lo, (float)(v & 0xFu)), m_lo);
            o[64 * g + 32 + lane] = __fsub_rn(__fmul_rn(d_hi, (float)(v >> 4)), m_hi);
        }
    } else if (KIND == 5) {
        const Q5Header h = q5_header(b);
        const uint32_t qh = b[16 + lane];
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint32_t v = b[48 + 32 * g + lane];
            const float q_lo = (float)((v & 0xFu) + (((qh >> (2 * g)) & 1u) << 4));
            const float q_hi = (float)((v >> 4) + (((qh >> (2 * g + 1)) & 1u) << 4));
            o[64 * g + lane] = __fsub_rn(__fmul_rn(h.dsc[2 * g], q_lo), h.dm[2 * g]);
            o[64 * g + 32 + lane] = __fsub_rn(__fmul_rn(h.dsc[2 * g + 1], q_hi), h.dm[2 * g + 1]);
        }
    } else {
        const float d = q6_d(b);
        const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
#pragma unroll
        for (int G = 0; G < 2; ++G) {
            int qv[4];
            q6_quants(b, G, lane, qv);
#pragma unroll
            for (int k = 0; k < 4; ++k)
                o[128 * G + 32 * k + lane] = __fmul_rn(__fmul_rn(d, (float)sc[8 * G + 2 * k + (lane >> 4)]), (float)qv[k]);
        }
    }
}

// The float 2^23 + b for byte I of `packed` (one byte permute): subtracting 2^23 (+ an offset) is exact.
template <int I>
__device__ __forceinline__ float byte_as_f(uint32_t packed) {
    return __uint_as_float(__byte_perm(packed, 0x4B000000u, 0x7540 + I));
}
__device__ __forceinline__ float2 ld_x2(const float* p, bool aligned) {
    return aligned ? *reinterpret_cast<const float2*>(p) : make_float2(p[0], p[1]);
}
__device__ __forceinline__ float4 ld_x4(const float* p, bool aligned) {
    return aligned ? *reinterpret_cast<const float4*>(p) : make_float4(p[0], p[1], p[2], p[3]);
}

// kind 5 / 6; x is read after the previous kernel of the stream has completed.
// A CTA of WARPS warps owns R consecutive rows at a time; its warps split the rows' super-blocks among
// them (warp w takes blocks w, w + WARPS, ...), so a long row is read by many loads in flight instead of
// one warp's serial walk, and every activation load serves R rows.  Within a block a lane owns a few
// adjacent columns of every quant group, extracts them four (Q5_K) or two (Q6_K) at a time from packed
// words, and applies each sub-block's scale once per group of columns, not once per weight.
template <int KIND, int R, int WARPS>
__global__ void __launch_bounds__(WARPS * 32) matvec_kquant_kernel(const uint8_t* __restrict__ w, const float* x,
                                                                   const float* add, float* y, int out_dim, int bpr,
                                                                   int x_aligned, int hold_trigger) {
    mg::pdl_prologue(hold_trigger);
    __shared__ float part[WARPS][R];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kBytes = KIND == 5 ? kQ5Bytes : kQ6Bytes;
    const bool xa = x_aligned != 0;
    for (int row0 = blockIdx.x * R; row0 < out_dim; row0 += gridDim.x * R) {
        float acc[R];
        const uint8_t* wr[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            acc[r] = 0.0f;
            wr[r] = w + (size_t)min(row0 + r, out_dim - 1) * bpr * kBytes;  // a row past the end repeats the last one
        }
        for (int blk = warp; blk < bpr; blk += WARPS) {
            const float* xb = x + (size_t)blk * 256;
            if (KIND == 5) {
                // lane: quant group g (64 columns), columns 4j..4j+3 of its low and of its high nibble half
                const int g = lane >> 3, j = lane & 7;
                const float4 xl = ld_x4(xb + 64 * g + 4 * j, xa), xh = ld_x4(xb + 64 * g + 32 + 4 * j, xa);
                const float sxl = (xl.x + xl.y) + (xl.z + xl.w), sxh = (xh.x + xh.y) + (xh.z + xh.w);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint8_t* b = wr[r] + (size_t)blk * kQ5Bytes;
                    const uint4 h = q4k::ld_nc_u4(b);
                    const uint32_t v = *reinterpret_cast<const uint32_t*>(b + 48 + 32 * g + 4 * j);
                    const uint32_t qh = *reinterpret_cast<const uint32_t*>(b + 16 + 4 * j);
                    const float d = q4k::half_bits_finite_or_zero(h.x), dmin = q4k::half_bits_finite_or_zero(h.x >> 16);
                    const q4k::ScaleMin sm = q4k::unpack_scales(h.y, h.z, h.w);
                    const uint32_t ql = (v & 0x0F0F0F0Fu) | (((qh >> (2 * g)) & 0x01010101u) << 4);
                    const uint32_t qu = ((v >> 4) & 0x0F0F0F0Fu) | (((qh >> (2 * g + 1)) & 0x01010101u) << 4);
                    constexpr float k23 = 8388608.0f;
                    float tl = (byte_as_f<0>(ql) - k23) * xl.x, tu = (byte_as_f<0>(qu) - k23) * xh.x;
                    tl = fmaf(byte_as_f<1>(ql) - k23, xl.y, tl); tu = fmaf(byte_as_f<1>(qu) - k23, xh.y, tu);
                    tl = fmaf(byte_as_f<2>(ql) - k23, xl.z, tl); tu = fmaf(byte_as_f<2>(qu) - k23, xh.z, tu);
                    tl = fmaf(byte_as_f<3>(ql) - k23, xl.w, tl); tu = fmaf(byte_as_f<3>(qu) - k23, xh.w, tu);
                    const float dl = d * (float)q4k::scale_of(sm, 2 * g), du = d * (float)q4k::scale_of(sm, 2 * g + 1);
                    const float ml = dmin * (float)q4k::min_of(sm, 2 * g), mu = dmin * (float)q4k::min_of(sm, 2 * g + 1);
                    acc[r] += fmaf(dl, tl, -ml * sxl) + fmaf(du, tu, -mu * sxh);
                }
            } else {
                // lane: half G of the block (128 columns), columns 2j, 2j+1 of each of its four 32-column groups
                // (Q6_K blocks are only 2-byte aligned: 16-bit loads)
                const int G = lane >> 4, j = lane & 15;
                const float* xg = xb + 128 * G + 2 * j;
                const float2 x0 = ld_x2(xg, xa), x1 = ld_x2(xg + 32, xa), x2 = ld_x2(xg + 64, xa), x3 = ld_x2(xg + 96, xa);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const uint8_t* b = wr[r] + (size_t)blk * kQ6Bytes;
                    const uint32_t a = *reinterpret_cast<const uint16_t*>(b + 64 * G + 2 * j);
                    const uint32_t c = *reinterpret_cast<const uint16_t*>(b + 64 * G + 32 + 2 * j);
                    const uint32_t h = *reinterpret_cast<const uint16_t*>(b + 128 + 32 * G + 2 * j);
                    const uint8_t* sc = b + 192 + 8 * G + (j >> 3);   // scales of groups k = 0..3 at sc[2k], as signed bytes
                    const float d = q4k::half_bits_finite_or_zero(*reinterpret_cast<const uint16_t*>(b + 208));
                    const uint32_t q0 = (a & 0x0F0Fu) | ((h & 0x0303u) << 4), q1 = (c & 0x0F0Fu) | (((h >> 2) & 0x0303u) << 4);
                    const uint32_t q2 = ((a >> 4) & 0x0F0Fu) | (((h >> 4) & 0x0303u) << 4),
                                   q3 = ((c >> 4) & 0x0F0Fu) | (((h >> 6) & 0x0303u) << 4);
                    constexpr float kq = 8388608.0f + 32.0f;     // quants are stored with +32
                    constexpr float ks = 8388608.0f + 128.0f;    // signed scale byte ^ 0x80 = scale + 128
                    const float t0 = fmaf(byte_as_f<1>(q0) - kq, x0.y, (byte_as_f<0>(q0) - kq) * x0.x);
                    const float t1 = fmaf(byte_as_f<1>(q1) - kq, x1.y, (byte_as_f<0>(q1) - kq) * x1.x);
                    const float t2 = fmaf(byte_as_f<1>(q2) - kq, x2.y, (byte_as_f<0>(q2) - kq) * x2.x);
                    const float t3 = fmaf(byte_as_f<1>(q3) - kq, x3.y, (byte_as_f<0>(q3) - kq) * x3.x);
                    const float s0 = byte_as_f<0>((uint32_t)sc[0] ^ 0x80u) - ks, s1 = byte_as_f<0>((uint32_t)sc[2] ^ 0x80u) - ks;
                    const float s2 = byte_as_f<0>((uint32_t)sc[4] ^ 0x80u) - ks, s3 = byte_as_f<0>((uint32_t)sc[6] ^ 0x80u) - ks;
                    acc[r] = fmaf(d, fmaf(s0, t0, s1 * t1) + fmaf(s2, t2, s3 * t3), acc[r]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = q4k::warp_sum(acc[r]);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; ++r) part[warp][r] = acc[r];
        }
        __syncthreads();
        if (threadIdx.x < R && row0 + threadIdx.x < out_dim) {
            float t = 0.0f;
#pragma unroll
            for (int wv = 0; wv < WARPS; ++wv) t += part[wv][threadIdx.x];   // fixed order: the same sum on every run
            y[row0 + threadIdx.x] = add ? add[row0 + threadIdx.x] + t : t;
        }
        __syncthreads();
    }
}

// ---- Q5_K / Q6_K on limb records ------------------------------------------------------------------
// The float kernel above spends about 12 lane-operations per weight (a byte permute, a subtraction
// and a multiply-add for each, plus the extraction) and is bound by instruction issue at a quarter of
// the memory bandwidth.  These kernels multiply the quants with the activations in integers, as the
// Q4_K kernels do (xlimbs.cuh): the activations are three byte limbs sharing one power-of-two scale
// per 32 elements, the quants are bytes (Q6_K: sign-extended; Q5_K: unsigned, the minimum applied
// through the records' sum word), and eight weights meet their activations in six dp4a.  The integer
// sums are exact; the result differs from the float kernel's by the rounding of the activations to
// 23 bits of their sub-block's largest element.
//
// Eight lanes cover a block, 32 weights each (the two formats split a block differently: Q6Fmt, Q5Fmt).
// Two kernel bodies: a warp takes four blocks per step of R rows at a time (many short rows), or a
// CTA per SM walks the (row, block) pairs of its rows with 96 eight-lane groups (few or long rows);
// every CTA keeps the whole activation vector as limb records in shared memory.
__device__ __forceinline__ int dp4a_su(uint32_t a_signed, uint32_t b_unsigned, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a_signed), "r"(b_unsigned), "r"(c));
    return d;
}
// Eight bytes from a 2-byte-aligned address inside a 4-byte-aligned array: three aligned words
// funnel-shifted.  Reads up to 2 bytes before and 6 bytes after the eight.
__device__ __forceinline__ uint2 ld8_align2(const uint8_t* p) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t* q = reinterpret_cast<const uint32_t*>(a & ~(uintptr_t)3);
    const uint32_t sh = (uint32_t)(a & 2u) * 8u;
    const uint32_t w0 = __ldg(q), w1 = __ldg(q + 1), w2 = __ldg(q + 2);
    return make_uint2(__funnelshift_r(w0, w1, sh), __funnelshift_r(w1, w2, sh));
}
// Four 6-bit quants (stored + 32) of group K as sign-extended bytes: nibbles of ql word `lo`,
// bits 2K, 2K+1 of every byte of qh word `h`.
template <int K>
__device__ __forceinline__ uint32_t q6_signed4(uint32_t lo, uint32_t h) {
    const uint32_t u = (K >= 2 ? lo >> 4 : lo) & 0x0F0F0F0Fu;
    const uint32_t hs = K == 0 ? h << 4 : K == 1 ? h << 2 : K == 2 ? h : h >> 2;
    const uint32_t q = u | (hs & 0x30303030u);            // 0..63
    const uint32_t neg = ~q & 0x20202020u;                // below 32: negative once 32 is taken off
    return (q ^ 0x20202020u) + neg * 6u;                  // bit 5 flipped, bits 6 and 7 set where negative
}

// A format for the limb kernels: the packed weights one lane keeps of one block (Lane), their loads, and
// the R rows' dot products with block `blk` of the activations.  `sub` = lane & 7: eight lanes cover a block.
//
// Q6_K: lane (G = sub / 4, qtr = sub % 4) owns columns 8 qtr .. 8 qtr + 7 of the four 32-column groups of half G.
struct Q6Fmt {
    static constexpr int kBytes = kQ6Bytes;
    struct Lane {
        uint2 ql0, ql1, qh;
        int sc[4];
        uint32_t d_bits;
    };
    static __device__ __forceinline__ void load(Lane& t, const uint8_t* b, int sub) {
        const int G = sub >> 2, qtr = sub & 3;
        t.ql0 = ld8_align2(b + 64 * G + 8 * qtr);
        t.ql1 = ld8_align2(b + 64 * G + 32 + 8 * qtr);
        t.qh = ld8_align2(b + 128 + 32 * G + 8 * qtr);
        const int8_t* s8 = reinterpret_cast<const int8_t*>(b + 192 + 8 * G + (qtr >> 1));
#pragma unroll
        for (int k = 0; k < 4; ++k) t.sc[k] = (int)s8[2 * k];
        t.d_bits = *reinterpret_cast<const uint16_t*>(b + 208);
    }
    // acc[r] += d_r * sum_k sc_rk * s_k * <q_rk, a_k>;  rec_w: the limb records of the whole vector
    template <int R>
    static __device__ __forceinline__ void dot(const Lane (&t)[R], const uint32_t* rec_w, int blk, int sub, float (&acc)[R]) {
        const int G = sub >> 2, qtr = sub & 3;
    float part[R];
#pragma unroll
    for (int r = 0; r < R; ++r) part[r] = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        // activations of sub-block 4G + k: record 2G + k/2, low or high plane set, words 2qtr, 2qtr + 1
        const uint32_t* rp = rec_w + (size_t)(blk * 4 + 2 * G + (k >> 1)) * xlimbs::kRecordWords;
        const uint32_t* lp = rp + (k & 1) * 24 + 2 * qtr;
        const uint2 a2 = *reinterpret_cast<const uint2*>(lp);
        const uint2 a1 = *reinterpret_cast<const uint2*>(lp + 8);
        const uint2 a0 = *reinterpret_cast<const uint2*>(lp + 16);
        const float s = __uint_as_float(rp[48 + (k & 1)]);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint2 lo = (k & 1) ? t[r].ql1 : t[r].ql0;
            uint32_t qa, qb;
            if (k == 0) { qa = q6_signed4<0>(lo.x, t[r].qh.x); qb = q6_signed4<0>(lo.y, t[r].qh.y); }
            else if (k == 1) { qa = q6_signed4<1>(lo.x, t[r].qh.x); qb = q6_signed4<1>(lo.y, t[r].qh.y); }
            else if (k == 2) { qa = q6_signed4<2>(lo.x, t[r].qh.x); qb = q6_signed4<2>(lo.y, t[r].qh.y); }
            else { qa = q6_signed4<3>(lo.x, t[r].qh.x); qb = q6_signed4<3>(lo.y, t[r].qh.y); }
            const int i2 = gemvdev::dp4a_ss(qb, a2.y, gemvdev::dp4a_ss(qa, a2.x, 0));
            const int i1 = dp4a_su(qb, a1.y, dp4a_su(qa, a1.x, 0));
            const int i0 = dp4a_su(qb, a0.y, dp4a_su(qa, a0.x, 0));
            // |i2| <= 2^15, |i1 * 256 + i0| < 2^24: both conversions are exact
            const float f = fmaf((float)i2, 65536.0f, (float)(i1 * 256 + i0));
            part[r] = fmaf(f * s, (float)t[r].sc[k], part[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = fmaf(q4k::half_bits_finite_or_zero(t[r].d_bits), part[r], acc[r]);
    }
};

// Q5_K: lane (g = sub / 2, half = sub % 2) owns columns 16 half .. 16 half + 15 of both 32-column sub-blocks of
// quant group g: 16 `ql` bytes (low nibbles: sub-block 2g, high: 2g + 1), the 16 `qh` bytes of those columns
// (bit 2g + hi of each) and the header, three 16-byte loads (blocks are 16-byte aligned).  The quants stay
// unsigned; the minimum enters once per sub-block through the record's s * sum(a) word, added by half 0.
struct Q5Fmt {
    static constexpr int kBytes = kQ5Bytes;
    struct Lane {
        uint4 hdr, ql, qh;
    };
    static __device__ __forceinline__ void load(Lane& t, const uint8_t* b, int sub) {
        const int g = sub >> 1, half = sub & 1;
        t.hdr = q4k::ld_nc_u4(b);
        t.qh = q4k::ld_nc_u4(b + 16 + 16 * half);
        t.ql = q4k::ld_nc_u4(b + 48 + 32 * g + 16 * half);
    }
    template <int R>
    static __device__ __forceinline__ void dot(const Lane (&t)[R], const uint32_t* rec_w, int blk, int sub, float (&acc)[R]) {
        const int g = sub >> 1, half = sub & 1;
        const uint32_t* rp = rec_w + (size_t)(blk * 4 + g) * xlimbs::kRecordWords;
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            // activations of sub-block 2g + hi: plane set hi of record g, words 4 half .. 4 half + 3
            const uint32_t* lp = rp + hi * 24 + 4 * half;
            const uint4 a2 = *reinterpret_cast<const uint4*>(lp);
            const uint4 a1 = *reinterpret_cast<const uint4*>(lp + 8);
            const uint4 a0 = *reinterpret_cast<const uint4*>(lp + 16);
            const float s = __uint_as_float(rp[48 + hi]);
            const float sx = half == 0 ? __uint_as_float(rp[50 + hi]) : 0.0f;   // s * sum(a) of the whole sub-block
            const int bit = 2 * g + hi;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const uint32_t v[4] = {t[r].ql.x, t[r].ql.y, t[r].ql.z, t[r].ql.w};
                const uint32_t h[4] = {t[r].qh.x, t[r].qh.y, t[r].qh.z, t[r].qh.w};
                const uint32_t l2[4] = {a2.x, a2.y, a2.z, a2.w}, l1[4] = {a1.x, a1.y, a1.z, a1.w}, l0[4] = {a0.x, a0.y, a0.z, a0.w};
                int i2 = 0;
                uint32_t i1 = 0, i0 = 0;
#pragma unroll
                for (int wd = 0; wd < 4; ++wd) {
                    const uint32_t q = ((hi ? v[wd] >> 4 : v[wd]) & 0x0F0F0F0Fu) | (((h[wd] >> bit) & 0x01010101u) << 4);   // 0..31
                    i2 = gemvdev::dp4a_us(q, l2[wd], i2);
                    i1 = gemvdev::dp4a_uu(q, l1[wd], i1);
                    i0 = gemvdev::dp4a_uu(q, l0[wd], i0);
                }
                // |i2| < 2^15, i1 and i0 < 2^17: the conversions are exact, the two fused adds round
                const float f = fmaf((float)i2, 65536.0f, fmaf((float)i1, 256.0f, (float)i0));
                const float d = q4k::half_bits_finite_or_zero(t[r].hdr.x), dmin = q4k::half_bits_finite_or_zero(t[r].hdr.x >> 16);
                const q4k::ScaleMin sm = q4k::unpack_scales(t[r].hdr.y, t[r].hdr.z, t[r].hdr.w);
                const float dsc = d * (float)q4k::scale_of(sm, bit), dm = dmin * (float)q4k::min_of(sm, bit);
                acc[r] = fmaf(dsc, f * s, fmaf(-dm, sx, acc[r]));
            }
        }
    }
};

// The activation vector as limb records in shared memory.  FROM_X = 1: src is the f32 vector, converted
// here; 0: src holds records (mg_q4k_x_to_limbs_on_stream, mg_swiglu_limbs_on_stream).  With norm_w
// (FROM_X only) the vector is RMS-normalised first (crates/modgrad-device/src/kfd/llm.rs:921-928, Plain):
// x * (1 / sqrt(mean(x^2) + eps)) * w, the sum of squares in one pass, the scaling in a second one that
// reads x again (it is in L2) instead of keeping it in registers.
template <int FROM_X, int THREADS>
__device__ __forceinline__ void limbs_stage_records(const void* src, int bpr, int x_aligned, uint4* rec_s,
                                                    const float* norm_w = nullptr, float eps = 0.0f) {
    if (FROM_X) {
        const float* x = static_cast<const float*>(src);
        const int n_chunks = bpr * 64;   // a multiple of 64: warps are whole
        float inv = 1.0f;
        const bool w_aligned = (reinterpret_cast<uintptr_t>(norm_w) & 15u) == 0;
        if (norm_w != nullptr) {
            __shared__ float red[THREADS / 32 + 1];
            float p = 0.0f;
            for (int c = threadIdx.x; c < n_chunks; c += THREADS) {
                float v[4];
                gemvdev::load_chunk<false>(v, x, c, x_aligned);
#pragma unroll
                for (int i = 0; i < 4; ++i) p = fmaf(v[i], v[i], p);
            }
            p = q4k::warp_sum(p);
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = p;
            __syncthreads();
            if (threadIdx.x < 32) {
                float t = threadIdx.x < THREADS / 32 ? red[threadIdx.x] : 0.0f;
                t = q4k::warp_sum(t);
                if (threadIdx.x == 0) red[THREADS / 32] = t;
            }
            __syncthreads();
            inv = 1.0f / sqrtf(red[THREADS / 32] / (float)(bpr * 256) + eps);
        }
        for (int c = threadIdx.x; c < n_chunks; c += THREADS) {
            float v[4];
            gemvdev::load_chunk<false>(v, x, c, x_aligned);
            if (norm_w != nullptr) {
                float wv[4];
                gemvdev::load_chunk<false>(wv, norm_w, c, w_aligned ? 1 : 0);
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = v[i] * inv * wv[i];
            }
            gemvdev::convert_chunk(v, c, reinterpret_cast<uint32_t*>(rec_s));
        }
    } else {
        const uint4* rec_g = static_cast<const uint4*>(src);
        const int n_vec = bpr * 4 * xlimbs::kRecordVec4;
        for (int i = threadIdx.x; i < n_vec; i += THREADS) gemvdev::cp_async16(&rec_s[i], &rec_g[i]);
        gemvdev::cp_async_wait_all();
    }
    __syncthreads();
}

constexpr int kLimbThreads = 256, kLimbWarps = kLimbThreads / 32;

// Short rows, many of them: a warp owns R rows at a time and walks their blocks four per step.
// y[row] = (add ? add[row] : 0) + W[row] . x.
template <class FMT, int R, int FROM_X>
__device__ __forceinline__ void limbs_short_body(const uint8_t* __restrict__ w, const void* src, const float* add, float* y,
                                                 int out_dim, int bpr, int x_aligned, int hold_trigger, const float* norm_w,
                                                 float eps) {
    extern __shared__ __align__(16) uint4 rec_s[];
    const uint32_t* rec_w = reinterpret_cast<const uint32_t*>(rec_s);
    mg::pdl_prologue(hold_trigger);
    limbs_stage_records<FROM_X, kLimbThreads>(src, bpr, x_aligned, rec_s, norm_w, eps);

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int bsel = lane >> 3, sub = lane & 7;
    const size_t row_bytes = (size_t)bpr * FMT::kBytes;
    for (int row0 = (blockIdx.x * kLimbWarps + warp) * R; row0 < out_dim; row0 += gridDim.x * kLimbWarps * R) {
        float acc[R];
        const uint8_t* wr[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            acc[r] = 0.0f;
            wr[r] = w + (size_t)min(row0 + r, out_dim - 1) * row_bytes;   // a row past the end repeats the last one
        }
        for (int blk = bsel; blk < bpr; blk += 4) {
            typename FMT::Lane t[R];
#pragma unroll
            for (int r = 0; r < R; ++r) FMT::load(t[r], wr[r] + (size_t)blk * FMT::kBytes, sub);
            FMT::template dot<R>(t, rec_w, blk, sub, acc);
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float t = q4k::warp_sum(acc[r]);
            if (lane == 0 && row0 + r < out_dim) y[row0 + r] = add ? add[row0 + r] + t : t;
        }
    }
}
template <int R, int FROM_X>
__global__ void __launch_bounds__(kLimbThreads, 4) matvec_q6k_limbs_kernel(const uint8_t* __restrict__ w, const void* src,
                                                                           const float* add, float* y, int out_dim, int bpr,
                                                                           int x_aligned, int hold_trigger, const float* norm_w,
                                                                           float eps) {
    limbs_short_body<Q6Fmt, R, FROM_X>(w, src, add, y, out_dim, bpr, x_aligned, hold_trigger, norm_w, eps);
}
template <int R, int FROM_X>
__global__ void __launch_bounds__(kLimbThreads, 3) matvec_q5k_limbs_kernel(const uint8_t* __restrict__ w, const void* src,
                                                                           const float* add, float* y, int out_dim, int bpr,
                                                                           int x_aligned, int hold_trigger, const float* norm_w,
                                                                           float eps) {
    limbs_short_body<Q5Fmt, R, FROM_X>(w, src, add, y, out_dim, bpr, x_aligned, hold_trigger, norm_w, eps);
}

// Long rows, few of them (a down projection): one CTA per SM keeps the records (one copy per SM, not
// per small CTA) and takes an even share of the rows; its 96 eight-lane groups walk the (row, block)
// pairs of up to 32 rows cyclically, so that every group has the same number of blocks whatever the
// row length, and leave one partial sum per (row, group) in shared memory, summed in a fixed order.
constexpr int kLongThreads = 768, kLongGroups = kLongThreads / 8, kLongRows = 32;

template <class FMT, int FROM_X>
__device__ __forceinline__ void limbs_long_body(const uint8_t* __restrict__ w, const void* src, const float* add, float* y,
                                                int out_dim, int bpr, int x_aligned, int hold_trigger, const float* norm_w,
                                                float eps) {
    extern __shared__ __align__(16) uint4 rec_s[];
    const uint32_t* rec_w = reinterpret_cast<const uint32_t*>(rec_s);
    float* part = reinterpret_cast<float*>(rec_s + (size_t)bpr * 4 * xlimbs::kRecordVec4);   // [kLongRows][kLongGroups]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = threadIdx.x >> 3, sub = lane & 7;
    const unsigned gmask = 0xFFu << (lane & 24);   // the eight lanes of this group
    const size_t row_bytes = (size_t)bpr * FMT::kBytes;
    const int row_begin = (int)((long long)blockIdx.x * out_dim / gridDim.x);
    const int row_end = (int)((long long)(blockIdx.x + 1) * out_dim / gridDim.x);
    const int step_rows = kLongGroups / bpr, step_blks = kLongGroups - step_rows * bpr;   // one stride of a group
    // The weights do not depend on the kernel before this one: the first block is requested before the
    // wait for the activations, the next one always before the current one is multiplied.
    typename FMT::Lane nxt[1];
    if (group < min(kLongRows, row_end - row_begin) * bpr)
        FMT::load(nxt[0], w + (size_t)row_begin * row_bytes + (size_t)group * FMT::kBytes, sub);
    mg::pdl_prologue(hold_trigger);
    limbs_stage_records<FROM_X, kLongThreads>(src, bpr, x_aligned, rec_s, norm_w, eps);

    for (int pass0 = row_begin; pass0 < row_end; pass0 += kLongRows) {
        const int n_rows = min(kLongRows, row_end - pass0);
        for (int i = threadIdx.x; i < kLongRows * kLongGroups; i += kLongThreads) part[i] = 0.0f;
        __syncthreads();
        const int n_items = n_rows * bpr;
        int cur = -1;
        float acc[1] = {0.0f};
        const uint8_t* wp = w + (size_t)pass0 * row_bytes;   // rows of a pass are one contiguous run of blocks
        if (pass0 != row_begin && group < n_items) FMT::load(nxt[0], wp + (size_t)group * FMT::kBytes, sub);
        int rl = group / bpr, blk = group - rl * bpr;   // (row, block) of item j
        for (int j = group; j < n_items; j += kLongGroups) {
            if (rl != cur) {   // the whole group moves on together
                if (cur >= 0) {
                    float v = acc[0];
                    v += __shfl_xor_sync(gmask, v, 4);
                    v += __shfl_xor_sync(gmask, v, 2);
                    v += __shfl_xor_sync(gmask, v, 1);
                    if (sub == 0) part[cur * kLongGroups + group] = v;
                }
                cur = rl;
                acc[0] = 0.0f;
            }
            typename FMT::Lane now[1];
            now[0] = nxt[0];
            if (j + kLongGroups < n_items) FMT::load(nxt[0], wp + (size_t)(j + kLongGroups) * FMT::kBytes, sub);
            FMT::template dot<1>(now, rec_w, blk, sub, acc);
            rl += step_rows;
            blk += step_blks;
            if (blk >= bpr) { blk -= bpr; ++rl; }
        }
        if (cur >= 0) {
            float v = acc[0];
            v += __shfl_xor_sync(gmask, v, 4);
            v += __shfl_xor_sync(gmask, v, 2);
            v += __shfl_xor_sync(gmask, v, 1);
            if (sub == 0) part[cur * kLongGroups + group] = v;
        }
        __syncthreads();
        for (int rr = warp; rr < n_rows; rr += kLongThreads / 32) {
            const float* pr = part + rr * kLongGroups;
            float t = (pr[lane] + pr[32 + lane]) + pr[64 + lane];
            t = q4k::warp_sum(t);
            if (lane == 0) y[pass0 + rr] = add ? add[pass0 + rr] + t : t;
        }
        __syncthreads();   // before the partial sums are cleared for the next rows
    }
}
template <int FROM_X>
__global__ void __launch_bounds__(kLongThreads, 1) matvec_q6k_limbs_long_kernel(const uint8_t* __restrict__ w, const void* src,
                                                                                const float* add, float* y, int out_dim,
                                                                                int bpr, int x_aligned, int hold_trigger,
                                                                                const float* norm_w, float eps) {
    limbs_long_body<Q6Fmt, FROM_X>(w, src, add, y, out_dim, bpr, x_aligned, hold_trigger, norm_w, eps);
}
template <int FROM_X>
__global__ void __launch_bounds__(kLongThreads, 1) matvec_q5k_limbs_long_kernel(const uint8_t* __restrict__ w, const void* src,
                                                                                const float* add, float* y, int out_dim,
                                                                                int bpr, int x_aligned, int hold_trigger,
                                                                                const float* norm_w, float eps) {
    limbs_long_body<Q5Fmt, FROM_X>(w, src, add, y, out_dim, bpr, x_aligned, hold_trigger, norm_w, eps);
}

// Q6_K weights x int8 activations (xq / xd / xsum from launch_quantize_q8_1):
// y[row] = sum over 32-element sub-blocks s of xd[s] * d * (sc_lo * <q, xq>[0..16) + sc_hi * <q, xq>[16..32)).
__global__ void __launch_bounds__(kThreads) matvec_q6k_q8_kernel(const uint8_t* __restrict__ w, const int8_t* xq,
                                                                 const float* xd, float* y, int out_dim, int bpr) {
    mg::pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < out_dim; row += gridDim.x * kWarps) {
        const uint8_t* wr = w + (size_t)row * bpr * kQ6Bytes;
        float acc = 0.0f;
        for (int blk = 0; blk < bpr; ++blk) {
            const uint8_t* b = wr + (size_t)blk * kQ6Bytes;
            const float d = q6_d(b);
            const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192);
#pragma unroll
            for (int G = 0; G < 2; ++G) {
                int qv[4];
                q6_quants(b, G, lane, qv);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int s32 = blk * 8 + G * 4 + k;  // the 32-element sub-block of x these weights meet
                    const int prod = qv[k] * (int)xq[(size_t)s32 * 32 + lane];
                    // exact integer products; per-lane f32 scaling then equals the per-half integer sums times the scale
                    acc = fmaf(xd[s32] * d, (float)((int)sc[8 * G + 2 * k + (lane >> 4)] * prod), acc);
                }
            }
        }
        acc = q4k::warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}

int grid_for(int work_items) {
    const mg::DeviceProps& dp = mg::device_props();
    const int sms = dp.ok ? dp.sm_count : 148;
    int grid = (work_items + kWarps - 1) / kWarps;
    if (grid > sms * 8) grid = sms * 8;
    return grid < 1 ? 1 : grid;
}

template <int KIND, int R, int WARPS>
int launch_matvec_shape(const uint8_t* w, const float* x, const float* add, float* y, int out_dim, int bpr, void* stream) {
    const mg::DeviceProps& dp = mg::device_props();
    const int sms = dp.ok ? dp.sm_count : 148;
    int grid = (out_dim + R - 1) / R;
    const int resident = sms * (2048 / (WARPS * 32));
    if (grid > resident) grid = resident;
    return (int)mg::launch_pdl(matvec_kquant_kernel<KIND, R, WARPS>, dim3((unsigned)grid), dim3(WARPS * 32), 0,
                               (cudaStream_t)stream, w, x, add, y, out_dim, bpr, mg::aligned16(x) ? 1 : 0,
                               mg::early_trigger_flag() ? 0 : 1);
}

template <int KIND>
int launch_matvec(const uint8_t* w, const float* x, const float* add, float* y, int out_dim, int bpr, void* stream) {
    // long rows: eight warps share two rows; short rows: four warps share four
    if (bpr >= 32) return launch_matvec_shape<KIND, 2, 8>(w, x, add, y, out_dim, bpr, stream);
    return launch_matvec_shape<KIND, 4, 4>(w, x, add, y, out_dim, bpr, stream);
}

// Few rows per SM (one pass of the long kernel), or rows of more than 32 blocks: the kernel that splits
// the rows' blocks over a whole CTA.  Many short rows: a warp per pair of rows.
bool limbs_long_shape(int out_dim, int bpr) {
    const mg::DeviceProps& dp = mg::device_props();
    return bpr > 32 || out_dim <= (dp.ok ? dp.sm_count : 148) * kLongRows;
}

// The limb kernels need the whole activation vector as records in one CTA's shared memory, and a Q6_K
// weight 4-byte aligned (its 8-byte loads round the address down; Q5_K is 16-byte aligned by contract).
size_t limbs_smem_bytes(int out_dim, int bpr) {
    return (size_t)bpr * 4 * xlimbs::kRecordBytes +
           (limbs_long_shape(out_dim, bpr) ? (size_t)kLongRows * kLongGroups * sizeof(float) : 0);
}
bool limbs_ok(const uint8_t* w, int out_dim, int bpr) {
    const mg::DeviceProps& dp = mg::device_props();
    // 256 bytes left for the kernels' static shared memory (the RMSNorm reduction)
    return (reinterpret_cast<uintptr_t>(w) & 3u) == 0 && dp.ok && limbs_smem_bytes(out_dim, bpr) + 256 <= (size_t)dp.max_smem_optin;
}

template <class Kernel>
int launch_limbs_kernel(Kernel kernel, size_t& configured, unsigned grid, int threads, size_t smem, const uint8_t* w,
                        const void* src, const float* add, float* y, int out_dim, int bpr, void* stream, const float* norm_w,
                        float eps) {
    if (smem > 48 * 1024 && smem > configured) {   // configured: the largest dynamic shared memory set for this kernel
        const mg::DeviceProps& dp = mg::device_props();
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, kernel);
        if (e != cudaSuccess) return (int)e;
        const int most = dp.max_smem_optin - (int)fa.sharedSizeBytes;   // the kernel's static shared memory counts too
        if ((size_t)most < smem) return (int)cudaErrorInvalidValue;
        if ((e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most)) != cudaSuccess) return (int)e;
        configured = (size_t)most;
    }
    // a collective of another library may follow and start on the early trigger: the host switches it off then
    return (int)mg::launch_pdl(kernel, dim3(grid), dim3((unsigned)threads), smem, (cudaStream_t)stream, w, src, add, y, out_dim,
                               bpr, mg::aligned16(src) ? 1 : 0, mg::early_trigger_flag() ? 0 : 1, norm_w, eps);
}

template <int KIND, int FROM_X>
int launch_limbs(const uint8_t* w, const void* src, const float* add, float* y, int out_dim, int bpr, void* stream,
                 const float* norm_w = nullptr, float eps = 0.0f) {
    const mg::DeviceProps& dp = mg::device_props();
    const size_t smem = limbs_smem_bytes(out_dim, bpr);
    if (limbs_long_shape(out_dim, bpr)) {
        static size_t configured = 0;
        const unsigned grid = (unsigned)(out_dim < dp.sm_count ? out_dim : dp.sm_count);
        if (KIND == 5)
            return launch_limbs_kernel(matvec_q5k_limbs_long_kernel<FROM_X>, configured, grid, kLongThreads, smem, w, src, add, y,
                                       out_dim, bpr, stream, norm_w, eps);
        return launch_limbs_kernel(matvec_q6k_limbs_long_kernel<FROM_X>, configured, grid, kLongThreads, smem, w, src, add, y,
                                   out_dim, bpr, stream, norm_w, eps);
    }
    constexpr int R = 2;
    static size_t configured = 0;
    // CTAs an SM holds: by shared memory (1 KiB reserved per CTA) and by threads
    int per_sm = (int)((228u * 1024u) / (smem + 1024));
    per_sm = per_sm > 2048 / kLimbThreads ? 2048 / kLimbThreads : (per_sm < 1 ? 1 : per_sm);
    int grid = (out_dim + R * kLimbWarps - 1) / (R * kLimbWarps);
    if (grid > dp.sm_count * per_sm) grid = dp.sm_count * per_sm;
    if (KIND == 5)
        return launch_limbs_kernel(matvec_q5k_limbs_kernel<R, FROM_X>, configured, (unsigned)grid, kLimbThreads, smem, w, src, add,
                                   y, out_dim, bpr, stream, norm_w, eps);
    return launch_limbs_kernel(matvec_q6k_limbs_kernel<R, FROM_X>, configured, (unsigned)grid, kLimbThreads, smem, w, src, add, y,
                               out_dim, bpr, stream, norm_w, eps);
}

// x_kind 0: f32 activations; 1: limb records.
template <int KIND>
int matvec_any(const uint8_t* w, const void* src, int x_kind, const float* add, float* y, int out_dim, int bpr, void* stream) {
    if (out_dim <= 0 || bpr <= 0 || !w || !src || !y || (x_kind != 0 && x_kind != 1)) return (int)cudaErrorInvalidValue;
    if (KIND == 5 && !mg::aligned16(w)) return (int)cudaErrorInvalidValue;
    if (KIND == 6 && (reinterpret_cast<uintptr_t>(w) & 1u)) return (int)cudaErrorInvalidValue;
    if (x_kind == 1) {
        if (!limbs_ok(w, out_dim, bpr) || !mg::aligned16(src)) return (int)cudaErrorInvalidValue;
        return launch_limbs<KIND, 0>(w, src, add, y, out_dim, bpr, stream);
    }
    if (limbs_ok(w, out_dim, bpr)) return launch_limbs<KIND, 1>(w, src, add, y, out_dim, bpr, stream);
    return launch_matvec<KIND>(w, static_cast<const float*>(src), add, y, out_dim, bpr, stream);
}

}  // namespace

extern "C" {

int launch_matvec_q5k_on_stream(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream) {
    return matvec_any<5>(w_q5, x, 0, nullptr, y, out_dim, blocks_per_row, stream);
}
int launch_matvec_q5k(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row) {
    return matvec_any<5>(w_q5, x, 0, nullptr, y, out_dim, blocks_per_row, nullptr);
}
int launch_matvec_q6k_on_stream(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream) {
    return matvec_any<6>(w_q6, x, 0, nullptr, y, out_dim, blocks_per_row, stream);
}
int launch_matvec_q6k(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row) {
    return matvec_any<6>(w_q6, x, 0, nullptr, y, out_dim, blocks_per_row, nullptr);
}
// y[row] = (add ? add[row] : 0) + W[row] . x for a Q5_K (ggml_type 13) or Q6_K (14) weight: the matvec
// with the residual add the decode loop puts behind it (crates/modgrad-gemma/src/rocm_gemma.rs:470-475,
// :497-500) folded in; y may alias add.  x_kind 0: x is the f32 activation vector; 1 (Q6_K only, weight
// 4-byte aligned): x holds the limb records of mg_q4k_x_to_limbs_on_stream / mg_swiglu_limbs_on_stream.
int mg_matvec_kquant_on_stream(int ggml_type, const uint8_t* w, const void* x, int x_kind, const float* add, float* y,
                               int out_dim, int blocks_per_row, void* stream) {
    if (ggml_type == 13) return matvec_any<5>(w, x, x_kind, add, y, out_dim, blocks_per_row, stream);
    if (ggml_type == 14) return matvec_any<6>(w, x, x_kind, add, y, out_dim, blocks_per_row, stream);
    return (int)cudaErrorInvalidValue;
}

int launch_matvec_q6k_dp4a_on_stream(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum, float* y,
                                     int out_dim, int bpr, void* stream) {
    (void)xsum;  // Q6_K has no per-block minimum: the sums are not needed (kept for the reference's signature)
    if (out_dim <= 0 || bpr <= 0) return (int)cudaErrorInvalidValue;
    if (!w || !xq || !xd || !y || (reinterpret_cast<uintptr_t>(w) & 1u)) return (int)cudaErrorInvalidValue;
    return (int)mg::launch_pdl(matvec_q6k_q8_kernel, dim3((unsigned)grid_for(out_dim)), dim3(kThreads), 0,
                               (cudaStream_t)stream, w, xq, xd, y, out_dim, bpr);
}
int launch_matvec_q6k_dp4a(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum, float* y, int out_dim,
                           int bpr) {
    return launch_matvec_q6k_dp4a_on_stream(w, xq, xd, xsum, y, out_dim, bpr, nullptr);
}

// y = W . rms_norm(x) for a Q5_K (ggml_type 13) or Q6_K (14) weight: the RMSNorm the decode loop runs in front
// of a projection (crates/modgrad-device/src/kfd/llm.rs:921-928, Plain) done by every CTA while it converts x,
// like mg_rmsnorm_matvec_q4k_multi_on_stream for Q4_K.  Runs on the limb kernels only: cudaErrorInvalidValue
// when the weight is not 4-byte aligned or the records of a row exceed one CTA's shared memory.
int mg_rmsnorm_matvec_kquant_on_stream(int ggml_type, const uint8_t* w, const float* x, const float* norm_w, float eps, float* y,
                                       int out_dim, int blocks_per_row, void* stream) {
    if (out_dim <= 0 || blocks_per_row <= 0 || !w || !x || !norm_w || !y) return (int)cudaErrorInvalidValue;
    if (ggml_type == 13 && !mg::aligned16(w)) return (int)cudaErrorInvalidValue;
    if (!limbs_ok(w, out_dim, blocks_per_row)) return (int)cudaErrorInvalidValue;
    if (ggml_type == 13) return launch_limbs<5, 1>(w, x, nullptr, y, out_dim, blocks_per_row, stream, norm_w, eps);
    if (ggml_type == 14) return launch_limbs<6, 1>(w, x, nullptr, y, out_dim, blocks_per_row, stream, norm_w, eps);
    return (int)cudaErrorInvalidValue;
}

// ggml_type: 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K); d_model a multiple of 256.
int mg_embed_kquant_on_stream(const void* table, int ggml_type, int token, const int* token_dev, float* out, int d_model,
                              int vocab, void* stream) {
    if (!table || !out || d_model <= 0 || d_model % 256 || vocab <= 0) return (int)cudaErrorInvalidValue;
    const int bpr = d_model / 256;
    const uint8_t* t = static_cast<const uint8_t*>(table);
    const dim3 grid((unsigned)((bpr + kWarps - 1) / kWarps)), block(kThreads);
    cudaStream_t st = (cudaStream_t)stream;
    switch (ggml_type) {
        case 12:
            if (!mg::aligned16(t)) return (int)cudaErrorInvalidValue;
            return (int)mg::launch_pdl(embed_kquant_kernel<4>, grid, block, 0, st, t, token_dev, token, out, bpr, vocab);
        case 13:
            if (!mg::aligned16(t)) return (int)cudaErrorInvalidValue;
            return (int)mg::launch_pdl(embed_kquant_kernel<5>, grid, block, 0, st, t, token_dev, token, out, bpr, vocab);
        case 14:
            if (reinterpret_cast<uintptr_t>(t) & 1u) return (int)cudaErrorInvalidValue;
            return (int)mg::launch_pdl(embed_kquant_kernel<6>, grid, block, 0, st, t, token_dev, token, out, bpr, vocab);
        default: return (int)cudaErrorInvalidValue;
    }
}

int mg_dequant_q5k_on_stream(const uint8_t* q5k, int n_blocks, float* fp32_out, void* stream) {
    if (n_blocks <= 0 || !q5k || !fp32_out || !mg::aligned16(q5k)) return (int)cudaErrorInvalidValue;
    dequant_q5k_kernel<<<grid_for(n_blocks), kThreads, 0, (cudaStream_t)stream>>>(q5k, fp32_out, n_blocks);
    return (int)cudaGetLastError();
}
int mg_dequant_q6k_on_stream(const uint8_t* q6k, int n_blocks, float* fp32_out, void* stream) {
    if (n_blocks <= 0 || !q6k || !fp32_out || (reinterpret_cast<uintptr_t>(q6k) & 1u)) return (int)cudaErrorInvalidValue;
    dequant_q6k_kernel<<<grid_for(n_blocks), kThreads, 0, (cudaStream_t)stream>>>(q6k, fp32_out, n_blocks);
    return (int)cudaGetLastError();
}

}  // extern "C"
