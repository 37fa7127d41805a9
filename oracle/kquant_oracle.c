/*
 * CPU ORACLE for the GGUF Q5_K and Q6_K dequantize / matvec path.  TEST INFRASTRUCTURE ONLY
 * (see q4k_oracle.c: never linked into or called from the shipped CUDA library).
 *
 * PARITY UNPINNED, as for Q4_K: the reference is Rust and cannot be run where this was written.
 * Its tree holds two hand-built Q6_K known-answer dots for the INTEGER (Q8_K-activation) path
 * (crates/modgrad-device/src/kfd/quant_dot.rs:366-393), none for these f32 functions; this
 * restatement is pinned by known-answer blocks derived from the format definition with exact
 * rational arithmetic (tests/golden/make_kquant_kats.py) and by an independent numpy restatement.
 *
 * Build with -ffp-contract=off: the specification is separate f32 roundings, no fused multiply-add.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

float orc_f16_to_f32(uint16_t h);
void orc_get_scale_min_k4(int j, const uint8_t* scales, uint8_t* sc, uint8_t* m);

#define Q5K_BLOCK_BYTES 176 /* crates/modgrad-device/src/kfd/gguf.rs:62 */
#define Q6K_BLOCK_BYTES 210 /* crates/modgrad-device/src/kfd/gguf.rs:63 */

/* crates/modgrad-device/src/kfd/gguf.rs:421-455: d, dmin (non-finite -> 0), scales[12] as Q4_K,
 * qh[32] one high bit per weight (bit 2g for the low-nibble half of group g, bit 2g+1 for the high
 * one), ql[128]; out = fl(fl(d*sc) * (nibble + 16*hbit)) - fl(dmin*m), ggml element order. */
void orc_dequantize_row_q5_k(const uint8_t* data, float* out, size_t n_blocks) {
    for (size_t blk = 0; blk < n_blocks; ++blk) {
        const uint8_t* b = data + blk * Q5K_BLOCK_BYTES;
        float d = orc_f16_to_f32((uint16_t)(b[0] | (b[1] << 8)));
        float dmin = orc_f16_to_f32((uint16_t)(b[2] | (b[3] << 8)));
        if (!isfinite(d)) d = 0.0f;
        if (!isfinite(dmin)) dmin = 0.0f;
        const uint8_t* scales = b + 4;
        const uint8_t* qh = b + 16;
        const uint8_t* ql = b + 48;
        float* o = out + blk * 256;
        int is = 0;
        uint8_t u1 = 1, u2 = 2;
        for (int j = 0; j < 256; j += 64) {
            uint8_t sc1, m1, sc2, m2;
            orc_get_scale_min_k4(is, scales, &sc1, &m1);
            orc_get_scale_min_k4(is + 1, scales, &sc2, &m2);
            const float d1 = d * (float)sc1, dm1 = dmin * (float)m1;
            const float d2 = d * (float)sc2, dm2 = dmin * (float)m2;
            for (int l = 0; l < 32; ++l) {
                const uint8_t hbit = (qh[l] & u1) ? 16 : 0;
                *o++ = d1 * (float)((ql[l] & 0xF) + hbit) - dm1;
            }
            for (int l = 0; l < 32; ++l) {
                const uint8_t hbit = (qh[l] & u2) ? 16 : 0;
                *o++ = d2 * (float)((ql[l] >> 4) + hbit) - dm2;
            }
            ql += 32;
            is += 2;
            u1 = (uint8_t)(u1 << 2);
            u2 = (uint8_t)(u2 << 2);
        }
    }
}

/* crates/modgrad-device/src/kfd/gguf.rs:458-484: ql[128], qh[64], sc[16] signed bytes, d (half at
 * +208, non-finite -> 0); q = (4 low bits | 2 high bits << 4) - 32; out = fl(fl(d * sc) * q). */
void orc_dequantize_row_q6_k(const uint8_t* data, float* out, size_t n_blocks) {
    for (size_t blk = 0; blk < n_blocks; ++blk) {
        const uint8_t* b = data + blk * Q6K_BLOCK_BYTES;
        const uint8_t* ql = b;
        const uint8_t* qh = b + 128;
        const int8_t* sc = (const int8_t*)(b + 192);
        float d = orc_f16_to_f32((uint16_t)(b[208] | (b[209] << 8)));
        if (!isfinite(d)) d = 0.0f;
        float* o = out + blk * 256;
        for (int grp = 0; grp < 2; ++grp) {
            const int qlb = grp * 64, qhb = grp * 32, scb = grp * 8, yb = grp * 128;
            for (int l = 0; l < 32; ++l) {
                const int is = l / 16;
                const int q1 = ((ql[qlb + l] & 0xF) | ((qh[qhb + l] & 3) << 4)) - 32;
                const int q2 = ((ql[qlb + l + 32] & 0xF) | (((qh[qhb + l] >> 2) & 3) << 4)) - 32;
                const int q3 = ((ql[qlb + l] >> 4) | (((qh[qhb + l] >> 4) & 3) << 4)) - 32;
                const int q4 = ((ql[qlb + l + 32] >> 4) | (((qh[qhb + l] >> 6) & 3) << 4)) - 32;
                o[yb + l] = d * (float)sc[scb + is] * (float)q1;
                o[yb + l + 32] = d * (float)sc[scb + is + 2] * (float)q2;
                o[yb + l + 64] = d * (float)sc[scb + is + 4] * (float)q3;
                o[yb + l + 96] = d * (float)sc[scb + is + 6] * (float)q4;
            }
        }
    }
}

/* y = W . x with the dequantised weights and an f64 accumulator: the reference's arm for quants
 * without a fused dot (crates/modgrad-device/src/kfd/llm.rs:524-531) and the scalar arm of
 * dot_q6k_row (llm.rs:547-552); an order-independent checker for reordered f32 sums.
 * kind: 5 = Q5_K, 6 = Q6_K. */
void orc_matvec_kquant_f64(int kind, const uint8_t* w, const float* x, double* y, int out_dim, int bpr) {
    const size_t bb = kind == 5 ? Q5K_BLOCK_BYTES : Q6K_BLOCK_BYTES;
    float tmp[256];
    for (int r = 0; r < out_dim; ++r) {
        double acc = 0.0;
        for (int b = 0; b < bpr; ++b) {
            const uint8_t* p = w + ((size_t)r * bpr + b) * bb;
            if (kind == 5) orc_dequantize_row_q5_k(p, tmp, 1);
            else orc_dequantize_row_q6_k(p, tmp, 1);
            for (int k = 0; k < 256; ++k) acc += (double)tmp[k] * (double)x[(size_t)b * 256 + k];
        }
        y[r] = acc;
    }
}

/* The int8-activation Q6_K matvec, crates/modgrad-device/kernels/matvec_q6k_dp4a.hip:56-138:
 * per 32-element sub-block s (group g = (s & 7) >> 2, quad = s & 3): integer dots of the low and
 * the high 16 weights, each with its own signed scale, term = (xd[s] * d) * (sc_lo * isum_lo +
 * sc_hi * isum_hi) in f32; the terms are summed in f64 here (order-independent checker). */
void orc_matvec_q6k_q8_1(const uint8_t* w, const int8_t* xq, const float* xd, float* y, int out_dim, int bpr) {
    for (int r = 0; r < out_dim; ++r) {
        const uint8_t* wrow = w + (size_t)r * bpr * Q6K_BLOCK_BYTES;
        double acc = 0.0;
        for (int s32 = 0; s32 < bpr * 8; ++s32) {
            const int blk = s32 >> 3, sub32 = s32 & 7;
            const uint8_t* b = wrow + (size_t)blk * Q6K_BLOCK_BYTES;
            float d = orc_f16_to_f32((uint16_t)(b[208] | (b[209] << 8)));
            if (!isfinite(d)) d = 0.0f;
            const int g = sub32 >> 2, quad = sub32 & 3;
            const uint8_t* ql = b + g * 64 + ((quad & 1) ? 32 : 0);
            const uint8_t* qh = b + 128 + g * 32;
            const int8_t* sc = (const int8_t*)(b + 192);
            const int sc_lo = sc[g * 8 + quad * 2], sc_hi = sc[g * 8 + quad * 2 + 1];
            int isum_lo = 0, isum_hi = 0;
            for (int l = 0; l < 32; ++l) {
                const int nib = (quad >> 1) ? (ql[l] >> 4) : (ql[l] & 0xF);
                const int q6 = (nib | (((qh[l] >> (quad * 2)) & 3) << 4)) - 32;
                const int prod = q6 * (int)xq[(size_t)s32 * 32 + l];
                if (l < 16) isum_lo += prod; else isum_hi += prod;
            }
            const float scl = xd[s32] * d;
            acc += (double)(scl * ((float)sc_lo * (float)isum_lo + (float)sc_hi * (float)isum_hi));
        }
        y[r] = (float)acc;
    }
}
