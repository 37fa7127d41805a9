// Q5_K and Q6_K: the other two K-quant formats real GGUF checkpoints mix with Q4_K (LM head and
// token embedding are Q6_K, attn_v / ffn_down often Q5_K: crates/modgrad-gemma/src/rocm_gemma.rs:295-297, :338).
//
//   launch_matvec_q5k       replaces crates/modgrad-device/kernels/matvec_q5k.hip:55-121
//   launch_matvec_q6k       replaces crates/modgrad-device/kernels/matvec_q6k.hip:32-94
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
// Kernel shape (both formats): one warp per row, lane l owns byte column l of every quant group, so
// every load instruction of the warp covers 32 consecutive bytes (or 128 bytes of x); eight weights
// per lane and super-block, f32 accumulate, warp-shuffle reduction.  HBM-bound work done with byte
// loads: correct and coalesced, not yet tuned like the Q4_K kernels.
#include <float.h>

#include "launch_common.cuh"
#include "q4k_device.cuh"

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

// kind 5 / 6; x is read after the previous kernel of the stream has completed.
template <int KIND>
__global__ void __launch_bounds__(kThreads) matvec_kquant_kernel(const uint8_t* __restrict__ w, const float* x, float* y,
                                                                 int out_dim, int bpr) {
    mg::pdl_prologue();
    const int lane = threadIdx.x & 31;
    constexpr int kBytes = KIND == 5 ? kQ5Bytes : kQ6Bytes;
    for (int row = blockIdx.x * kWarps + (threadIdx.x >> 5); row < out_dim; row += gridDim.x * kWarps) {
        const uint8_t* wr = w + (size_t)row * bpr * kBytes;
        float acc = 0.0f;
        for (int blk = 0; blk < bpr; ++blk) {
            const uint8_t* b = wr + (size_t)blk * kBytes;
            const float* xb = x + (size_t)blk * 256;
            if (KIND == 5) {
                const Q5Header h = q5_header(b);
                const uint32_t qh = b[16 + lane];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t v = b[48 + 32 * g + lane];
                    const float q_lo = (float)((v & 0xFu) + (((qh >> (2 * g)) & 1u) << 4));
                    const float q_hi = (float)((v >> 4) + (((qh >> (2 * g + 1)) & 1u) << 4));
                    acc = fmaf(fmaf(h.dsc[2 * g], q_lo, -h.dm[2 * g]), xb[64 * g + lane], acc);
                    acc = fmaf(fmaf(h.dsc[2 * g + 1], q_hi, -h.dm[2 * g + 1]), xb[64 * g + 32 + lane], acc);
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
                        acc = fmaf(d * (float)sc[8 * G + 2 * k + (lane >> 4)] * (float)qv[k], xb[128 * G + 32 * k + lane], acc);
                }
            }
        }
        acc = q4k::warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
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

template <int KIND>
int launch_matvec(const uint8_t* w, const float* x, float* y, int out_dim, int bpr, void* stream) {
    if (out_dim <= 0 || bpr <= 0) return (int)cudaErrorInvalidValue;
    if (!w || !x || !y) return (int)cudaErrorInvalidValue;
    if (KIND == 5 && !mg::aligned16(w)) return (int)cudaErrorInvalidValue;
    if (KIND == 6 && (reinterpret_cast<uintptr_t>(w) & 1u)) return (int)cudaErrorInvalidValue;
    return (int)mg::launch_pdl(matvec_kquant_kernel<KIND>, dim3((unsigned)grid_for(out_dim)), dim3(kThreads), 0,
                               (cudaStream_t)stream, w, x, y, out_dim, bpr);
}

}  // namespace

extern "C" {

int launch_matvec_q5k_on_stream(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream) {
    return launch_matvec<5>(w_q5, x, y, out_dim, blocks_per_row, stream);
}
int launch_matvec_q5k(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row) {
    return launch_matvec<5>(w_q5, x, y, out_dim, blocks_per_row, nullptr);
}
int launch_matvec_q6k_on_stream(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream) {
    return launch_matvec<6>(w_q6, x, y, out_dim, blocks_per_row, stream);
}
int launch_matvec_q6k(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row) {
    return launch_matvec<6>(w_q6, x, y, out_dim, blocks_per_row, nullptr);
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
