// The int8-activation pair of the reference: launch_quantize_q8_1 + launch_matvec_q4k_dp4a
// (crates/modgrad-device/kernels/matvec_q4k_dp4a.hip:30-116; Rust declarations
// crates/modgrad-device/src/backend/rocm.rs:477-479).  RocmGemma::qmatvec takes this pair by
// default (crates/modgrad-gemma/src/rocm_gemma.rs:283, :298-305), so a drop-in library has to
// export it.  It is LOSSY by design (activations rounded to 8 bits per 32-element sub-block,
// about 1 % error); the f32-accurate path is launch_matvec_q4k.
//
//   quantize:  per sub-block s of 32 activations: amax = max|x|, xd[s] = amax / 127,
//              xq = clamp(rint(x * (127 / amax)), -127, 127), xsum[s] = sum(xq) as f32; a sub-block whose
//              inverse scale is not finite (amax == 0 or denormal) becomes all zero with xd = 0.
//   matvec:    y[row] = sum_s xd[s] * (d * sc[s] * <nibbles, xq> - dmin * m[s] * xsum[s]),
//              integer dot per sub-block, f32 across sub-blocks, a non-finite row sum -> 0
//              (matvec_q4k_dp4a.hip:104-106).
//
// Kernel shape: x (int8 + the two f32 arrays) is staged once per CTA in shared memory; a warp
// streams rows two at a time, lane = (super-block of an 8-block window, 32-byte quant group) with
// 16-byte loads, four dp4a chains per lane and row, warp-shuffle reduction.
#include <float.h>

#include "gemv_q4k_device.cuh"
#include "launch_common.cuh"
#include "q4k_device.cuh"

namespace {

using gemvdev::dp4a_us;

__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const float* x, int8_t* xq, float* xd, float* xsum,
                                                           int nsub) {
    mg::pdl_prologue();  // x may come from the kernel launched just before
    // 8 threads per sub-block, 4 activations each; nsub * 8 threads in all (whole warps: 4 sub-blocks)
    const int gid = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = gid >> 3, part = gid & 7;
    const bool valid = s < nsub;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) {
        const float* p = x + (size_t)s * 32 + part * 4;
        if ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
            const float4 f = *reinterpret_cast<const float4*>(p);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
            v[0] = p[0]; v[1] = p[1]; v[2] = p[2]; v[3] = p[3];
        }
    }
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
    float d = __fdiv_rn(amax, 127.0f);
    float id = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    if (!(fabsf(id) <= FLT_MAX)) {  // not finite: emit a zero sub-block
        id = 0.0f;
        d = 0.0f;
    }
    int sum = 0;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int q = __float2int_rn(__fmul_rn(v[i], id));
        q = max(-127, min(127, q));
        sum += q;
        packed |= ((uint32_t)q & 0xFFu) << (8 * i);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (!valid) return;
    *reinterpret_cast<uint32_t*>(xq + (size_t)s * 32 + part * 4) = packed;
    if (part == 0) {
        xd[s] = d;
        xsum[s] = (float)sum;
    }
}

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kRows = 2;  // rows per warp and step

// STAGED: xq / xd / xsum copied to shared memory first (x up to ~180k activations).
template <bool STAGED>
__global__ void __launch_bounds__(kThreads) matvec_q4k_q8_kernel(const uint8_t* __restrict__ w, const int8_t* xq_g,
                                                                 const float* xd_g, const float* xsum_g, float* y,
                                                                 int out_dim, int bpr) {
    extern __shared__ __align__(16) uint8_t smem[];
    mg::pdl_prologue();  // the quantised activations come from the kernel launched just before
    const int nsub = bpr * 8;
    const int8_t* xq = xq_g;
    const float* xd = xd_g;
    const float* xsum = xsum_g;
    if (STAGED) {
        int8_t* sq = reinterpret_cast<int8_t*>(smem);
        float* sd = reinterpret_cast<float*>(smem + (size_t)nsub * 32);
        float* ss = sd + nsub;
        const uint4* src = reinterpret_cast<const uint4*>(xq_g);  // 16-byte aligned (checked by the launcher)
        for (int i = threadIdx.x; i < nsub * 2; i += kThreads) reinterpret_cast<uint4*>(sq)[i] = src[i];
        for (int i = threadIdx.x; i < nsub; i += kThreads) {
            sd[i] = xd_g[i];
            ss[i] = xsum_g[i];
        }
        __syncthreads();
        xq = sq; xd = sd; xsum = ss;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bl = lane >> 2, g = lane & 3;
    const size_t row_bytes = (size_t)bpr * q4k::kBlockBytes;
    const int n_groups = (out_dim + kRows - 1) / kRows;
    for (int grp = blockIdx.x * kWarps + warp; grp < n_groups; grp += gridDim.x * kWarps) {
        const int row0 = grp * kRows;
        float acc[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
        for (int b0 = 0; b0 < bpr; b0 += 8) {
            const int blk = b0 + bl;
            if (blk >= bpr) continue;
            const int s_lo = blk * 8 + 2 * g;
            const uint4 xa = *reinterpret_cast<const uint4*>(xq + (size_t)s_lo * 32);
            const uint4 xb = *reinterpret_cast<const uint4*>(xq + (size_t)s_lo * 32 + 16);
            const uint4 xc = *reinterpret_cast<const uint4*>(xq + (size_t)s_lo * 32 + 32);
            const uint4 xe = *reinterpret_cast<const uint4*>(xq + (size_t)s_lo * 32 + 48);
            const uint32_t xl[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
            const uint32_t xh[8] = {xc.x, xc.y, xc.z, xc.w, xe.x, xe.y, xe.z, xe.w};
            const float xd_lo = xd[s_lo], xd_hi = xd[s_lo + 1];
            const float xs_lo = xsum[s_lo], xs_hi = xsum[s_lo + 1];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int row = min(row0 + r, out_dim - 1);  // a tail row is computed twice, stored once
                const uint8_t* p = w + (size_t)row * row_bytes + (size_t)blk * q4k::kBlockBytes;
                const uint4 hdr = q4k::ld_nc_u4(p);
                const uint4 q0 = q4k::ld_stream_u4(p + 16 + g * 32);
                const uint4 q1 = q4k::ld_stream_u4(p + 32 + g * 32);
                const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                int i_lo = 0, i_hi = 0;
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    i_lo = dp4a_us(qw[t] & 0x0F0F0F0Fu, xl[t], i_lo);
                    i_hi = dp4a_us((qw[t] >> 4) & 0x0F0F0F0Fu, xh[t], i_hi);
                }
                const float d = q4k::half_bits_finite_or_zero(hdr.x);
                const float dmin = q4k::half_bits_finite_or_zero(hdr.x >> 16);
                const q4k::ScaleMin sm = q4k::unpack_scales(hdr.y, hdr.z, hdr.w);
                const float sc_lo = (float)q4k::scale_of(sm, 2 * g), sc_hi = (float)q4k::scale_of(sm, 2 * g + 1);
                const float m_lo = (float)q4k::min_of(sm, 2 * g), m_hi = (float)q4k::min_of(sm, 2 * g + 1);
                acc[r] += xd_lo * (d * sc_lo * (float)i_lo - dmin * m_lo * xs_lo);
                acc[r] += xd_hi * (d * sc_hi * (float)i_hi - dmin * m_hi * xs_hi);
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            float s = q4k::warp_sum(acc[r]);
            if (!(fabsf(s) <= FLT_MAX)) s = 0.0f;  // a degenerate sub-block must not poison the residual stream
            if (lane == 0 && row0 + r < out_dim) y[row0 + r] = s;
        }
    }
}

constexpr size_t kStageLimit = 200 * 1024;

}  // namespace

extern "C" int launch_quantize_q8_1_on_stream(const float* x, int8_t* xq, float* xd, float* xsum, int n,
                                              void* stream) {
    if (x == nullptr || xq == nullptr || xd == nullptr || xsum == nullptr || n < 0) return (int)cudaErrorInvalidValue;
    const int nsub = n / 32;  // a tail of fewer than 32 activations is ignored, as in the reference
    if (nsub == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(xq) & 3u) != 0) return (int)cudaErrorInvalidValue;
    const int threads = nsub * 8;
    return (int)mg::launch_pdl(quantize_q8_1_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0,
                               (cudaStream_t)stream, x, xq, xd, xsum, nsub);
}

extern "C" int launch_quantize_q8_1(const float* x, int8_t* xq, float* xd, float* xsum, int n) {
    return launch_quantize_q8_1_on_stream(x, xq, xd, xsum, n, nullptr);
}

extern "C" int launch_matvec_q4k_dp4a_on_stream(const uint8_t* w, const int8_t* xq, const float* xd,
                                                const float* xsum, float* y, int out_dim, int bpr, void* stream) {
    if (out_dim <= 0 || bpr <= 0) return (int)cudaErrorInvalidValue;
    if (!w || !xq || !xd || !xsum || !y) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(w) || !mg::aligned16(xq)) return (int)cudaErrorInvalidValue;
    const mg::DeviceProps& dp = mg::device_props();
    const int sms = dp.ok ? dp.sm_count : 148;
    const int n_groups = (out_dim + kRows - 1) / kRows;
    int grid = (n_groups + kWarps - 1) / kWarps;
    if (grid > sms * 4) grid = sms * 4;
    const size_t smem = (size_t)bpr * 8 * (32 + 8);
    cudaStream_t s = (cudaStream_t)stream;
    if (smem <= kStageLimit) {
        static bool attr_set[64] = {};
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            cudaError_t e = cudaFuncSetAttribute(matvec_q4k_q8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)kStageLimit);
            if (e != cudaSuccess) return (int)e;
            attr_set[dev] = true;
        }
        return (int)mg::launch_pdl(matvec_q4k_q8_kernel<true>, dim3((unsigned)grid), dim3(kThreads), smem, s, w, xq, xd,
                                   xsum, y, out_dim, bpr);
    }
    return (int)mg::launch_pdl(matvec_q4k_q8_kernel<false>, dim3((unsigned)grid), dim3(kThreads), 0, s, w, xq, xd, xsum,
                               y, out_dim, bpr);
}

extern "C" int launch_matvec_q4k_dp4a(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum, float* y,
                                      int out_dim, int bpr) {
    return launch_matvec_q4k_dp4a_on_stream(w, xq, xd, xsum, y, out_dim, bpr, nullptr);
}
