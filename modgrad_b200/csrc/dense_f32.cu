// Dense f32 matvec y = W[out_dim][in_dim] . x + bias: the op LinearResidentQuantized's expanded mode
// dispatches after the dequantisation (ops::matvec_resident -> hipblasSgemv in the reference,
// crates/modgrad-compute/src/neuron.rs:1093-1101).  One warp per row, 16-byte loads when aligned.
#include "launch_common.cuh"
#include "q4k_device.cuh"

namespace {
__global__ void __launch_bounds__(256) matvec_f32_kernel(const float* __restrict__ w, const float* x, const float* bias,
                                                         float* y, int out_dim, int in_dim, int vec_ok) {
    mg::pdl_prologue();
    const int lane = threadIdx.x & 31;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < out_dim; row += gridDim.x * 8) {
        const float* wr = w + (size_t)row * in_dim;
        float acc = 0.0f;
        if (vec_ok) {
            for (int i = lane * 4; i < in_dim; i += 128) {
                const float4 a = *reinterpret_cast<const float4*>(wr + i);
                const float4 b = *reinterpret_cast<const float4*>(x + i);
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (int i = lane; i < in_dim; i += 32) acc = fmaf(wr[i], x[i], acc);
        }
        acc = q4k::warp_sum(acc);
        if (lane == 0) y[row] = bias ? acc + bias[row] : acc;
    }
}
}  // namespace

extern "C" int mg_matvec_f32_on_stream(const float* w, const float* x, const float* bias, float* y, int out_dim, int in_dim,
                                       void* stream) {
    if (!w || !x || !y || out_dim <= 0 || in_dim <= 0) return (int)cudaErrorInvalidValue;
    const mg::DeviceProps& dp = mg::device_props();
    int grid = (out_dim + 7) / 8;
    const int cap = (dp.ok ? dp.sm_count : 148) * 8;
    if (grid > cap) grid = cap;
    const int vec_ok = (in_dim % 4 == 0) && mg::aligned16(w) && mg::aligned16(x);
    return (int)mg::launch_pdl(matvec_f32_kernel, dim3((unsigned)grid), dim3(256), 0, (cudaStream_t)stream, w, x, bias, y,
                               out_dim, in_dim, vec_ok);
}
