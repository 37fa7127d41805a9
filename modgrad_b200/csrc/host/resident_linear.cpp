// Q4_K residency container: the counterpart of LinearResidentQuantized
// (crates/modgrad-compute/src/neuron.rs:866-1250).  The weight lives on the HOST as Q4_K
// super-blocks (about 14 % of fp32); device buffers exist only between ensure_resident and evict.
//
// Two forward modes:
//   direct   (default): the Q4_K bytes are uploaded and the matvec runs on them as they are
//            (launch_matvec_q4k + bias): 0.5625 bytes per weight of device memory and traffic.
//   expanded (the reference's behaviour, neuron.rs:989-1108): the bytes are also dequantised once per
//            residency into an fp32 copy and the forward is a dense fp32 matvec: 7x the memory and
//            the bandwidth of the direct mode.
// Contract kept from the reference: from_* allocates nothing on the device; forward(auto_evict)
// leaves the layer resident or evicted accordingly; an evict followed by a forward reproduces the
// previous output bit for bit (neuron.rs:1943-1994); host_size_bytes / dequant_size_bytes.
//
// The quantiser writes the CANONICAL ggml element order that the dequantiser reads
// (crates/modgrad-device/src/kfd/gguf.rs:364-404).  The reference's own quantize_row_q4_k still
// writes the older all-low-then-all-high sub-block map (gguf.rs:590-601), which its dequantiser no
// longer matches; this one is written against the dequantiser.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "modgrad_cuda.h"

namespace {

uint16_t f32_to_f16_rne(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7FFFFFFFu;
    if (x >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (x > 0x7F800000u ? 0x200u : 0));
    if (x >= 0x477FF000u) return (uint16_t)(sign | 0x7BFFu);  // clamp to the largest finite half
    if (x < 0x33000001u) return (uint16_t)sign;                // below half of the smallest sub-normal
    int e = (int)(x >> 23) - 127;
    uint32_t m = (x & 0x7FFFFFu) | 0x800000u;
    int shift = e < -14 ? (13 + (-14 - e)) : 13;
    uint32_t half = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    if (e < -14) return (uint16_t)(sign | half);               // sub-normal (a carry lands in the exponent correctly)
    return (uint16_t)(sign | (((uint32_t)(e + 15) << 10) + (half - 0x400u)));
}
float f16_to_f32(uint16_t h) {
    const uint32_t s = (h >> 15) & 1u, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) {
        const float v = (float)m / 1024.0f * 6.103515625e-05f;
        return s ? -v : v;
    }
    const uint32_t bits = (s << 31) | ((e + 112u) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

}  // namespace

struct mg_linear_q4k {
    std::vector<uint8_t> host_q4k;
    std::vector<float> host_bias;
    int in_dim = 0, out_dim = 0;
    bool expand = false;
    uint8_t* q4k_dev = nullptr;
    float* w_dev = nullptr;  // expanded mode only
    float* bias_dev = nullptr;
};

extern "C" {

// x[n] (n % 256 == 0) -> n / 256 Q4_K super-blocks in the canonical element order: per 32-element
// sub-block an affine 4-bit grid from min(x, 0) to max(x), its step and offset stored as 6-bit
// multiples of the super-block's half-precision d and dmin.  Host code (construction time).
int mg_quantize_row_q4_k(const float* x, uint8_t* out, size_t n) {
    if (!x || !out || n == 0 || n % 256) return -4;
    for (size_t blk = 0; blk < n / 256; ++blk) {
        const float* xb = x + blk * 256;
        uint8_t* b = out + blk * 144;
        float step[8], off[8], max_step = 0.f, max_off = 0.f;
        for (int s = 0; s < 8; ++s) {
            float mn = 0.f, mx = 0.f;
            for (int l = 0; l < 32; ++l) {
                const float v = std::isfinite(xb[32 * s + l]) ? xb[32 * s + l] : 0.f;
                mn = v < mn ? v : mn;
                mx = v > mx ? v : mx;
            }
            step[s] = (mx - mn) / 15.0f;
            off[s] = -mn;
            max_step = step[s] > max_step ? step[s] : max_step;
            max_off = off[s] > max_off ? off[s] : max_off;
        }
        const uint16_t dh = f32_to_f16_rne(max_step / 63.0f), mh = f32_to_f16_rne(max_off / 63.0f);
        const float d = f16_to_f32(dh), dmin = f16_to_f32(mh);
        uint8_t sc[8], m[8];
        for (int s = 0; s < 8; ++s) {
            int a = d > 0.f ? (int)lrintf(step[s] / d) : 0, c = dmin > 0.f ? (int)lrintf(off[s] / dmin) : 0;
            sc[s] = (uint8_t)(a < 0 ? 0 : (a > 63 ? 63 : a));
            m[s] = (uint8_t)(c < 0 ? 0 : (c > 63 ? 63 : c));
        }
        b[0] = (uint8_t)(dh & 0xFF); b[1] = (uint8_t)(dh >> 8); b[2] = (uint8_t)(mh & 0xFF); b[3] = (uint8_t)(mh >> 8);
        for (int i = 0; i < 4; ++i) {  // the 12-byte packing of gguf.rs:349-358
            b[4 + i] = (uint8_t)((sc[i] & 0x3F) | (((sc[i + 4] >> 4) & 3) << 6));
            b[8 + i] = (uint8_t)((m[i] & 0x3F) | (((m[i + 4] >> 4) & 3) << 6));
            b[12 + i] = (uint8_t)((sc[i + 4] & 0xF) | ((m[i + 4] & 0xF) << 4));
        }
        memset(b + 16, 0, 128);
        for (int s = 0; s < 8; ++s) {
            const float ds = d * (float)sc[s], dm = dmin * (float)m[s];
            for (int l = 0; l < 32; ++l) {
                const float v = std::isfinite(xb[32 * s + l]) ? xb[32 * s + l] : 0.f;
                int q = ds > 0.f ? (int)lrintf((v + dm) / ds) : 0;
                q = q < 0 ? 0 : (q > 15 ? 15 : q);
                uint8_t* p = b + 16 + 32 * (s >> 1) + l;  // sub-block 2g: low nibbles of group g, 2g+1: high nibbles
                *p = (uint8_t)((s & 1) ? (*p | (q << 4)) : (*p | q));
            }
        }
    }
    return 0;
}

static int make(const uint8_t* q4k, const float* weight, const float* bias, int in_dim, int out_dim, mg_linear_q4k** out) {
    if (!out || in_dim <= 0 || out_dim <= 0) return -4;
    *out = nullptr;
    // the reference refuses a weight that is not a whole number of blocks (neuron.rs:925-931); the direct
    // matvec additionally needs whole blocks per ROW
    if (in_dim % 256) return -4;
    mg_linear_q4k* l = new mg_linear_q4k();
    l->in_dim = in_dim; l->out_dim = out_dim;
    l->host_q4k.resize((size_t)out_dim * (in_dim / 256) * 144);
    if (q4k) memcpy(l->host_q4k.data(), q4k, l->host_q4k.size());
    else mg_quantize_row_q4_k(weight, l->host_q4k.data(), (size_t)out_dim * in_dim);
    l->host_bias.assign(out_dim, 0.0f);
    if (bias) memcpy(l->host_bias.data(), bias, (size_t)out_dim * 4);
    *out = l;
    return 0;
}

// LinearResidentQuantized::from_linear (neuron.rs:923-949): quantise a row-major fp32 weight
// [out_dim][in_dim]; no device allocation.  bias may be NULL (zeros).  -4: in_dim % 256 != 0.
int mg_linear_q4k_from_f32(const float* weight, const float* bias, int in_dim, int out_dim, mg_linear_q4k** out) {
    if (!weight) return -4;
    return make(nullptr, weight, bias, in_dim, out_dim, out);
}
// The same from ready-made super-blocks (e.g. a tensor of a GGUF file), copied to the host store.
int mg_linear_q4k_from_blocks(const uint8_t* q4k, const float* bias, int in_dim, int out_dim, mg_linear_q4k** out) {
    if (!q4k) return -4;
    return make(q4k, nullptr, bias, in_dim, out_dim, out);
}

void mg_linear_q4k_evict(mg_linear_q4k* l) {
    if (!l) return;
    cudaFree(l->q4k_dev); cudaFree(l->w_dev); cudaFree(l->bias_dev);
    l->q4k_dev = nullptr; l->w_dev = nullptr; l->bias_dev = nullptr;
}
void mg_linear_q4k_destroy(mg_linear_q4k* l) {
    mg_linear_q4k_evict(l);
    delete l;
}
int mg_linear_q4k_is_resident(const mg_linear_q4k* l) {
    return l && l->q4k_dev && l->bias_dev && (!l->expand || l->w_dev);
}
// 1: keep an fp32 copy on the device and run dense matvecs (the reference's behaviour); 0: run the
// matvec on the Q4_K bytes (default).  Evicts, so that the next forward builds the chosen form.
int mg_linear_q4k_set_expanded(mg_linear_q4k* l, int expanded) {
    if (!l) return -4;
    mg_linear_q4k_evict(l);
    l->expand = expanded != 0;
    return 0;
}
size_t mg_linear_q4k_host_size_bytes(const mg_linear_q4k* l) {
    return l ? l->host_q4k.size() + l->host_bias.size() * 4 : 0;
}
// Device footprint when resident: Q4_K bytes + bias (+ the fp32 copy in the expanded mode; the
// reference's dequant_size_bytes, neuron.rs:978-980).
size_t mg_linear_q4k_device_size_bytes(const mg_linear_q4k* l) {
    if (!l) return 0;
    return l->host_q4k.size() + l->host_bias.size() * 4 + (l->expand ? (size_t)l->in_dim * l->out_dim * 4 : 0);
}
const uint8_t* mg_linear_q4k_host_blocks(const mg_linear_q4k* l, size_t* bytes) {
    if (!l) return nullptr;
    if (bytes) *bytes = l->host_q4k.size();
    return l->host_q4k.data();
}

// Upload (and, expanded, dequantise once); no-op when already resident (neuron.rs:989-1030).
int mg_linear_q4k_ensure_resident(mg_linear_q4k* l, void* stream) {
    if (!l) return -4;
    if (mg_linear_q4k_is_resident(l)) return 0;
    mg_linear_q4k_evict(l);
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&l->q4k_dev), l->host_q4k.size());
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&l->bias_dev), l->host_bias.size() * 4);
    if (e == cudaSuccess && l->expand) e = cudaMalloc(reinterpret_cast<void**>(&l->w_dev), (size_t)l->in_dim * l->out_dim * 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (e == cudaSuccess) e = cudaMemcpyAsync(l->q4k_dev, l->host_q4k.data(), l->host_q4k.size(), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(l->bias_dev, l->host_bias.data(), l->host_bias.size() * 4, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess && l->expand)
        e = (cudaError_t)launch_dequant_q4k_on_stream(l->q4k_dev, (int)(l->host_q4k.size() / 144), l->w_dev, stream);
    if (e != cudaSuccess) {
        mg_linear_q4k_evict(l);
        return (int)e;
    }
    return 0;
}

// out = W . x + bias on device vectors (neuron.rs:1059-1108): ensure_resident, one matvec launch,
// then evict when asked (the eviction waits for the stream: the buffers are still in use until then).
int mg_linear_q4k_forward(mg_linear_q4k* l, const float* x_dev, float* out_dev, int auto_evict, void* stream) {
    if (!l || !x_dev || !out_dev) return -4;
    int rc = mg_linear_q4k_ensure_resident(l, stream);
    if (rc) return rc;
    if (l->expand) rc = mg_matvec_f32_on_stream(l->w_dev, x_dev, l->bias_dev, out_dev, l->out_dim, l->in_dim, stream);
    else rc = mg_matvec_q4k_bias_on_stream(l->q4k_dev, x_dev, l->bias_dev, out_dev, l->out_dim, l->in_dim / 256, stream);
    if (rc) return rc;
    if (auto_evict) {
        const cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
        mg_linear_q4k_evict(l);
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

}  // extern "C"
