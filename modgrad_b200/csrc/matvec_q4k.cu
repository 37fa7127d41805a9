// Batch-1 Q4_K matvec (GEMV): y[row] = sum_e dequant(W)[row][e] * x[e] (+ bias[row]).
//
// Replaces the reference's one-block-per-row, byte-load kernel
// (crates/modgrad-device/kernels/matvec_q4k.hip:55-124).  The op is HBM-bound (0.5625 bytes
// per weight), but at B200 bandwidth only about 3.4 lane-operations per weight are available,
// so the arithmetic is arranged to need about half of that:
//
//   1. The activations are rewritten as block-fixed-point byte limbs (xlimbs.cuh): by every
//      CTA into its own shared-memory table when the matvec is a single launch
//      (launch_matvec_q4k), or once by x_to_limbs_kernel into global memory when several
//      matvecs share one activation vector (the *_limbs entry points).
//   2. matvec_q4k_dp4a_kernel streams the weights with 16-byte loads.  One lane owns one
//      32-byte group of a super-block (two complete sub-blocks), a warp covers eight
//      consecutive super-blocks (1152 contiguous bytes of a row) per step and works on R
//      rows at once so the limb registers are reused R times.  Nibbles are unpacked four at a
//      time in registers and multiplied with dp4a (exact int32 sums per sub-block); the 6-bit
//      scales are unpacked in registers; per sub-block
//          d*sc * s * sum(q*a)  -  dmin*m * sum(x)
//      is accumulated in f32 and rows are reduced with warp shuffles.
//      One persistent 512-thread CTA per SM, row groups interleaved over all warps.  Before
//      it touches x the kernel issues its first weight loads, so the weight stream starts
//      while x is still being converted; with programmatic dependent launch that part can
//      also overlap the tail of the previous kernel in the stream.
//
// matvec_q4k_f32_kernel is the plain-f32 variant (x staged as f32, one fma per weight) kept
// for vectors too long for the shared-memory record table.
//
// Accuracy contract: a different summation order than the CPU reference
// (crates/modgrad-device/src/kfd/llm.rs:695-735); within 1e-5 of an f64-accumulated
// reference relative to the RMS of the output.
#include <float.h>
#include <stdio.h>
#include <stdlib.h>

#include <atomic>
#include <map>
#include <mutex>

#include "gemv_q4k_device.cuh"
#include "gemv_q4k_mma.hpp"
#include "launch_common.cuh"
#include "q4k_device.cuh"
#include "xlimbs.cuh"

namespace {

using namespace gemvdev;

// up == nullptr: records of x.  up != nullptr: records of silu(x) * up, the SwiGLU product
// (exact logistic, crates/modgrad-device/src/kfd/llm.rs:1065-1069), also stored as f32 to
// `act_out` when that is given.
template <int PEER>
__global__ void __launch_bounds__(256) x_to_limbs_kernel(const float* x,
                                                         const float* up, float* act_out,
                                                         uint32_t* rec, int n_chunks,
                                                         int aligned, int hold_trigger,
                                                         const mgpeer::PeerSync peer) {
    // Let the kernel that follows be scheduled now (unless held back), then wait for whatever
    // produced x: this kernel may itself have been launched early.
    if (!hold_trigger) griddep_launch_dependents();
    griddep_wait();
    // n_chunks is a multiple of 8, so whole 8-thread sub-block teams are in or out of range;
    // threads past the end stay for the warp shuffles and store nothing.
    const int chunk = blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = chunk < n_chunks;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (valid) load_chunk(v, x, chunk, aligned);
    if (up != nullptr && valid) {
        float u[4];
        load_chunk(u, up, chunk, aligned);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float sig = 1.0f / (1.0f + expf(-v[i]));
            v[i] = (v[i] * sig) * u[i];
        }
        if (act_out != nullptr) {
#pragma unroll
            for (int i = 0; i < 4; ++i) act_out[(size_t)chunk * 4 + i] = v[i];
        }
    }
    convert_chunk<PEER>(v, chunk, rec, valid, &peer);
    if (PEER == kPeerFused) mgpeer::peer_finish(peer);
}

// FROM_X = 1: `src` is the f32 activation vector and every CTA converts it into its
// shared-memory record table itself (one kernel per matvec); FROM_X = 0: `src` is a record
// table in global memory made by x_to_limbs_kernel (several matvecs share one conversion).
template <int R, int FROM_X, int PEER>
__global__ void __launch_bounds__(kGemvThreads, 1)
matvec_q4k_dp4a_kernel(const MatList ml, const void* src, int x_aligned, int bpr) {
    gemv_body<R, FROM_X, false, true, PEER>(ml, src, x_aligned, bpr, (int)blockIdx.x, (int)gridDim.x);
}

// Warps of the ring kernel that gave up waiting for a bulk copy (never expected; a non-zero
// count means some rows of some result were left unwritten).
__device__ unsigned g_ring_timeouts = 0;

// The same arithmetic with the weight stream staged in shared memory by bulk asynchronous
// copies (gemv_ring_body): the default path.
// PEER (gemv_q4k_device.cuh): which exchange the launch ends with / reads its input from; the
// instantiation for none carries none of that code.
template <int R, int FROM_X, int PEER>
__global__ void __launch_bounds__(kGemvThreads, 1)
matvec_q4k_ring_kernel(const MatList ml, const void* src, int x_aligned, int bpr, int depth) {
    gemv_ring_body<R, FROM_X, PEER>(ml, src, x_aligned, bpr, depth, &g_ring_timeouts);
}

// ---------------------------------------------------------------------------------------------
// Plain-f32 variant: lane = (block in a 4-block window, 16-byte chunk), x staged as f32.
// ---------------------------------------------------------------------------------------------
constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kChunkBlocksMax = 112;  // super-blocks of x staged per pass (112 KiB of f32)

template <int R>
__global__ void __launch_bounds__(kThreads)
matvec_q4k_f32_kernel(const uint8_t* __restrict__ w, const float* __restrict__ x,
                      const float* __restrict__ bias, float* __restrict__ y, int out_dim, int bpr,
                      int chunk_blocks, int x_aligned) {
    extern __shared__ __align__(16) float xs[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int c = lane & 7;    // 16-byte chunk of qs inside the block: group c>>1, half c&1
    const int bl = lane >> 3;  // block inside the 4-block window
    const int x_off = 64 * (c >> 1) + 16 * (c & 1);
    const int sub_lo = 2 * (c >> 1);
    const size_t row_bytes = (size_t)bpr * q4k::kBlockBytes;
    const int row0 = (blockIdx.x * kWarps + warp) * R;

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    for (int cb = 0; cb < bpr; cb += chunk_blocks) {
        const int nb = min(chunk_blocks, bpr - cb);
        if (cb > 0) __syncthreads();
        const float* xg = x + (size_t)cb * q4k::kBlockElems;
        if (x_aligned) {
            for (int i = threadIdx.x * 4; i < nb * q4k::kBlockElems; i += kThreads * 4)
                cp_async16(&xs[i], &xg[i]);
            cp_async_wait_all();
        } else {
            for (int i = threadIdx.x; i < nb * q4k::kBlockElems; i += kThreads) xs[i] = xg[i];
        }
        __syncthreads();

        if (row0 < out_dim) {
            for (int b0 = 0; b0 < nb; b0 += 4) {
                const int blk = b0 + bl;
                const bool active = blk < nb;
                uint4 hdr[R], q[R];
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    hdr[r] = make_uint4(0, 0, 0, 0);
                    q[r] = make_uint4(0, 0, 0, 0);
                    if (active && row0 + r < out_dim) {
                        const uint8_t* p =
                            w + (size_t)(row0 + r) * row_bytes + (size_t)(cb + blk) * q4k::kBlockBytes;
                        hdr[r] = q4k::ld_nc_u4(p);
                        q[r] = q4k::ld_stream_u4(p + 16 + c * 16);
                    }
                }
                if (!active) continue;
                float xlo[16], xhi[16];
                const float4* xp = reinterpret_cast<const float4*>(xs + blk * q4k::kBlockElems + x_off);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 a = xp[i], b = xp[8 + i];
                    xlo[4 * i] = a.x; xlo[4 * i + 1] = a.y; xlo[4 * i + 2] = a.z; xlo[4 * i + 3] = a.w;
                    xhi[4 * i] = b.x; xhi[4 * i + 1] = b.y; xhi[4 * i + 2] = b.z; xhi[4 * i + 3] = b.w;
                }
                float sx_lo = 0.0f, sx_hi = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; ++i) { sx_lo += xlo[i]; sx_hi += xhi[i]; }
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float d = q4k::half_bits_finite_or_zero(hdr[r].x);
                    const float dmin = q4k::half_bits_finite_or_zero(hdr[r].x >> 16);
                    const q4k::ScaleMin sm = q4k::unpack_scales(hdr[r].y, hdr[r].z, hdr[r].w);
                    const float dsc_lo = d * (float)q4k::scale_of(sm, sub_lo);
                    const float dsc_hi = d * (float)q4k::scale_of(sm, sub_lo + 1);
                    const float dm_lo = dmin * (float)q4k::min_of(sm, sub_lo);
                    const float dm_hi = dmin * (float)q4k::min_of(sm, sub_lo + 1);
                    const uint32_t qw[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
                    float s_lo = 0.0f, s_hi = 0.0f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t lo4 = qw[k] & 0x0F0F0F0Fu;
                        const uint32_t hi4 = (qw[k] >> 4) & 0x0F0F0F0Fu;
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            s_lo = fmaf((float)((lo4 >> (8 * b)) & 0xFFu), xlo[4 * k + b], s_lo);
                            s_hi = fmaf((float)((hi4 >> (8 * b)) & 0xFFu), xhi[4 * k + b], s_hi);
                        }
                    }
                    acc[r] += dsc_lo * s_lo - dm_lo * sx_lo + dsc_hi * s_hi - dm_hi * sx_hi;
                }
            }
        }
    }
    if (row0 < out_dim) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float s = q4k::warp_sum(acc[r]);
            if (lane == 0 && row0 + r < out_dim) y[row0 + r] = bias ? s + bias[row0 + r] : s;
        }
    }
}

cudaError_t launch_f32(const uint8_t* w, const float* x, const float* bias, float* y, int out_dim,
                       int bpr, cudaStream_t stream) {
    constexpr int R = 2;
    const int chunk_blocks = bpr < kChunkBlocksMax ? bpr : kChunkBlocksMax;
    const size_t smem = (size_t)chunk_blocks * q4k::kBlockElems * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(matvec_q4k_f32_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kChunkBlocksMax * q4k::kBlockElems * (int)sizeof(float));
    if (e != cudaSuccess) return e;
    const int rows_per_cta = kWarps * R;
    const unsigned grid = (unsigned)((out_dim + rows_per_cta - 1) / rows_per_cta);
    matvec_q4k_f32_kernel<R><<<grid, kThreads, smem, stream>>>(w, x, bias, y, out_dim, bpr, chunk_blocks,
                                                               mg::aligned16(x) ? 1 : 0);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
constexpr int kMaxRecordSmem = 200 * 1024;  // limb-record table limit: bpr <= 246

template <int R, int FROM_X, int PEER>
cudaError_t launch_dp4a(const MatList& ml, const void* src, int bpr, int sms, cudaStream_t stream) {
    const size_t smem = xlimbs::record_bytes((size_t)bpr * 256);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(matvec_q4k_dp4a_kernel<R, FROM_X, PEER>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxRecordSmem);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    int groups = 0;
    for (int i = 0; i < ml.n; ++i) groups += (ml.rows[i] + R - 1) / R;
    const int grid = groups < sms ? groups : sms;  // row groups go to warp slots warp-major
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int x_aligned = mg::aligned16(src) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, matvec_q4k_dp4a_kernel<R, FROM_X, PEER>, ml, src, x_aligned, bpr);
}

// Stages per warp the ring kernel can have for rows of `bpr` super-blocks at R rows per stage
// (0: the shared memory left beside the record table is too small).
constexpr int kRingSmemBudget = 226 * 1024;
int ring_depth(int bpr, int rows) {
    const int per_warp = (kRingSmemBudget - ring_record_bytes(bpr)) / kGemvWarps;
    const int d = per_warp / ring_stage_bytes(bpr, rows);
    return d > kRingMaxDepth ? kRingMaxDepth : (d < 0 ? 0 : d);
}

template <int R, int FROM_X, int PEER>
cudaError_t launch_ring(const MatList& ml, const void* src, int bpr, int depth, int sms, cudaStream_t stream) {
    const size_t smem = (size_t)ring_record_bytes(bpr) + (size_t)kGemvWarps * depth * ring_stage_bytes(bpr, R);
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(matvec_q4k_ring_kernel<R, FROM_X, PEER>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kRingSmemBudget);
        if (e != cudaSuccess) return e;
        attr_set[dev] = true;
    }
    int groups = 0;
    for (int i = 0; i < ml.n; ++i) groups += (ml.rows[i] + R - 1) / R;
    const int grid = groups < sms ? groups : sms;  // row groups go to warp slots warp-major
    return mg::launch_pdl(matvec_q4k_ring_kernel<R, FROM_X, PEER>, dim3((unsigned)grid), dim3(kGemvThreads), smem, stream,
                          ml, src, mg::aligned16(src) ? 1 : 0, bpr, depth);
}

// Ring kernel when at least two stages per warp fit, else the register-load kernel.
template <int R, int FROM_X>
cudaError_t launch_gemv(const MatList& ml, const void* src, int bpr, int sms, cudaStream_t stream) {
    const int depth = ring_depth(bpr, R);
    const bool stamped = (ml.peer.world > 1 && ml.peer.stamp_slots != nullptr) || ml.xin.slots != nullptr;
    const bool fused = ml.peer.world > 1 && ml.peer.stamp_slots == nullptr;
    if (stamped && fused) return cudaErrorInvalidValue;  // a stamped input with a handshake output: not built
    if (depth >= 2) {
        if (stamped) return launch_ring<R, FROM_X, kPeerStamped>(ml, src, bpr, depth, sms, stream);
        if (fused) return launch_ring<R, FROM_X, kPeerFused>(ml, src, bpr, depth, sms, stream);
        return launch_ring<R, FROM_X, kPeerNone>(ml, src, bpr, depth, sms, stream);
    }
    if (stamped) return launch_dp4a<R, FROM_X, kPeerStamped>(ml, src, bpr, sms, stream);
    if (fused) return launch_dp4a<R, FROM_X, kPeerFused>(ml, src, bpr, sms, stream);
    return launch_dp4a<R, FROM_X, kPeerNone>(ml, src, bpr, sms, stream);
}

// Per (device, stream) scratch for the limb records of long activation vectors.  Every kernel of
// this library waits for its predecessor in the stream to COMPLETE before it writes (or reads)
// anything the predecessor touches, so one table per stream would do; two halves used alternately
// keep the conversion of call N+1 off the lines the GEMV of call N has just read.
struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;  // of one half
    unsigned turn = 0;
};
std::mutex g_ws_mu;
std::map<std::pair<int, cudaStream_t>, Workspace> g_ws;

cudaError_t workspace_for(cudaStream_t stream, size_t bytes, void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> lock(g_ws_mu);
    Workspace& ws = g_ws[{dev, stream}];
    if (ws.bytes < bytes) {
        // Growing allocates, which a capturing stream cannot do: the first call on a stream
        // (and the first call with a longer x) has to come before stream capture.
        cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st != cudaStreamCaptureStatusNone)
            return cudaErrorStreamCaptureUnsupported;
        if (ws.ptr) {
            e = cudaFree(ws.ptr);
            ws.ptr = nullptr;
            ws.bytes = 0;
            if (e != cudaSuccess) return e;
        }
        const size_t want = bytes < (size_t)(128 << 10) ? (size_t)(128 << 10) : ((bytes + 255) & ~(size_t)255);
        e = cudaMalloc(&ws.ptr, 2 * want);
        if (e != cudaSuccess) return e;
        ws.bytes = want;
    }
    *out = static_cast<char*>(ws.ptr) + (ws.turn++ & 1u) * ws.bytes;
    return cudaSuccess;
}

// Above this many super-blocks per row the per-CTA conversion of x costs more than a separate
// conversion kernel plus a scratch table.
constexpr int kFusedConvertMaxBpr = 32;
// From this many rows on (two or more 16-row tiles per SM) the tensor-core kernel wins.
constexpr int kMmaMinRows = 4736;

// Speculation of the tensor-core GEMV (gemv_q4k_mma.cu): it converts x and computes while the kernel
// queued before it may still run, and publishes only after x has been re-checked.  A stale x costs
// a second pass, so the launcher does not speculate when it KNOWS the input is still being produced:
// when x or the addend overlaps the output of the previous matvec this library queued on the same
// stream.  (Kernels of other libraries in between are invisible here; the re-check covers them.)
std::atomic<int> g_speculation{-1};  // -1: not read from the environment yet
struct LastOutput {
    const char* lo = nullptr;
    const char* hi = nullptr;
};
std::mutex g_last_mu;
std::map<std::pair<int, cudaStream_t>, LastOutput> g_last_out;

bool overlaps(const void* p, size_t n, const LastOutput& o) {
    const char* a = static_cast<const char*>(p);
    return p != nullptr && o.lo != nullptr && a < o.hi && o.lo < a + n;
}
int speculation_for(cudaStream_t stream, const void* x, size_t x_bytes, const void* addend, const void* y,
                    size_t y_bytes) {
    int on = g_speculation.load(std::memory_order_relaxed);
    if (on < 0) {
        const char* e = getenv("MODGRAD_Q4K_SPECULATE");
        on = (e && e[0] == '0') ? 0 : 1;
        g_speculation.store(on, std::memory_order_relaxed);
    }
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_last_mu);
    LastOutput& last = g_last_out[{dev, stream}];
    const bool dependent = overlaps(x, x_bytes, last) || overlaps(addend, y_bytes, last);
    last.lo = static_cast<const char*>(y);
    last.hi = last.lo + y_bytes;
    return on && !dependent ? 1 : 0;
}

// An armed exchange stores the output at the same offset of every peer's arena: the target must
// lie inside this rank's arena, behind the flag block.
bool peer_target_ok(const mgpeer::PeerSync& ps, const void* out, size_t bytes) {
    if (ps.world <= 1) return true;
    if (ps.stamp_slots != nullptr)  // one 8-byte slot per 4-byte result word
        return ps.epoch_dev != nullptr && ps.stamp_index0 >= 0 &&
               mgpeer::in_arena(ps, ps.stamp_slots + ps.stamp_index0, bytes * 2);
    return mgpeer::in_arena(ps, out, bytes);
}

bool limbs_path_ok(int bpr) { return xlimbs::record_bytes((size_t)bpr * 256) <= (size_t)kMaxRecordSmem; }

}  // namespace

// x[k] -> limb records (xlimbs.cuh); k % 256 == 0; records: mg_q4k_limb_record_bytes(k) bytes,
// 16-byte aligned.
extern "C" int mg_q4k_x_to_limbs_on_stream(const float* x, int k, void* records, void* stream) {
    if (x == nullptr || records == nullptr || k <= 0 || (k % 256) != 0) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(records)) return (int)cudaErrorInvalidValue;
    const int threads = k / 4;  // one thread per 4 activations
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, x_to_limbs_kernel<kPeerNone>, x, (const float*)nullptr, (float*)nullptr,
                                   static_cast<uint32_t*>(records), threads,
                                   ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) ? 1 : 0,
                                   mg::early_trigger_flag() ? 0 : 1, mgpeer::PeerSync{});
}

// records (and act_out, optional f32 copy) of silu(gate) * up: the input of the down
// projection, produced directly in limb form.
extern "C" int mg_swiglu_limbs_on_stream(const float* gate, const float* up, float* act_out, int n,
                                         void* records, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    if (!gate || !up || !records || n <= 0 || (n % 64) != 0) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(records)) return (int)cudaErrorInvalidValue;
    if (!peer_target_ok(peer, records, xlimbs::record_bytes((size_t)n))) return (int)cudaErrorInvalidValue;
    const int threads = n / 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)((threads + 255) / 256));
    cfg.blockDim = dim3(256);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const int aligned = (mg::aligned16(gate) && mg::aligned16(up)) ? 1 : 0;
    if (peer.world > 1 && peer.stamp_slots != nullptr)
        return (int)cudaLaunchKernelEx(&cfg, x_to_limbs_kernel<kPeerStamped>, gate, up, act_out, static_cast<uint32_t*>(records),
                                       threads, aligned, mg::early_trigger_flag() ? 0 : 1, peer);
    if (peer.world > 1)
        return (int)cudaLaunchKernelEx(&cfg, x_to_limbs_kernel<kPeerFused>, gate, up, act_out, static_cast<uint32_t*>(records),
                                       threads, aligned, mg::early_trigger_flag() ? 0 : 1, peer);
    return (int)cudaLaunchKernelEx(&cfg, x_to_limbs_kernel<kPeerNone>, gate, up, act_out, static_cast<uint32_t*>(records),
                                   threads, aligned, mg::early_trigger_flag() ? 0 : 1, peer);
}

// Number of warps of the GEMV that ever gave up waiting for a weight copy on the current
// device (0 in a healthy process); synchronises the device.  Negative: a CUDA error code, negated.
extern "C" long long mg_matvec_q4k_timeouts(void) {
    unsigned n = 0;
    const cudaError_t e = cudaMemcpyFromSymbol(&n, g_ring_timeouts, sizeof(n));
    return e == cudaSuccess ? (long long)n : -(long long)e;
}

// Switches the speculative start of launch_matvec_q4k / mg_matvec_q4k_bias_on_stream on (default) or
// off for the whole process; returns the previous setting.
extern "C" int mg_matvec_q4k_speculation(int enabled) {
    int prev = g_speculation.exchange(enabled ? 1 : 0);
    return prev < 0 ? 1 : prev;
}

extern "C" size_t mg_q4k_limb_record_bytes(int k) { return k > 0 ? xlimbs::record_bytes((size_t)k) : 0; }

// `peer`: the exchange armed for this launch by an engine that wants the output all-gathered
// (taken from the host thread's slot by the extern "C" entry point, whatever path it then takes).
template <int FROM_X>
int dispatch_multi(const MatList& ml_in, const void* src, int blocks_per_row, const mgpeer::PeerSync& peer,
                   cudaStream_t s) {
    MatList ml = ml_in;
    ml.hold_trigger = mg::early_trigger_flag() ? 0 : 1;
    ml.peer = peer;
    if (ml.peer.world > 1 && ml.n != 1) return (int)cudaErrorInvalidValue;
    const mg::DeviceProps& dp = mg::device_props();
    const int sms = dp.ok ? dp.sm_count : 148;
    const int slots = sms * kGemvWarps;
    int rows = 0;
    for (int i = 0; i < ml.n; ++i) rows += ml.rows[i];
    // Rows per warp: reuse of the limb registers against keeping every warp slot busy.
    if (rows >= 4 * slots && (ring_depth(blocks_per_row, 4) >= 2 || ring_depth(blocks_per_row, 2) < 2))
        return (int)launch_gemv<4, FROM_X>(ml, src, blocks_per_row, sms, s);
    if (rows >= slots) return (int)launch_gemv<2, FROM_X>(ml, src, blocks_per_row, sms, s);
    return (int)launch_gemv<1, FROM_X>(ml, src, blocks_per_row, sms, s);
}
template <int FROM_X>
int dispatch_dp4a(const uint8_t* w_q4, const void* src, const float* addend, float* y, int out_dim,
                  int blocks_per_row, const mgpeer::PeerSync& peer, cudaStream_t s) {
    MatList ml = {};
    ml.w[0] = w_q4; ml.y[0] = y; ml.addend[0] = addend; ml.rows[0] = out_dim; ml.n = 1;
    return dispatch_multi<FROM_X>(ml, src, blocks_per_row, peer, s);
}

bool fill_matlist(MatList& ml, int n_mats, const uint8_t* const* w, float* const* y, const float* const* addend,
                  const int* out_dims) {
    if (n_mats < 1 || n_mats > kMaxMats || !w || !y || !out_dims) return false;
    ml = MatList{};
    ml.n = n_mats;
    for (int i = 0; i < n_mats; ++i) {
        if (!w[i] || !y[i] || out_dims[i] <= 0 || !mg::aligned16(w[i])) return false;
        ml.w[i] = w[i]; ml.y[i] = y[i]; ml.rows[i] = out_dims[i];
        ml.addend[i] = addend ? addend[i] : nullptr;
    }
    return true;
}

// y = dequant(W) . x (+ bias) with x given as limb records (several matvecs that share one
// activation vector convert it once).
extern "C" int mg_matvec_q4k_limbs_on_stream(const uint8_t* w_q4, const void* records, const float* bias,
                                             float* y, int out_dim, int blocks_per_row, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    (void)mgpeer::take_next_stamp_in();  // only the multi entry points read stamped input
    if (out_dim <= 0 || blocks_per_row <= 0) return (int)cudaErrorInvalidValue;
    if (w_q4 == nullptr || records == nullptr || y == nullptr) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(w_q4) || !mg::aligned16(records)) return (int)cudaErrorInvalidValue;
    if (!limbs_path_ok(blocks_per_row)) return (int)cudaErrorInvalidValue;
    if (!peer_target_ok(peer, y, (size_t)out_dim * sizeof(float))) return (int)cudaErrorInvalidValue;
    return dispatch_dp4a<0>(w_q4, records, bias, y, out_dim, blocks_per_row, peer, (cudaStream_t)stream);
}

// y = dequant(W) . x + bias (bias may be null): the semantics of Op::Matvec
// (crates/modgrad-device/src/backend/op.rs:175-186) and of the KFD kernel's kernarg
// (crates/modgrad-device/src/kfd/dispatch_queue.rs:235-262).  Rows of up to 8192 weights: one
// kernel, every CTA converts x into its own record table.  Longer rows: a conversion kernel
// into a per-stream scratch table, then the GEMV (the first call on a stream, and the first
// with a longer x, allocates the scratch and therefore has to precede any stream capture).
extern "C" int mg_matvec_q4k_bias_on_stream(const uint8_t* w_q4, const float* x, const float* bias,
                                            float* y, int out_dim, int blocks_per_row, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    (void)mgpeer::take_next_stamp_in();  // only the multi entry points read stamped input
    if (out_dim <= 0 || blocks_per_row <= 0) return (int)cudaErrorInvalidValue;
    if (w_q4 == nullptr || x == nullptr || y == nullptr) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(w_q4)) return (int)cudaErrorInvalidValue;
    if (blocks_per_row > 0x7FFFFFFF / 256) return (int)cudaErrorInvalidValue;
    if (!peer_target_ok(peer, y, (size_t)out_dim * sizeof(float))) return (int)cudaErrorInvalidValue;
    cudaStream_t s = (cudaStream_t)stream;
    // Matrices of many short rows go to the tensor-core kernel (half an SM per CTA, speculative
    // start: consecutive launches overlap); few rows or long rows are faster on the dp4a ring
    // kernel below, whose x conversion is lighter.
    // Measured (graph-replayed chains, rotating weight copies): 18944 x 3584 9.6 against 12.3 us, 8192 x 8192
    // 12.2 against 14.0 us, 28672 x 8192 27.0 against 31.3 us in favour of the tensor-core kernel (the last two
    // with three windows per row and one CTA per SM); rows of 18944 and 28672 weights (down projections)
    // 18.6 against 17.3 and 52.8 against 36.1 us in favour of the ring kernel.
    const bool want_mma = (out_dim >= kMmaMinRows &&
                           (gemvmma::fits_half_sm(blocks_per_row) || blocks_per_row <= kFusedConvertMaxBpr)) ||
                          !limbs_path_ok(blocks_per_row);
    if (peer.world <= 1 && want_mma && gemvmma::supported(blocks_per_row)) {
        // the tensor-core kernel: one launch, x converted inside, no scratch
        const mg::DeviceProps& dp = mg::device_props();
        unsigned* timeouts = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&timeouts), g_ring_timeouts);
        if (e != cudaSuccess) return (int)e;
        return (int)gemvmma::launch(w_q4, x, bias, y, out_dim, blocks_per_row, mg::early_trigger_flag() ? 0 : 1,
                                    speculation_for(s, x, (size_t)blocks_per_row * 256 * sizeof(float), bias, y,
                                                    (size_t)out_dim * sizeof(float)),
                                    timeouts, dp.ok ? dp.sm_count : 148, s);
    }
    if (!limbs_path_ok(blocks_per_row)) {
        if (peer.world > 1) return (int)cudaErrorInvalidValue;  // the f32 kernel has no fused exchange
        return (int)launch_f32(w_q4, x, bias, y, out_dim, blocks_per_row, s);
    }
    if (blocks_per_row <= kFusedConvertMaxBpr)
        return dispatch_dp4a<1>(w_q4, x, bias, y, out_dim, blocks_per_row, peer, s);
    void* ws = nullptr;
    const int k = blocks_per_row * 256;
    cudaError_t e = workspace_for(s, xlimbs::record_bytes((size_t)k), &ws);
    if (e != cudaSuccess) return (int)e;
    const int rc = mg_q4k_x_to_limbs_on_stream(x, k, ws, stream);
    if (rc) return rc;
    return dispatch_dp4a<0>(w_q4, ws, bias, y, out_dim, blocks_per_row, peer, s);
}

// Up to three matrices times ONE activation vector in one launch (q/k/v, gate/up):
// y[i] = dequant(w[i]) . x + addend[i].  `x_is_records` selects f32 x (rows of up to 8192
// weights, converted inside the kernel) or limb records.  addend may be null, its entries
// may be null, and an entry may alias the matching y (in-place residual add).
extern "C" int mg_matvec_q4k_multi_on_stream(int n_mats, const uint8_t* const* w_q4, const void* x,
                                             int x_is_records, const float* const* addend, float* const* y,
                                             const int* out_dims, int blocks_per_row, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    const mgpeer::StampIn xin = mgpeer::take_next_stamp_in();
    if (blocks_per_row <= 0 || x == nullptr || !limbs_path_ok(blocks_per_row)) return (int)cudaErrorInvalidValue;
    MatList ml;
    if (!fill_matlist(ml, n_mats, w_q4, y, addend, out_dims)) return (int)cudaErrorInvalidValue;
    ml.xin = xin;
    if (!peer_target_ok(peer, ml.y[0], (size_t)ml.rows[0] * sizeof(float))) return (int)cudaErrorInvalidValue;
    if (x_is_records) {
        if (!mg::aligned16(x)) return (int)cudaErrorInvalidValue;
        return dispatch_multi<0>(ml, x, blocks_per_row, peer, (cudaStream_t)stream);
    }
    if (blocks_per_row > kFusedConvertMaxBpr) return (int)cudaErrorInvalidValue;
    return dispatch_multi<1>(ml, x, blocks_per_row, peer, (cudaStream_t)stream);
}

// The same with RMSNorm fused in front: y[i] = dequant(w[i]) . (x * rsqrt(mean(x^2)+eps) * norm_weight)
// + addend[i]; x is f32, blocks_per_row <= 32.  Saves the separate norm launch of the decode
// loop (RocmGemma::layer launches kern::rms_norm before the q/k/v and the gate/up matvecs).
extern "C" int mg_rmsnorm_matvec_q4k_multi_on_stream(int n_mats, const uint8_t* const* w_q4, const float* x,
                                                     const float* norm_weight, float eps,
                                                     const float* const* addend, float* const* y,
                                                     const int* out_dims, int blocks_per_row, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    const mgpeer::StampIn xin = mgpeer::take_next_stamp_in();
    if (blocks_per_row <= 0 || blocks_per_row > kFusedConvertMaxBpr || !x || !norm_weight) return (int)cudaErrorInvalidValue;
    MatList ml;
    if (!fill_matlist(ml, n_mats, w_q4, y, addend, out_dims)) return (int)cudaErrorInvalidValue;
    ml.xin = xin;
    if (!peer_target_ok(peer, ml.y[0], (size_t)ml.rows[0] * sizeof(float))) return (int)cudaErrorInvalidValue;
    ml.norm_w = norm_weight;
    ml.eps = eps;
    return dispatch_multi<1>(ml, x, blocks_per_row, peer, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant.
//
// Some hosts must never see this library allocate device memory: an engine that carves every
// buffer out of one arena it sized itself (the reference's resident decoder packs all weights
// into a single buffer and refuses loads that would over-commit the GPU), a serving process
// with a fixed memory budget, or a latency-critical loop in which cudaMalloc — which may
// synchronise the whole device — is not acceptable.  For them the limb records of x live in
// the fixed array below instead of a scratch buffer obtained at run time.  The array is part of
// the loaded library image: every GPU that loads the library holds these 104 KiB until exit.
constexpr int kNoAllocMaxBpr = 128;  // rows of up to 32768 weights
static __device__ __align__(256) unsigned char g_noalloc_records[kNoAllocMaxBpr * 4 * xlimbs::kRecordBytes];

// y = dequant(W) . x like launch_matvec_q4k_on_stream, without any allocation: no cudaMalloc /
// cudaFree and no allocating library routine on any call.  blocks_per_row above 128 is refused
// with cudaErrorInvalidValue (and a line on stderr).
// The first call on a device looks up the device address of the built-in array (with that
// device current) and remembers it; make that first call before any stream capture.
// All calls share the one array, which always holds the records of the most recent call and
// is completely rewritten for the length in use, so nothing has to be cleared between calls —
// but two calls that overlap on the GPU (different streams, or the same graph launched twice
// concurrently) race on it: keep calls of this entry point ordered on one stream.
extern "C" int launch_matvec_q4k_noalloc_on_stream(const uint8_t* w_q4, const float* x, float* y, int out_dim,
                                                   int blocks_per_row, void* stream) {
    const mgpeer::PeerSync peer = mgpeer::take_next_peer_sync();  // consumed on every path, errors included
    if (out_dim <= 0 || blocks_per_row <= 0) return (int)cudaErrorInvalidValue;
    if (w_q4 == nullptr || x == nullptr || y == nullptr) return (int)cudaErrorInvalidValue;
    if (!mg::aligned16(w_q4)) return (int)cudaErrorInvalidValue;
    if (!peer_target_ok(peer, y, (size_t)out_dim * sizeof(float))) return (int)cudaErrorInvalidValue;
    if (blocks_per_row > kNoAllocMaxBpr) {
        fprintf(stderr,
                "launch_matvec_q4k_noalloc_on_stream: blocks_per_row %d exceeds the built-in scratch "
                "(limit %d, i.e. rows of %d weights); use launch_matvec_q4k_on_stream\n",
                blocks_per_row, kNoAllocMaxBpr, kNoAllocMaxBpr * 256);
        return (int)cudaErrorInvalidValue;
    }
    // In host code the array's name is only a stand-in; the kernels need its device address.
    // (host threads may race to be first on a device: the slot is atomic and every racer stores the same address)
    static std::atomic<void*> dev_ptr[64] = {};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    void* records = dev_ptr[dev].load(std::memory_order_acquire);
    if (records == nullptr) {
        e = cudaGetSymbolAddress(&records, g_noalloc_records);
        if (e != cudaSuccess) return (int)e;
        dev_ptr[dev].store(records, std::memory_order_release);
    }
    const int rc = mg_q4k_x_to_limbs_on_stream(x, blocks_per_row * 256, records, stream);
    if (rc) return rc;
    return dispatch_dp4a<0>(w_q4, records, nullptr, y, out_dim, blocks_per_row, peer, (cudaStream_t)stream);
}

extern "C" int launch_matvec_q4k_on_stream(const uint8_t* w_q4, const float* x, float* y, int out_dim,
                                           int blocks_per_row, void* stream) {
    return mg_matvec_q4k_bias_on_stream(w_q4, x, nullptr, y, out_dim, blocks_per_row, stream);
}

extern "C" int launch_matvec_q4k(const uint8_t* w_q4, const float* x, float* y, int out_dim,
                                 int blocks_per_row) {
    return mg_matvec_q4k_bias_on_stream(w_q4, x, nullptr, y, out_dim, blocks_per_row, nullptr);
}
