// Device code of the batch-1 Q4_K GEMV shared by the stand-alone kernels (matvec_q4k.cu) and
// the persistent decode kernel (decode_persistent.cu): activation -> limb-record conversion,
// the per-window dp4a arithmetic and the GEMV body.  See matvec_q4k.cu for the design.
#pragma once
#include <float.h>

#include "peer_sync.cuh"
#include "q4k_device.cuh"
#include "xlimbs.cuh"

namespace gemvdev {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------------------------
// x -> limb records.  One thread converts 4 consecutive activations; 8 threads share a
// sub-block (max and sum by shuffles); 16 threads write one record.
// ---------------------------------------------------------------------------------------------
// Converts activations 4*chunk .. 4*chunk+3 (v) and writes this thread's share of the record
// of their sub-block; the 8 threads of a sub-block (8 consecutive lanes) call it together.
// PEER selects the exchange code that is compiled in: 0 none, 1 plain peer stores + handshake,
// 2 stamped words (peer_sync.cuh).  Kernels carry only the form they use: their code size decides
// how well the instruction cache serves the hot loop (the single-GPU GEMV lost 20 % when all of it
// was compiled into one kernel).
constexpr int kPeerNone = 0, kPeerFused = 1, kPeerStamped = 2;
template <int PEER = kPeerNone>
__device__ __forceinline__ void convert_chunk(const float (&v)[4], int chunk, uint32_t* __restrict__ rec,
                                              bool store = true, const mgpeer::PeerSync* peer = nullptr) {
    const int sub = chunk >> 3, t = chunk & 7;
    float amax = 0.f;
    int bad = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float a = fabsf(v[i]);
        bad |= !(a <= FLT_MAX);  // inf or NaN
        amax = fmaxf(amax, a);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
        bad |= __shfl_xor_sync(0xFFFFFFFFu, bad, o);
    }
    int E = (int)(__float_as_uint(amax) >> 23) - 127;  // floor(log2(amax)); -127 for 0 / sub-normal
    E = max(E, -100);
    const float s = __uint_as_float((uint32_t)(E - 21 + 127) << 23);    // 2^(E-21)
    const float inv = __uint_as_float((uint32_t)(21 - E + 127) << 23);  // 2^(21-E)
    uint32_t l2 = 0, l1 = 0, l0 = 0;
    int sum = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int a = bad ? 0 : __float2int_rn(v[i] * inv);  // |a| <= 2^22
        sum += a;
        l2 |= ((uint32_t)(a >> 16) & 0xFFu) << (8 * i);
        l1 |= ((uint32_t)(a >> 8) & 0xFFu) << (8 * i);
        l0 |= ((uint32_t)a & 0xFFu) << (8 * i);
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    if (!store) return;  // after the shuffles: lanes past the end only take part in them
    uint32_t* r = rec + (size_t)(sub >> 1) * xlimbs::kRecordWords;
    uint32_t* plane = r + (sub & 1) * 24;
    // A non-finite activation poisons its sub-block: the scale becomes NaN, so every
    // row's sum becomes NaN as it does in the reference (w * NaN).
    const float sc = bad ? __uint_as_float(0x7FC00000u) : s;
    if (PEER == kPeerStamped && peer != nullptr && peer->world > 1 && peer->stamp_slots != nullptr) {
        // records all-gathered word by word, every word stamped with the exchange's epoch
        const unsigned epoch = mgpeer::exchange_epoch(peer->epoch_dev, peer->epoch_mul, peer->epoch_add);
        const long long w0 = plane - rec, r0 = r - rec;  // word offsets inside this rank's record slice
        mgpeer::store_stamped_all(*peer, w0 + t, l2, epoch);
        mgpeer::store_stamped_all(*peer, w0 + 8 + t, l1, epoch);
        mgpeer::store_stamped_all(*peer, w0 + 16 + t, l0, epoch);
        if (t == 0) {
            mgpeer::store_stamped_all(*peer, r0 + 48 + (sub & 1), __float_as_uint(sc), epoch);
            mgpeer::store_stamped_all(*peer, r0 + 50 + (sub & 1), __float_as_uint(sc * (float)sum), epoch);
        }
        return;
    }
    if (PEER == kPeerFused && peer != nullptr && peer->world > 1) {  // records all-gathered by the producing kernel
        mgpeer::store_all(*peer, plane + t, l2);
        mgpeer::store_all(*peer, plane + 8 + t, l1);
        mgpeer::store_all(*peer, plane + 16 + t, l0);
        if (t == 0) {
            mgpeer::store_all(*peer, r + 48 + (sub & 1), __float_as_uint(sc));
            mgpeer::store_all(*peer, r + 50 + (sub & 1), __float_as_uint(sc * (float)sum));
        }
        return;
    }
    plane[t] = l2;
    plane[8 + t] = l1;
    plane[16 + t] = l0;
    if (t == 0) {
        r[48 + (sub & 1)] = __float_as_uint(sc);
        r[50 + (sub & 1)] = __float_as_uint(sc * (float)sum);
    }
}

// COHERENT: L2-level loads (ld.global.cg) for data other CTAs wrote earlier in this kernel.
template <bool COHERENT>
__device__ __forceinline__ float ld_f32(const float* p) {
    if (COHERENT) {
        float v;
        asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
        return v;
    }
    return *p;
}
template <bool COHERENT = false>
__device__ __forceinline__ void load_chunk(float (&v)[4], const float* x, int chunk, int aligned) {
    const float* p = x + (size_t)chunk * 4;
    if (COHERENT) {
        if (aligned) {
            asm volatile("ld.global.cg.v4.f32 {%0,%1,%2,%3}, [%4];"
                         : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]) : "l"(p));
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = ld_f32<true>(p + i);
        }
    } else if (aligned) {
        const float4 f = *reinterpret_cast<const float4*>(p);
        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
        v[0] = p[0]; v[1] = p[1]; v[2] = p[2]; v[3] = p[3];
    }
}

// ---------------------------------------------------------------------------------------------
// The streaming GEMV on limb records.
// ---------------------------------------------------------------------------------------------
constexpr int kGemvThreads = 512;
constexpr int kGemvWarps = kGemvThreads / 32;
constexpr int kWindowBytes = 8 * q4k::kBlockBytes;  // 1152: eight super-blocks of one row

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) { return __dp4a((int)a, (int)b, c); }
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) { return __dp4a(a, b, c); }
// unsigned bytes (a) times signed bytes (b)
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// Up to three weight matrices that multiply the same activation vector (q/k/v, gate/up) in
// one launch: their row groups are enumerated back to back.
constexpr int kMaxMats = 3;
struct MatList {
    const uint8_t* w[kMaxMats];
    float* y[kMaxMats];
    const float* addend[kMaxMats];  // y = W.x + addend (bias or residual; may alias y; may be null)
    int rows[kMaxMats];
    int n;
    // Optional RMSNorm fused in front (FROM_X kernels only): x <- x * rsqrt(mean(x^2)+eps) * norm_w
    const float* norm_w;
    float eps;
    // Non-zero: do not let the next kernel of the stream launch before this one has finished
    // (set when a kernel of another library, which may not wait for completion, follows).
    int hold_trigger;
    // world > 1: every result is also stored into the peers' arenas and the kernel ends with the
    // exchange handshake (peer_sync.cuh): matvec and all-gather of the output slices in one kernel.
    // y (and addend) then point into this rank's arena.
    mgpeer::PeerSync peer;
    // x (or the limb records) arrive as a stamped vector written by the peers: poll while staging.
    mgpeer::StampIn xin;
};
template <int R>
__device__ __forceinline__ int total_groups(const MatList& ml) {
    int t = 0;
#pragma unroll
    for (int i = 0; i < kMaxMats; ++i)
        if (i < ml.n) t += (ml.rows[i] + R - 1) / R;
    return t;
}
// group index -> (matrix, first row)
template <int R>
__device__ __forceinline__ void locate_group(const MatList& ml, int grp, int& mat, int& row0) {
    mat = 0;
    row0 = grp * R;
#pragma unroll
    for (int i = 0; i < kMaxMats - 1; ++i) {
        const int gi = (ml.rows[i] + R - 1) / R;
        if (i + 1 < ml.n && mat == i && grp >= gi) {
            grp -= gi;
            mat = i + 1;
            row0 = grp * R;
        }
    }
}
__device__ __forceinline__ const uint8_t* mat_w(const MatList& ml, int m) {
    return m == 0 ? ml.w[0] : (m == 1 ? ml.w[1] : ml.w[2]);
}
__device__ __forceinline__ int mat_rows(const MatList& ml, int m) {
    return m == 0 ? ml.rows[0] : (m == 1 ? ml.rows[1] : ml.rows[2]);
}

// One window of R rows: per lane the 16-byte header and the lane's 32-byte group.
template <int R>
struct Window {
    uint4 hdr[R], q0[R], q1[R];
};

template <int R>
__device__ __forceinline__ void load_window(Window<R>& wd, const uint8_t* lane_base, size_t row_bytes,
                                            int row0, int out_dim, int win, int g) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int row = min(row0 + r, out_dim - 1);  // tail rows re-read the last row
        const uint8_t* p = lane_base + (size_t)row * row_bytes + (size_t)win * kWindowBytes;
        wd.hdr[r] = q4k::ld_nc_u4(p);
        wd.q0[r] = q4k::ld_nc_u4(p + 16 + g * 32);
        wd.q1[r] = q4k::ld_nc_u4(p + 32 + g * 32);
    }
}

template <int R>
__device__ __forceinline__ void compute_window(const Window<R>& wd, const uint4* __restrict__ rec, int g,
                                               uint32_t sel_sc, float (&acc)[R]) {
    const uint4 tail = rec[12];
    const float s_lo = __uint_as_float(tail.x);
    const float s_hi = __uint_as_float(tail.y) * 0.0625f;  // high nibbles are used as 16*q
    const float x_lo = __uint_as_float(tail.z), x_hi = __uint_as_float(tail.w);
    float S_lo[R], S_hi[R];
    {   // low nibbles: sub-block 2g
        uint32_t L2[8], L1[8], L0[8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 a = rec[i], b = rec[2 + i], c = rec[4 + i];
            L2[4 * i] = a.x; L2[4 * i + 1] = a.y; L2[4 * i + 2] = a.z; L2[4 * i + 3] = a.w;
            L1[4 * i] = b.x; L1[4 * i + 1] = b.y; L1[4 * i + 2] = b.z; L1[4 * i + 3] = b.w;
            L0[4 * i] = c.x; L0[4 * i + 1] = c.y; L0[4 * i + 2] = c.z; L0[4 * i + 3] = c.w;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t qw[8] = {wd.q0[r].x, wd.q0[r].y, wd.q0[r].z, wd.q0[r].w,
                                    wd.q1[r].x, wd.q1[r].y, wd.q1[r].z, wd.q1[r].w};
            int s2 = 0;
            uint32_t s1 = 0, s0 = 0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const uint32_t n4 = qw[t] & 0x0F0F0F0Fu;
                s2 = dp4a_ss(n4, L2[t], s2);
                s1 = dp4a_uu(n4, L1[t], s1);
                s0 = dp4a_uu(n4, L0[t], s0);
            }
            S_lo[r] = (float)(s2 * 65536 + (int)(s1 * 256u + s0));  // |.| < 2^31, exact
        }
    }
    {   // high nibbles: sub-block 2g+1, taken in place as 16*q (no shift)
        uint32_t L2[8], L1[8], L0[8];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 a = rec[6 + i], b = rec[8 + i], c = rec[10 + i];
            L2[4 * i] = a.x; L2[4 * i + 1] = a.y; L2[4 * i + 2] = a.z; L2[4 * i + 3] = a.w;
            L1[4 * i] = b.x; L1[4 * i + 1] = b.y; L1[4 * i + 2] = b.z; L1[4 * i + 3] = b.w;
            L0[4 * i] = c.x; L0[4 * i + 1] = c.y; L0[4 * i + 2] = c.z; L0[4 * i + 3] = c.w;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const uint32_t qw[8] = {wd.q0[r].x, wd.q0[r].y, wd.q0[r].z, wd.q0[r].w,
                                    wd.q1[r].x, wd.q1[r].y, wd.q1[r].z, wd.q1[r].w};
            int s2 = 0;
            uint32_t s1 = 0, s0 = 0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const uint32_t n4 = qw[t] & 0xF0F0F0F0u;
                s2 = dp4a_us(n4, L2[t], s2);
                s1 = dp4a_uu(n4, L1[t], s1);
                s0 = dp4a_uu(n4, L0[t], s0);
            }
            // |s2| <= 240*64*32, s1*256+s0 < 2^29: exact in int32, combined in f32
            S_hi[r] = fmaf((float)s2, 65536.0f, (float)(s1 * 256u + s0));
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float2 dd = __half22float2(*reinterpret_cast<const __half2*>(&wd.hdr[r].x));
        const float d = fabsf(dd.x) <= 65504.0f ? dd.x : 0.0f;      // inf / NaN -> 0
        const float dmin = fabsf(dd.y) <= 65504.0f ? dd.y : 0.0f;
        const q4k::ScaleMin sm = q4k::unpack_scales(wd.hdr[r].y, wd.hdr[r].z, wd.hdr[r].w);
        const uint32_t scw = g < 2 ? sm.sc_lo : sm.sc_hi;
        const uint32_t mw = g < 2 ? sm.m_lo : sm.m_hi;
        const float sc_a = (float)__byte_perm(scw, 0, sel_sc);
        const float sc_b = (float)__byte_perm(scw, 0, sel_sc + 1);
        const float m_a = (float)__byte_perm(mw, 0, sel_sc);
        const float m_b = (float)__byte_perm(mw, 0, sel_sc + 1);
        const float t1 = fmaf(sc_a, S_lo[r] * s_lo, sc_b * (S_hi[r] * s_hi));
        const float t2 = fmaf(m_a, x_lo, m_b * x_hi);
        acc[r] = fmaf(d, t1, acc[r]);
        acc[r] = fmaf(-dmin, t2, acc[r]);
    }
}

// Fills the CTA's shared-memory record table: from the f32 activation vector (FROM_X = 1,
// optional RMSNorm in front; bpr <= 32 so four chunks per thread cover the vector in one pass)
// or by copying records made by x_to_limbs_kernel (FROM_X = 0).  Ends with __syncthreads().
template <int FROM_X, bool COHERENT, int PEER>
__device__ __forceinline__ void stage_records(const MatList& ml, const void* src, int x_aligned, int bpr,
                                              uint4* rec_s) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (FROM_X) {
        // bpr <= 32 on this path, so four chunks per thread cover the whole vector in one pass.
        const float* x = static_cast<const float*>(src);
        uint32_t* rec_w = reinterpret_cast<uint32_t*>(rec_s);
        const int n_chunks = bpr * 64;  // multiple of 64: whole warps stay in or out of range
        constexpr int kU = 4;
        float v[kU][4];
        if (PEER == kPeerStamped && ml.xin.slots != nullptr) {
            // the thread's sixteen activations out of a stamped vector, polled together
            long long idx[kU * 4];
            unsigned bits[kU * 4], live = 0u;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int c = threadIdx.x + u * kGemvThreads;
#pragma unroll
                for (int i = 0; i < 4; ++i) idx[u * 4 + i] = (long long)c * 4 + i;
                if (c < n_chunks) live |= 0xFu << (4 * u);
            }
            mgpeer::ld_stamped_n<kU * 4>(ml.xin, idx, live, mgpeer::exchange_epoch(ml.xin.epoch_dev, ml.xin.epoch_mul, ml.xin.epoch_add), bits);
#pragma unroll
            for (int u = 0; u < kU; ++u)
#pragma unroll
                for (int i = 0; i < 4; ++i) v[u][i] = __uint_as_float(bits[u * 4 + i]);
        } else {
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int c = threadIdx.x + u * kGemvThreads;
                if (c < n_chunks) load_chunk<COHERENT>(v[u], x, c, x_aligned);
            }
        }
        if (ml.norm_w != nullptr) {
            // RMSNorm in front of the matvec (crates/modgrad-device/src/kfd/llm.rs:921-928, Plain)
            __shared__ float red[kGemvWarps + 1];
            // the norm weights are requested before the reduction's barriers, so that their trip to L2
            // overlaps it instead of following it
            float wv[kU][4];
            const bool w_aligned = (reinterpret_cast<uintptr_t>(ml.norm_w) & 15u) == 0;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int c = threadIdx.x + u * kGemvThreads;
                if (c < n_chunks) load_chunk<false>(wv[u], ml.norm_w, c, w_aligned);
            }
            float p = 0.0f;
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                if (threadIdx.x + u * kGemvThreads < n_chunks) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) p = fmaf(v[u][i], v[u][i], p);
                }
            }
            p = q4k::warp_sum(p);
            if (lane == 0) red[warp] = p;
            __syncthreads();
            if (warp == 0) {
                float t = lane < kGemvWarps ? red[lane] : 0.0f;
                t = q4k::warp_sum(t);
                if (lane == 0) red[kGemvWarps] = t;
            }
            __syncthreads();
            const float inv = 1.0f / sqrtf(red[kGemvWarps] / (float)(bpr * 256) + ml.eps);
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int c = threadIdx.x + u * kGemvThreads;
                if (c < n_chunks) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[u][i] = v[u][i] * inv * wv[u][i];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kU; ++u) {
            const int c = threadIdx.x + u * kGemvThreads;
            if (c < n_chunks) convert_chunk(v[u], c, rec_w);
        }
    } else {
        const uint4* rec_g = static_cast<const uint4*>(src);
        const int n_vec = bpr * 4 * xlimbs::kRecordVec4;
        if (PEER == kPeerStamped && ml.xin.slots != nullptr) {  // stamped records: one slot per record word
            const unsigned epoch = mgpeer::exchange_epoch(ml.xin.epoch_dev, ml.xin.epoch_mul, ml.xin.epoch_add);
            for (int base = threadIdx.x; base < n_vec; base += 4 * kGemvThreads) {  // four record vectors per round
                long long idx[16];
                unsigned bits[16], live = 0u;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base + j * kGemvThreads;
#pragma unroll
                    for (int k = 0; k < 4; ++k) idx[j * 4 + k] = (long long)i * 4 + k;
                    if (i < n_vec) live |= 0xFu << (4 * j);
                }
                mgpeer::ld_stamped_n<16>(ml.xin, idx, live, epoch, bits);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = base + j * kGemvThreads;
                    if (i < n_vec) rec_s[i] = make_uint4(bits[j * 4], bits[j * 4 + 1], bits[j * 4 + 2], bits[j * 4 + 3]);
                }
            }
        } else {
            for (int i = threadIdx.x; i < n_vec; i += kGemvThreads) cp_async16(&rec_s[i], &rec_g[i]);
            cp_async_wait_all();
        }
    }
    __syncthreads();
}

// FROM_X = 1: `src` is the f32 activation vector and every CTA converts it into its
// shared-memory record table itself (one kernel per matvec); FROM_X = 0: `src` is a record
// table in global memory made by x_to_limbs_kernel (several matvecs share one conversion).
// COHERENT = true: x / records / addend were written earlier in the SAME kernel by other CTAs
// (persistent decode kernel): they are read with L2-level loads.  PDL = true: stand-alone
// kernel chained with programmatic dependent launch.  block_id / n_blocks replace blockIdx /
// gridDim so that a persistent kernel can run the body as one of its phases.
template <int R, int FROM_X, bool COHERENT, bool PDL, int PEER>
__device__ __forceinline__ void gemv_body(const MatList& ml, const void* src, int x_aligned, int bpr,
                                          int block_id, int n_blocks) {
    extern __shared__ __align__(16) uint4 rec_s[];  // the kernel's dynamic shared memory
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bl = lane >> 2;  // super-block inside the 8-block window
    const int g = lane & 3;    // 32-byte group inside the super-block
    const size_t row_bytes = (size_t)bpr * q4k::kBlockBytes;
    const int n_slots = n_blocks * kGemvWarps;
    const int n_win = (bpr + 7) >> 3;
    const int n_groups = total_groups<R>(ml);
    const int first = warp * n_blocks + block_id;  // warp-major: a short matrix still spreads over all CTAs
    const int my_groups = first < n_groups ? (n_groups - first + n_slots - 1) / n_slots : 0;
    const uint32_t sel_sc = 0x4440u + (uint32_t)((g & 1) * 2);  // byte (g&1)*2 of the word, zero-extended
    const size_t lane_off = (size_t)bl * q4k::kBlockBytes;

    // Let the next kernel in the stream be scheduled as soon as CTAs of this one retire.
    if (PDL && !ml.hold_trigger) griddep_launch_dependents();
    // Weights do not depend on the kernel before this one: issue the first window's loads
    // before waiting for x, so the weight stream starts while x is converted.
    const int total = my_groups * n_win;  // flattened (group, window) steps of this warp
    Window<R> wa;
    int mat = 0, row0 = 0;
    if (total > 0) {
        locate_group<R>(ml, first, mat, row0);
        if (bl < bpr) load_window<R>(wa, mat_w(ml, mat) + lane_off, row_bytes, row0, mat_rows(ml, mat), 0, g);
    }

    if (PDL) griddep_wait();  // x / the records may be produced by the kernel launched just before this one
    stage_records<FROM_X, COHERENT, PEER>(ml, src, x_aligned, bpr, rec_s);

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    int gi = 0, win = 0;  // position of the window held in `wa`
    for (int t = 0; t < total; ++t) {
        if (win * 8 + bl < bpr)
            compute_window<R>(wa, rec_s + ((win * 8 + bl) * 4 + g) * xlimbs::kRecordVec4, g, sel_sc, acc);
        if (win == n_win - 1) {
            const int rows = mat_rows(ml, mat);
            float* y = mat == 0 ? ml.y[0] : (mat == 1 ? ml.y[1] : ml.y[2]);
            const float* add = mat == 0 ? ml.addend[0] : (mat == 1 ? ml.addend[1] : ml.addend[2]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float s = q4k::warp_sum(acc[r]);
                if (lane == 0 && row0 + r < rows) {
                    const float v = add ? s + ld_f32<COHERENT>(add + row0 + r) : s;
                    if (PEER == kPeerStamped && ml.peer.world > 1 && ml.peer.stamp_slots != nullptr) {
                        y[row0 + r] = v;
                        mgpeer::store_stamped_all(ml.peer, row0 + r, __float_as_uint(v),
                                                  mgpeer::exchange_epoch(ml.peer.epoch_dev, ml.peer.epoch_mul, ml.peer.epoch_add));
                    } else if (PEER == kPeerFused && ml.peer.world > 1) mgpeer::store_all(ml.peer, y + row0 + r, v);
                    else y[row0 + r] = v;
                }
                acc[r] = 0.0f;
            }
        }
        if (++win == n_win) {
            win = 0;
            ++gi;
            if (gi < my_groups) locate_group<R>(ml, first + gi * n_slots, mat, row0);
        }
        if (t + 1 < total && win * 8 + bl < bpr)
            load_window<R>(wa, mat_w(ml, mat) + lane_off, row_bytes, row0, mat_rows(ml, mat), win, g);
    }
    if (!COHERENT) mgpeer::peer_finish(ml.peer);
}

// ---------------------------------------------------------------------------------------------
// Ring variant: the weight stream is staged in shared memory by bulk asynchronous copies.
//
// With register loads the bytes in flight are limited by the register file (a warp can hold one
// window per row), and the stream only starts once every warp has run its prologue.  Here each
// warp owns `depth` stages of R rows x one 8-block window; its lanes fill them with
// cp.async.bulk copies (one per row) that complete on the stage's mbarrier, the warp reads a
// full stage into registers, hands the stage straight back to the copy engine for the unit
// `depth` steps ahead and only then does the arithmetic.  All of a CTA's first copies are issued
// before the kernel waits for its predecessor, so the stream is already running while x is
// converted.
// ---------------------------------------------------------------------------------------------
constexpr int kRingMaxDepth = 4;
constexpr uint32_t kRingSpinLimit = 1u << 22;  // polls of one stage before the warp gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// global -> this CTA's shared memory, completion counted in bytes on `bar`; both addresses and
// the size are multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Position of a warp in its sequence of units (row group x window).
struct UnitCursor {
    int gi, win;    // group index within the warp's groups, window within the row
    int mat, row0;  // matrix and first row of group gi
};

// Bytes of the record table inside the dynamic shared memory (padded to 128).
__host__ __device__ inline int ring_record_bytes(int bpr) { return (bpr * 4 * xlimbs::kRecordBytes + 127) & ~127; }
// Bytes of one stage: `rows` rows of min(bpr, 8) super-blocks.
__host__ __device__ inline int ring_stage_bytes(int bpr, int rows) {
    return rows * (bpr < 8 ? bpr : 8) * q4k::kBlockBytes;
}

template <int R>
__device__ __forceinline__ void load_window_smem(Window<R>& wd, const uint8_t* stage, int row_stride, int bl, int g) {
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const uint8_t* p = stage + r * row_stride + bl * q4k::kBlockBytes;
        wd.hdr[r] = *reinterpret_cast<const uint4*>(p);
        wd.q0[r] = *reinterpret_cast<const uint4*>(p + 16 + g * 32);
        wd.q1[r] = *reinterpret_cast<const uint4*>(p + 32 + g * 32);
    }
}

// Dynamic shared memory: the record table, then kGemvWarps * depth stages.  `timeouts` counts
// warps that gave up waiting for a stage (their rows are then left unwritten).
template <int R, int FROM_X, int PEER>
__device__ __forceinline__ void gemv_ring_body(const MatList& ml, const void* src, int x_aligned, int bpr,
                                               int depth, unsigned* timeouts) {
    extern __shared__ __align__(16) uint4 rec_s[];
    __shared__ __align__(8) uint64_t full_bar[kGemvWarps * kRingMaxDepth];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bl = lane >> 2, g = lane & 3;
    const int n_win = (bpr + 7) >> 3;
    const int row_stride = min(bpr, 8) * q4k::kBlockBytes;
    const int stage_bytes = R * row_stride;
    const size_t row_bytes = (size_t)bpr * q4k::kBlockBytes;
    uint8_t* ring = reinterpret_cast<uint8_t*>(rec_s) + ring_record_bytes(bpr) + (size_t)warp * depth * stage_bytes;
    uint64_t* bars = full_bar + warp * kRingMaxDepth;
    const int n_slots = (int)gridDim.x * kGemvWarps;
    const int n_groups = total_groups<R>(ml);
    const int first = warp * (int)gridDim.x + (int)blockIdx.x;  // warp-major: a short matrix still spreads over all CTAs
    const int my_groups = first < n_groups ? (n_groups - first + n_slots - 1) / n_slots : 0;
    const int total = my_groups * n_win;
    const uint32_t sel_sc = 0x4440u + (uint32_t)((g & 1) * 2);

    if (!ml.hold_trigger) griddep_launch_dependents();

    // Fills stage `st` with the unit at cursor `c`; all lanes call it, lanes 0..R-1 copy.
    auto issue = [&](const UnitCursor& c, int st) {
        const int valid = min(R, mat_rows(ml, c.mat) - c.row0);
        const int nb = min(8, bpr - c.win * 8);
        const uint8_t* base = mat_w(ml, c.mat) + (size_t)c.row0 * row_bytes + (size_t)c.win * kWindowBytes;
        uint8_t* dst = ring + st * stage_bytes;
        if (n_win == 1) {  // whole rows, contiguous in memory: one copy
            if (lane == 0) {
                mbar_arrive_expect_tx(bars + st, (uint32_t)(valid * row_stride));
                bulk_copy_g2s(dst, base, (uint32_t)(valid * row_stride), bars + st);
            }
        } else {
            if (lane == 0) mbar_arrive_expect_tx(bars + st, (uint32_t)(valid * nb * q4k::kBlockBytes));
            __syncwarp();
            if (lane < valid)
                bulk_copy_g2s(dst + lane * row_stride, base + (size_t)lane * row_bytes,
                              (uint32_t)(nb * q4k::kBlockBytes), bars + st);
        }
    };
    auto advance = [&](UnitCursor& c) {
        if (++c.win == n_win) {
            c.win = 0;
            ++c.gi;
            if (c.gi < my_groups) locate_group<R>(ml, first + c.gi * n_slots, c.mat, c.row0);
        }
    };

    UnitCursor prod = {0, 0, 0, 0}, cons = {0, 0, 0, 0};
    if (lane == 0) {
        for (int d = 0; d < depth; ++d) mbar_init(bars + d, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (total > 0) {
        locate_group<R>(ml, first, prod.mat, prod.row0);
        cons = prod;
    }
    int issued = 0;
    for (; (issued < depth) && (issued < total); ++issued) {  // weights do not depend on the previous kernel
        issue(prod, issued);
        advance(prod);
    }

    griddep_wait();  // x / the records may be produced by the kernel launched just before this one
    stage_records<FROM_X, false, PEER>(ml, src, x_aligned, bpr, rec_s);

    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;

    int st = 0;
    uint32_t parity = 0;
    for (int t = 0; t < total; ++t) {
        uint32_t spins = 0;
        bool arrived = true;
        while (!mbar_try_wait(bars + st, parity)) {
            if (++spins > kRingSpinLimit) {  // never expected: give up instead of hanging the GPU
                arrived = false;
                break;
            }
        }
        if (!arrived) {
            if (lane == 0) atomicAdd(timeouts, 1u);
            break;
        }
        const bool active = cons.win * 8 + bl < bpr;
        Window<R> wd;
        if (active) load_window_smem<R>(wd, ring + st * stage_bytes, row_stride, bl, g);
        __syncwarp();  // every lane has read the stage: refill it
        if (issued < total) {
            issue(prod, st);
            advance(prod);
            ++issued;
        }
        if (active)
            compute_window<R>(wd, rec_s + ((cons.win * 8 + bl) * 4 + g) * xlimbs::kRecordVec4, g, sel_sc, acc);
        if (cons.win == n_win - 1) {
            const int rows = mat_rows(ml, cons.mat);
            float* y = cons.mat == 0 ? ml.y[0] : (cons.mat == 1 ? ml.y[1] : ml.y[2]);
            const float* add = cons.mat == 0 ? ml.addend[0] : (cons.mat == 1 ? ml.addend[1] : ml.addend[2]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float s = q4k::warp_sum(acc[r]);
                if (lane == 0 && cons.row0 + r < rows) {
                    const float v = add ? s + add[cons.row0 + r] : s;
                    if (PEER == kPeerStamped && ml.peer.world > 1 && ml.peer.stamp_slots != nullptr) {
                        y[cons.row0 + r] = v;
                        mgpeer::store_stamped_all(ml.peer, cons.row0 + r, __float_as_uint(v),
                                                  mgpeer::exchange_epoch(ml.peer.epoch_dev, ml.peer.epoch_mul, ml.peer.epoch_add));
                    } else if (PEER == kPeerFused && ml.peer.world > 1) mgpeer::store_all(ml.peer, y + cons.row0 + r, v);
                    else y[cons.row0 + r] = v;
                }
                acc[r] = 0.0f;
            }
        }
        advance(cons);
        if (++st == depth) {
            st = 0;
            parity ^= 1u;
        }
    }
    if (PEER == kPeerFused) mgpeer::peer_finish(ml.peer);
}

}  // namespace gemvdev
