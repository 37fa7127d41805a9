// Resident Q4_K decoder engine: the CUDA counterpart of the reference's resident decode loop
//   RocmGemma::{load, qmatvec, layer, forward_token, generate}
//   (crates/modgrad-gemma/src/rocm_gemma.rs:94, :291, :429, :312, :372)
// computing the arithmetic of the reference's CPU decoder
//   kfd::llm::forward_token (crates/modgrad-device/src/kfd/llm.rs:1177-1298)
// for the 7B-class configuration: plain RMSNorm, NEOX RoPE, grouped-query attention over a
// half-precision KV cache, SwiGLU, dense half embedding and LM head, greedy arg-max.
//
// Like RocmGemma every weight lives in device memory, the activation never leaves it, all
// kernels of a token are queued without synchronising and the host synchronises once per
// token (forward_token) or once per generate() call.  One token is captured once as a CUDA
// graph; position, sequence length and the fed-back token are device-side integers, so the
// same graph is replayed for every step.
//
// Row sharding (world > 1, one process per GPU): rank r holds the rows of every projection
// that belong to its query heads / its slice of the FFN / of the hidden state / of the
// vocabulary (the unmodified row-major block arrays cut at row boundaries, nothing repacked).
// Attention is head-parallel, so q/k/v and the attention itself need no exchange; four
// all-gathers per layer remain (attention output, o_proj output, the SwiGLU activation in
// limb-record form, down_proj output) plus one of (value, index) pairs for the arg-max.
// They are NCCL calls captured in the same per-token graph.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../launch_common.cuh"
#include "../peer_gather.hpp"
#include "modgrad_cuda.h"
#include "nccl_dl.hpp"

namespace {

struct Layer {
    uint8_t *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr, *wgate = nullptr, *wup = nullptr,
            *wdown = nullptr;
    float *attn_norm = nullptr, *ffn_norm = nullptr;
    __half *k_cache = nullptr, *v_cache = nullptr;
    // GGUF tensor types of wq, wk, wv, wo, wgate, wup, wdown (12 Q4_K, 13 Q5_K, 14 Q6_K)
    uint8_t type[7] = {12, 12, 12, 12, 12, 12, 12};
};

constexpr int kTypeF16 = 1, kTypeQ4K = 12, kTypeQ5K = 13, kTypeQ6K = 14;
// Bytes of a [rows][cols] tensor of GGUF type `type` (cols a multiple of 256 for the K-quants);
// 0 for a type the engine does not run.
size_t typed_bytes(int type, size_t rows, size_t cols) {
    switch (type) {
        case kTypeF16: return rows * cols * 2;
        case kTypeQ4K: return rows * (cols / 256) * 144;
        case kTypeQ5K: return rows * (cols / 256) * 176;
        case kTypeQ6K: return rows * (cols / 256) * 210;
        default: return 0;
    }
}

}  // namespace

struct mg_decoder {
    mg_decoder_config cfg{};
    std::vector<Layer> layers;
    uint8_t* weights = nullptr;  // the one allocation that holds every weight tensor
    size_t weights_bytes = 0;
    __half *embed = nullptr, *lm_head = nullptr;  // raw bytes of embed_type / head_type (half by default)
    int embed_type = 1, head_type = 1;            // GGUF type ids (1 = F16)
    // Some tensor is not of the default type (a Q5_K / Q6_K projection, a quantised embedding or head):
    // the token is then queued one projection per launch through the launchers of each type.
    bool mixed = false;
    int mixed_launches = 0;  // kernels the last queued token of that path launched
    float* out_norm = nullptr;
    float* rope_freq = nullptr;  // base^(-2i/head_dim), i < head_dim/2
    // activations
    float *hidden = nullptr, *cur = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *gate = nullptr,
          *up = nullptr, *logits = nullptr;
    void *records = nullptr, *attn_scratch = nullptr, *argmax_scratch = nullptr;
    int* state = nullptr;    // [0] position, [1] sequence length (position + 1), [2] step, [3] token,
                             // [4] tokens decoded since creation (never reset: the epoch of the stamped exchanges)
    int* history = nullptr;  // generated tokens
    int history_cap = 0;
    int n_splits = 1;
    cudaStream_t stream = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t graph_exec = nullptr;
    std::vector<void*> allocs;
    std::string last_error;
    int pos_host = 0;
    // ---- row sharding -------------------------------------------------------------------
    int rank = 0, world = 1;
    int h0 = 0, h1 = 0, kv0 = 0, kv1 = 0;  // this rank's query heads [h0,h1) and KV heads [kv0,kv1)
    int d_loc = 0, f_loc = 0, v_loc = 0;    // rows of the hidden state / FFN / vocabulary held here
    std::vector<int> head_lo;               // first query head of every rank (world + 1 entries)
    mgnccl::Comm comm = nullptr;
    float* att_full = nullptr;   // gathered attention output [q_dim]
    float* tmp_full = nullptr;   // gathered projection output [d_model]
    float* tmp_down = nullptr;   // the same for the down projection (consecutive gathers use different buffers)
    float* pair_buf = nullptr;   // arg-max (value, index) pairs [2 * world]
    // Gathers by direct peer stores (peer_gather.hpp) instead of NCCL: the gathered buffers then
    // live in one arena that the other ranks' processes map with CUDA IPC.
    bool peer = false;   // gathers by peer stores (else NCCL)
    bool fused = false;  // ... done by the producing kernels themselves instead of a gather kernel
    bool stamped = false;  // ... as stamped words (flag in data): no fence, no handshake, the consumer polls
    unsigned long long *s_att = nullptr, *s_out = nullptr, *s_down = nullptr, *s_rec = nullptr;  // stamped vectors
    mgpeer::Exchange px;
    unsigned char* arena = nullptr;
    size_t arena_bytes = 0;
    std::vector<void*> ipc_opened;
};

namespace {

__global__ void advance_state_kernel(int* state) {
    mg::pdl_prologue();
    state[0] += 1;
    state[1] += 1;
    state[2] += 1;
    state[4] += 1;
}

int fail(mg_decoder* d, int code, const char* what) {
    if (d) d->last_error = std::string(what) + ": " + cudaGetErrorString((cudaError_t)code);
    return code;
}

template <class T>
int dev_alloc(mg_decoder* d, T** out, size_t count) {
    void* p = nullptr;
    const size_t bytes = count * sizeof(T);
    cudaError_t e = cudaMalloc(&p, bytes != 0 ? bytes : 16);
    if (e != cudaSuccess) return fail(d, (int)e, "cudaMalloc");
    d->allocs.push_back(p);
    *out = static_cast<T*>(p);
    return 0;
}

// hidden += x (the residual add after a gathered projection output)
__global__ void residual_add_kernel(float* h, const float* x, int n) {
    mg::pdl_prologue();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] += x[i];
}
// Global arg-max from per-rank (value, vocabulary index) pairs; first maximum wins.
__global__ void argmax_pairs_kernel(const float* pairs, int world, int* tok,
                                    int* history, const int* step) {
    mg::pdl_prologue();
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int r = 0; r < world; ++r) {
        const float v = pairs[2 * r];
        const int i = __float_as_int(pairs[2 * r + 1]);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
    if (bi == 0x7FFFFFFF) bi = 0;
    *tok = bi;
    if (history) history[*step] = bi;
}
// (best value, best global index) of this rank's logits slice -> pairs[2*rank..]
__global__ void local_pair_kernel(const float* logits, const int* local_tok, int offset,
                                  float* pair, const mgpeer::PeerSync peer) {
    // no early trigger: an NCCL all-gather that follows may start on it and send a stale pair
    mg::pdl_prologue(1);
    const int i = *local_tok;
    if (peer.world > 1) {  // the pair goes to every rank from here
        mgpeer::store_all(peer, pair, logits[i]);
        mgpeer::store_all(peer, pair + 1, __int_as_float(i + offset));
    } else {
        pair[0] = logits[i];
        pair[1] = __int_as_float(i + offset);
    }
    mgpeer::peer_finish(peer);
}

// RMSNorm (crates/modgrad-device/src/kfd/llm.rs:921-928, Plain) of a stamped vector: the final norm
// reads the hidden state straight out of the last down-projection's exchange.
__global__ void __launch_bounds__(1024) rms_norm_stamped_kernel(const mgpeer::StampIn in, const float* weight, float* y,
                                                                 int n, float eps) {
    mg::pdl_prologue();
    __shared__ float red[33];
    const unsigned epoch = mgpeer::exchange_epoch(in.epoch_dev, in.epoch_mul, in.epoch_add);
    float v[8], p = 0.0f;  // n <= 8192
    {
        long long idx[8];
        unsigned bits[8], live = 0u;
        for (int k = 0; k < 8; ++k) {
            idx[k] = threadIdx.x + k * 1024;
            if (idx[k] < n) live |= 1u << k;
        }
        mgpeer::ld_stamped_n<8>(in, idx, live, epoch, bits);
        for (int k = 0; k < 8; ++k) {
            v[k] = ((live >> k) & 1u) ? __uint_as_float(bits[k]) : 0.0f;
            p = fmaf(v[k], v[k], p);
        }
    }
    for (int o = 16; o > 0; o >>= 1) p += __shfl_xor_sync(0xFFFFFFFFu, p, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = p;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = red[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    const float inv = 1.0f / sqrtf(red[32] / (float)n + eps);
    for (int k = 0; k < 8; ++k) {
        const int i = threadIdx.x + k * 1024;
        if (i < n) y[i] = v[k] * inv * weight[i];
    }
}

int nccl_fail(mg_decoder* d, int code, const char* what) {
    d->last_error = std::string(what) + ": " + (mgnccl::api().GetErrorString ? mgnccl::api().GetErrorString(code) : "nccl");
    return (int)cudaErrorUnknown;
}

enum GatherSite { kSiteHeads = 0, kSiteOut = 1, kSiteRecords = 2, kSiteDown = 3, kSitePairs = 4 };

// All-gather of equal slices, in place: every rank's slice already sits at rank*count.
int gather_equal(mg_decoder* d, int site, void* buf, size_t count, int dtype, size_t elem) {
    if (d->world == 1) return 0;
    if (d->peer) {
        const size_t off = (size_t)(static_cast<unsigned char*>(buf) - d->arena);
        cudaError_t e = mgpeer::launch_gather(d->px, site, off, (size_t)d->rank * count * elem, count * elem, d->stream);
        return e == cudaSuccess ? 0 : fail(d, (int)e, "peer gather");
    }
    const mgnccl::Api& n = mgnccl::api();
    int rc = n.AllGather(static_cast<char*>(buf) + (size_t)d->rank * count * elem, buf, count, dtype, d->comm, d->stream);
    return rc ? nccl_fail(d, rc, "ncclAllGather") : 0;
}
// All-gather of the attention output, whose slices follow the (possibly uneven) head split.
int gather_heads(mg_decoder* d) {
    if (d->world == 1) return 0;
    if (d->peer) {
        const size_t off = (size_t)(reinterpret_cast<unsigned char*>(d->att_full) - d->arena);
        const size_t hb = (size_t)d->cfg.head_dim * sizeof(float);
        cudaError_t e = mgpeer::launch_gather(d->px, kSiteHeads, off, d->head_lo[d->rank] * hb,
                                              (d->head_lo[d->rank + 1] - d->head_lo[d->rank]) * hb, d->stream);
        return e == cudaSuccess ? 0 : fail(d, (int)e, "peer gather");
    }
    const mgnccl::Api& n = mgnccl::api();
    const int hd = d->cfg.head_dim;
    int rc = n.GroupStart();
    if (rc) return nccl_fail(d, rc, "ncclGroupStart");
    for (int r = 0; r < d->world && !rc; ++r) {
        float* p = d->att_full + (size_t)d->head_lo[r] * hd;
        rc = n.Broadcast(p, p, (size_t)(d->head_lo[r + 1] - d->head_lo[r]) * hd, mgnccl::kFloat32, r, d->comm, d->stream);
    }
    int rc2 = n.GroupEnd();
    if (rc) return nccl_fail(d, rc, "ncclBroadcast");
    return rc2 ? nccl_fail(d, rc2, "ncclGroupEnd") : 0;
}

int queue_token_impl(mg_decoder* d);
int queue_token_mixed(mg_decoder* d);

// Stamped exchanges: the epoch of exchange `site` of layer `layer` in the current token is
// tokens_decoded * (4 * n_layers + 4) + 4 * layer + site + 1: unique, increasing, never 0 (a zeroed
// arena holds epoch 0), computed by producer and consumer from the same device counter.
mgpeer::PeerSync stamp_out(mg_decoder* d, int site, unsigned long long* slots, long long index0, int layer) {
    mgpeer::PeerSync ps = mgpeer::make_sync(d->px, site);
    ps.stamp_slots = slots;
    ps.epoch_dev = d->state + 4;
    ps.epoch_mul = 4 * d->cfg.n_layers + 4;
    ps.epoch_add = 4 * layer + site + 1;
    ps.stamp_index0 = index0;
    return ps;
}
mgpeer::StampIn stamp_in(mg_decoder* d, int site, const unsigned long long* slots, int layer) {
    mgpeer::StampIn in;
    in.slots = slots;
    in.epoch_dev = d->state + 4;
    in.epoch_mul = 4 * d->cfg.n_layers + 4;
    in.epoch_add = 4 * layer + site + 1;
    in.err = d->px.ctl + 2 * mgpeer::kMaxSites;
    in.site = site;
    in.spin_limit = d->px.spin_limit;
    return in;
}

// One token: embedding of state[3] -> logits -> arg-max into state[3].  Everything is queued
// on d->stream; nothing synchronises.  The sharded engine chains NCCL collectives behind its
// kernels, which may start as soon as their predecessor lets its successor launch: there the
// kernels that feed a collective keep their trigger until they have finished.
int queue_token(mg_decoder* d) {
    int (*impl)(mg_decoder*) = d->mixed ? queue_token_mixed : queue_token_impl;
    if (d->world == 1 || d->peer) return impl(d);  // the peer-store gathers are our own kernels
    const int before = mg_pdl_early_trigger(0);
    const int rc = impl(d);
    mg_pdl_early_trigger(before);
    return rc;
}

int queue_token_impl(mg_decoder* d) {
    const mg_decoder_config& c = d->cfg;
    void* s = d->stream;
    const int D = c.d_model, hd = c.head_dim, F = c.d_ff;
    const int q_dim = c.n_heads * hd;
    const int Hl = d->h1 - d->h0, KVl = d->kv1 - d->kv0;
    const int q_loc = Hl * hd, kv_loc = KVl * hd;
    const bool sharded = d->world > 1;
    const float scale = 1.0f / sqrtf((float)hd);
    int e;
    int* pos_dev = d->state;
    int* step_dev = d->state + 2;
    int* tok_dev = d->state + 3;

    if ((e = mg_embed_f16_on_stream(d->embed, 0, tok_dev, d->hidden, D, c.vocab, s))) return fail(d, e, "embed");
    for (int l = 0; l < c.n_layers; ++l) {
        const Layer& L = d->layers[l];
        {   // q, k, v share the normalised hidden state: one launch, RMSNorm fused in front
            const uint8_t* w[3] = {L.wq, L.wk, L.wv};
            float* y[3] = {d->q, d->k, d->v};
            const int rows[3] = {q_loc, kv_loc, kv_loc};
            // stamped: the hidden state is read out of the previous layer's down-projection exchange
            if (d->stamped && l > 0) mgpeer::set_next_stamp_in(stamp_in(d, kSiteDown, d->s_down, l - 1));
            if ((e = mg_rmsnorm_matvec_q4k_multi_on_stream(3, w, d->hidden, L.attn_norm, c.rms_eps, nullptr, y, rows,
                                                           D / 256, s)))
                return fail(d, e, "qkv");
        }
        // RoPE, cache append, attention and the merge of its splits in one launch.  This rank's heads land
        // at their place in the full attention vector (and, fused, in every peer's: the kernel ends with
        // the exchange).
        if (d->stamped) mgpeer::set_next_peer_sync(stamp_out(d, kSiteHeads, d->s_att, (long long)d->h0 * hd, l));
        else if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteHeads));
        if ((e = mg_sdpa_rope_decode_f16kv_on_stream(d->q, d->k, d->v, L.k_cache, L.v_cache, d->att_full + (size_t)d->h0 * hd,
                                                     Hl, KVl, hd, 0, pos_dev, scale, c.rope_base, d->rope_freq,
                                                     d->attn_scratch, d->n_splits, s)))
            return fail(d, e, "attention");
        if (!d->fused && (e = gather_heads(d))) return e;
        {   // hidden += Wo . att.  One GPU: in place.  Fused: this rank's rows are added in place and
            // stored into every rank's hidden state by the matvec itself.  Otherwise the rows are
            // gathered into a scratch vector and added by a separate kernel.
            const bool in_place = !sharded || d->fused;
            float* mine = d->hidden + (sharded ? (size_t)d->rank * d->d_loc : 0);
            const uint8_t* w[1] = {L.wo};
            float* y[1] = {in_place ? mine : d->tmp_full + (size_t)d->rank * d->d_loc};
            const float* add[1] = {in_place ? mine : nullptr};
            const int rows[1] = {d->d_loc};
            if (d->stamped) {
                mgpeer::set_next_stamp_in(stamp_in(d, kSiteHeads, d->s_att, l));
                mgpeer::set_next_peer_sync(stamp_out(d, kSiteOut, d->s_out, (long long)d->rank * d->d_loc, l));
            } else if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteOut));
            if ((e = mg_matvec_q4k_multi_on_stream(1, w, d->att_full, 0, add, y, rows, q_dim / 256, s))) return fail(d, e, "o_proj");
        }
        if (sharded && !d->fused) {
            if ((e = gather_equal(d, kSiteOut, d->tmp_full, (size_t)d->d_loc, mgnccl::kFloat32, 4))) return e;
            mg::launch_pdl(residual_add_kernel, dim3((D + 255) / 256), dim3(256), 0, d->stream, d->hidden, (const float*)d->tmp_full, D);
        }
        {   // gate and up share their input: one launch, RMSNorm fused in front
            const uint8_t* w[2] = {L.wgate, L.wup};
            float* y[2] = {d->gate, d->up};
            const int rows[2] = {d->f_loc, d->f_loc};
            if (d->stamped) mgpeer::set_next_stamp_in(stamp_in(d, kSiteOut, d->s_out, l));
            if ((e = mg_rmsnorm_matvec_q4k_multi_on_stream(2, w, d->hidden, L.ffn_norm, c.rms_eps, nullptr, y, rows,
                                                           D / 256, s)))
                return fail(d, e, "gate_up");
        }
        {   // SwiGLU straight into limb records; a rank's slice is a whole number of records
            uint8_t* rec = static_cast<uint8_t*>(d->records) + mg_q4k_limb_record_bytes(d->f_loc) * d->rank;
            if (d->stamped)
                mgpeer::set_next_peer_sync(stamp_out(d, kSiteRecords, d->s_rec, (long long)d->rank * (d->f_loc / 64) * 52, l));
            else if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteRecords));
            if ((e = mg_swiglu_limbs_on_stream(d->gate, d->up, nullptr, d->f_loc, rec, s))) return fail(d, e, "swiglu");
            if (!d->fused &&
                (e = gather_equal(d, kSiteRecords, d->records, mg_q4k_limb_record_bytes(d->f_loc), mgnccl::kUint8, 1)))
                return e;
        }
        {   // hidden += Wdown . act
            const uint8_t* w[1] = {L.wdown};
            const bool in_place = !sharded || d->fused;
            float* mine = d->hidden + (sharded ? (size_t)d->rank * d->d_loc : 0);
            float* y[1] = {in_place ? mine : d->tmp_down + (size_t)d->rank * d->d_loc};
            const float* add[1] = {in_place ? mine : nullptr};
            const int rows[1] = {d->d_loc};
            if (d->stamped) {
                mgpeer::set_next_stamp_in(stamp_in(d, kSiteRecords, d->s_rec, l));
                mgpeer::set_next_peer_sync(stamp_out(d, kSiteDown, d->s_down, (long long)d->rank * d->d_loc, l));
            } else if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteDown));
            if ((e = mg_matvec_q4k_multi_on_stream(1, w, d->records, 1, add, y, rows, F / 256, s))) return fail(d, e, "down");
        }
        if (sharded && !d->fused) {
            if ((e = gather_equal(d, kSiteDown, d->tmp_down, (size_t)d->d_loc, mgnccl::kFloat32, 4))) return e;
            mg::launch_pdl(residual_add_kernel, dim3((D + 255) / 256), dim3(256), 0, d->stream, d->hidden, (const float*)d->tmp_down, D);
        }
    }
    if (d->stamped) {
        if ((e = (int)mg::launch_pdl(rms_norm_stamped_kernel, dim3(1), dim3(1024), 0, d->stream,
                                     stamp_in(d, kSiteDown, d->s_down, c.n_layers - 1), (const float*)d->out_norm, d->cur, D,
                                     c.rms_eps)))
            return fail(d, e, "rms_norm");
    } else if ((e = launch_rms_norm_on_stream(d->hidden, d->out_norm, d->cur, 1, D, c.rms_eps, s))) return fail(d, e, "rms_norm");
    if ((e = mg_matvec_f16_on_stream(d->lm_head, d->cur, d->logits, d->v_loc, D, s))) return fail(d, e, "lm_head");
    if (!sharded) {
        if ((e = mg_argmax_on_stream(d->logits, c.vocab, tok_dev, d->argmax_scratch, d->history, step_dev, s)))
            return fail(d, e, "argmax");
    } else {
        // local best -> (value, global index) pairs of all ranks -> the same global choice everywhere
        int* local_tok = reinterpret_cast<int*>(static_cast<char*>(d->argmax_scratch) + 2048);
        if ((e = mg_argmax_on_stream(d->logits, d->v_loc, local_tok, d->argmax_scratch, nullptr, nullptr, s)))
            return fail(d, e, "argmax");
        mg::launch_pdl(local_pair_kernel, dim3(1), dim3(1), 0, d->stream, (const float*)d->logits, (const int*)local_tok, d->rank * d->v_loc, d->pair_buf + 2 * d->rank,
                       d->fused ? mgpeer::make_sync(d->px, kSitePairs) : mgpeer::PeerSync{});
        if (!d->fused && (e = gather_equal(d, kSitePairs, d->pair_buf, 2, mgnccl::kFloat32, 4))) return e;
        mg::launch_pdl(argmax_pairs_kernel, dim3(1), dim3(1), 0, d->stream, (const float*)d->pair_buf, d->world, tok_dev, d->history, (const int*)step_dev);
    }
    mg::launch_pdl(advance_state_kernel, dim3(1), dim3(1), 0, d->stream, d->state);
    if ((e = (int)cudaGetLastError())) return fail(d, e, "advance");
    return 0;
}

// y = W x for one tensor of GGUF type `type` (the per-tensor dispatch of RocmGemma::qmatvec,
// crates/modgrad-gemma/src/rocm_gemma.rs:291-309).
int typed_matvec(mg_decoder* d, int type, const void* w, const float* x, float* y, int rows, int cols) {
    const uint8_t* wb = static_cast<const uint8_t*>(w);
    switch (type) {
        case kTypeQ4K: return launch_matvec_q4k_on_stream(wb, x, y, rows, cols / 256, d->stream);
        case kTypeQ5K: return launch_matvec_q5k_on_stream(wb, x, y, rows, cols / 256, d->stream);
        case kTypeQ6K: return launch_matvec_q6k_on_stream(wb, x, y, rows, cols / 256, d->stream);
        case kTypeF16: return mg_matvec_f16_on_stream(w, x, y, rows, cols, d->stream);
        default: return (int)cudaErrorInvalidValue;
    }
}

// y[i] = W[i] . rms_norm(hidden) for n tensors of one input.  All Q4_K: the one fused launch of the
// default path.  Otherwise the Q4_K tensors share one launch and every other tensor takes the launcher
// of its type, each with the RMSNorm fused in front; only for rows too long for that is the normalised
// vector written once by a launch of its own.
int norm_project(mg_decoder* d, int n, const uint8_t* const* w, const uint8_t* types, const float* norm_w, float* const* y,
                 const int* rows, int cols, const char* what) {
    int e, n4 = 0;
    const uint8_t* w4[3];
    float* y4[3];
    int rows4[3];
    for (int i = 0; i < n; ++i)
        if (types[i] == kTypeQ4K) { w4[n4] = w[i]; y4[n4] = y[i]; rows4[n4] = rows[i]; ++n4; }
    if (n4 == n) {
        e = mg_rmsnorm_matvec_q4k_multi_on_stream(n, w, d->hidden, norm_w, d->cfg.rms_eps, nullptr, y, rows, cols / 256, d->stream);
        d->mixed_launches += 1;
        return e ? fail(d, e, what) : 0;
    }
    if ((size_t)(cols / 256) * 4 * 208 <= (size_t)200 * 1024) {
        // every launch normalises for itself while it converts the activations: no separate RMSNorm launch
        if (n4) {
            if ((e = mg_rmsnorm_matvec_q4k_multi_on_stream(n4, w4, d->hidden, norm_w, d->cfg.rms_eps, nullptr, y4, rows4, cols / 256,
                                                           d->stream)))
                return fail(d, e, what);
            d->mixed_launches += 1;
        }
        for (int i = 0; i < n; ++i) {
            if (types[i] == kTypeQ4K) continue;
            if ((e = mg_rmsnorm_matvec_kquant_on_stream(types[i], w[i], d->hidden, norm_w, d->cfg.rms_eps, y[i], rows[i], cols / 256,
                                                        d->stream)))
                return fail(d, e, what);
            d->mixed_launches += 1;
        }
        return 0;
    }
    if ((e = launch_rms_norm_on_stream(d->hidden, norm_w, d->cur, 1, cols, d->cfg.rms_eps, d->stream))) return fail(d, e, "rms_norm");
    d->mixed_launches += 1;
    if (n4) {
        if ((e = mg_matvec_q4k_multi_on_stream(n4, w4, d->cur, 0, nullptr, y4, rows4, cols / 256, d->stream))) return fail(d, e, what);
        d->mixed_launches += 1;
    }
    for (int i = 0; i < n; ++i) {
        if (types[i] == kTypeQ4K) continue;
        if ((e = typed_matvec(d, types[i], w[i], d->cur, y[i], rows[i], cols))) return fail(d, e, what);
        d->mixed_launches += 1;
    }
    return 0;
}

// hidden += W x for one projection whose rows are split over the ranks: one GPU adds in place (the matvec
// itself adds); a sharded rank either does the same and ends its kernel with the exchange, or writes its
// rows into `gathered`, the rows are all-gathered and a small kernel adds the whole vector.
// x_kind 0: f32 activations, 1: limb records.
int project_add(mg_decoder* d, int type, const uint8_t* w, const void* x, int x_kind, float* gathered, int site, int cols,
                const char* what) {
    const int D = d->cfg.d_model;
    const bool sharded = d->world > 1;
    // a Q4_K matvec can end with the exchange itself (it stores its rows, added in place, into every rank's
    // hidden state); the other types write a slice that a gather kernel then distributes
    const bool in_place = !sharded || (d->fused && type == kTypeQ4K);
    float* mine = d->hidden + (sharded ? (size_t)d->rank * d->d_loc : 0);
    float* y = in_place ? mine : gathered + (size_t)d->rank * d->d_loc;
    const float* add = in_place ? mine : nullptr;
    int e;
    if (type == kTypeQ4K) {
        const uint8_t* ws[1] = {w};
        float* ys[1] = {y};
        const float* adds[1] = {add};
        const int rows[1] = {d->d_loc};
        if (sharded && in_place) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, site));
        e = mg_matvec_q4k_multi_on_stream(1, ws, x, x_kind, adds, ys, rows, cols / 256, d->stream);
    } else {
        e = mg_matvec_kquant_on_stream(type, w, x, x_kind, add, y, d->d_loc, cols / 256, d->stream);
    }
    if (e) return fail(d, e, what);
    d->mixed_launches += 1;
    if (!in_place) {
        if ((e = gather_equal(d, site, gathered, (size_t)d->d_loc, mgnccl::kFloat32, 4))) return e;
        mg::launch_pdl(residual_add_kernel, dim3((D + 255) / 256), dim3(256), 0, d->stream, d->hidden, (const float*)gathered, D);
        d->mixed_launches += 2;
    }
    return 0;
}

// One token of an engine whose tensors are not all of the default types: the same arithmetic, queued
// through the launchers of each tensor's type.  A real checkpoint mixes Q4_K with Q6_K (attn_v, ffn_down,
// token embedding, LM head) and Q5_K.  Row-sharded, the exchanges of a layer are fused into the producing
// kernels that can do it (attention, Q4_K matvecs, SwiGLU: flag handshake at their end) and are a peer-store
// gather kernel with the same handshake behind a Q5_K / Q6_K matvec; or all of them NCCL.
int queue_token_mixed(mg_decoder* d) {
    const mg_decoder_config& c = d->cfg;
    void* s = d->stream;
    const int D = c.d_model, hd = c.head_dim, F = c.d_ff;
    const int q_dim = c.n_heads * hd;
    const int Hl = d->h1 - d->h0, KVl = d->kv1 - d->kv0;
    const int q_loc = Hl * hd, kv_loc = KVl * hd;
    const bool sharded = d->world > 1;
    const float scale = 1.0f / sqrtf((float)hd);
    int e;
    int* pos_dev = d->state;
    int* step_dev = d->state + 2;
    int* tok_dev = d->state + 3;
    d->mixed_launches = 0;
    if (d->embed_type == kTypeF16) e = mg_embed_f16_on_stream(d->embed, 0, tok_dev, d->hidden, D, c.vocab, s);
    else e = mg_embed_kquant_on_stream(d->embed, d->embed_type, 0, tok_dev, d->hidden, D, c.vocab, s);
    if (e) return fail(d, e, "embed");
    d->mixed_launches += 1;
    // the SwiGLU output goes to limb records while a row of them fits one CTA's shared memory (always, sharded)
    const bool records_fit = (size_t)(F / 256) * 4 * 208 <= (size_t)200 * 1024;
    for (int l = 0; l < c.n_layers; ++l) {
        const Layer& L = d->layers[l];
        {
            const uint8_t* w[3] = {L.wq, L.wk, L.wv};
            float* y[3] = {d->q, d->k, d->v};
            const int rows[3] = {q_loc, kv_loc, kv_loc};
            if ((e = norm_project(d, 3, w, L.type, L.attn_norm, y, rows, D, "qkv"))) return e;
        }
        // this rank's heads land at their place in the full attention vector (and, fused, in every peer's)
        if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteHeads));
        if ((e = mg_sdpa_rope_decode_f16kv_on_stream(d->q, d->k, d->v, L.k_cache, L.v_cache, d->att_full + (size_t)d->h0 * hd, Hl,
                                                     KVl, hd, 0, pos_dev, scale, c.rope_base, d->rope_freq, d->attn_scratch,
                                                     d->n_splits, s)))
            return fail(d, e, "attention");
        d->mixed_launches += 1;
        if (!d->fused && (e = gather_heads(d))) return e;
        if ((e = project_add(d, L.type[3], L.wo, d->att_full, 0, d->tmp_full, kSiteOut, q_dim, "o_proj"))) return e;
        {
            const uint8_t* w[2] = {L.wgate, L.wup};
            float* y[2] = {d->gate, d->up};
            const int rows[2] = {d->f_loc, d->f_loc};
            if ((e = norm_project(d, 2, w, L.type + 4, L.ffn_norm, y, rows, D, "gate_up"))) return e;
        }
        if (L.type[6] == kTypeQ4K || records_fit) {
            // SwiGLU straight into limb records (a rank's slice is a whole number of records), which the Q4_K,
            // Q5_K and Q6_K down projections all read
            uint8_t* rec = static_cast<uint8_t*>(d->records) + mg_q4k_limb_record_bytes(d->f_loc) * d->rank;
            if (d->fused) mgpeer::set_next_peer_sync(mgpeer::make_sync(d->px, kSiteRecords));
            if ((e = mg_swiglu_limbs_on_stream(d->gate, d->up, nullptr, d->f_loc, rec, s))) return fail(d, e, "swiglu");
            d->mixed_launches += 1;
            if (!d->fused &&
                (e = gather_equal(d, kSiteRecords, d->records, mg_q4k_limb_record_bytes(d->f_loc), mgnccl::kUint8, 1)))
                return e;
            if ((e = project_add(d, L.type[6], L.wdown, d->records, 1, d->tmp_down, kSiteDown, F, "down"))) return e;
        } else {   // one GPU only (refused at creation otherwise)
            if ((e = launch_swiglu_on_stream(d->gate, d->up, d->gate, F, s))) return fail(d, e, "swiglu");
            d->mixed_launches += 1;
            if ((e = project_add(d, L.type[6], L.wdown, d->gate, 0, d->tmp_down, kSiteDown, F, "down"))) return e;
        }
    }
    if (d->head_type != kTypeF16 && (size_t)(D / 256) * 4 * 208 <= (size_t)200 * 1024) {   // final RMSNorm inside the head's launch
        const uint8_t* w[1] = {reinterpret_cast<const uint8_t*>(d->lm_head)};
        float* y[1] = {d->logits};
        const int rows[1] = {d->v_loc};
        const uint8_t t[1] = {(uint8_t)d->head_type};
        if ((e = norm_project(d, 1, w, t, d->out_norm, y, rows, D, "lm_head"))) return e;
        d->mixed_launches -= 2;   // counted with the tail below
    } else {
        if ((e = launch_rms_norm_on_stream(d->hidden, d->out_norm, d->cur, 1, D, c.rms_eps, s))) return fail(d, e, "rms_norm");
        if ((e = typed_matvec(d, d->head_type, d->lm_head, d->cur, d->logits, d->v_loc, D))) return fail(d, e, "lm_head");
    }
    if (!sharded) {
        if ((e = mg_argmax_on_stream(d->logits, c.vocab, tok_dev, d->argmax_scratch, d->history, step_dev, s)))
            return fail(d, e, "argmax");
    } else {
        // local best -> (value, global index) pairs of all ranks -> the same global choice everywhere
        int* local_tok = reinterpret_cast<int*>(static_cast<char*>(d->argmax_scratch) + 2048);
        if ((e = mg_argmax_on_stream(d->logits, d->v_loc, local_tok, d->argmax_scratch, nullptr, nullptr, s)))
            return fail(d, e, "argmax");
        mg::launch_pdl(local_pair_kernel, dim3(1), dim3(1), 0, d->stream, (const float*)d->logits, (const int*)local_tok,
                       d->rank * d->v_loc, d->pair_buf + 2 * d->rank,
                       d->fused ? mgpeer::make_sync(d->px, kSitePairs) : mgpeer::PeerSync{});
        if (!d->fused && (e = gather_equal(d, kSitePairs, d->pair_buf, 2, mgnccl::kFloat32, 4))) return e;
        mg::launch_pdl(argmax_pairs_kernel, dim3(1), dim3(1), 0, d->stream, (const float*)d->pair_buf, d->world, tok_dev, d->history,
                       (const int*)step_dev);
        d->mixed_launches += 2;
    }
    mg::launch_pdl(advance_state_kernel, dim3(1), dim3(1), 0, d->stream, d->state);
    d->mixed_launches += 5;
    if ((e = (int)cudaGetLastError())) return fail(d, e, "advance");
    return 0;
}

// Maps every rank's arena into this process (CUDA IPC handles exchanged with an NCCL all-gather)
// so that the per-layer gathers can be direct peer stores.  Falls back to NCCL gathers — on all
// ranks together — when any rank cannot map its peers, or when MODGRAD_DECODER_GATHER=nccl.
int setup_peer_exchange(mg_decoder* d) {
    const mgnccl::Api& n = mgnccl::api();
    const int world = d->world;
    // MODGRAD_DECODER_GATHER: "nccl" (NCCL collectives), "peer" (one peer-store gather kernel per
    // collective), "fused" (the producing kernels store to the peers themselves and end with a flag
    // handshake), default "stamped" (the same stores, every word carrying its epoch: no handshake,
    // the consuming kernel polls the words it reads).
    const char* mode = getenv("MODGRAD_DECODER_GATHER");
    int want = !(mode && strcmp(mode, "nccl") == 0) && world <= mgpeer::kMaxRanks;
    struct Slot { cudaIpcMemHandle_t h; int ok; int pad[15]; };  // 128 bytes
    static_assert(sizeof(Slot) == 128, "slot size");
    std::vector<Slot> host(world);
    Slot mine{};
    mine.ok = want && cudaIpcGetMemHandle(&mine.h, d->arena) == cudaSuccess;
    uint8_t* dev_slots = nullptr;
    int rc;
    if ((rc = dev_alloc(d, &dev_slots, sizeof(Slot) * world))) return rc;
    cudaError_t e = cudaMemcpy(dev_slots + sizeof(Slot) * d->rank, &mine, sizeof mine, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(d, (int)e, "ipc slot");
    // two passes: the handles, then whether every rank managed to open every handle
    for (int pass = 0; pass < 2; ++pass) {
        if (n.AllGather(dev_slots + sizeof(Slot) * d->rank, dev_slots, sizeof(Slot), mgnccl::kUint8, d->comm, d->stream))
            return fail(d, (int)cudaErrorUnknown, "ncclAllGather (ipc handles)");
        if ((e = cudaStreamSynchronize(d->stream)) != cudaSuccess) return fail(d, (int)e, "ipc exchange");
        if ((e = cudaMemcpy(host.data(), dev_slots, sizeof(Slot) * world, cudaMemcpyDeviceToHost)) != cudaSuccess)
            return fail(d, (int)e, "ipc slots");
        bool all = true;
        for (int r = 0; r < world; ++r) all = all && host[r].ok;
        if (pass == 0) {
            int opened = all ? 1 : 0;
            d->px.rank = d->rank; d->px.world = world; d->px.bytes = d->arena_bytes;
            for (int r = 0; r < world && opened; ++r) {
                if (r == d->rank) { d->px.base[r] = d->arena; continue; }
                void* p = nullptr;
                if (cudaIpcOpenMemHandle(&p, host[r].h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    opened = 0;
                    break;
                }
                d->ipc_opened.push_back(p);
                d->px.base[r] = static_cast<unsigned char*>(p);
            }
            mine.ok = opened;
            if ((e = cudaMemcpy(dev_slots + sizeof(Slot) * d->rank, &mine, sizeof mine, cudaMemcpyHostToDevice)) != cudaSuccess)
                return fail(d, (int)e, "ipc slot");
        } else {
            d->peer = all;
            d->fused = all && !(mode && strcmp(mode, "peer") == 0);
            d->stamped = d->fused && !(mode && strcmp(mode, "fused") == 0);
        }
    }
    if (d->peer) {
        if ((rc = dev_alloc(d, &d->px.ctl, mgpeer::kCtlWords))) return rc;
        if ((e = cudaMemset(d->px.ctl, 0, mgpeer::kCtlWords * sizeof(unsigned))) != cudaSuccess) return fail(d, (int)e, "ctl");
    }
    return 0;
}
int check_peer_error(mg_decoder* d) {
    if (!d->peer) return 0;
    int site = 0;
    cudaError_t e = mgpeer::read_error(d->px, &site);
    if (e != cudaSuccess) return fail(d, (int)e, "peer error word");
    if (site) {
        d->last_error = "peer gather: a rank did not arrive within the wait limit (site " + std::to_string(site - 1) + ")";
        return (int)cudaErrorLaunchTimeout;
    }
    return 0;
}

int ensure_graph(mg_decoder* d) {
    if (d->graph_exec) return 0;
    // A first pass outside capture sets every kernel attribute (function attributes cannot be
    // changed while capturing); it is undone by restoring the device state afterwards.
    int saved[4];
    cudaError_t e = cudaMemcpy(saved, d->state, sizeof saved, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(d, (int)e, "state read");
    int rc = queue_token(d);
    if (rc) return rc;
    if ((e = cudaStreamSynchronize(d->stream)) != cudaSuccess) return fail(d, (int)e, "warm-up token");
    if ((e = cudaMemcpy(d->state, saved, sizeof saved, cudaMemcpyHostToDevice)) != cudaSuccess)
        return fail(d, (int)e, "state restore");
    if ((e = cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal)) != cudaSuccess)
        return fail(d, (int)e, "begin capture");
    rc = queue_token(d);
    cudaError_t ee = cudaStreamEndCapture(d->stream, &d->graph);
    if (rc) return rc;
    if (ee != cudaSuccess) return fail(d, (int)ee, "end capture");
    if ((e = cudaGraphInstantiate(&d->graph_exec, d->graph, 0)) != cudaSuccess) return fail(d, (int)e, "instantiate");
    return 0;
}

}  // namespace

extern "C" {

// A fresh NCCL unique id (128 bytes) for mg_decoder_create_sharded; rank 0 makes it and the
// host distributes it to the other ranks by whatever channel it has.
int mg_nccl_unique_id(void* out128) {
    if (!out128) return (int)cudaErrorInvalidValue;
    const mgnccl::Api& n = mgnccl::api();
    if (!n.ok) return (int)cudaErrorNotSupported;
    mgnccl::UniqueId id;
    if (n.GetUniqueId(&id)) return (int)cudaErrorUnknown;
    memcpy(out128, &id, sizeof id);
    return 0;
}

// Row ranges of rank `rank` of `world` (the same arithmetic as modgrad_b200/shard.py):
// query heads [h0,h1) = [rank*H/world, (rank+1)*H/world), the KV heads they use, and equal
// slices of the hidden state, the FFN and the vocabulary.
int mg_decoder_shard_ranges(const mg_decoder_config* cfg, int rank, int world, int* out8) {
    if (!cfg || !out8 || world < 1 || rank < 0 || rank >= world) return (int)cudaErrorInvalidValue;
    const int H = cfg->n_heads, grp = cfg->n_heads / cfg->n_kv_heads;
    const int h0 = (int)((long long)rank * H / world), h1 = (int)((long long)(rank + 1) * H / world);
    if (h1 <= h0) return (int)cudaErrorInvalidValue;
    const int kv0 = h0 / grp, kv1 = (h1 - 1) / grp + 1;
    // the local heads must form whole groups over the local KV heads, or share ONE KV head
    const bool one_kv = (kv1 - kv0) == 1;
    const bool whole = (h0 % grp == 0) && (h1 % grp == 0);
    if (!one_kv && !whole) return (int)cudaErrorInvalidValue;
    if (cfg->d_model % world || cfg->d_ff % world || (cfg->d_ff / world) % 64 || cfg->vocab % world)
        return (int)cudaErrorInvalidValue;
    out8[0] = h0; out8[1] = h1; out8[2] = kv0; out8[3] = kv1;
    out8[4] = cfg->d_model / world; out8[5] = cfg->d_ff / world; out8[6] = cfg->vocab / world; out8[7] = grp;
    return 0;
}

}  // extern "C"

namespace {

// proj_types: n_layers * 7 GGUF type ids in the order wq, wk, wv, wo, wgate, wup, wdown, or null for
// all Q4_K.
int create_impl(const mg_decoder_config* cfg, int rank, int world, const void* nccl_id128, const int* proj_types,
                int embed_type, int head_type, mg_decoder** out) {
    if (!cfg || !out) return (int)cudaErrorInvalidValue;
    *out = nullptr;
    const mg_decoder_config& c = *cfg;
    if (c.n_layers <= 0 || c.d_model <= 0 || c.d_model % 256 || c.d_ff <= 0 || c.d_ff % 256 || c.n_heads <= 0 ||
        c.n_kv_heads <= 0 || c.n_heads % c.n_kv_heads || (c.n_heads * c.head_dim) % 256 || c.vocab <= 0 ||
        c.max_seq <= 0 || c.d_model / 256 > 32 || (c.n_heads * c.head_dim) / 256 > 32)
        return (int)cudaErrorInvalidValue;
    if (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) return (int)cudaErrorInvalidValue;
    int rg[8];
    int rc = mg_decoder_shard_ranges(cfg, rank, world, rg);
    if (rc) return rc;
    if (world > 1 && (!nccl_id128 || !mgnccl::api().ok)) return (int)cudaErrorNotSupported;
    mg_decoder* d = new mg_decoder();
    d->cfg = c;
    d->rank = rank; d->world = world;
    d->h0 = rg[0]; d->h1 = rg[1]; d->kv0 = rg[2]; d->kv1 = rg[3];
    d->d_loc = rg[4]; d->f_loc = rg[5]; d->v_loc = rg[6];
    d->head_lo.resize(world + 1);
    for (int r = 0; r <= world; ++r) d->head_lo[r] = (int)((long long)r * c.n_heads / world);
    auto bail = [&](int code) {
        mg_decoder_destroy(d);
        return code;
    };
    cudaError_t e = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return bail((int)e);
    if (world > 1) {
        mgnccl::UniqueId id;
        memcpy(&id, nccl_id128, sizeof id);
        if (mgnccl::api().CommInitRank(&d->comm, world, id, rank)) return bail((int)cudaErrorUnknown);
    }
    const int D = c.d_model, F = c.d_ff, hd = c.head_dim, q_dim = c.n_heads * hd;
    const int q_loc = (d->h1 - d->h0) * hd, kv_loc = (d->kv1 - d->kv0) * hd;
    d->layers.resize(c.n_layers);
    d->embed_type = embed_type;
    d->head_type = head_type;
    d->mixed = embed_type != kTypeF16 || head_type != kTypeF16;
    if (proj_types)
        for (int l = 0; l < c.n_layers; ++l)
            for (int i = 0; i < 7; ++i) {
                d->layers[l].type[i] = (uint8_t)proj_types[l * 7 + i];
                d->mixed = d->mixed || proj_types[l * 7 + i] != kTypeQ4K;
            }
    // a sharded typed engine exchanges the SwiGLU output as limb records, which one CTA must be able to hold
    if (d->mixed && world > 1 && (size_t)(c.d_ff / 256) * 4 * 208 > (size_t)200 * 1024) return bail((int)cudaErrorInvalidValue);
    {   // Every weight lives in ONE device allocation addressed by offset, as the reference's engine
        // packs its quantised tensors (crates/modgrad-gemma/src/rocm_gemma.rs:206-224); 256-byte
        // aligned sub-ranges, so every Q4_K row stays 16-byte aligned.
        size_t off = 0;
        auto take = [&](size_t bytes) {
            const size_t at = off;
            off += (bytes + 255) & ~(size_t)255;
            return at;
        };
        struct Slots { size_t wq, wk, wv, wo, wgate, wup, wdown, attn_norm, ffn_norm; };
        std::vector<Slots> slots(c.n_layers);
        for (int l = 0; l < c.n_layers; ++l) {
            Slots& sl = slots[l];
            const uint8_t* t = d->layers[l].type;
            sl.wq = take(typed_bytes(t[0], q_loc, D)); sl.wk = take(typed_bytes(t[1], kv_loc, D));
            sl.wv = take(typed_bytes(t[2], kv_loc, D)); sl.wo = take(typed_bytes(t[3], d->d_loc, q_dim));
            sl.wgate = take(typed_bytes(t[4], d->f_loc, D)); sl.wup = take(typed_bytes(t[5], d->f_loc, D));
            sl.wdown = take(typed_bytes(t[6], d->d_loc, F));
            sl.attn_norm = take((size_t)D * 4); sl.ffn_norm = take((size_t)D * 4);
        }
        const size_t o_embed = take(typed_bytes(embed_type, c.vocab, D)), o_head = take(typed_bytes(head_type, d->v_loc, D)),
                     o_norm = take((size_t)D * 4);
        if ((rc = dev_alloc(d, &d->weights, off))) return bail(rc);
        d->weights_bytes = off;
        for (int l = 0; l < c.n_layers; ++l) {
            Layer& L = d->layers[l];
            const Slots& sl = slots[l];
            L.wq = d->weights + sl.wq; L.wk = d->weights + sl.wk; L.wv = d->weights + sl.wv; L.wo = d->weights + sl.wo;
            L.wgate = d->weights + sl.wgate; L.wup = d->weights + sl.wup; L.wdown = d->weights + sl.wdown;
            L.attn_norm = reinterpret_cast<float*>(d->weights + sl.attn_norm);
            L.ffn_norm = reinterpret_cast<float*>(d->weights + sl.ffn_norm);
        }
        d->embed = reinterpret_cast<__half*>(d->weights + o_embed);
        d->lm_head = reinterpret_cast<__half*>(d->weights + o_head);
        d->out_norm = reinterpret_cast<float*>(d->weights + o_norm);
    }
    for (Layer& L : d->layers) {
        if ((rc = dev_alloc(d, &L.k_cache, (size_t)c.max_seq * kv_loc))) return bail(rc);
        if ((rc = dev_alloc(d, &L.v_cache, (size_t)c.max_seq * kv_loc))) return bail(rc);
    }
    if ((rc = dev_alloc(d, &d->cur, (size_t)D))) return bail(rc);
    if ((rc = dev_alloc(d, &d->q, (size_t)q_loc))) return bail(rc);
    if ((rc = dev_alloc(d, &d->k, (size_t)kv_loc))) return bail(rc);
    if ((rc = dev_alloc(d, &d->v, (size_t)kv_loc))) return bail(rc);
    {   // the gathered buffers, in one allocation that peers can map: flags, then the buffers
        auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
        const size_t o_att = mgpeer::kFlagBytes, o_out = o_att + up((size_t)q_dim * 4), o_down = o_out + up((size_t)D * 4),
                     o_rec = o_down + up((size_t)D * 4), o_pair = o_rec + up(mg_q4k_limb_record_bytes(F)),
                     o_hid = o_pair + up((size_t)2 * mgpeer::kMaxRanks * 4), o_satt = o_hid + up((size_t)D * 4),
                     o_sout = o_satt + up((size_t)q_dim * 8), o_sdown = o_sout + up((size_t)D * 8),
                     o_srec = o_sdown + up((size_t)D * 8), total = o_srec + up((size_t)(F / 64) * 52 * 8);
        if ((rc = dev_alloc(d, &d->arena, total))) return bail(rc);
        if ((e = cudaMemset(d->arena, 0, total)) != cudaSuccess) return bail((int)e);
        d->arena_bytes = total;
        d->att_full = reinterpret_cast<float*>(d->arena + o_att);
        d->tmp_full = reinterpret_cast<float*>(d->arena + o_out);
        d->tmp_down = reinterpret_cast<float*>(d->arena + o_down);
        d->records = d->arena + o_rec;
        d->pair_buf = reinterpret_cast<float*>(d->arena + o_pair);
        d->hidden = reinterpret_cast<float*>(d->arena + o_hid);
        d->s_att = reinterpret_cast<unsigned long long*>(d->arena + o_satt);
        d->s_out = reinterpret_cast<unsigned long long*>(d->arena + o_sout);
        d->s_down = reinterpret_cast<unsigned long long*>(d->arena + o_sdown);
        d->s_rec = reinterpret_cast<unsigned long long*>(d->arena + o_srec);
    }
    if ((rc = dev_alloc(d, &d->gate, (size_t)d->f_loc))) return bail(rc);
    if ((rc = dev_alloc(d, &d->up, (size_t)d->f_loc))) return bail(rc);
    if ((rc = dev_alloc(d, &d->logits, (size_t)d->v_loc))) return bail(rc);
    uint8_t* tmp = nullptr;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int kv_n = d->kv1 - d->kv0;
    d->n_splits = sms / kv_n > 0 ? (sms / kv_n < 160 ? sms / kv_n : 160) : 1;  // the one-launch attention takes up to 160
    {
        const size_t nb = mg_sdpa_rope_f16kv_scratch_bytes(d->h1 - d->h0, kv_n, hd, d->n_splits);
        if ((rc = dev_alloc(d, &tmp, nb))) return bail(rc);
        if ((e = cudaMemset(tmp, 0, nb)) != cudaSuccess) return bail((int)e);  // the ticket counters start at zero
        d->attn_scratch = tmp;
    }
    if ((rc = dev_alloc(d, &tmp, (size_t)2 * 256 * 4 + 64))) return bail(rc);
    d->argmax_scratch = tmp;
    if ((rc = dev_alloc(d, &d->state, (size_t)8))) return bail(rc);
    if ((e = cudaMemset(d->state, 0, 8 * sizeof(int))) != cudaSuccess) return bail((int)e);
    d->history_cap = c.max_seq + 1;
    if ((rc = dev_alloc(d, &d->history, (size_t)d->history_cap))) return bail(rc);
    {   // inv_freq = base^(-2i/head_dim) as the CPU decoder evaluates it (llm.rs:958), rounded once
        std::vector<float> f((size_t)hd / 2);
        for (int i = 0; i < hd / 2; ++i) f[i] = (float)pow((double)c.rope_base, (double)(-2.0f * (float)i / (float)hd));
        if ((rc = dev_alloc(d, &d->rope_freq, f.size()))) return bail(rc);
        if ((e = cudaMemcpy(d->rope_freq, f.data(), f.size() * 4, cudaMemcpyHostToDevice)) != cudaSuccess) return bail((int)e);
    }
    int init[4] = {0, 1, 0, 0};
    if ((e = cudaMemcpy(d->state, init, sizeof init, cudaMemcpyHostToDevice)) != cudaSuccess) return bail((int)e);
    if (world > 1 && (rc = setup_peer_exchange(d))) return bail(rc);
    // the typed path ends its Q4_K / attention / SwiGLU kernels with the handshake exchange and gathers behind
    // the other types with a kernel using the same handshake; its consumers read plain arrays, not stamped words
    if (d->mixed) d->stamped = false;
    *out = d;
    return 0;
}

}  // namespace

extern "C" {

int mg_decoder_create_sharded(const mg_decoder_config* cfg, int rank, int world, const void* nccl_id128,
                              mg_decoder** out) {
    return create_impl(cfg, rank, world, nccl_id128, nullptr, kTypeF16, kTypeF16, out);
}

// An engine whose tensors carry their own GGUF types, as real checkpoints mix them
// (crates/modgrad-gemma/src/rocm_gemma.rs:291-309 dispatches per tensor the same way): every projection
// Q4_K (12), Q5_K (13) or Q6_K (14); the token embedding and the LM head F16 (1) or one of the three.
// proj_types holds n_layers * 7 ids in the order q, k, v, o, gate, up, down.  An engine whose types are
// all the defaults is the one mg_decoder_create_sharded builds.  Row-sharded like that one (same row
// ranges, same uploads); see queue_token_mixed for its exchanges.
int mg_decoder_create_typed_sharded(const mg_decoder_config* cfg, const int* proj_types, int embed_type, int head_type,
                                    int rank, int world, const void* nccl_id128, mg_decoder** out) {
    if (!cfg || !proj_types || !out) return (int)cudaErrorInvalidValue;
    auto quant = [](int t) { return t == kTypeQ4K || t == kTypeQ5K || t == kTypeQ6K; };
    for (int i = 0; i < cfg->n_layers * 7; ++i)
        if (!quant(proj_types[i])) return (int)cudaErrorInvalidValue;
    if ((embed_type != kTypeF16 && !quant(embed_type)) || (head_type != kTypeF16 && !quant(head_type)))
        return (int)cudaErrorInvalidValue;
    return create_impl(cfg, rank, world, nccl_id128, proj_types, embed_type, head_type, out);
}
int mg_decoder_create_typed(const mg_decoder_config* cfg, const int* proj_types, int embed_type, int head_type,
                            mg_decoder** out) {
    return mg_decoder_create_typed_sharded(cfg, proj_types, embed_type, head_type, 0, 1, nullptr, out);
}

int mg_decoder_create(const mg_decoder_config* cfg, mg_decoder** out) {
    return mg_decoder_create_sharded(cfg, 0, 1, nullptr, out);
}

void mg_decoder_destroy(mg_decoder* d) {
    if (!d) return;
    if (d->graph_exec) cudaGraphExecDestroy(d->graph_exec);
    if (d->graph) cudaGraphDestroy(d->graph);
    for (void* p : d->ipc_opened) cudaIpcCloseMemHandle(p);
    if (d->comm) mgnccl::api().CommDestroy(d->comm);
    for (void* p : d->allocs) cudaFree(p);
    if (d->stream) cudaStreamDestroy(d->stream);
    delete d;
}

const char* mg_decoder_last_error(const mg_decoder* d) { return d ? d->last_error.c_str() : ""; }

// Uploads one tensor verbatim (the super-blocks of its type, f32 norm weights, half embedding / LM head).
int mg_decoder_upload(mg_decoder* d, int layer, int which, const void* host, size_t bytes) {
    if (!d || !host) return (int)cudaErrorInvalidValue;
    const mg_decoder_config& c = d->cfg;
    const int D = c.d_model, F = c.d_ff, q_dim = c.n_heads * c.head_dim;
    const int q_loc = (d->h1 - d->h0) * c.head_dim, kv_loc = (d->kv1 - d->kv0) * c.head_dim;
    void* dst = nullptr;
    size_t want = 0;
    if (which >= MG_W_EMBED) {
        switch (which) {
            case MG_W_EMBED: dst = d->embed; want = typed_bytes(d->embed_type, c.vocab, D); break;
            case MG_W_LM_HEAD: dst = d->lm_head; want = typed_bytes(d->head_type, d->v_loc, D); break;
            case MG_W_OUT_NORM: dst = d->out_norm; want = (size_t)D * 4; break;
            default: return (int)cudaErrorInvalidValue;
        }
    } else {
        if (layer < 0 || layer >= c.n_layers) return (int)cudaErrorInvalidValue;
        Layer& L = d->layers[layer];
        switch (which) {
            case MG_W_Q: dst = L.wq; want = typed_bytes(L.type[0], q_loc, D); break;
            case MG_W_K: dst = L.wk; want = typed_bytes(L.type[1], kv_loc, D); break;
            case MG_W_V: dst = L.wv; want = typed_bytes(L.type[2], kv_loc, D); break;
            case MG_W_O: dst = L.wo; want = typed_bytes(L.type[3], d->d_loc, q_dim); break;
            case MG_W_GATE: dst = L.wgate; want = typed_bytes(L.type[4], d->f_loc, D); break;
            case MG_W_UP: dst = L.wup; want = typed_bytes(L.type[5], d->f_loc, D); break;
            case MG_W_DOWN: dst = L.wdown; want = typed_bytes(L.type[6], d->d_loc, F); break;
            case MG_W_ATTN_NORM: dst = L.attn_norm; want = (size_t)D * 4; break;
            case MG_W_FFN_NORM: dst = L.ffn_norm; want = (size_t)D * 4; break;
            default: return (int)cudaErrorInvalidValue;
        }
    }
    if (bytes != want) {
        d->last_error = "upload: size mismatch, expected " + std::to_string(want) + " got " + std::to_string(bytes);
        return (int)cudaErrorInvalidValue;
    }
    return (int)cudaMemcpy(dst, host, bytes, cudaMemcpyHostToDevice);
}

// Prefills positions [0, n_pos) of one layer's half KV cache and sets the position to n_pos.
int mg_decoder_set_kv(mg_decoder* d, int layer, const void* k_f16, const void* v_f16, int n_pos) {
    if (!d || layer < 0 || layer >= d->cfg.n_layers || n_pos < 0 || n_pos >= d->cfg.max_seq) return (int)cudaErrorInvalidValue;
    const size_t bytes = (size_t)n_pos * (d->kv1 - d->kv0) * d->cfg.head_dim * 2;  // this rank's KV heads
    if (bytes) {
        if (!k_f16 || !v_f16) return (int)cudaErrorInvalidValue;
        cudaError_t e = cudaMemcpy(d->layers[layer].k_cache, k_f16, bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return (int)e;
        e = cudaMemcpy(d->layers[layer].v_cache, v_f16, bytes, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) return (int)e;
    }
    return mg_decoder_set_position(d, n_pos);
}

int mg_decoder_set_position(mg_decoder* d, int pos) {
    if (!d || pos < 0 || pos >= d->cfg.max_seq) return (int)cudaErrorInvalidValue;
    int st[3] = {pos, pos + 1, 0};
    d->pos_host = pos;
    return (int)cudaMemcpy(d->state, st, sizeof st, cudaMemcpyHostToDevice);
}

// One token in, logits out (RocmGemma::forward_token, rocm_gemma.rs:312-356): one graph
// launch, ONE synchronisation, then the logits are copied to the host when asked for.
// Returns the greedy next token through *next_token (may be null).
int mg_decoder_forward_token(mg_decoder* d, int token, float* logits_host, int* next_token) {
    if (!d || token < 0 || token >= d->cfg.vocab) return (int)cudaErrorInvalidValue;
    if (d->pos_host >= d->cfg.max_seq) {
        d->last_error = "forward_token: KV cache full";
        return (int)cudaErrorInvalidValue;
    }
    int rc = ensure_graph(d);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(d->state + 3, &token, sizeof(int), cudaMemcpyHostToDevice, d->stream);
    if (e != cudaSuccess) return fail(d, (int)e, "token upload");
    if ((e = cudaGraphLaunch(d->graph_exec, d->stream)) != cudaSuccess) return fail(d, (int)e, "graph launch");
    if ((e = cudaStreamSynchronize(d->stream)) != cudaSuccess) return fail(d, (int)e, "sync");
    if ((rc = check_peer_error(d))) return rc;
    d->pos_host += 1;
    if (logits_host) {
        e = cudaMemcpy(logits_host, d->logits, (size_t)d->v_loc * 4, cudaMemcpyDeviceToHost);  // this rank's slice
        if (e != cudaSuccess) return fail(d, (int)e, "logits download");
    }
    if (next_token) {
        e = cudaMemcpy(next_token, d->state + 3, sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return fail(d, (int)e, "token download");
    }
    return 0;
}

// Greedy decode of n_tokens starting from first_token (RocmGemma::generate, rocm_gemma.rs:372):
// the arg-max of each step is fed back on the device; the host synchronises once at the end
// and downloads the generated ids.  device_ms (may be null) receives the device time of the
// loop measured with events on the engine's stream.
int mg_decoder_generate(mg_decoder* d, int first_token, int n_tokens, int* out_tokens, float* device_ms) {
    if (!d || n_tokens <= 0 || first_token < 0 || first_token >= d->cfg.vocab) return (int)cudaErrorInvalidValue;
    if (d->pos_host + n_tokens > d->cfg.max_seq || n_tokens > d->history_cap) {
        d->last_error = "generate: KV cache too small for the requested tokens";
        return (int)cudaErrorInvalidValue;
    }
    int rc = ensure_graph(d);
    if (rc) return rc;
    int st[2] = {0, first_token};
    cudaError_t e = cudaMemcpyAsync(d->state + 2, st, sizeof st, cudaMemcpyHostToDevice, d->stream);
    if (e != cudaSuccess) return fail(d, (int)e, "state upload");
    cudaEvent_t a = nullptr, b = nullptr;
    cudaEventCreate(&a);
    cudaEventCreate(&b);
    cudaEventRecord(a, d->stream);
    for (int i = 0; i < n_tokens; ++i) {
        if ((e = cudaGraphLaunch(d->graph_exec, d->stream)) != cudaSuccess) break;
    }
    cudaEventRecord(b, d->stream);
    cudaError_t es = cudaStreamSynchronize(d->stream);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    if (e != cudaSuccess) return fail(d, (int)e, "graph launch");
    if (es != cudaSuccess) return fail(d, (int)es, "sync");
    if ((rc = check_peer_error(d))) return rc;
    d->pos_host += n_tokens;
    if (device_ms) *device_ms = ms;
    if (out_tokens) {
        e = cudaMemcpy(out_tokens, d->history, (size_t)n_tokens * sizeof(int), cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return fail(d, (int)e, "history download");
    }
    return 0;
}

// Device pointers of the engine's buffers, for parity tests of intermediate activations.
void* mg_decoder_buffer(mg_decoder* d, int which) {
    if (!d) return nullptr;
    switch (which) {
        case 0: return d->hidden;
        case 1: return d->logits;
        case 2: return d->state;
        case 3: return d->pair_buf;
        case 4: return static_cast<char*>(d->argmax_scratch) + 2048;
        default: return nullptr;
    }
}
// Base and size of the single device allocation that holds all weights (offsets of the tensors
// inside it follow from mg_decoder_weight_ptr).
void* mg_decoder_weight_arena(mg_decoder* d, size_t* bytes) {
    if (!d) return nullptr;
    if (bytes) *bytes = d->weights_bytes;
    return d->weights;
}
// Device pointer of one weight tensor (the `which` codes of mg_decoder_upload).
void* mg_decoder_weight_ptr(mg_decoder* d, int layer, int which) {
    if (!d) return nullptr;
    if (which >= MG_W_EMBED) {
        switch (which) {
            case MG_W_EMBED: return d->embed;
            case MG_W_LM_HEAD: return d->lm_head;
            case MG_W_OUT_NORM: return d->out_norm;
            default: return nullptr;
        }
    }
    if (layer < 0 || layer >= d->cfg.n_layers) return nullptr;
    Layer& L = d->layers[layer];
    switch (which) {
        case MG_W_Q: return L.wq;
        case MG_W_K: return L.wk;
        case MG_W_V: return L.wv;
        case MG_W_O: return L.wo;
        case MG_W_GATE: return L.wgate;
        case MG_W_UP: return L.wup;
        case MG_W_DOWN: return L.wdown;
        case MG_W_ATTN_NORM: return L.attn_norm;
        case MG_W_FFN_NORM: return L.ffn_norm;
        default: return nullptr;
    }
}
// GGUF type id of one weight tensor (the `which` codes of mg_decoder_upload); 0 (F32) for the norms, -1 on error.
int mg_decoder_weight_type(const mg_decoder* d, int layer, int which) {
    if (!d) return -1;
    if (which == MG_W_EMBED) return d->embed_type;
    if (which == MG_W_LM_HEAD) return d->head_type;
    if (which == MG_W_OUT_NORM || which == MG_W_ATTN_NORM || which == MG_W_FFN_NORM) return 0;
    if (layer < 0 || layer >= d->cfg.n_layers || which < MG_W_Q || which > MG_W_DOWN) return -1;
    return d->layers[layer].type[which - MG_W_Q];
}
int mg_decoder_kernels_per_token(const mg_decoder* d) {
    if (!d) return 0;
    if (d->mixed) return d->mixed_launches;  // launcher calls of the last queued token (0 before the first)
    // per layer: qkv, attention (RoPE + append + splits + merge), o, gate/up, SwiGLU, down
    if (d->world == 1) return 1 + d->cfg.n_layers * 6 + 5;
    // sharded: + the pair kernels at the end; + two residual adds per layer unless the matvecs
    // add in place (fused); + one gather kernel per collective in the peer-kernel mode
    int n = 1 + d->cfg.n_layers * (d->fused ? 6 : 8) + 7;
    if (d->peer && !d->fused) n += 4 * d->cfg.n_layers + 1;
    return n;
}
// Polls a bounded wait of the engine's peer exchanges makes before it gives up (default 1 << 22).
// Takes effect for graphs captured afterwards: call it before the first token.
int mg_decoder_set_exchange_spin_limit(mg_decoder* d, unsigned polls) {
    if (!d || polls == 0 || d->graph_exec) return (int)cudaErrorInvalidValue;
    d->px.spin_limit = polls;
    return 0;
}
// How the sharded engine gathers: 0 NCCL collectives, 1 one peer-store gather kernel per
// collective, 2 fused into the producing kernels; -1 for a single-GPU engine.
int mg_decoder_gather_mode(const mg_decoder* d) {
    if (!d || d->world == 1) return -1;
    return d->stamped ? 3 : (d->fused ? 2 : (d->peer ? 1 : 0));
}

}  // extern "C"
