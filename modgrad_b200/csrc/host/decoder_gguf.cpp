// GGUF checkpoint -> resident decoder: the counterpart of
//   LlmConfig::populate_from_gguf     (crates/modgrad-device/src/kfd/llm.rs:145-180)
//   LlmWeights::load_from_gguf        (crates/modgrad-device/src/kfd/llm.rs:233-296)
//   RocmGemma::load                   (crates/modgrad-gemma/src/rocm_gemma.rs:94-262: VRAM guard,
//                                      every tensor uploaded verbatim into one packed allocation)
// for the engine in decoder.cpp: Q4_K / Q5_K / Q6_K projections, f32 norm weights, token embedding and
// LM head in half or one of the three K-quants (the head tied to the embedding when the file has no
// output.weight, llm.rs:1281-1286).  A file whose projections are all Q4_K with half embedding and
// head gets the default engine; any other mix gets the typed engine (both row-shard the same way).  Tensor bytes go
// from the memory-mapped file straight to the device, never re-encoded; a row-sharded rank
// uploads only its row ranges (rows are contiguous byte ranges of the row-major block array).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <string>
#include <vector>

#include "gguf.hpp"
#include "modgrad_cuda.h"

const mggguf::File& mg_gguf_file(const mg_gguf* g);
const uint8_t* mg_gguf_bytes(const mg_gguf* g, size_t* n);

namespace {

thread_local std::string g_load_error;

int fail(int code, const std::string& msg) {
    g_load_error = msg;
    return code;
}

// (dims[0], dims[1]) = (in_dim, out_dim) of a matrix tensor.
bool matrix_dims(const mggguf::TensorInfo& t, size_t* in_dim, size_t* out_dim) {
    if (t.dims.size() != 2) return false;
    *in_dim = t.dims[0];
    *out_dim = t.dims[1];
    return true;
}

}  // namespace

extern "C" {

const char* mg_decoder_load_error(void) { return g_load_error.c_str(); }

// Architecture numbers from the metadata, as LlmConfig::populate_from_gguf reads them:
// {arch}.block_count, embedding_length, feed_forward_length, attention.head_count (required),
// attention.head_count_kv (default: head_count), attention.key_length (default d_model / heads),
// attention.layer_norm_rms_epsilon (default 1e-5), rope.freq_base (default 500000), vocabulary
// size from token_embd.weight's shape, else {arch}.vocab_size.  0, or -4 with mg_decoder_load_error().
int mg_decoder_config_from_gguf(const mg_gguf* g, int max_seq, mg_decoder_config* out) {
    if (!g || !out || max_seq <= 0) return fail(-4, "bad arguments");
    const mggguf::File& f = mg_gguf_file(g);
    const std::string* archp = f.architecture();
    if (!archp) return fail(-4, "no general.architecture");
    const std::string arch = *archp;
    uint32_t v = 0;
    mg_decoder_config c{};
    auto need = [&](const char* key, int* dst) {
        if (!f.meta_u32(arch + "." + key, &v)) return false;
        *dst = (int)v;
        return true;
    };
    if (!need("block_count", &c.n_layers)) return fail(-4, "missing " + arch + ".block_count");
    if (!need("embedding_length", &c.d_model)) return fail(-4, "missing " + arch + ".embedding_length");
    if (!need("feed_forward_length", &c.d_ff)) return fail(-4, "missing " + arch + ".feed_forward_length");
    if (!need("attention.head_count", &c.n_heads)) return fail(-4, "missing " + arch + ".attention.head_count");
    if (!need("attention.head_count_kv", &c.n_kv_heads)) c.n_kv_heads = c.n_heads;
    if (!need("attention.key_length", &c.head_dim)) c.head_dim = c.d_model / (c.n_heads > 0 ? c.n_heads : 1);
    c.rms_eps = 1e-5f;
    c.rope_base = 500000.0f;
    float fv = 0.f;
    if (f.meta_f32(arch + ".attention.layer_norm_rms_epsilon", &fv)) c.rms_eps = fv;
    if (f.meta_f32(arch + ".rope.freq_base", &fv)) c.rope_base = fv;
    const mggguf::TensorInfo* embd = f.tensor("token_embd.weight");
    if (embd && embd->dims.size() >= 2) c.vocab = (int)embd->dims[1];
    else if (!need("vocab_size", &c.vocab)) return fail(-4, "can't determine vocab_size");
    c.max_seq = max_seq;
    *out = c;
    return 0;
}

// Builds the engine for rank `rank` of `world` from the file at `path`: parse, check shapes and
// types, VRAM guard, create, upload every tensor (its row range on a sharded rank).
// Returns 0; -4 (Runtime: malformed or unsupported file), 2 (cudaErrorMemoryAllocation: the
// resident footprint plus a margin would over-commit the device), or a CUDA error code;
// mg_decoder_load_error() has the message.  MODGRAD_VRAM_MARGIN_MB overrides the 512 MiB margin.
int mg_decoder_load_gguf(const char* path, int max_seq, int rank, int world, const void* nccl_id128,
                         mg_decoder** out) {
    if (!out) return fail(-4, "null out");
    *out = nullptr;
    mg_gguf* g = nullptr;
    if (mg_gguf_open(path, &g)) return fail(-4, mg_gguf_last_error());
    struct Closer {
        mg_gguf* g;
        ~Closer() { mg_gguf_close(g); }
    } closer{g};
    mg_decoder_config c{};
    int rc = mg_decoder_config_from_gguf(g, max_seq, &c);
    if (rc) return rc;
    int rg[8];
    if (mg_decoder_shard_ranges(&c, rank, world, rg)) return fail(-4, "this model cannot be split over " + std::to_string(world) + " ranks");
    const int h0 = rg[0], h1 = rg[1], kv0 = rg[2], kv1 = rg[3], d_loc = rg[4], f_loc = rg[5], v_loc = rg[6];
    const mggguf::File& f = mg_gguf_file(g);
    size_t file_bytes = 0;
    const uint8_t* base = mg_gguf_bytes(g, &file_bytes);
    const int D = c.d_model, F = c.d_ff, hd = c.head_dim, q_dim = c.n_heads * hd, kv_dim = c.n_kv_heads * hd;

    struct Piece {
        int layer, which;
        const uint8_t* src;
        size_t bytes;
    };
    std::vector<Piece> pieces;
    size_t resident = 0;
    enum Accept { kF32Only, kQuant, kQuantOrHalf };
    std::vector<int> proj_types((size_t)c.n_layers * 7, (int)mggguf::kQ4_K);
    int embed_type = (int)mggguf::kF16, head_type = (int)mggguf::kF16;
    bool all_default = true;
    // rows [row0, row0 + rows) of matrix `name` ([out_dim][in_dim], a tensor type that `accept` allows)
    auto add_rows = [&](const std::string& name, int layer, int which, Accept accept, size_t in_dim, size_t out_dim,
                        size_t row0, size_t rows) -> int {
        const mggguf::TensorInfo* t = f.tensor(name);
        if (!t) return fail(-4, "missing " + name);
        size_t in_d = 0, out_d = 0;
        if (t->dims.size() == 1 && out_dim == 1) { in_d = t->dims[0]; out_d = 1; }
        else if (!matrix_dims(*t, &in_d, &out_d)) return fail(-4, name + ": not a matrix");
        if (in_d != in_dim || out_d != out_dim)
            return fail(-4, name + ": shape [" + std::to_string(in_d) + ", " + std::to_string(out_d) + "], expected [" +
                                std::to_string(in_dim) + ", " + std::to_string(out_dim) + "]");
        const uint32_t want = t->dtype;
        const bool quant = want == mggguf::kQ4_K || want == mggguf::kQ5_K || want == mggguf::kQ6_K;
        const bool ok = accept == kF32Only ? want == mggguf::kF32 : (quant || (accept == kQuantOrHalf && want == mggguf::kF16));
        if (!ok)
            return fail(-4, name + ": tensor type " + std::to_string(t->dtype) + " is not supported here (expected " +
                                (accept == kF32Only ? "F32" : accept == kQuant ? "Q4_K, Q5_K or Q6_K" : "F16, Q4_K, Q5_K or Q6_K") +
                                ")");
        if (which <= MG_W_DOWN) {
            proj_types[(size_t)layer * 7 + (which - MG_W_Q)] = (int)want;
            all_default = all_default && want == mggguf::kQ4_K;
        } else if (which == MG_W_EMBED || which == MG_W_LM_HEAD) {
            (which == MG_W_EMBED ? embed_type : head_type) = (int)want;
            all_default = all_default && want == mggguf::kF16;
        }
        size_t bb, be;
        mggguf::block_size(want, &bb, &be);
        if (in_dim % be) return fail(-4, name + ": row length is not a whole number of blocks");
        const size_t row_bytes = in_dim / be * bb;
        const size_t start = f.data_offset + t->offset;
        if (start > file_bytes || out_dim * row_bytes > file_bytes - start) return fail(-4, name + ": data runs past the end of the file");
        pieces.push_back({layer, which, base + start + row0 * row_bytes, rows * row_bytes});
        resident += rows * row_bytes;
        return 0;
    };
    for (int l = 0; l < c.n_layers; ++l) {
        const std::string p = "blk." + std::to_string(l) + ".";
        if ((rc = add_rows(p + "attn_q.weight", l, MG_W_Q, kQuant, D, q_dim, (size_t)h0 * hd, (size_t)(h1 - h0) * hd))) return rc;
        if ((rc = add_rows(p + "attn_k.weight", l, MG_W_K, kQuant, D, kv_dim, (size_t)kv0 * hd, (size_t)(kv1 - kv0) * hd))) return rc;
        if ((rc = add_rows(p + "attn_v.weight", l, MG_W_V, kQuant, D, kv_dim, (size_t)kv0 * hd, (size_t)(kv1 - kv0) * hd))) return rc;
        if ((rc = add_rows(p + "attn_output.weight", l, MG_W_O, kQuant, q_dim, D, (size_t)rank * d_loc, d_loc))) return rc;
        if ((rc = add_rows(p + "ffn_gate.weight", l, MG_W_GATE, kQuant, D, F, (size_t)rank * f_loc, f_loc))) return rc;
        if ((rc = add_rows(p + "ffn_up.weight", l, MG_W_UP, kQuant, D, F, (size_t)rank * f_loc, f_loc))) return rc;
        if ((rc = add_rows(p + "ffn_down.weight", l, MG_W_DOWN, kQuant, F, D, (size_t)rank * d_loc, d_loc))) return rc;
        if ((rc = add_rows(p + "attn_norm.weight", l, MG_W_ATTN_NORM, kF32Only, D, 1, 0, 1))) return rc;
        if ((rc = add_rows(p + "ffn_norm.weight", l, MG_W_FFN_NORM, kF32Only, D, 1, 0, 1))) return rc;
    }
    if ((rc = add_rows("token_embd.weight", 0, MG_W_EMBED, kQuantOrHalf, D, c.vocab, 0, c.vocab))) return rc;
    const char* head = f.tensor("output.weight") ? "output.weight" : "token_embd.weight";  // tied when absent
    if ((rc = add_rows(head, 0, MG_W_LM_HEAD, kQuantOrHalf, D, c.vocab, (size_t)rank * v_loc, v_loc))) return rc;
    if ((rc = add_rows("output_norm.weight", 0, MG_W_OUT_NORM, kF32Only, D, 1, 0, 1))) return rc;

    // VRAM guard (rocm_gemma.rs:110-138): weights + KV cache + activations must fit with headroom.
    resident += (size_t)c.n_layers * 2 * (size_t)max_seq * (kv1 - kv0) * hd * 2;  // half K and V
    resident += (size_t)(4 * D + 2 * f_loc + q_dim + v_loc) * 4 + (size_t)F * 4 + (8u << 20);
    size_t margin = (size_t)512 << 20;
    if (const char* e = getenv("MODGRAD_VRAM_MARGIN_MB")) margin = (size_t)strtoull(e, nullptr, 10) << 20;
    size_t free_b = 0, total_b = 0;
    cudaError_t ce = cudaMemGetInfo(&free_b, &total_b);
    if (ce != cudaSuccess) return fail((int)ce, std::string("cudaMemGetInfo: ") + cudaGetErrorString(ce));
    if (resident + margin > free_b) {
        char msg[256];
        snprintf(msg, sizeof msg, "would over-commit VRAM: need %.2f GiB + %.2f GiB margin > %.2f GiB free",
                 resident / 1.073741824e9, margin / 1.073741824e9, free_b / 1.073741824e9);
        return fail((int)cudaErrorMemoryAllocation, msg);
    }

    mg_decoder* d = nullptr;
    rc = all_default ? mg_decoder_create_sharded(&c, rank, world, nccl_id128, &d)
                     : mg_decoder_create_typed_sharded(&c, proj_types.data(), embed_type, head_type, rank, world, nccl_id128, &d);
    if (rc) return fail(rc, std::string("mg_decoder_create: ") + cudaGetErrorString((cudaError_t)rc));
    for (const Piece& pc : pieces) {
        rc = mg_decoder_upload(d, pc.layer, pc.which, pc.src, pc.bytes);
        if (rc) {
            const std::string msg = std::string("upload: ") + mg_decoder_last_error(d);
            mg_decoder_destroy(d);
            return fail(rc, msg);
        }
    }
    *out = d;
    return 0;
}

}  // extern "C"
