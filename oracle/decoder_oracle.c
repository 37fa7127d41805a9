/*
 * CPU ORACLE for one decoder token built from Q4_K matvecs.  TEST INFRASTRUCTURE ONLY
 * (same rules as q4k_oracle.c: never linked into or called from the shipped library).
 *
 * Restates the reference's CPU decoder `forward_token`
 * (crates/modgrad-device/src/kfd/llm.rs:1177-1298) with the choices the 7B-class
 * benchmark configuration fixes: plain RMSNorm, NEOX RoPE without frequency scaling,
 * grouped-query softmax attention, SwiGLU with the exact logistic, no soft-caps, an
 * untied LM head.  Two storage choices differ from the reference, which keeps both in
 * f32: the K/V cache holds IEEE half values (written round-to-nearest-even, widened with
 * gguf.rs:281-292 on read) and the embedding / LM head are dense half matrices (the
 * reference's dense-matrix matvec arm accumulates in f64, llm.rs:478-492; kept).
 *
 * PARITY UNPINNED: see q4k_oracle.c.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

float orc_f16_to_f32(uint16_t h);
int orc_matvec_q4k(const uint8_t* w, const float* x, float* y, int out_dim, int blocks_per_row,
                   int mode, int n_threads);
typedef void (*orc_range_fn)(int begin, int end, void* ctx);
int orc_parallel_for(int n, orc_range_fn fn, void* ctx, int n_threads);

/* f32 -> half, round to nearest even (IEEE convert; what a GPU's cvt.rn.f16.f32 does). */
uint16_t orc_f32_to_f16_rne(float f) {
    _Float16 h = (_Float16)f;
    uint16_t u;
    memcpy(&u, &h, 2);
    return u;
}

/* llm.rs:921-933, NormKind::Plain: ss = (sequential f32 sum of squares)/n;
 * dst = src * (1/sqrt(ss+eps)) * weight. */
void orc_rms_norm(const float* src, const float* weight, float* dst, int n, float eps) {
    float ss = 0.0f;
    for (int i = 0; i < n; ++i) ss += src[i] * src[i];
    ss /= (float)n;
    float inv = 1.0f / sqrtf(ss + eps);
    for (int i = 0; i < n; ++i) dst[i] = src[i] * inv * weight[i];
}

/* llm.rs:944-982 without scaling: inv_freq = base^(-2i/head_dim), pairs (i, i+half). */
void orc_apply_rope(float* data, int pos, int n_heads, int head_dim, float base) {
    int half = head_dim / 2;
    for (int h = 0; h < n_heads; ++h) {
        float* v = data + (size_t)h * head_dim;
        for (int i = 0; i < half; ++i) {
            float inv_freq = powf(base, -2.0f * (float)i / (float)head_dim);
            float angle = (float)pos * inv_freq;
            float s = sinf(angle), c = cosf(angle);
            float x0 = v[i], x1 = v[i + half];
            v[i] = x0 * c - x1 * s;
            v[i + half] = x0 * s + x1 * c;
        }
    }
}

/* llm.rs:986-1032 over a cache laid out [seq][kv_dim] (token-major): half precision (k_buf / v_buf,
 * the 7B-class configuration of this build) or f32 (k32 / v32, what the reference itself keeps:
 * llm.rs:305-310, :1232-1234). */
typedef struct {
    const float* q; const uint16_t* k_buf; const uint16_t* v_buf; float* out;
    int seq_len, n_heads, n_kv_heads, head_dim;
    const float* k32; const float* v32;
} orc_att_ctx;
static void orc_att_range(int h0, int h1, void* p) {
    orc_att_ctx* c = (orc_att_ctx*)p;
    int head_dim = c->head_dim, seq_len = c->seq_len;
    int kv_dim = c->n_kv_heads * head_dim;
    int heads_per_kv = c->n_heads / (c->n_kv_heads > 0 ? c->n_kv_heads : 1);
    float scale = 1.0f / sqrtf((float)head_dim);
    float* scores = (float*)malloc(sizeof(float) * (size_t)seq_len);
    for (int h = h0; h < h1; ++h) {
        int kv_h = h / heads_per_kv;
        const float* qh = c->q + (size_t)h * head_dim;
        size_t kv_off = (size_t)kv_h * head_dim;
        for (int t = 0; t < seq_len; ++t) {
            float s = 0.0f;
            if (c->k32) {
                const float* kt = c->k32 + (size_t)t * kv_dim + kv_off;
                for (int i = 0; i < head_dim; ++i) s += qh[i] * kt[i];
            } else {
                const uint16_t* kt = c->k_buf + (size_t)t * kv_dim + kv_off;
                for (int i = 0; i < head_dim; ++i) s += qh[i] * orc_f16_to_f32(kt[i]);
            }
            scores[t] = s * scale;
        }
        float mx = -INFINITY;
        for (int t = 0; t < seq_len; ++t) mx = fmaxf(mx, scores[t]);
        float sum = 0.0f;
        for (int t = 0; t < seq_len; ++t) { scores[t] = expf(scores[t] - mx); sum += scores[t]; }
        for (int t = 0; t < seq_len; ++t) scores[t] /= sum;
        float* dst = c->out + (size_t)h * head_dim;
        for (int i = 0; i < head_dim; ++i) dst[i] = 0.0f;
        for (int t = 0; t < seq_len; ++t) {
            float pr = scores[t];
            if (c->v32) {
                const float* vt = c->v32 + (size_t)t * kv_dim + kv_off;
                for (int i = 0; i < head_dim; ++i) dst[i] += pr * vt[i];
            } else {
                const uint16_t* vt = c->v_buf + (size_t)t * kv_dim + kv_off;
                for (int i = 0; i < head_dim; ++i) dst[i] += pr * orc_f16_to_f32(vt[i]);
            }
        }
    }
    free(scores);
}
void orc_attention_f16kv(const float* q, const uint16_t* k_buf, const uint16_t* v_buf, float* out,
                         int seq_len, int n_heads, int n_kv_heads, int head_dim) {
    orc_att_ctx c = { q, k_buf, v_buf, out, seq_len, n_heads, n_kv_heads, head_dim, 0, 0 };
    orc_parallel_for(n_heads, orc_att_range, &c, 0);
}
void orc_attention_f32kv(const float* q, const float* k_buf, const float* v_buf, float* out,
                         int seq_len, int n_heads, int n_kv_heads, int head_dim) {
    orc_att_ctx c = { q, 0, 0, out, seq_len, n_heads, n_kv_heads, head_dim, k_buf, v_buf };
    orc_parallel_for(n_heads, orc_att_range, &c, 0);
}

/* llm.rs:1065-1069 (the exact-logistic arm, not the AVX-512 rational approximation). */
void orc_swiglu_inplace(float* gate, const float* up, int n) {
    for (int i = 0; i < n; ++i) {
        float g = gate[i];
        float sig = 1.0f / (1.0f + expf(-g));
        gate[i] = (g * sig) * up[i];
    }
}

/* Dense half matrix [out_dim][in_dim] times f32 x, f64 accumulate (llm.rs:478-492). */
typedef struct { const uint16_t* w; const float* x; float* y; int in_dim; } orc_mvh_ctx;
static void orc_mvh_range(int r0, int r1, void* p) {
    orc_mvh_ctx* c = (orc_mvh_ctx*)p;
    for (int r = r0; r < r1; ++r) {
        const uint16_t* row = c->w + (size_t)r * c->in_dim;
        double acc = 0.0;
        for (int k = 0; k < c->in_dim; ++k) acc += (double)orc_f16_to_f32(row[k]) * (double)c->x[k];
        c->y[r] = (float)acc;
    }
}
void orc_matvec_f16(const uint16_t* w, const float* x, float* y, int out_dim, int in_dim) {
    orc_mvh_ctx c = { w, x, y, in_dim };
    orc_parallel_for(out_dim, orc_mvh_range, &c, 0);
}

/* First-maximum argmax, NaN never wins (crates/modgrad-gemma/src/rocm_gemma.rs:34-41). */
uint32_t orc_argmax(const float* v, int n) {
    int best = 0;
    float bv = -INFINITY;
    for (int i = 0; i < n; ++i)
        if (v[i] > bv) { bv = v[i]; best = i; }
    return (uint32_t)best;
}

typedef struct {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_seq;
    float rms_eps, rope_base;
} orc_decoder_cfg;

typedef struct {
    const uint8_t *wq, *wk, *wv, *wo, *wgate, *wup, *wdown; /* Q4_K, row-major blocks */
    const float *attn_norm, *ffn_norm;
    uint16_t *k_cache, *v_cache; /* [max_seq][n_kv_heads*head_dim] half */
} orc_decoder_layer;

/* One token at position `pos` (the number of positions already in the cache).
 * llm.rs:1177-1298.  matvec_mode: 0 scalar f32, 1 reference selector, 2 f64. */
static void forward_token_impl(const orc_decoder_cfg* cfg, const orc_decoder_layer* layers, float* const* k32,
                               float* const* v32, const uint16_t* embed, const uint16_t* lm_head,
                               const float* out_norm_w, int pos, uint32_t token, float* logits, int matvec_mode) {
    int D = cfg->d_model, H = cfg->n_heads, KVH = cfg->n_kv_heads, hd = cfg->head_dim;
    int q_dim = H * hd, kv_dim = KVH * hd, F = cfg->d_ff;
    float* hidden = (float*)malloc(sizeof(float) * D);
    float* cur = (float*)malloc(sizeof(float) * (D > q_dim ? D : q_dim));
    float* q = (float*)malloc(sizeof(float) * q_dim);
    float* k = (float*)malloc(sizeof(float) * kv_dim);
    float* v = (float*)malloc(sizeof(float) * kv_dim);
    float* att = (float*)malloc(sizeof(float) * q_dim);
    float* tmp = (float*)malloc(sizeof(float) * D);
    float* gate = (float*)malloc(sizeof(float) * F);
    float* up = (float*)malloc(sizeof(float) * F);

    for (int i = 0; i < D; ++i) hidden[i] = orc_f16_to_f32(embed[(size_t)token * D + i]);

    for (int l = 0; l < cfg->n_layers; ++l) {
        const orc_decoder_layer* L = &layers[l];
        orc_rms_norm(hidden, L->attn_norm, cur, D, cfg->rms_eps);
        orc_matvec_q4k(L->wq, cur, q, q_dim, D / 256, matvec_mode, 0);
        orc_matvec_q4k(L->wk, cur, k, kv_dim, D / 256, matvec_mode, 0);
        orc_matvec_q4k(L->wv, cur, v, kv_dim, D / 256, matvec_mode, 0);
        orc_apply_rope(q, pos, H, hd, cfg->rope_base);
        orc_apply_rope(k, pos, KVH, hd, cfg->rope_base);
        if (k32) {  /* the reference's own cache: f32, appended unrounded (llm.rs:1232-1234) */
            for (int i = 0; i < kv_dim; ++i) {
                k32[l][(size_t)pos * kv_dim + i] = k[i];
                v32[l][(size_t)pos * kv_dim + i] = v[i];
            }
            orc_attention_f32kv(q, k32[l], v32[l], att, pos + 1, H, KVH, hd);
        } else {
            for (int i = 0; i < kv_dim; ++i) {
                L->k_cache[(size_t)pos * kv_dim + i] = orc_f32_to_f16_rne(k[i]);
                L->v_cache[(size_t)pos * kv_dim + i] = orc_f32_to_f16_rne(v[i]);
            }
            orc_attention_f16kv(q, L->k_cache, L->v_cache, att, pos + 1, H, KVH, hd);
        }
        orc_matvec_q4k(L->wo, att, tmp, D, q_dim / 256, matvec_mode, 0);
        for (int i = 0; i < D; ++i) hidden[i] += tmp[i];
        orc_rms_norm(hidden, L->ffn_norm, cur, D, cfg->rms_eps);
        orc_matvec_q4k(L->wgate, cur, gate, F, D / 256, matvec_mode, 0);
        orc_matvec_q4k(L->wup, cur, up, F, D / 256, matvec_mode, 0);
        orc_swiglu_inplace(gate, up, F);
        orc_matvec_q4k(L->wdown, gate, tmp, D, F / 256, matvec_mode, 0);
        for (int i = 0; i < D; ++i) hidden[i] += tmp[i];
    }
    orc_rms_norm(hidden, out_norm_w, cur, D, cfg->rms_eps);
    orc_matvec_f16(lm_head, cur, logits, cfg->vocab, D);

    free(hidden); free(cur); free(q); free(k); free(v); free(att); free(tmp); free(gate); free(up);
}

/* ---- tensors of mixed types -----------------------------------------------------------------------
 * The reference's matvec dispatches on the tensor's GGML type (llm.rs:498-533: Q4_K fused dot, Q6_K its own
 * dot, every other quant dequantise-then-f64-dot) and its embedding lookup dequantises one row of a quantised
 * table (embed_token, llm.rs:898-918).  orc_forward_token_typed is forward_token (llm.rs:1177-1298) over such
 * tensors: type ids are GGML's (1 F16, 12 Q4_K, 13 Q5_K, 14 Q6_K); matvecs accumulate in f64 and round once,
 * as the f64 arms of the reference do. */
void orc_dequantize_row_q4_k(const uint8_t* data, float* out, size_t n_blocks);
void orc_dequantize_row_q5_k(const uint8_t* data, float* out, size_t n_blocks);
void orc_dequantize_row_q6_k(const uint8_t* data, float* out, size_t n_blocks);
void orc_matvec_kquant_f64(int kind, const uint8_t* w, const float* x, double* y, int out_dim, int bpr);

typedef struct {
    const void* w[7];   /* wq, wk, wv, wo, wgate, wup, wdown */
    int type[7];
    const float *attn_norm, *ffn_norm;
    uint16_t *k_cache, *v_cache; /* [max_seq][n_kv_heads*head_dim] half */
} orc_typed_layer;

static void typed_matvec(int type, const void* w, const float* x, float* y, int out_dim, int in_dim) {
    if (type == 12) { orc_matvec_q4k((const uint8_t*)w, x, y, out_dim, in_dim / 256, 2 /* f64 */, 0); return; }
    if (type == 1) { orc_matvec_f16((const uint16_t*)w, x, y, out_dim, in_dim); return; }
    double* t = (double*)malloc(sizeof(double) * (size_t)out_dim);
    orc_matvec_kquant_f64(type == 13 ? 5 : 6, (const uint8_t*)w, x, t, out_dim, in_dim / 256);
    for (int i = 0; i < out_dim; ++i) y[i] = (float)t[i];
    free(t);
}

void orc_forward_token_typed(const orc_decoder_cfg* cfg, const orc_typed_layer* layers, const void* embed, int embed_type,
                             const void* lm_head, int head_type, const float* out_norm_w, int pos, uint32_t token,
                             float* logits) {
    int D = cfg->d_model, H = cfg->n_heads, KVH = cfg->n_kv_heads, hd = cfg->head_dim;
    int q_dim = H * hd, kv_dim = KVH * hd, F = cfg->d_ff;
    float* hidden = (float*)malloc(sizeof(float) * D);
    float* cur = (float*)malloc(sizeof(float) * D);
    float* q = (float*)malloc(sizeof(float) * q_dim);
    float* k = (float*)malloc(sizeof(float) * kv_dim);
    float* v = (float*)malloc(sizeof(float) * kv_dim);
    float* att = (float*)malloc(sizeof(float) * q_dim);
    float* tmp = (float*)malloc(sizeof(float) * D);
    float* gate = (float*)malloc(sizeof(float) * F);
    float* up = (float*)malloc(sizeof(float) * F);

    if (embed_type == 1) {
        const uint16_t* e = (const uint16_t*)embed;
        for (int i = 0; i < D; ++i) hidden[i] = orc_f16_to_f32(e[(size_t)token * D + i]);
    } else {
        size_t bb = embed_type == 12 ? 144 : embed_type == 13 ? 176 : 210;
        const uint8_t* row = (const uint8_t*)embed + (size_t)token * (D / 256) * bb;
        if (embed_type == 12) orc_dequantize_row_q4_k(row, hidden, D / 256);
        else if (embed_type == 13) orc_dequantize_row_q5_k(row, hidden, D / 256);
        else orc_dequantize_row_q6_k(row, hidden, D / 256);
    }
    for (int l = 0; l < cfg->n_layers; ++l) {
        const orc_typed_layer* L = &layers[l];
        orc_rms_norm(hidden, L->attn_norm, cur, D, cfg->rms_eps);
        typed_matvec(L->type[0], L->w[0], cur, q, q_dim, D);
        typed_matvec(L->type[1], L->w[1], cur, k, kv_dim, D);
        typed_matvec(L->type[2], L->w[2], cur, v, kv_dim, D);
        orc_apply_rope(q, pos, H, hd, cfg->rope_base);
        orc_apply_rope(k, pos, KVH, hd, cfg->rope_base);
        for (int i = 0; i < kv_dim; ++i) {
            L->k_cache[(size_t)pos * kv_dim + i] = orc_f32_to_f16_rne(k[i]);
            L->v_cache[(size_t)pos * kv_dim + i] = orc_f32_to_f16_rne(v[i]);
        }
        orc_attention_f16kv(q, L->k_cache, L->v_cache, att, pos + 1, H, KVH, hd);
        typed_matvec(L->type[3], L->w[3], att, tmp, D, q_dim);
        for (int i = 0; i < D; ++i) hidden[i] += tmp[i];
        orc_rms_norm(hidden, L->ffn_norm, cur, D, cfg->rms_eps);
        typed_matvec(L->type[4], L->w[4], cur, gate, F, D);
        typed_matvec(L->type[5], L->w[5], cur, up, F, D);
        orc_swiglu_inplace(gate, up, F);
        typed_matvec(L->type[6], L->w[6], gate, tmp, D, F);
        for (int i = 0; i < D; ++i) hidden[i] += tmp[i];
    }
    orc_rms_norm(hidden, out_norm_w, cur, D, cfg->rms_eps);
    typed_matvec(head_type, lm_head, cur, logits, cfg->vocab, D);
    free(hidden); free(cur); free(q); free(k); free(v); free(att); free(tmp); free(gate); free(up);
}

/* Half-precision KV cache: the 7B-class configuration this build benchmarks. */
void orc_forward_token(const orc_decoder_cfg* cfg, const orc_decoder_layer* layers,
                       const uint16_t* embed, const uint16_t* lm_head, const float* out_norm_w,
                       int pos, uint32_t token, float* logits, int matvec_mode) {
    forward_token_impl(cfg, layers, 0, 0, embed, lm_head, out_norm_w, pos, token, logits, matvec_mode);
}
/* f32 KV cache, as the reference keeps it (llm.rs:305-310): k32[l] / v32[l] are [max_seq][kv_dim] floats;
 * the half caches inside `layers` are not touched. */
void orc_forward_token_f32kv(const orc_decoder_cfg* cfg, const orc_decoder_layer* layers, float* const* k32,
                             float* const* v32, const uint16_t* embed, const uint16_t* lm_head,
                             const float* out_norm_w, int pos, uint32_t token, float* logits, int matvec_mode) {
    forward_token_impl(cfg, layers, k32, v32, embed, lm_head, out_norm_w, pos, token, logits, matvec_mode);
}
