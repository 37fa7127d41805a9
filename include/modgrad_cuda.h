/*
 * modgrad_cuda.h — C ABI of libmodgrad_cuda.so, the sm_100a (B200) backend for modgrad's
 * GGUF Q4_K dequantize / matvec path.
 *
 * The entry points are the `extern "C"` launcher symbols modgrad's device crate already
 * binds for its HIP backend (crates/modgrad-device/src/backend/rocm.rs:433-563), with the
 * same names, argument order and types, so a `cuda` feature of that crate can bind them
 * unchanged.  Conventions, identical to the reference launchers:
 *   - every pointer is a DEVICE pointer owned by the caller; Q4_K weights are the
 *     unmodified 144-byte GGUF super-blocks, rows contiguous ([out_dim][bpr][144]);
 *   - the return value is the CUDA runtime's error code as int, 0 = success; a
 *     non-positive dimension or a null pointer returns cudaErrorInvalidValue (1);
 *   - launches are asynchronous, no synchronisation inside; the un-suffixed symbols use
 *     the default stream like the reference, the `_on_stream` variants take a
 *     cudaStream_t passed as void*;
 *   - weight pointers must be 16-byte aligned (GGUF aligns tensor data to 32 bytes and a
 *     row is a multiple of 144 = 9 x 16 bytes, so every row of an aligned tensor is).
 * There is no CPU fallback: without a CUDA device every launcher returns the runtime's
 * error code.
 */
#ifndef MODGRAD_CUDA_H
#define MODGRAD_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MG_Q4K_BLOCK_BYTES 144 /* crates/modgrad-device/src/kfd/gguf.rs:272 */
#define MG_Q4K_BLOCK_ELEMS 256 /* crates/modgrad-device/src/kfd/gguf.rs:275 */

/* ---- runtime shims: the CUDA counterparts of the hip* calls the Rust side binds --------
 * (crates/modgrad-device/src/backend/rocm.rs:57-85: hipMalloc, hipFree, hipMemcpy,
 *  hipDeviceSynchronize, hipGetErrorString, hipMemGetInfo, hipGetDeviceCount). */
int mg_get_device_count(int* count);
int mg_set_device(int device);
int mg_malloc(void** ptr, size_t bytes);
int mg_free(void* ptr);
int mg_memcpy_h2d(void* dst_dev, const void* src_host, size_t bytes);
int mg_memcpy_d2h(void* dst_host, const void* src_dev, size_t bytes);
int mg_memcpy_d2d(void* dst_dev, const void* src_dev, size_t bytes);
int mg_memset(void* dst_dev, int value, size_t bytes);
int mg_device_synchronize(void);
int mg_mem_get_info(size_t* free_bytes, size_t* total_bytes);
const char* mg_get_error_string(int code);
/* Library build identification: "modgrad_cuda <version> sm_100a". */
const char* mg_version(void);

/* ---- Q4_K -------------------------------------------------------------------------------- */

/* y[out_dim] = dequant(w_q4) . x, f32 accumulate, no bias.
 * Replaces launch_matvec_q4k, crates/modgrad-device/kernels/matvec_q4k.hip:111-124
 * (Rust declaration rocm.rs:457-463).  w_q4: out_dim*blocks_per_row*144 bytes;
 * x: blocks_per_row*256 f32; y: out_dim f32. */
int launch_matvec_q4k(const uint8_t* w_q4, const float* x, float* y, int out_dim, int blocks_per_row);
int launch_matvec_q4k_on_stream(const uint8_t* w_q4, const float* x, float* y, int out_dim,
                                int blocks_per_row, void* stream);

/* fp32_out[n_blocks*256] = dequant(q4k[n_blocks*144]) in the canonical ggml element order
 * of the host dequantiser (crates/modgrad-device/src/kfd/gguf.rs:364-404), bit-exact.
 * Replaces launch_dequant_q4k, crates/modgrad-device/kernels/dequant_q4k.hip:147-157
 * (Rust declaration rocm.rs:448-452; note the argument order). */
int launch_dequant_q4k(const uint8_t* q4k, int n_blocks, float* fp32_out);
int launch_dequant_q4k_on_stream(const uint8_t* q4k, int n_blocks, float* fp32_out, void* stream);

/* The int8-activation pair RocmGemma::qmatvec takes by default
 * (crates/modgrad-gemma/src/rocm_gemma.rs:283, :298-305): LOSSY (about 1 %), not the parity path.
 * launch_quantize_q8_1 replaces crates/modgrad-device/kernels/matvec_q4k_dp4a.hip:30-56 (Rust
 * declaration rocm.rs:477): per 32 activations xq = clamp(rint(x * 127/amax), -127, 127),
 * xd = amax/127, xsum = sum(xq) as f32; n / 32 sub-blocks (a shorter tail is ignored).
 * launch_matvec_q4k_dp4a replaces matvec_q4k_dp4a.hip:57-116 (rocm.rs:478-479):
 * y[row] = sum_s xd[s] * (d*sc[s]*<nibbles, xq> - dmin*m[s]*xsum[s]); a non-finite row sum is
 * stored as 0 (matvec_q4k_dp4a.hip:104-106).  xq: 16-byte aligned for the matvec. */
int launch_quantize_q8_1(const float* x, int8_t* xq, float* xd, float* xsum, int n);
int launch_quantize_q8_1_on_stream(const float* x, int8_t* xq, float* xd, float* xsum, int n, void* stream);
int launch_matvec_q4k_dp4a(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum, float* y,
                           int out_dim, int bpr);
int launch_matvec_q4k_dp4a_on_stream(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum,
                                     float* y, int out_dim, int bpr, void* stream);

/* The other two K-quant formats of real GGUF checkpoints, same launcher ABI as Q4_K:
 * launch_matvec_q5k replaces crates/modgrad-device/kernels/matvec_q5k.hip:112-121 (Rust declaration
 * rocm.rs:466-472; weight out_dim*blocks_per_row*176 bytes, 16-byte aligned), launch_matvec_q6k
 * replaces matvec_q6k.hip:85-94 (rocm.rs:481-484; 210-byte blocks, 2-byte aligned),
 * launch_matvec_q6k_dp4a replaces matvec_q6k_dp4a.hip:139-150 (rocm.rs:489-490; int8 activations
 * from launch_quantize_q8_1, lossy; xsum is unused: Q6_K has no per-block minimum).  f32 results
 * within 1e-5 of the output RMS of an f64-accumulated dot of the host dequantiser's weights
 * (crates/modgrad-device/src/kfd/gguf.rs:421-455, :458-484). */
int launch_matvec_q5k(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row);
int launch_matvec_q5k_on_stream(const uint8_t* w_q5, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream);
int launch_matvec_q6k(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row);
int launch_matvec_q6k_on_stream(const uint8_t* w_q6, const float* x, float* y, int out_dim, int blocks_per_row,
                                void* stream);
/* y[row] = (add ? add[row] : 0) + W[row] . x for a Q5_K (ggml_type 13) or Q6_K (14) weight: the matvec with
 * the residual add the decode loop puts behind it (crates/modgrad-gemma/src/rocm_gemma.rs:470-475, :497-500)
 * folded in; y may alias add.  x_kind 0: x is the f32 activation vector.  x_kind 1 (weight 4-byte aligned,
 * blocks_per_row * 832 bytes (+ 12 KiB for few or long rows) within one CTA's shared memory): x holds the limb
 * records of mg_q4k_x_to_limbs_on_stream / mg_swiglu_limbs_on_stream, multiplied with dp4a.
 * launch_matvec_q5k / launch_matvec_q6k take the same integer path under the same conditions (they convert x
 * themselves): the result then carries the activations' rounding to 23 bits of each 32-element sub-block's
 * largest element, like the Q4_K launchers'; otherwise a float kernel runs.  The kernels request their
 * first weights before they wait for the previous kernel of the stream: the weight must not be produced by
 * the kernel launched immediately before on the same stream. */
int mg_matvec_kquant_on_stream(int ggml_type, const uint8_t* w, const void* x, int x_kind, const float* add, float* y,
                               int out_dim, int blocks_per_row, void* stream);
/* y = W . rms_norm(x) for a Q5_K (13) or Q6_K (14) weight: the RMSNorm of the decode loop
 * (crates/modgrad-device/src/kfd/llm.rs:921-928, Plain) done by every CTA while it converts x, like
 * mg_rmsnorm_matvec_q4k_multi_on_stream for Q4_K.  Integer kernels only: cudaErrorInvalidValue when the weight
 * is not 4-byte aligned or a row's records exceed one CTA's shared memory. */
int mg_rmsnorm_matvec_kquant_on_stream(int ggml_type, const uint8_t* w, const float* x, const float* norm_w, float eps,
                                       float* y, int out_dim, int blocks_per_row, void* stream);
int launch_matvec_q6k_dp4a(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum, float* y,
                           int out_dim, int bpr);
int launch_matvec_q6k_dp4a_on_stream(const uint8_t* w, const int8_t* xq, const float* xd, const float* xsum,
                                     float* y, int out_dim, int bpr, void* stream);
/* Bulk dequantisation on the device, bit-exact against the host dequantisers (gguf.rs:421-455,
 * :458-484); the reference has no device kernel for these (it dequantises Q5_K / Q6_K rows on the
 * host, e.g. one embedding row per token, rocm_gemma.rs:316-323). */
int mg_dequant_q5k_on_stream(const uint8_t* q5k, int n_blocks, float* fp32_out, void* stream);
int mg_dequant_q6k_on_stream(const uint8_t* q6k, int n_blocks, float* fp32_out, void* stream);

/* y = dequant(w_q4) . x + bias, bias may be NULL.  The semantics of Op::Matvec{quant: Q4K}
 * (crates/modgrad-device/src/backend/op.rs:175-186) and of the KFD kernel's kernarg block
 * (crates/modgrad-device/src/kfd/dispatch_queue.rs:235-262); the HIP launcher has no bias. */
int mg_matvec_q4k_bias_on_stream(const uint8_t* w_q4, const float* x, const float* bias, float* y,
                                 int out_dim, int blocks_per_row, void* stream);

/* launch_matvec_q4k_on_stream for hosts that must not see the library allocate: an engine
 * that owns all device memory through its own arena, a process with a fixed memory budget, a
 * loop where cudaMalloc's device-wide synchronisation is unacceptable.  It has no counterpart
 * in the reference.  The converted activations go into a 104 KiB array built into the
 * library image (held by every GPU that loads the library) instead of run-time scratch; the
 * call performs no allocation of any kind.  blocks_per_row <= 128 (rows of up to 32768
 * weights), otherwise cudaErrorInvalidValue.  The first call on a device resolves the
 * array's device address and should precede any stream capture.  All calls share the array:
 * calls that overlap on the GPU race, so keep them ordered on one stream. */
int launch_matvec_q4k_noalloc_on_stream(const uint8_t* w_q4, const float* x, float* y, int out_dim,
                                        int blocks_per_row, void* stream);

/* The matvec in two steps, for callers that multiply several matrices by one activation
 * vector (q/k/v, gate/up): convert x once into block-fixed-point limb records, then run any
 * number of matvecs on the records.  launch_matvec_q4k does exactly these two steps with an
 * internal per-stream workspace.  No counterpart in the reference (its int8 pair
 * launch_quantize_q8_1 / launch_matvec_q4k_dp4a, matvec_q4k_dp4a.hip:51,109, is the nearest
 * shape, but lossy); this pair keeps 23 bits per activation and meets the f32 tolerance.
 * k % 256 == 0; `records` is device memory of mg_q4k_limb_record_bytes(k) bytes, 16-byte
 * aligned; blocks_per_row <= 135 on this path. */
size_t mg_q4k_limb_record_bytes(int k);
/* The library's kernels are chained with programmatic dependent launch: each lets its successor
 * launch early and waits for its predecessor's completion before it reads.  A kernel of another
 * library queued behind them (an NCCL collective) may start on that early trigger and read
 * results that are not written yet.  mg_pdl_early_trigger(0) makes the kernels whose output such
 * a kernel would consume (the Q4_K matvecs, the activation conversion / SwiGLU, the attention
 * merge) hold their trigger until they have finished; mg_pdl_early_trigger(1) restores the
 * default.  The setting belongs to the calling host thread and applies to launches made (or
 * captured) afterwards; the previous setting is returned. */
int mg_pdl_early_trigger(int enabled);

/* launch_matvec_q4k / mg_matvec_q4k_bias_on_stream start SPECULATIVELY: the kernel converts x and
 * computes while the kernel queued before it on the stream may still run, and publishes y only
 * after that kernel has completed and x has been re-checked against what was converted (results
 * are exact either way; an x that changed in between costs a second pass).  The launcher already
 * skips the speculation when x or the bias is the output of the previous matvec it queued on the
 * same stream.  mg_matvec_q4k_speculation(0) switches it off for the process (also
 * MODGRAD_Q4K_SPECULATE=0 in the environment), (1) on; the previous setting is returned.  Weights
 * must not be written by the kernel queued directly before a matvec: they are prefetched early. */
int mg_matvec_q4k_speculation(int enabled);

/* Health counter of the GEMV kernels on the current device: warps that gave up waiting for a
 * weight copy (every wait in the kernels is bounded).  0 in a healthy process; non-zero means
 * rows of some result were left unwritten.  Synchronises the device; negative = -(CUDA error). */
long long mg_matvec_q4k_timeouts(void);
int mg_q4k_x_to_limbs_on_stream(const float* x, int k, void* records, void* stream);
int mg_matvec_q4k_limbs_on_stream(const uint8_t* w_q4, const void* records, const float* bias, float* y,
                                  int out_dim, int blocks_per_row, void* stream);

/* Up to three matrices times ONE activation vector in one launch (q/k/v, gate/up share their
 * input): y[i] = dequant(w_q4[i]) . x + addend[i].  x_is_records = 0: x is f32 and
 * blocks_per_row <= 32 (converted inside the kernel); 1: x is a limb-record table.
 * addend may be NULL, entries may be NULL, and an entry may alias the matching y (in-place
 * residual add, as the reference's launch_residual_add after a matvec).  The reference
 * issues one launch per matrix (RocmGemma::layer, crates/modgrad-gemma/src/rocm_gemma.rs:440-481). */
int mg_matvec_q4k_multi_on_stream(int n_mats, const uint8_t* const* w_q4, const void* x, int x_is_records,
                                  const float* const* addend, float* const* y, const int* out_dims,
                                  int blocks_per_row, void* stream);
/* The same with RMSNorm fused in front of the matvecs (llm.rs:921-928, Plain): x is f32,
 * blocks_per_row <= 32. */
int mg_rmsnorm_matvec_q4k_multi_on_stream(int n_mats, const uint8_t* const* w_q4, const float* x,
                                          const float* norm_weight, float eps, const float* const* addend,
                                          float* const* y, const int* out_dims, int blocks_per_row, void* stream);
/* Limb records (and, if act_out != NULL, the f32 values) of silu(gate) * up: the SwiGLU
 * activation (crates/modgrad-device/src/kfd/llm.rs:1065-1069) produced directly in the form
 * the down projection consumes.  n % 64 == 0 (whole records). */
int mg_swiglu_limbs_on_stream(const float* gate, const float* up, float* act_out, int n, void* records,
                              void* stream);

/* ---- multi-sequence dequant-GEMM on the tensor cores (tcgen05 + TMEM), M <= 64 per call --------
 * Y[m][out_dim] = X[m][K] . dequant(W)^T: the batched contract of Linear::forward_batched
 * (crates/modgrad-device/src/backend/tensor.rs:1839-1853) for Q4_K weights; no reference kernel
 * exists for it (compared with M independent CPU matvecs on the same f32 X, 1e-5 of the output
 * rms).  X is f32 [m_rows][K]; each row is carried as two half-precision limbs after a power-of-two
 * scale (22 significant bits relative to the row's largest magnitude).  Exactly m_rows * out_dim
 * floats of y are written.
 * `scratch`: mg_matmul_q4k_scratch_bytes(m_rows, blocks_per_row) bytes of device memory,
 * 1024-byte aligned.  mg_matmul_q4k_status (after a synchronise) returns 702 if a bounded
 * wait inside the kernel expired, else 0. */
size_t mg_matmul_q4k_scratch_bytes(int m_rows, int blocks_per_row);
int launch_matmul_q4k_on_stream(const uint8_t* w_q4, const float* x, float* y, int m_rows, int out_dim,
                                int blocks_per_row, void* scratch, void* stream);
int mg_matmul_q4k_status(const void* scratch, int m_rows, int blocks_per_row);

/* ---- decode-loop glue: the launchers of crates/modgrad-device/kernels/rms_norm.hip:79-94 and
 * transformer_ops.hip:15-100 (Rust declarations rocm.rs:433-446, :501-507), same names and
 * argument order; launch_swiglu is new (the reference GPU engine has GeGLU only). ------------ */
int launch_rms_norm(const float* x, const float* weight, float* y, int n, int hidden, float eps);
int launch_rms_norm_on_stream(const float* x, const float* weight, float* y, int n, int hidden, float eps,
                              void* stream);
int launch_residual_add(float* h, const float* x, int n);
int launch_residual_add_on_stream(float* h, const float* x, int n, void* stream);
int launch_scale(float* h, float s, int n);
int launch_scale_on_stream(float* h, float s, int n, void* stream);
int launch_geglu(const float* gate, const float* up, float* out, int n);
int launch_geglu_on_stream(const float* gate, const float* up, float* out, int n, void* stream);
int launch_swiglu(const float* gate, const float* up, float* out, int n);
int launch_swiglu_on_stream(const float* gate, const float* up, float* out, int n, void* stream);
int launch_softcap(float* y, float cap, int n);
int launch_softcap_on_stream(float* y, float cap, int n, void* stream);
int launch_rope_neox(float* data, int pos, int n_heads, int head_dim, float base, const float* freq_factors);
int launch_rope_neox_on_stream(float* data, int pos, int n_heads, int head_dim, float base,
                               const float* freq_factors, void* stream);
int launch_copy(float* dst, const float* src, int n);
int launch_copy_on_stream(float* dst, const float* src, int n, void* stream);

/* One-query grouped-query attention over an f32 cache [seq][kv_dim]: the launchers of
 * crates/modgrad-device/kernels/sdpa_decode.hip:77-89 and sdpa_decode_flash.hip:102-115
 * (positions win_start .. seq_len-1 take part). */
int launch_sdpa_decode(const float* q, const float* k_cache, const float* v_cache, float* out, int n_heads,
                       int n_kv_heads, int head_dim, int seq_len, int kv_dim, float scale, int win_start);
int launch_sdpa_decode_flash(const float* q, const float* k_cache, const float* v_cache, float* out, int n_heads,
                             int n_kv_heads, int head_dim, int seq_len, int kv_dim, float scale, int win_start);
int launch_sdpa_decode_on_stream(const float* q, const float* k_cache, const float* v_cache, float* out,
                                 int n_heads, int n_kv_heads, int head_dim, int seq_len, int kv_dim, float scale,
                                 int win_start, void* stream);
int launch_sdpa_decode_flash_on_stream(const float* q, const float* k_cache, const float* v_cache, float* out,
                                       int n_heads, int n_kv_heads, int head_dim, int seq_len, int kv_dim, float scale,
                                       int win_start, void* stream);

/* The same attention over a HALF cache, split over the sequence (the 7B-class decoder keeps
 * K/V in half precision; the reference keeps f32, rocm_gemma.rs:256-261).  `scratch` holds the
 * per-split partial results: mg_sdpa_f16kv_scratch_bytes(...) bytes of device memory.
 * seq_len_dev / pos_dev: device integers read by the kernels (NULL -> the by-value argument),
 * so that one captured graph serves every step.  head_dim 64, 128 or 256. */
size_t mg_sdpa_f16kv_scratch_bytes(int n_heads, int head_dim, int n_splits);
int mg_sdpa_decode_f16kv_on_stream(const float* q, const void* k_cache, const void* v_cache, float* out,
                                   int n_heads, int n_kv_heads, int head_dim, int seq_len,
                                   const int* seq_len_dev, float scale, void* scratch, int n_splits,
                                   void* stream);
/* NEOX RoPE on q and k in place (llm.rs:944-982, no frequency scaling), then k and v stored
 * as halves at position pos of the cache (llm.rs:1232-1234 appends f32).  freq_table: device
 * array of head_dim/2 precomputed base^(-2i/head_dim), or NULL. */
int mg_rope_kv_append_f16_on_stream(float* q, float* k, const float* v, void* k_cache, void* v_cache, int pos,
                                    const int* pos_dev, int n_heads, int n_kv_heads, int head_dim, float base,
                                    const float* freq_table, void* stream);

/* Both steps and the merge of the split results in ONE launch: q, k_new, v_new as the projections
 * left them (f32, not rotated, not modified); k_new is rotated, both are rounded to half, appended
 * at position pos (or *pos_dev) and used; the output is the attention over positions 0 .. pos
 * (rocm_gemma.rs:429-489 issues rope, cache write and attention as separate launches).
 * `scratch`: mg_sdpa_rope_f16kv_scratch_bytes(...) bytes, ZEROED ONCE by the caller after allocation
 * (ticket counters that every launch leaves at zero).  n_splits <= 160. */
size_t mg_sdpa_rope_f16kv_scratch_bytes(int n_heads, int n_kv_heads, int head_dim, int n_splits);
int mg_sdpa_rope_decode_f16kv_on_stream(const float* q, const float* k_new, const float* v_new, void* k_cache,
                                        void* v_cache, float* out, int n_heads, int n_kv_heads, int head_dim, int pos,
                                        const int* pos_dev, float scale, float rope_base, const float* freq_table,
                                        void* scratch, int n_splits, void* stream);

/* Dense half pieces: y = W_half[out_dim][in_dim] . x (the dense-matrix arm of the reference
 * matvec, llm.rs:478-492; in_dim % 256 == 0, <= 12288), embedding row lookup (llm.rs:898-918)
 * and first-maximum arg-max where NaN never wins (rocm_gemma.rs:34-41; scratch: 2048 bytes). */
int mg_matvec_f16_on_stream(const void* w_f16, const float* x, float* y, int out_dim, int in_dim, void* stream);
/* One row of a Q4_K (12) / Q5_K (13) / Q6_K (14) embedding table, dequantised bit-exactly as the bulk
 * dequantisers do (the reference dequantises the row on the host: rocm_gemma.rs:316-323). */
int mg_embed_kquant_on_stream(const void* table, int ggml_type, int token, const int* token_dev, float* out, int d_model,
                              int vocab, void* stream);
int mg_embed_f16_on_stream(const void* table_f16, int token, const int* token_dev, float* out, int d_model,
                           int vocab, void* stream);
int mg_argmax_on_stream(const float* v, int n, int* out_token_dev, void* scratch, int* history, int* step_dev,
                        void* stream);

/* ---- resident decoder engine: RocmGemma::{load, layer, forward_token, generate}
 * (crates/modgrad-gemma/src/rocm_gemma.rs:94, :429, :312, :372) with the arithmetic of
 * kfd::llm::forward_token (crates/modgrad-device/src/kfd/llm.rs:1177-1298). ------------------- */
typedef struct mg_decoder_config {
    int n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, max_seq;
    float rms_eps, rope_base;
} mg_decoder_config;
enum {
    MG_W_Q = 0, MG_W_K, MG_W_V, MG_W_O, MG_W_GATE, MG_W_UP, MG_W_DOWN, /* Q4_K, per layer */
    MG_W_ATTN_NORM, MG_W_FFN_NORM,                                      /* f32, per layer */
    MG_W_EMBED = 100, MG_W_LM_HEAD, MG_W_OUT_NORM                       /* half, half, f32 */
};
typedef struct mg_decoder mg_decoder;
int mg_decoder_create(const mg_decoder_config* cfg, mg_decoder** out);
/* Engine whose tensors carry their own GGUF types, as real checkpoints mix them: the per-tensor dispatch of
 * RocmGemma::qmatvec (crates/modgrad-gemma/src/rocm_gemma.rs:291-309).  proj_types: n_layers * 7 type ids in
 * the order q, k, v, o, gate, up, down, each 12 (Q4_K), 13 (Q5_K) or 14 (Q6_K); embed_type / head_type: 1 (F16)
 * or one of the three.  mg_decoder_upload then expects the byte size of each tensor's type (of this rank's
 * rows); mg_decoder_weight_type reports the type (0 for the f32 norms).  All-default types build the engine of
 * mg_decoder_create[_sharded].  The _sharded form splits rows over the ranks exactly as
 * mg_decoder_create_sharded does; a typed engine ends its Q4_K / attention / SwiGLU kernels with the flag-handshake
 * exchange and puts a peer-store gather kernel behind a Q5_K / Q6_K matvec, or uses NCCL (the stamped exchanges
 * belong to the all-Q4_K engine). */
int mg_decoder_create_typed(const mg_decoder_config* cfg, const int* proj_types, int embed_type, int head_type,
                            mg_decoder** out);
int mg_decoder_create_typed_sharded(const mg_decoder_config* cfg, const int* proj_types, int embed_type, int head_type,
                                    int rank, int world, const void* nccl_id128, mg_decoder** out);
int mg_decoder_weight_type(const mg_decoder* d, int layer, int which);
/* Row-sharded engine, one process per GPU (no counterpart in the reference, which has no
 * multi-device code): rank r of `world` holds the rows of its query heads, of its slice of
 * the FFN, the hidden state and the vocabulary, and uploads / prefills only those slices;
 * output slices are all-gathered with NCCL inside the per-token graph.  nccl_id128: the
 * 128-byte id made by mg_nccl_unique_id on rank 0 (NULL when world == 1).
 * mg_decoder_shard_ranges fills {h0, h1, kv0, kv1, d_model/world, d_ff/world, vocab/world,
 * heads per KV head} and rejects splits the engine cannot run. */
int mg_nccl_unique_id(void* out128);
int mg_decoder_shard_ranges(const mg_decoder_config* cfg, int rank, int world, int* out8);
int mg_decoder_create_sharded(const mg_decoder_config* cfg, int rank, int world, const void* nccl_id128,
                              mg_decoder** out);
void mg_decoder_destroy(mg_decoder* d);
const char* mg_decoder_last_error(const mg_decoder* d);
int mg_decoder_upload(mg_decoder* d, int layer, int which, const void* host, size_t bytes);
int mg_decoder_set_kv(mg_decoder* d, int layer, const void* k_f16, const void* v_f16, int n_pos);
int mg_decoder_set_position(mg_decoder* d, int pos);
int mg_decoder_forward_token(mg_decoder* d, int token, float* logits_host, int* next_token);
int mg_decoder_generate(mg_decoder* d, int first_token, int n_tokens, int* out_tokens, float* device_ms);
void* mg_decoder_buffer(mg_decoder* d, int which);
int mg_decoder_kernels_per_token(const mg_decoder* d);
/* Sharded engines: 0 = NCCL collectives, 1 = one peer-store gather kernel per collective,
 * 2 = the all-gathers are fused into the producing kernels (default when every rank can map its
 * peers; MODGRAD_DECODER_GATHER=nccl|peer|fused overrides); -1 on a single GPU. */
int mg_decoder_gather_mode(const mg_decoder* d);
/* Polls a bounded wait of the engine's peer exchanges makes before it gives up and the token fails
 * with cudaErrorLaunchTimeout (default 1 << 22, seconds); call before the first token. */
int mg_decoder_set_exchange_spin_limit(mg_decoder* d, unsigned polls);

/* The single device allocation that holds every weight tensor of the engine (the reference packs
 * its quantised tensors the same way, crates/modgrad-gemma/src/rocm_gemma.rs:206-224) and the
 * device pointer of one tensor inside it (`which` as for mg_decoder_upload). */
void* mg_decoder_weight_arena(mg_decoder* d, size_t* bytes);
void* mg_decoder_weight_ptr(mg_decoder* d, int layer, int which);

/* ---- Q4_K residency: LinearResidentQuantized (crates/modgrad-compute/src/neuron.rs:866-1250) ------
 * The weight lives on the host as Q4_K super-blocks; device buffers exist between ensure_resident
 * and evict.  Default forward: the matvec runs on the Q4_K bytes themselves (launch_matvec_q4k +
 * bias; 0.5625 bytes per weight).  mg_linear_q4k_set_expanded(l, 1) selects the reference's
 * behaviour: dequantise once per residency into an fp32 copy (Op::DequantQ4KResident) and run a
 * dense fp32 matvec (7x the memory and traffic).  from_* allocate nothing on the device; an evict
 * followed by a forward reproduces the previous output bit for bit.  -4: bad arguments or
 * in_dim % 256 != 0; positive: CUDA error codes.  mg_quantize_row_q4_k is the host quantiser
 * (canonical ggml element order, the one dequantize_row_q4_k reads, gguf.rs:364-404). */
typedef struct mg_linear_q4k mg_linear_q4k;
int mg_quantize_row_q4_k(const float* x, uint8_t* out, size_t n);
int mg_linear_q4k_from_f32(const float* weight, const float* bias, int in_dim, int out_dim, mg_linear_q4k** out);
int mg_linear_q4k_from_blocks(const uint8_t* q4k, const float* bias, int in_dim, int out_dim, mg_linear_q4k** out);
void mg_linear_q4k_destroy(mg_linear_q4k* l);
int mg_linear_q4k_set_expanded(mg_linear_q4k* l, int expanded);
int mg_linear_q4k_is_resident(const mg_linear_q4k* l);
size_t mg_linear_q4k_host_size_bytes(const mg_linear_q4k* l);
size_t mg_linear_q4k_device_size_bytes(const mg_linear_q4k* l);
const uint8_t* mg_linear_q4k_host_blocks(const mg_linear_q4k* l, size_t* bytes);
int mg_linear_q4k_ensure_resident(mg_linear_q4k* l, void* stream);
void mg_linear_q4k_evict(mg_linear_q4k* l);
int mg_linear_q4k_forward(mg_linear_q4k* l, const float* x_dev, float* out_dev, int auto_evict, void* stream);
/* Dense fp32 matvec y = W[out_dim][in_dim] . x + bias (bias may be NULL): what the expanded mode
 * dispatches (ops::matvec_resident -> hipblasSgemv in the reference, neuron.rs:1093-1101). */
int mg_matvec_f32_on_stream(const float* w, const float* x, const float* bias, float* y, int out_dim, int in_dim,
                            void* stream);

/* ---- GGUF: header parser and checkpoint loader ---------------------------------------------------
 * GgufFile::parse / TensorInfo / MetaValue / GgmlType::block_size of the reference
 * (crates/modgrad-device/src/kfd/gguf.rs:11-234, :665-694): GGUF v2 and v3, little endian,
 * metadata key/values of the thirteen value types (arrays nest), tensor infos, data section
 * aligned to 32 bytes.  Only the header is decoded; the file is memory-mapped and tensor bytes are
 * addressed by offset.  Return codes: 0, or -4 (Runtime) with the message in mg_gguf_last_error()
 * ("not a GGUF file", "unsupported GGUF version N", "string too long", "unknown GGUF value type N",
 * a short read).  Needs no GPU. */
typedef struct mg_gguf mg_gguf;
int mg_gguf_open(const char* path, mg_gguf** out);
int mg_gguf_parse_memory(const void* data, size_t bytes, mg_gguf** out);
void mg_gguf_close(mg_gguf* g);
const char* mg_gguf_last_error(void);
int mg_gguf_version(const mg_gguf* g);
size_t mg_gguf_data_offset(const mg_gguf* g);
int mg_gguf_n_tensors(const mg_gguf* g);
int mg_gguf_n_meta(const mg_gguf* g);
int mg_gguf_find_tensor(const mg_gguf* g, const char* name);
/* dims4: dims[0] (the row length, in_dim) .. dims[3], 1 where absent; file_offset = data_offset + the
 * tensor's offset (GgufFile::tensor_file_offset, gguf.rs:232-234). */
int mg_gguf_tensor(const mg_gguf* g, int index, const char** name, int* n_dims, uint64_t* dims4, uint32_t* dtype,
                   uint64_t* file_offset, uint64_t* data_bytes);
const void* mg_gguf_tensor_data(const mg_gguf* g, int index);
int mg_gguf_meta_u32(const mg_gguf* g, const char* key, uint32_t* out); /* U32, I32, U64: gguf.rs:117-124 */
int mg_gguf_meta_f32(const mg_gguf* g, const char* key, float* out);    /* F32, F64: gguf.rs:125-131 */
const char* mg_gguf_meta_str(const mg_gguf* g, const char* key);
long long mg_gguf_meta_array_len(const mg_gguf* g, const char* key);
void mg_gguf_block_size(uint32_t dtype, size_t* block_bytes, size_t* block_elems); /* gguf.rs:48-67 */

/* LlmConfig::populate_from_gguf (crates/modgrad-device/src/kfd/llm.rs:145-180) and
 * LlmWeights::load_from_gguf / RocmGemma::load (llm.rs:233-296; rocm_gemma.rs:94-262): engine
 * configuration from the metadata, then every tensor uploaded verbatim from the mapped file into
 * the engine's single weight allocation (rank `rank` of `world` uploads its row ranges only),
 * behind a VRAM guard: weights + KV cache + activations plus a margin (512 MiB,
 * MODGRAD_VRAM_MARGIN_MB) must fit the free device memory, else cudaErrorMemoryAllocation (2).
 * Tensors: blk.N.{attn_q,attn_k,attn_v,attn_output,ffn_gate,ffn_up,ffn_down}.weight Q4_K,
 * blk.N.{attn_norm,ffn_norm}.weight and output_norm.weight F32, token_embd.weight and
 * output.weight F16 (LM head tied to the embedding when output.weight is absent, llm.rs:1281-1286).
 * -4 with mg_decoder_load_error() for a malformed file, a missing tensor, a wrong shape or an
 * unsupported tensor type. */
int mg_decoder_config_from_gguf(const mg_gguf* g, int max_seq, mg_decoder_config* out);
int mg_decoder_load_gguf(const char* path, int max_seq, int rank, int world, const void* nccl_id128,
                         mg_decoder** out);
const char* mg_decoder_load_error(void);

/* ---- all-gather by direct peer stores over NVLink, fused into the producing kernel -----------
 * For row-sharded engines (one process per GPU of one box).  Every rank owns an `arena` of
 * device memory that the other ranks map with CUDA IPC; all ranks lay it out identically, the
 * first mg_peer_arena_offset() bytes hold flags.  After mg_peer_fuse_next(x, site) the next
 * supporting launch from this host thread — launch_matvec_q4k[_on_stream] /
 * mg_matvec_q4k_*_on_stream with ONE matrix and y inside the arena, mg_swiglu_limbs_on_stream,
 * mg_sdpa_decode_f16kv_on_stream — stores every result into all peers' arenas as well and ends
 * with a handshake (a per-(site, source) epoch flag on every peer, bounded wait for the peers'):
 * when the kernel has finished, the whole gathered buffer is in local memory.  Rules: every
 * rank issues the exchanges of a site in the same order; consecutive exchanges use different
 * buffers (a rank may run one exchange ahead of a peer).  No counterpart in the reference (its
 * engine is single-GPU).  Setup: create on every rank, exchange the 64-byte handles through
 * any host channel, open.  mg_peer_exchange_status: 0, or 1 + the site whose wait ran out. */
typedef struct mg_peer_exchange mg_peer_exchange;
int mg_peer_exchange_create(size_t bytes, int rank, int world, void* ipc_handle_out64, mg_peer_exchange** out);
int mg_peer_exchange_open(mg_peer_exchange* x, const void* handles_world_x_64);
void* mg_peer_arena(mg_peer_exchange* x);
size_t mg_peer_arena_offset(void);
int mg_peer_fuse_next(mg_peer_exchange* x, int site);
int mg_peer_gather_on_stream(mg_peer_exchange* x, int site, size_t offset, size_t my_off, size_t my_bytes,
                             void* stream);
int mg_peer_exchange_status(mg_peer_exchange* x);
int mg_peer_exchange_set_spin_limit(mg_peer_exchange* x, unsigned polls);
void mg_peer_exchange_destroy(mg_peer_exchange* x);

/* ---- the operator/plugin tier above the launchers ------------------------------------------
 * A CUDA `Backend` (crates/modgrad-device/src/backend/mod.rs:148-176) that claims the two
 * Q4_K ops no reference backend claims today.  Return codes: 0 ok; -1 Unsupported,
 * -2 OutOfMemory, -3 DeviceLost, -4 Runtime (BackendError, backend/mod.rs:109-123);
 * mg_backend_last_error gives the message.  `quant`: 0 = F32, 1 = Q4K (op.rs:22-29). */
typedef struct mg_backend mg_backend;
int mg_backend_create(int device, mg_backend** out); /* -1 when no CUDA device answers */
void mg_backend_destroy(mg_backend* b);
const char* mg_backend_name(const mg_backend* b); /* "cuda" */
const char* mg_backend_device_info(mg_backend* b);
const char* mg_backend_last_error(const mg_backend* b);
/* Op::Matvec with HOST slices (op.rs:178-186), blocking like Backend::dispatch: uploads x
 * (and bias), keeps the weight bytes resident keyed by their host address until
 * mg_backend_invalidate_cache, launches, downloads `out`.  bias_len 0 = no bias. */
int mg_backend_supports_matvec(const mg_backend* b, const float* x, size_t x_len, const void* weight,
                               size_t weight_bytes, const float* bias, size_t bias_len, float* out,
                               size_t out_len, size_t out_dim, size_t in_dim, int quant);
int mg_backend_dispatch_matvec(mg_backend* b, const float* x, size_t x_len, const void* weight,
                               size_t weight_bytes, const float* bias, size_t bias_len, float* out,
                               size_t out_len, size_t out_dim, size_t in_dim, int quant);
/* Op::DequantQ4KResident (op.rs:479-483; facade backend/ops.rs:531-539): device pointers. */
int mg_backend_supports_dequant_q4k_resident(const mg_backend* b, const uint8_t* q4k_dev,
                                             float* fp32_dev, size_t n_blocks);
int mg_backend_dispatch_dequant_q4k_resident(mg_backend* b, const uint8_t* q4k_dev, float* fp32_dev,
                                             size_t n_blocks);
void mg_backend_invalidate_cache(mg_backend* b); /* Backend::invalidate_cache, mod.rs:172-176 */
size_t mg_backend_cached_weights(const mg_backend* b);

/* HipBuffer::matvec_q4k (crates/modgrad-device/src/backend/rocm.rs:681-710): resident weight,
 * HOST x in, HOST y out; upload, launch, one sync, download.  CUDA error code. */
int mg_buffer_matvec_q4k(const uint8_t* w_dev, size_t w_bytes, const float* x_host, float* y_host,
                         size_t out_dim, size_t bpr);
/* HipBuffer::matvec_q4k_into (rocm.rs:717-738): device x / y, synchronises before returning. */
int mg_buffer_matvec_q4k_into(const uint8_t* w_dev, const float* x_dev, float* y_dev, size_t out_dim,
                              size_t bpr);

#ifdef __cplusplus
}
#endif
#endif /* MODGRAD_CUDA_H */
