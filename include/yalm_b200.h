/* yalm_b200 — C ABI of the B200-native token-generation forward pass.
 *
 * This is the drop-in boundary for xiaguan/yalm's `-d cuda` path.  Three layers:
 *
 *  (1) the seven memory/stream helpers the reference already exports from src/infer.cu and declares
 *      in src/model.h:33-39 — same names, same meaning;
 *  (2) one entry point per fused device op (device pointers + sizes + stream, returns the
 *      cudaError_t as int) — what replaces the kernel launches inside Block::_block_cuda
 *      (src/infer.cu:699-888) and Model::_forward_cuda_build_graph (src/infer.cu:1041-1128);
 *  (3) host-pointer test entry points with the semantics of the reference's "exposed for tests"
 *      functions matmul_cuda / mha_cuda / ffn_cuda (src/model.h:353-384, src/infer.cu:890-1007),
 *      and opaque-handle wrappers over Model / InferenceState (src/model.h:84-327) for bindings
 *      that cannot consume C++ classes (ctypes, cgo, JNI).
 *
 * Error convention: layer (1) keeps the reference's (CUDA failure -> message on stderr + abort(),
 * src/infer.cu:13-31).  Layers (2)/(3) return 0 on success, a cudaError_t or a negative YALM_E*
 * code otherwise, and never fall back to a CPU path.
 */
#ifndef YALM_B200_H
#define YALM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Weight element types; values are the reference's DType enum (src/codec.h:15-25). */
#define YALM_F32 0
#define YALM_F16 1
#define YALM_BF16 2 /* layered architectures (checkpoint directories); the .yalm kernels do not take it */
#define YALM_F8E5M2 3 /* parsed, but no arithmetic exists for it: rejected */
#define YALM_F8E4M3 4 /* net-new: e4m3 codes + one fp32 scale per output row */

#define YALM_ACT_GELU 0 /* ActivationType, src/model.h:14-17 */
#define YALM_ACT_SILU 1

#define YALM_MODE_HYDRATE 0 /* InferenceMode, src/model.h:28-31 */
#define YALM_MODE_LOGITS 1

#define YALM_EINVAL (-1)  /* unsupported shape / dtype / null pointer */
#define YALM_ENOGPU (-2)  /* no CUDA device: there is deliberately no CPU fallback */
#define YALM_EFORMAT (-3) /* bad .yalm container */

typedef void *yalm_stream_t; /* cudaStream_t */

/* ---- (1) reference C ABI, src/model.h:33-39 / src/infer.cu:59-90 ------------------------------ */
void *upload_cuda(void *host, size_t size);            /* cudaMalloc + H2D, returns device pointer */
void *download_cuda_raw(void *device, size_t size);    /* C-clean form of download_cuda (the reference's takes a std::string) */
void register_cuda_host(void *host, size_t size);
void free_cuda(void *device);
void unregister_cuda_host(void *host);
void set_cuda_device(int device);
void init_cuda_stream(yalm_stream_t *stream);

/* ---- (2) fused device ops ---------------------------------------------------------------------
 * Decode control block `ctl` (device, 8 ints): [0] token [1] pos [2] kv_sink [3] kv_pos [4] kv_len
 * [5] step counter [6..7] reserved.  Keeping pos/kv_* in device memory is what lets one CUDA graph be
 * replayed for every token with zero per-token node updates (the reference patches 129-161 kernel
 * nodes per token, src/infer.cu:1146-1163).                                                        */
#define YALM_CTL_INTS 8

/* x = float(E[token,:]) (src/infer.cu:622-640) and derive the KV ring position from pos
 * (src/infer.cu:1081-1083: kv_sink/kv_pos/kv_len with KV_SINKS = 2) into ctl.  token >= 0: token and
 * pos are taken from the arguments (copied at launch, so back-to-back calls never race); token < 0:
 * ctl[0..1] are taken as already set on the device (by yalm_argmax_advance). */
int yalm_embed(float *x, const void *table, const float *row_scale, int dim, int dtype, int *ctl, int token,
               int pos, int max_seq_len, yalm_stream_t s);

/* KV cache layout on the device: HEAD-MAJOR fp16 ring, (n_kv_heads, max_seq_len, head_dim) — one contiguous
 * slab per KV head, so a run of rows of one head is one 1-D bulk (TMA) copy.  The reference keeps
 * (max_seq_len, n_kv_heads, head_dim) (src/model.cpp:171-172); the host-pointer test entry yalm_mha_host and
 * the yalm_state_read taps take / return the reference layout and convert. */

/* rmsnorm -> q,k,v GEMVs -> clip -> RoPE(q,k) -> fp16 KV append at ctl.kv_pos -> sink re-rotation.
 * Replaces rmsnorm + fused_qkv_matmul_clip + fused_rope_and_cache_update + rotate_sink_tokens
 * (src/infer.cu:526-539, 291-336, 642-697).  Weights are (out,in) row-major, y = W x. */
int yalm_qkv_rope_append(float *q_out, uint16_t *key_cache, uint16_t *value_cache, const float *x,
                         const float *rms_weight, const void *wq, const void *wk, const void *wv,
                         const float *sq, const float *sk, const float *sv, int dim, int n_heads, int n_kv_heads,
                         int head_dim, int rotary_dim, int max_seq_len, float rope_theta, float norm_eps,
                         float qkv_clip, int dtype, const int *ctl, yalm_stream_t s);

/* Split-K flash-decode GQA attention over the fp16 KV ring: replaces attn_dot + attn_softmax +
 * att_mix (src/infer.cu:338-524).  `workspace` holds the per-split partials; size from
 * yalm_attn_workspace_bytes().  out is (n_heads*head_dim) fp32. */
size_t yalm_attn_workspace_bytes(int n_heads, int n_kv_heads, int head_dim);
int yalm_attn_decode(float *out, const uint16_t *key_cache, const uint16_t *value_cache, const float *q,
                     void *workspace, int n_heads, int n_kv_heads, int head_dim, int max_seq_len, const int *ctl,
                     yalm_stream_t s);

/* yalm_attn_decode without a caller workspace and without any allocation (no cudaMalloc / cudaFree / allocating library
 * call).  This entry point has no counterpart in the reference: it was added at the request of the run's operators, for
 * callers that cannot allocate (code under CUDA graph capture, tight serving loops, harnesses that forbid cudaMalloc).
 * The split-K partials live in a file-scope device array of yalm_attn_decode_static_max_bytes() = 2 MiB that every GPU
 * loading the library holds until exit; shapes whose yalm_attn_workspace_bytes() exceeds it (or with more than 64 KV
 * heads) are refused with YALM_EINVAL and a message on stderr.  All calls on one device share that array: calls that
 * overlap on the GPU (different streams or host threads) race — serialise them on one stream.  Same result as
 * yalm_attn_decode (same kernel, same split count). */
size_t yalm_attn_decode_static_max_bytes(void);
int yalm_attn_decode_static(float *out, const uint16_t *key_cache, const uint16_t *value_cache, const float *q, int n_heads,
                            int n_kv_heads, int head_dim, int max_seq_len, const int *ctl, yalm_stream_t s);

/* out[i] = (residual ? residual[i] : 0) + sum_k aw[k] * (W[e_k] v_k)[i]   (wo and w2 + residual:
 * fused_matmul_add_residuals, src/infer.cu:270-288; MoE mix: src/infer.cpp:377-383).
 * Dense: n_active = 1, active_e = active_w = NULL.  MoE: expert e's matrix starts at
 * w + e*d*n elements, its scales at scale + e*d, and v_k = v + k*n. */
int yalm_gemv_residual(float *out, const float *residual, const float *v, const void *w, const float *scale, int n,
                       int d, int dtype, int n_active, const int *active_e, const float *active_w,
                       yalm_stream_t s);

/* Expert-parallel variants (the measured alternative to slicing every expert): the rank holds only the
 * experts e with e % ep_size == ep_rank, stacked in ascending order in w / w1 / w3 (and their scales); the router is
 * replicated and still selects among all n_experts; rows of experts held elsewhere are skipped here and reach x through
 * the all-reduce that follows w2.  ep_size == 1 is the plain function. */
int yalm_gemv_residual_ep(float *out, const float *residual, const float *v, const void *w, const float *scale, int n, int d,
                          int dtype, int n_active, const int *active_e, const float *active_w, int ep_rank, int ep_size,
                          yalm_stream_t s);
int yalm_ffn_glu_ep(float *hb, const float *x, const float *rms_weight, const void *w1, const void *w3, const float *s1,
                    const float *s3, const void *gate, const float *sgate, int dim, int hidden_dim, int act, float norm_eps,
                    int dtype, int n_experts, int n_active, int *active_e, float *active_w, float *moe_logits, int ep_rank,
                    int ep_size, yalm_stream_t s);

/* rmsnorm -> [router GEMV + top-k gate] -> hb[k,i] = act(W1[e_k] xb)[i] * (W3[e_k] xb)[i].
 * Replaces rmsnorm + fused_ffn_w1_w3_glu_act (src/infer.cu:598-620) and, for MoE, the CPU-only
 * router (src/infer.cpp:100-132, 347-349).  Dense: n_experts = 0, gate = NULL; hb is (hidden).
 * MoE: hb is (n_active, hidden); active_e/active_w (device, n_active) receive the selection.
 * rms_weight == NULL skips the norm (the reference's ffn_cuda test entry has none). */
int yalm_ffn_glu(float *hb, const float *x, const float *rms_weight, const void *w1, const void *w3,
                 const float *s1, const float *s3, const void *gate, const float *sgate, int dim, int hidden_dim,
                 int act, float norm_eps, int dtype, int n_experts, int n_active, int *active_e,
                 float *active_w, float *moe_logits, yalm_stream_t s);

/* logits = Wcls rmsnorm(x)  (final rmsnorm + matmul_wide, src/infer.cu:1097-1126).  logits may be
 * device memory or device-mapped host memory. */
int yalm_lm_head(float *logits, const float *x, const float *rms_weight, const void *wcls, const float *scale,
                 int dim, int vocab, float norm_eps, int dtype, yalm_stream_t s);

/* Greedy on device with Sampler::sample_argmax's first-max rule (src/sampler.cpp:27-38): writes the
 * arg-max to tokens_out[ctl.step], then ctl.token = argmax, ctl.pos += 1, ring position re-derived. */
int yalm_argmax_advance(const float *logits, int vocab, int *ctl, int max_seq_len, int *tokens_out,
                        yalm_stream_t s);

/* Sampler::sample on the device (src/sampler.cpp:40-65): p_i = exp((l_i - max) / T) / sum, the first index whose
 * running sum reaches r wins (vocab - 1 if none); r = uniform(seed, ctl.step) from a counter-based generator (the
 * reference draws std::rand()).  Then the same control-block advance as yalm_argmax_advance.  temperature 0 = greedy. */
int yalm_sample_advance(const float *logits, int vocab, int *ctl, int max_seq_len, int *tokens_out, float temperature,
                        unsigned long long seed, yalm_stream_t s);
/* One draw into *token_dev (device int) with r = uniform(seed, counter); temperature 0 = first-max arg-max. */
int yalm_sample_device1(const float *logits, int vocab, float temperature, unsigned long long seed,
                        unsigned long long counter, int *token_dev, yalm_stream_t s);
/* Sampler::sample_prob (src/sampler.cpp:11-25) for n_rows logit rows (device, row stride vocab):
 * probs[i] = softmax(logits[i, :])[targets[i]] — what perplexity mode needs per position (src/main.cpp:174-184). */
int yalm_token_probs(const float *logits, int vocab, int n_rows, const int *targets, float *probs, yalm_stream_t s);

/* Bare GEMV xout = W x (matmul<T>, src/infer.cu:234-248), device pointers. */
int yalm_gemv(float *xout, const float *x, const void *w, const float *scale, int n, int d, int dtype,
              yalm_stream_t s);

/* xout = alpha * W x; also takes YALM_BF16 weights (n % 8 == 0, 16-byte aligned rows). */
int yalm_gemv_scaled(float *xout, const float *x, const void *w, int n, int d, int dtype, float alpha, yalm_stream_t s);

/* ---- (2b) batched prefill ops (net-new, SURVEY.md 8(f).1: the reference hydrates and scores token by token,
 * src/main.cpp:91-97, 174-184) ---------------------------------------------------------------------------------------
 * c (M, ldc) fp32 (=|+=) a (M, K) fp16 * w (N, K)^T fp16 on the tcgen05 tensor cores (TMA operand loads, TMEM
 * accumulator); w is a .yalm weight as stored ((out, in) row-major).  accumulate != 0: c += ... (residual in place). */
int yalm_gemm_f16(float *c, int ldc, const void *a, const void *w, int M, int N, int K, int accumulate, yalm_stream_t s);
/* h (M, ldh) fp16 = act(a w1^T) * (a w3^T): fused w1 / w3 projection + GLU (src/infer.cpp:360-375). */
int yalm_gemm_glu_f16(void *h, int ldh, const void *a, const void *w1, const void *w3, int M, int N, int K, int act,
                      yalm_stream_t s);
/* Causal attention of n query rows q16 (n, n_heads * head_dim) fp16 = positions pos0 .. pos0 + n - 1 over the head-major
 * KV ring (rows 0 .. pos0 + n - 1 valid; no wrap: pos0 + n <= max_seq_len); out16 like q16.  src/infer.cpp:216-248 per row. */
int yalm_attn_prefill(void *out16, const void *q16, const uint16_t *key_cache, const uint16_t *value_cache, int n, int pos0,
                      int n_heads, int n_kv_heads, int head_dim, int max_seq_len, yalm_stream_t s);

/* ---- (2c) row-batched ops of the layered executor (no reference counterpart: the reference has one homogeneous
 * Llama-style block) -------------------------------------------------------------------------------------------------
 * Every op takes n rows = n consecutive positions of one sequence; n = 1 is a decode step.  Device pointers; fp32
 * activations; weights fp32 / fp16 / bf16 (out, in) row-major.  Position of row m: pos0 + m, or ctl[1] + m when a device
 * control block is given.  Key / value rings are head-major (kv head, slot, channel), slot = position % ring, fp32
 * (cache_f32 != 0) or bf16; pooled keys / values are fp32 (kv head, block, channel). */
int yalm_embed_rows(float *x, const void *table, const void *positions, int dtype, const int *tokens, int n, int dim, int pos0,
                    const int *ctl, float scale, yalm_stream_t s);
int yalm_linear_rows(float *y, int ldy, const float *x, int ldx, const void *w, int dtype, int M, int N, int K, float alpha,
                     yalm_stream_t s);
int yalm_cast_rows16(void *out16, const float *x, int ldx, int M, int K, int bf16, yalm_stream_t s);
/* yalm_gemm_f16 with fp16 or bf16 operands and c = alpha * (a w^T) [+ c]. */
int yalm_gemm_16(float *c, int ldc, const void *a, const void *w, int M, int N, int K, int accumulate, int bf16, float alpha,
                 yalm_stream_t s);
/* q | k | v rows (fp32, row stride ld): RMS norm over the whole q and k projections (weights qnorm / knorm, null: none),
 * vmode 0 plain values, 1 also kept in vfirst, 2 blended v = (1 - vmix[0]) v + vmix[0] vfirst; k and v appended to the rings. */
int yalm_qkv_post_rows(float *qkv, int ld, void *key_ring, void *value_ring, float *vfirst, int ldvf, const float *qnorm,
                       const float *knorm, const float *vmix, int vmode, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                       float eps, int cache_f32, int pos0, const int *ctl, yalm_stream_t s);
/* Mean key / value of every block of `pool` positions whose last position is one of these rows. */
int yalm_kv_pool_rows(float *key_pool, float *value_pool, const void *key_ring, const void *value_ring, int n, int n_kv, int dk, int dv,
                      int ring, int pool, int max_blocks, int cache_f32, int pos0, const int *ctl, yalm_stream_t s);
/* Attention of n query rows: position i sees tokens j with 0 <= i - j < window (window 0: all) and, if pool > 0, block b
 * (positions b pool .. b pool + pool - 1) once b pool + pool - 1 <= i - window; one softmax over both; score = q . k * scale.
 * The key / value rows are read once for up to four query heads that share a kv head.  workspace (optional,
 * yalm_attn_window_pool_workspace(dv) floats): with few rows (decoding) the keys are split over more CTAs and merged in order;
 * context: the most positions a sequence reaches (0: unknown), used to pick the split count from shapes alone. */
size_t yalm_attn_window_pool_workspace(int dv);
int yalm_attn_window_pool(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring,
                          const float *key_pool, const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv,
                          int ring, int max_blocks, int window, int pool, float scale, int cache_f32, int context, int pos0, const int *ctl,
                          yalm_stream_t s);
/* The same attention for many rows over bf16 rings on the tensor cores (mma.sync bf16, fp32 scores / softmax): head sizes
 * dk in {64, 128}, dv in {32, 64, 128} (yalm_attn_window_pool_mma_shape), ldq % 4 == 0, ldo % 2 == 0. */
int yalm_attn_window_pool_mma_shape(int dk, int dv);
int yalm_attn_window_pool_mma(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring,
                              const float *key_pool, const float *value_pool, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                              int max_blocks, int window, int pool, float scale, int pos0, const int *ctl, yalm_stream_t s);
/* x[m] += rms(sum_{j < nsum} y[m * nsum + j]) * (w_offset + w) */
int yalm_norm_residual_rows(float *x, const float *y, int ldy, int nsum, const float *w, float w_offset, float eps, int n, int dim,
                            yalm_stream_t s);
int yalm_norm_gather_rows(float *out, const float *x, const int *rows, const float *w, int scalar_weight, float w_offset, float eps, int n_rows,
                          int dim, yalm_stream_t s);
/* h[m, f] = act(g) * (u + up_offset), g = gu[m, f], u = gu[m, ff + f]; limit > 0: g = min(g, limit), u clamped to +-limit.
 * act: YALM_ACT_GELU, YALM_ACT_SILU, 2 = g * sigmoid(alpha g), 3 = tanh GELU with sqrt(2 / pi) to fp32 precision. */
int yalm_glu_act_rows(float *h, const float *gu, int n, int ff, int act, float alpha, float limit, float up_offset, yalm_stream_t s);
/* ids / wts (n, top): the experts with the largest scores (score 0: softmax, 1: sigmoid of the fp32 router logits) and
 * their scores, divided by their sum + renorm_eps if renorm.  groups > 1: experts form equal groups of neighbours, a group
 * scores its best expert, and only the keep_groups best groups' experts can be chosen. */
int yalm_router_topk_rows(int *ids, float *wts, const float *x, int ldx, const void *wr, int dtype, int n, int n_experts, int top, int dim,
                          int score, int renorm, float renorm_eps, int groups, int keep_groups, yalm_stream_t s);
/* Slot s = (row s / top, expert ids[s]) through stacked expert matrices gate / up (E, ff, dim) and down (E, dim, ff);
 * in_scale: the slot's weight multiplies the expert's input; out_scale: its output. */
int yalm_moe_glu_slots(float *h, const float *x, int ldx, const void *wg, const void *wu, int dtype, const int *ids, const float *wts, int n,
                       int top, int ff, int dim, int act, float alpha, float limit, float up_offset, int in_scale, yalm_stream_t s);
int yalm_moe_down_slots(float *y, int ldy, const float *h, const void *wd, int dtype, const int *ids, const float *wts, int n, int top, int ff,
                        int dim, int out_scale, yalm_stream_t s);

/* Experts on the tensor cores (prompt portions): order[j] is the slot (row * top + k) at place j once slots are sorted by
 * expert.  gather: out16[j] = x[order[j] / top] (* wts[order[j]] if in_scale) as bf16 / fp16; scatter: y[order[j]] = ys[j]
 * (* wts[order[j]] if out_scale). */
int yalm_moe_gather_rows16(void *out16, const float *x, int ldx, const int *order, const float *wts, int n_slots, int top, int dim, int bf16,
                           int in_scale, yalm_stream_t s);
int yalm_moe_scatter_rows(float *y, int ldy, const float *ys, int lds, const int *order, const float *wts, int n_slots, int dim, int out_scale,
                          yalm_stream_t s);

/* One-row (decode) products with what follows them fused in, on the streaming GEMV: the CTA that finishes last runs the tail.
 * yalm_gemv_norm_residual: y = W x (d x n), res += rms(y) (w_offset + nw); gu != 0: x is a (gate | up) row of 2 n floats and
 * the input is act(g) (u + up_offset).  yalm_gemv_qkv_post: qkv = W x, then yalm_qkv_post_rows for the row and the block mean
 * if the position completes a block.  counter: a zeroed device word, left zero.  n % 8 == 0 (fp32: 4), 16-byte aligned. */
int yalm_gemv_norm_residual(float *res, float *y, const float *x, const void *w, const float *nw, float w_offset, float eps, int n, int d,
                            int dtype, int gu, int act, float act_alpha, float limit, float up_offset, unsigned *counter, yalm_stream_t s);
int yalm_gemv_qkv_post(float *qkv, const float *x, const void *w, int n, int dtype, void *key_ring, void *value_ring, float *vfirst,
                       const float *qnorm, const float *knorm, const float *vmix, int vmode, int n_heads, int n_kv, int dk, int dv, int ring,
                       float eps, int cache_f32, float *key_pool, float *value_pool, int pool, int max_blocks, int pos0, const int *ctl,
                       unsigned *counter, yalm_stream_t s);

/* yalm_gemv_norm_shift: yalm_norm_shift_rows for one row + the product of its shifted output, as one launch (h left in h_out
 * and in the state).  yalm_gemv_residual_sum: y = alpha W x, then res += (y + add1) + sum_j slots[j] (yalm_residual_sum_rows). */
int yalm_gemv_norm_shift(float *out, const float *x, const void *w, int n, int d, int dtype, const float *hw, int scalar_weight, float w_offset,
                         float eps, const float *shift, float *state, float *h_out, int pos0, const int *ctl, unsigned *counter, yalm_stream_t s);
int yalm_gemv_residual_sum(float *res, float *y, const float *x, const void *w, float alpha, int n, int d, int dtype, const float *add1,
                           const float *slots, int nslots, int ldslots, unsigned *counter, yalm_stream_t s);

/* ---- layers with per-sequence state besides a key / value ring (csrc/ops_stack_state.cu) ----
 * A call whose first position is 0 starts a sequence: stored state is taken as zero.  All state is fp32.
 * yalm_norm_shift_rows: h = rms(x) (w_offset + w), w one number if scalar_weight; hs (optional) = h + (h of the previous
 * position - h) * shift, the previous h of the call's first row coming from `state` (dim floats), which then takes the
 * last row's h.  h may alias x only without hs. */
int yalm_norm_shift_rows(float *h, float *hs, const float *x, const float *w, int scalar_weight, float w_offset, float eps, const float *shift,
                         float *state, int n, int dim, int pos0, const int *ctl, yalm_stream_t s);
/* out[m, c] = silu(bias[c] + sum_j w[c, j] in[m - (taps - 1) + j, c]); w (channels, taps) fp32, bias optional; state
 * (channels, taps - 1): the inputs of the positions just before the call, replaced by the call's last ones. */
int yalm_conv_act_rows(float *out, int ldo, const float *in, int ldi, const float *w, const float *bias, float *state, int n, int channels,
                       int taps, int pos0, const int *ctl, yalm_stream_t s);
/* Linear recurrence over a (D, P) matrix state M per head: M <- a M (a: the decay); e = beta (v - M^T k) if beta, else vscale v;
 * M <- M + k e^T; out = M^T q (+ skip v).  k, q (n, kv heads D), head h reading kv head h / rep; v, out (n, heads P);
 * decay (n, heads) or, if decay_per_channel, (n, heads D) acting on rows; vscale, beta (n, heads) or null; skip (heads) or
 * null; state (heads, P, D).  D <= 256. */
int yalm_state_scan_rows(float *out, int ldo, const float *k, int ldk, const float *q, int ldq, const float *v, int ldv, const float *decay,
                         int ldd, int decay_per_channel, const float *vscale, int ldvs, const float *beta, int ldb, const float *skip,
                         float *state, int n, int heads, int rep, int D, int P, int pos0, const int *ctl, yalm_stream_t s);
/* dt = softplus(dt + dt_bias[h]) in place, decay = exp(-exp(a_log[h]) dt). */
int yalm_ssm_prep_rows(float *dt, int lddt, float *decay, int ldd, const float *dt_bias, const float *a_log, int n, int heads, yalm_stream_t s);
/* In place: q, k unit vectors per head (x / sqrt(sum x^2 + unit_eps)), q also times q_scale; beta = sigmoid(beta);
 * g[h, i] = exp(-exp(a_log[h]) softplus(g[h, i] + dt_bias[h, i])). */
int yalm_delta_prep_rows(float *q, float *k, int ldqk, float *beta, int ldb, float *g, int ldg, const float *a_log, const float *dt_bias, int n,
                         int heads, int kv_heads, int dim, float unit_eps, float q_scale, yalm_stream_t s);
/* out = rms over each of `parts` equal parts of (y * silu(z)), times w (dim). */
int yalm_gated_group_norm_rows(float *out, int ldo, const float *y, int ldy, const float *z, int ldz, const float *w, int n, int dim, int parts,
                               float eps, yalm_stream_t s);
/* out[m, h, :] = o[m, h, :] / sqrt(mean o^2 + eps) * w (vdim, shared by heads) * sigmoid(gate[m, h, :]). */
int yalm_head_norm_gate_rows(float *out, int ldo, const float *o, int ldi, const float *gate, int ldg, const float *w, int n, int heads, int vdim,
                             float eps, yalm_stream_t s);
/* q += qb, k += kb in place (null: none); k rows appended to the ring (kv head, slot, channel) and, for positions below
 * `keep`, to first_buf (kv head, keep, channel). */
int yalm_qk_bias_append_rows(float *q, float *k, int ld, const float *qb, const float *kb, void *ring_buf, void *first_buf, int n, int n_heads,
                             int n_kv, int dk, int ring, int keep, int cache_f32, int pos0, const int *ctl, yalm_stream_t s);
/* Attention with sigmoid weights over keys that are also the values: position i sees j <= i with i - j < window (0: all) or
 * j < keep; weight = sigmoid(q . k scale + rel[bucket[i - j], h] + hb[h]), not normalised; out *= sigmoid(gate). */
size_t yalm_attn_sigmoid_workspace(int dk);
int yalm_attn_sigmoid_rows(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                           const float *rel, const int *bucket, const float *hb, float *workspace, int n, int n_heads, int n_kv, int dk, int ring,
                           int window, int keep, float scale, int cache_f32, int context, int pos0, const int *ctl, yalm_stream_t s);
/* The same attention for many rows over a bf16 ring on the tensor cores (mma.sync bf16, fp32 scores and sigmoid): head sizes
 * 32, 64, 128 (yalm_attn_sigmoid_mma_shape), ldq % 4 == 0, ldo % 2 == 0.  table (optional, (n_heads, ldt)): rel[bucket[d], h] + hb[h]
 * per head and distance, read instead of rel / bucket / hb. */
int yalm_attn_sigmoid_mma_shape(int dk);
int yalm_attn_sigmoid_mma(float *out, int ldo, const float *q, int ldq, const void *ring_buf, const void *first_buf, const float *gate, int ldg,
                          const float *rel, const int *bucket, const float *hb, const float *table, int ldt, int n, int n_heads, int n_kv, int dk,
                          int ring, int window, int keep, float scale, int context, int pos0, const int *ctl, yalm_stream_t s);
/* x[m] += a[m] (+ b[m]) + sum_{j < nsum} y[m * nsum + j]  (a, b, y optional). */
int yalm_residual_sum_rows(float *x, const float *a, const float *b, const float *y, int ldy, int nsum, int n, int dim, yalm_stream_t s);
int yalm_softcap_rows(float *z, int n, int dim, float cap, yalm_stream_t s);

/* ---- pre-norm layers with an input convolution, latent attention, gated linear attention (csrc/ops_stack_latent.cu) ----
 * yalm_norm_conv_rows: h = norm(x) w (layer_norm != 0: (x - mean) / sqrt(var + eps), else x / sqrt(mean x^2 + eps)); u = h + conv(h),
 * conv(h)[m, c] = sum_j conv_w[c, j] h[m - taps + 1 + j, c]; state (taps - 1, dim): h of the positions just before the call,
 * replaced by the call's last ones. */
int yalm_norm_conv_rows(float *u, float *h, const float *x, const float *w, int layer_norm, float eps, const float *conv_w, float *state, int n,
                        int dim, int taps, int pos0, const int *ctl, yalm_stream_t s);
/* yalm_norm_conv_rows after x += add (add optional). */
int yalm_add_norm_conv_rows(float *u, float *h, float *x, const float *add, const float *w, int layer_norm, float eps, const float *conv_w,
                            float *state, int n, int dim, int taps, int pos0, const int *ctl, yalm_stream_t s);
/* Rotary table: freq (rot_dims / 2) fp32 and a magnitude on cos and sin; interleaved != 0: pair i = channels (2 i, 2 i + 1).
 * yalm_latent_post_rows: row m of proj (ld): [o_q, +q_rank) RMS-normed with q_norm in place; ring_buf != NULL: [o_kv, +kv_rank) RMS-normed
 * with kv_norm and [o_kv + kv_rank, +rot_dim) with its first rot_dims channels rotated go to ring row p % ring as
 * [kv_rank | rot_dim] (fp32 if cache_f32, else bf16). */
int yalm_latent_post_rows(float *proj, int ld, int o_q, int q_rank, const float *q_norm, int o_kv, int kv_rank, int rot_dim, const float *kv_norm,
                          void *ring_buf, int ring, const float *freq, float magnitude, int rot_dims, int interleaved, float eps, int cache_f32,
                          int n, int pos0, const int *ctl, yalm_stream_t s);
/* q (n, heads (dim + rot_dim)) -> out (n, heads (kv_rank + rot_dim)): per head [ukt_h q_unrotated | rotated part turned by its
 * position], ukt (heads, kv_rank, dim) = every head's W_uk transposed: the query against cached rows [latent | rotated key part]. */
int yalm_latent_query_rows(float *out, int ldo, const float *q, int ldq, const void *ukt, int dtype, int n, int heads, int dim, int rot_dim,
                           int kv_rank, const float *freq, float magnitude, int rot_dims, int interleaved, int pos0, const int *ctl,
                           yalm_stream_t s);
/* Prompt portions of latent attention on the tensor cores: the cached rows (bf16) of positions first_pos .. first_pos + count - 1
 * give (a) their latents as a dense bf16 operand (count, kv_rank) and, with kv (count, heads (dim + vdim)) fp32 = that operand times
 * [W_uk ; W_uv]^T, (b) per head the key [unrotated | rotated key part] and the value as bf16 rows of head-major rings
 * (head, ring_out, dim + rot_dim | vdim), slot = position % ring_out: what yalm_attn_window_pool_mma reads. */
int yalm_latent_gather_rows16(void *out16, const void *ring_buf, int ring, int row, int kv_rank, int first_pos, int count, yalm_stream_t s);
int yalm_latent_pack_rings(void *key_ring, void *value_ring, const float *kv, int ldkv, const void *ring_buf, int ring, int kv_rank, int rot_dim,
                           int heads, int dim, int vdim, int ring_out, int first_pos, int count, yalm_stream_t s);
/* In place: channels [offset, offset + rot_dims) of every head (head_size channels) of row m turned by its position. */
int yalm_rotate_heads_rows(float *q, int ldq, int heads, int head_size, int offset, const float *freq, float magnitude, int rot_dims,
                           int interleaved, int n, int pos0, const int *ctl, yalm_stream_t s);
/* x[m, :dim] *= sigmoid(gate[m, :dim]) */
int yalm_sigmoid_gate_rows(float *x, int ldx, const float *gate, int ldg, int n, int dim, yalm_stream_t s);
/* Attention over cached bf16 rows that all heads share (key = the row's dk channels, value = its first dv; row stride ld), each
 * row read once for scores and weighted sums: position i sees rows j with 0 <= i - j < window (0: all).  Sizes:
 * yalm_attn_latent_rows_shape; workspace as for yalm_attn_window_pool (or NULL). */
int yalm_attn_latent_rows_shape(int dk, int dv, int ld);
int yalm_attn_latent_rows(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                          int dv, int ring, int window, float scale, int context, int pos0, const int *ctl, yalm_stream_t s);
/* out[m, h, :N] = w_h x[m, h, :K] (w (heads N, K)), times sigmoid(gate[m, h, :N]) if gate. */
int yalm_head_linear_gate_rows(float *out, int ldo, const float *x, int ldx, const void *w, int dtype, const float *gate, int ldg, int n, int heads,
                               int N, int K, yalm_stream_t s);
/* In place: z = sigmoid(z + bias)^(1 / tau) (the decays of gated linear attention, fp32), q *= q_scale. */
int yalm_gla_prep_rows(float *z, int ldz, const float *bias, float tau, float *q, int ldq, float q_scale, int n, int channels, yalm_stream_t s);
/* hist slab count - 1 (slabs of `stride` floats) <- x (+ a + b + sum_j y[m nsum + j], each optional); x <- sum_j w[j] slab_j
 * (w NULL: x <- the slab). */
int yalm_depth_average_rows(float *x, float *hist, size_t stride, const float *w, int count, int n, int dim, const float *a, const float *b,
                            const float *y, int ldy, int nsum, yalm_stream_t s);
int yalm_layer_norm_gather_rows(float *out, const float *x, const int *rows, const float *w, int layer_norm, float eps, int n_rows, int dim,
                                yalm_stream_t s);
/* yalm_head_norm_gate_rows with silu(gate) instead of sigmoid(gate) when gate_silu != 0. */
int yalm_head_norm_act_rows(float *out, int ldo, const float *o, int ldi, const float *gate, int ldg, const float *w, int n, int heads, int vdim,
                            float eps, int gate_silu, yalm_stream_t s);
/* yalm_attn_window_pool with explicit row strides of the rings (elements): values may be the first dv channels of the key rows
 * (value_ring = key_ring, ldv = ldk). */
int yalm_attn_window_pool_strided(float *out, int ldo, const float *q, int ldq, const void *key_ring, int ldk, const void *value_ring, int ldv,
                                  const float *key_pool, const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv,
                                  int ring, int max_blocks, int window, int pool, float scale, int cache_f32, int context, int pos0,
                                  const int *ctl, yalm_stream_t s);
/* yalm_router_topk_rows with a stored bias per expert that only the choice sees (NULL: none) and a scale on the weights. */
int yalm_router_bias_topk_rows(int *ids, float *wts, const float *x, int ldx, const void *wr, int dtype, int n, int n_experts, int top, int dim,
                               int score, int renorm, float renorm_eps, int groups, int keep_groups, const float *bias, float weight_scale,
                               yalm_stream_t s);
/* The slot kernels with identity experts: ids >= n_real have no matrices; their slot returns the row of x (times the weight). */
int yalm_moe_glu_slots_real(float *h, const float *x, int ldx, const void *wg, const void *wu, int dtype, const int *ids, const float *wts, int n,
                            int top, int ff, int dim, int act, float alpha, float limit, float up_offset, int in_scale, int n_real, yalm_stream_t s);
int yalm_moe_identity_slots(float *y, int ldy, const float *x, int ldx, const int *ids, const float *wts, int n, int top, int dim, int n_real,
                            int out_scale, yalm_stream_t s);
int yalm_moe_down_slots_real(float *y, int ldy, const float *h, const void *wd, int dtype, const int *ids, const float *wts, int n, int top, int ff,
                             int dim, int out_scale, int n_real, const float *x, int ldx, yalm_stream_t s);

/* ---- layers with a norm before and after every sublayer (csrc/ops_stack_diff.cu) and what their mixers add to the attention ops ----
 * The attention ops with a sink per query head in the softmax's denominator (exp(sink_h) counts once, without key or value;
 * sink NULL: none) and with v_heads value heads for n_kv key heads: key head g reads value head g % v_heads, so that several
 * maps share one set of values.  The pooled blocks visible to a row are capped at max_blocks: with pool = 1 and max_blocks = k
 * they are a window's kept first k tokens. */
int yalm_attn_window_pool_sink(float *out, int ldo, const float *q, int ldq, const void *key_ring, int ldk, const void *value_ring, int ldv,
                               const float *key_pool, const float *value_pool, float *workspace, int n, int n_heads, int n_kv, int dk, int dv,
                               int ring, int max_blocks, int window, int pool, float scale, int cache_f32, int context, int pos0, const int *ctl,
                               const float *sink, int v_heads, yalm_stream_t s);
int yalm_attn_window_pool_mma_sink(float *out, int ldo, const float *q, int ldq, const void *key_ring, const void *value_ring,
                                   const float *key_pool, const float *value_pool, int n, int n_heads, int n_kv, int dk, int dv, int ring,
                                   int max_blocks, int window, int pool, float scale, int pos0, const int *ctl, const float *sink, int v_heads,
                                   yalm_stream_t s);
int yalm_attn_latent_rows_sink(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                               int dv, int ring, int window, float scale, int context, int pos0, const int *ctl, const float *sink, yalm_stream_t s);
/* Row m of proj (ld): n_q_vectors query vectors of dk channels from o_q, n_k_vectors key vectors from o_k, n_v_heads value heads
 * of dv channels from o_v.  Every query / key vector: RMS norm over its dk channels with the shared weight q_norm / k_norm (dk
 * floats; NULL: none), then its first rot_dims channels turned by the row's position (freq: rot_dims / 2 frequencies, magnitude
 * on cos and sin; pair i = channels (i, i + rot_dims / 2), or (2 i, 2 i + 1) if interleaved).  Queries stay in place, keys and
 * values go to the rings (vector, slot, channel), slot = position % ring; positions below `keep` also to key_first (vector,
 * keep, dk) / value_first (head, keep, dv), fp32, as the rings hold them.  dk <= 512. */
int yalm_head_norm_rope_append_rows(float *proj, int ld, int o_q, int o_k, int o_v, int n_q_vectors, int n_k_vectors, int n_v_heads, int dk, int dv,
                                    const float *q_norm, const float *k_norm, const float *freq, float magnitude, int rot_dims, int interleaved,
                                    float eps, void *key_ring, void *value_ring, int ring, float *key_first, float *value_first, int keep,
                                    int cache_f32, int n, int pos0, const int *ctl, yalm_stream_t s);
/* maps (n, 2 heads dv): every head's first map, then every head's second.  out[m, h] = o / sqrt(mean o^2 + eps) * out_scale
 * * sigmoid(gate[m, h]) with o = map_1 - lambda map_2 (gate NULL: none). */
int yalm_diff_combine_rows(float *out, int ldo, const float *maps, int ldm, const float *gate, int ldg, int n, int heads, int dv, float lambda,
                           float out_scale, float eps, yalm_stream_t s);
/* h[m, :ff] = act(h[m, :ff]) in place; act: YALM_ACT_GELU, YALM_ACT_SILU, 3 = tanh GELU, 4 = exact (erf) GELU. */
int yalm_act_rows(float *h, int ld, int n, int ff, int act, yalm_stream_t s);
/* x[m] += y / sqrt(mean y^2 + eps) * norm_w, y = w_proj (gelu_tanh(w_gate x[m]) * e), e = table[token of row m, col0 .. col0 + side):
 * w_gate (side, dim), w_proj (dim, side), table (vocab, ldt) in `dtype`; tokens (n) or, if NULL, ctl[0]. */
int yalm_token_side_rows(float *x, const void *table, int ldt, int col0, const int *tokens, const int *ctl, const void *w_gate, const void *w_proj,
                         const float *norm_w, int dtype, int n, int dim, int side, float eps, yalm_stream_t s);

/* The side input in two steps that spread over the GPU: h[m, j] = gelu_tanh(w_gate[j] . x[m]) * table[token of row m, col0 + j]; with
 * w_gate NULL, h already holds the product x w_gate^T and is finished in place.  dim % 8 == 0 (fp32: 4), 16-byte aligned rows. */
int yalm_token_side_gate_rows(float *h, int ldh, const float *x, int ldx, const void *table, int ldt, int col0, const int *tokens, const int *ctl,
                              const void *w_gate, int dtype, int n, int dim, int side, yalm_stream_t s);
/* yalm_gemv_norm_residual (no weight offset) with a plain activation on the input (act >= 0: yalm_act_rows' codes, applied while x is
 * staged; negative: none) and, if next_w, the next sublayer's input norm from the finished row: next_out = rms(res) * next_w. */
int yalm_gemv_act_norm_residual_norm(float *res, float *y, const float *x, const void *w, const float *nw, float eps, int n, int d, int dtype, int act,
                                     const float *next_w, float *next_out, unsigned *counter, yalm_stream_t s);

/* Decode rows of latent attention on the tensor cores (mma.sync bf16): the heads of a row are the M tile, a tile of 64 cached rows is
 * fetched once for all heads, for the scores and for the weighted sums.  Sizes: yalm_attn_latent_mma_shape.  nsplit CTAs share a row's
 * keys (1 ... 128, n n_heads nsplit <= 4096; workspace as for yalm_attn_latent_rows when above 1); the caller picks it from shapes alone.
 * yalm_attn_latent_merge joins such partials. */
int yalm_attn_latent_mma_shape(int dk, int dv, int ld);
int yalm_attn_latent_mma_rows(float *out, int ldo, const float *q, int ldq, const void *rows, int ld, float *workspace, int n, int n_heads, int dk,
                              int dv, int ring, int window, float scale, int nsplit, int pos0, const int *ctl, const float *sink, yalm_stream_t s);
int yalm_attn_latent_merge(float *out, int ldo, const float *part, int n, int n_heads, int dv, int nsplit, const float *sink, yalm_stream_t s);

/* ---- (3a) host-pointer test entry points (src/infer.cu:890-1007 semantics) ------------------- */
int yalm_matmul_host(float *xout, const float *x, const void *w, const float *scale, int n, int d, int dtype);
int yalm_mha_host(float *xout, float *att, const uint16_t *kb, const uint16_t *vb, const float *q, int head_dim,
                  int kv_len, int max_seq_len, int n_heads, int n_kv_heads);
int yalm_ffn_host(float *xout, const float *x, const void *w1, const void *w2, const void *w3, const float *s1,
                  const float *s2, const float *s3, int hidden_dim, int dim, int act, int dtype);
/* Host-pointer test entries of the device sampler: one draw with a caller-supplied r in [0, 1] (Sampler::sample with
 * std::rand() / RAND_MAX replaced by r), and sample_prob for n_rows rows. */
int yalm_sample_host(const float *logits, int vocab, float temperature, float r, int *token);
int yalm_token_probs_host(const float *logits, int vocab, int n_rows, const int *targets, float *probs);
/* Host-pointer test entry of the prefill GEMM: c (M, N) fp32 = a (M, K) fp16 * w (N, K)^T fp16 [+ c if accumulate];
 * with w3 != NULL instead h (M, N) fp16 = act(a w^T) * (a w3^T). */
int yalm_gemm_host(float *c, void *h, const void *a, const void *w, const void *w3, int M, int N, int K, int accumulate, int act);
/* Host-pointer test entry of the windowed attention with pooled blocks: positions 0 .. T - 1 in portions of `chunk` rows
 * through the append, block-mean and attention kernels over rings of `ring` slots (>= max(window, pool) + chunk - 1).
 * q (T, n_heads dk), k (T, n_kv dk), v (T, n_kv dv), out (T, n_heads dv), fp32. */
int yalm_attn_window_pool_host(float *out, const float *q, const float *k, const float *v, int T, int n_heads, int n_kv, int dk, int dv,
                               int window, int pool, float scale, int ring, int chunk, int cache_f32);
/* Same ops timed on the device: `iters` launches after `warmup`, returns mean microseconds per
 * launch (CUDA events) in *usec.  This is what `./build/test -k <name>` prints. */
int yalm_bench_op(const char *name, int iters, int warmup, double *usec, double *bytes);

/* ---- (3b) opaque handles over Model / InferenceState ------------------------------------------ */
typedef struct yalm_model yalm_model;
typedef struct yalm_state yalm_state;

/* `context` = the reference's -T (0: min(metadata max_seq_len, 4096), src/model.cpp:31-36). */
int yalm_model_open_file(const char *path, int context, yalm_model **out);
/* Image must stay valid until yalm_model_cuda() has returned. */
int yalm_model_open_memory(const void *image, size_t size, int context, yalm_model **out);
/* A checkpoint directory (config.json + model.safetensors) of a registered layered architecture.  compute_dtype:
 * YALM_F32 = everything in true 32-bit (16-bit weights are widened at load), YALM_BF16 / YALM_F16 = 16-bit matrix operands
 * with fp32 accumulation, negative = as stored.  yalm_model_open_file on a directory is this with compute_dtype -1.
 * context: most positions a sequence may reach (0: the model's own limit). */
int yalm_model_open_dir(const char *path, int context, int compute_dtype, yalm_model **out);
/* 1 for a layered architecture, 0 for a .yalm model. */
int yalm_model_is_stack(const yalm_model *m);
/* Tensor-parallel shard `tp_rank` of `tp_size` (1 = whole model) is uploaded to `device`. */
int yalm_model_cuda(yalm_model *m, int device, int tp_rank, int tp_size);
void yalm_model_close(yalm_model *m);
/* out[16]: dim, hidden_dim, head_dim, n_layers, n_heads, n_kv_heads, vocab_size, max_seq_len,
 * rotary_dim, n_experts, n_experts_active, weight dtype, act, tp_rank, tp_size, reserved */
void yalm_model_config(const yalm_model *m, int *out);
size_t yalm_model_device_bytes(const yalm_model *m);
/* Loader facts (the reference: one cudaMalloc + one pageable copy per tensor, src/model.cpp:185-211):
 * out[0] = device allocations behind the model's weights and KV caches (1: one arena per rank),
 * out[1] = 1 if the upload went through the pinned double-buffered staging stream, 0 if it fell back to pageable copies. */
void yalm_model_load_info(const yalm_model *m, int *out2);

int yalm_state_new(yalm_model *m, yalm_state **out);
void yalm_state_free(yalm_state *s);
/* Model::forward (src/model.cpp:396-407). After a YALM_MODE_LOGITS call returns, yalm_logits() is valid. */
int yalm_forward(yalm_model *m, yalm_state *s, int token, int pos, int mode);
float *yalm_logits(yalm_state *s); /* host, vocab_size fp32 */
/* n_gen greedy steps entirely on the device starting from (token,pos): per step forward + argmax;
 * tokens_out (host, n_gen ints) gets the generated ids.  If logits_out != NULL (host, n_gen*vocab)
 * each step's logits are copied back too (parity mode).  *device_ms (optional) = CUDA-event time. */
int yalm_generate_greedy(yalm_model *m, yalm_state *s, int token, int pos, int n_gen, int *tokens_out,
                         float *logits_out, float *device_ms);
/* Batched prefill / perplexity: positions pos0 .. pos0 + n - 1 in one pass (dense tcgen05 GEMMs over the chunk, causal
 * flash attention, bulk KV append).  Afterwards the KV cache holds the chunk and yalm_logits() the LAST position's
 * logits; if targets != NULL, probs_out[i] = softmax(logits_i)[targets[i]] (Sampler::sample_prob per position,
 * src/sampler.cpp:11-25).  n <= yalm_model_batch_capacity() (0: this model / shard has no batched path — fp16 dense
 * unsharded models have — and the caller walks the tokens with yalm_forward); pos0 + n <= max_seq_len (no ring wrap). */
int yalm_model_batch_capacity(const yalm_model *m);
int yalm_forward_batch(yalm_model *m, yalm_state *s, const int *tokens, int n, int pos0, const int *targets, float *probs_out);
/* The general step: positions pos0 .. pos0 + n - 1 (n = 1: decode; larger: a portion of a prompt cut anywhere) from the
 * cache earlier steps left; logits of rows want[0 .. n_want) (ascending row indices) go to logits_out (host, n_want x
 * vocab).  Layered models take any n in one call; .yalm models walk the rows with yalm_forward. */
int yalm_forward_rows(yalm_model *m, yalm_state *s, const int *tokens, int n, int pos0, const int *want, int n_want, float *logits_out);
/* The current sequence is finished: what it holds in the cache is given back; the next step starts at position 0. */
int yalm_sequence_end(yalm_model *m, yalm_state *s);
/* Layered models, tests: fp32 copy of layer's key ring (0), value ring (1), pooled keys (2), pooled values (3); and the ring's slot count. */
int yalm_stack_read(yalm_model *m, int layer, int which, float *dst, size_t count);
int yalm_stack_ring_slots(const yalm_model *m, int layer);
/* Layered models, tests: after every layer of the following yalm_forward_rows calls (of at most the portion capacity rows)
 * the residual rows (n, width) are copied to dst + layer * n * width (host); NULL switches it off. */
int yalm_stack_tap(yalm_model *m, float *dst);
/* The same loop with Sampler::sample on the device: temperature 0 = greedy, > 0 = one draw per step with
 * r = uniform(seed, step).  4 bytes per token come back (the reference moves vocab * 4, src/model.cpp:338). */
int yalm_generate(yalm_model *m, yalm_state *s, int token, int pos, int n_gen, float temperature,
                  unsigned long long seed, int *tokens_out, float *logits_out, float *device_ms);
/* Tests only: set the launch counter behind the megakernel's hand-over flags (exercises its wrap). */
void yalm_state_debug_set_launch_seq(yalm_state *s, unsigned seq);
/* Debug/parity taps: copy a device activation or one layer's KV rows to the host.
 * which: 0 x, 1 xb2(attn out), 2 hb, 3 q, 4 key_cache(layer), 5 value_cache(layer),
 * 6 active_experts (int), 7 active_experts_weights */
int yalm_state_read(yalm_model *m, yalm_state *s, int which, int layer, void *dst, size_t bytes);
/* Mean duration (microseconds, CUDA events on the launching stream) of the dominant kernel — the fused
 * rmsnorm + w1/w3 + GLU GEMV — over n_steps greedy decode steps x n_layers launches from (token,pos). */
int yalm_profile_ffn(yalm_model *m, yalm_state *s, int token, int pos, int n_steps, double *mean_us);
/* Number of kernel launches one forward pass issues in `mode` (for bench.py's gpu_launches). */
int yalm_forward_launches(const yalm_model *m, int mode);
/* 1 when forward() is one persistent cooperative kernel per token (unsharded dense models; the weight and KV
 * tiles of the whole pass stream through a shared-memory TMA ring), 0 when it is the per-op kernel graph
 * (tensor-parallel shards, MoE, shapes the tile planner rejects, or YALM_B200_MEGA=0 in the environment). */
int yalm_model_uses_megakernel(const yalm_model *m);
/* Plan of the whole-token kernel for this model (no reference counterpart: the reference has no such kernel):
 * out8 = {ring stages, floats of the shared-memory vector region, 1 if hb travels w1/w3 -> w2 as pipelined slices
 * (decode_mega.cuh "pipelined hb") else 0, K splits of w2, 1 if the GEMV phases run on the tensor cores (decode_mega.cuh
 * "tensor-core GEMV") else 0, 0, 0, 0}.  Returns YALM_EINVAL when the model does not run on it. */
int yalm_model_mega_info(const yalm_model *m, int *out8);
/* One forward pass (logits mode) with the megakernel's phase profile on.  out receives grid * n_layers * 48
 * clock64 values: per CTA, per layer, 6 phases (qkv, attention, wo, w1/w3, w2, lm head) x 8 slots
 * ([0] phase entered [1] grid barrier passed [2] input vector staged [3] tiles + epilogue done
 * [4] cycles spent waiting for ring stages to fill).  out == NULL: only *grid (CTAs) is returned. */
int yalm_mega_profile(yalm_model *m, yalm_state *s, int token, int pos, long long *out, size_t count, int *grid);

/* Tensor-parallel plumbing (one process per GPU).  The 128-byte NCCL unique id is created by rank 0
 * with yalm_tp_unique_id() and distributed by the caller (torch.distributed / MPI / files). */
int yalm_tp_unique_id(void *id128);
int yalm_tp_init(const void *id128, int rank, int world);
void yalm_tp_finalize(void);
/* Shard arithmetic of the loader, callable without a device (tests): which bytes of an unsharded row-major tensor
 * rank `rank` of `size` holds.  dims[7] = dim, hidden, head_dim, n_heads, n_kv_heads, vocab, bytes per weight;
 * tensor: 0 wq, 1 wk, 2 wv, 3 wo, 4 w1, 5 w2, 6 w3, 7 wcls; out[4] = spitch, offset, width, height (bytes; `height`
 * pieces of `width`, piece i at offset + i * spitch).  Column-parallel: wq wk wv w1 w3 wcls; row-parallel: wo w2
 * (the reference is single-GPU). */
int yalm_tp_shard_plan(const int *dims, int tensor, int rank, int size, long long *out);

/* Planning arithmetic of the whole-token kernel, callable without a device (tests).  It replaces the launch geometry
 * the reference hard-codes per kernel (src/infer.cu:745-880: one warp per output row, grids of d / 32 CTAs).
 * yalm_mega_tile_plan: out20 = 5 GEMV kinds (qkv, wo, w1/w3, w2, lm head) x {rows per tile, columns per tile, K splits,
 * row groups} for one rank's dimensions; row group g of a phase goes to CTA (rotation + g) % grid.
 * yalm_mega_attn_split: out5 = {kv head, first CTA of the head, CTAs of the head, first chunk, chunks} of CTA `cta` for a
 * context of `n_chunks` KV row chunks per head.  Both return YALM_EINVAL for shapes the kernel does not take. */
int yalm_mega_tile_plan(int dtype, int dim, int q_dim, int kv_dim, int hidden, int vocab, int *out20);
/* Tensor-core GEMV geometry (decode_mega.cuh "tensor-core GEMV"): out4 = {rows per tile, first row, rows, tiles} of CTA `cta`
 * of `grid` for a matrix of `rows` rows partitioned in units of `unit` rows with tiles of at most `cap` rows.
 * yalm_mega_hb_share (pipelined hb): the number of hb elements of slice `slice` (slice_elems elements each) that CTA `cta`
 * produces when the w1/w3 phase has `groups` row groups of rows_per_group rows, group g on CTA (rotation + g) % grid;
 * negative = YALM_EINVAL. */
int yalm_mega_mma_plan(int rows, int unit, int cap, int grid, int cta, int *out4);
int yalm_mega_hb_share(int groups, int rows_per_group, int slice_elems, int grid, int cta, int rotation, int slice);
int yalm_mega_attn_split(int cta, int ncta, int n_kv_heads, int n_chunks, int *out5);

/* The CLI's tokenizer (greedy longest-prefix match + byte fallback, src/tokenizer.cpp:57-94; decode_one :44-55) over an
 * in-memory .yalm image; host only.  yalm_tokenize returns the number of ids (out receives at most cap of them),
 * yalm_detokenize the byte length of the text (out receives at most cap - 1 bytes + NUL); negative = error. */
int yalm_tokenize(const void *image, size_t size, const char *text, int add_bos, int *out, int cap);
int yalm_detokenize(const void *image, size_t size, const int *ids, int n, char *out, int cap);

const char *yalm_error_string(int code);
const char *yalm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* YALM_B200_H */
