/*
 * inkq_glue.h - device-resident stand-ins for the operators between the quantized linear
 * layers of a Qwen3 decoder (C ABI, same conventions as inkq.h).
 *
 * They exist so that a whole synthetic Qwen3-8B forward can be timed with its activations on
 * the GPU (prompt prefill + greedy decode); they are simple and correct, not tuned, and they
 * are not part of the quantized-matmul path itself.  Each cites the reference code whose
 * behaviour it follows.  Activations are fp32 row-major [tokens][features]; `pos0_dev` points
 * to the position of the call's first token in device memory, so a captured CUDA graph of one
 * decode step can be replayed for every step.
 */
#ifndef INKQ_GLUE_H
#define INKQ_GLUE_H

#include "inkq.h"

#ifdef __cplusplus
extern "C" {
#endif

/* out[t][:] = table[tokens[t]][:]  (fp16 table [vocab][dim]; ids are clamped to the table).  qwen3/src/ops/embedding.cc:11-26 */
int inkq_glue_embedding(inkq_ctx *ctx, const uint16_t *table16_dev, const int *tokens_dev, int T, int dim, int vocab, float *out_dev);
/* y = x * rsqrt(mean(x^2) + eps) * w per row.  Qwen3RMSNorm::forward, qwen3/src/qwen/QwenOperator.cc:24-53 */
int inkq_glue_rmsnorm(inkq_ctx *ctx, const float *x_dev, const float *w_dev, int rows, int dim, float eps, float *y_dev);
/* Fused qkv output [T][(nq + 2 nkv) * 128] -> per-head RMSNorm of q and k, RoPE (rotate-half form,
 * cos/sin tables [max_pos][128]) at positions pos0 + t, q to q_out [T][nq][128] fp32, k and v
 * appended to the fp16 caches [nkv][max_pos][128].  qwen3/src/qwen/QwenAttention.cc:78-121,
 * qwen3/src/ops/RotaryPosEmb.cc:6-79 */
int inkq_glue_qknorm_rope_cache(inkq_ctx *ctx, const float *qkv_dev, const float *q_norm_w, const float *k_norm_w, const float *cos_dev,
                                const float *sin_dev, const int *pos0_dev, int T, int nq, int nkv, int max_pos, float eps, float *q_out_dev,
                                uint16_t *k_cache_dev, uint16_t *v_cache_dev);
/* Causal grouped-query attention of T query tokens over cache positions 0 .. pos0 + t, softmax in
 * fp32; out [T][nq * 128].  qwen3/src/qwen/QwenAttention.cc:154-190, qwen3/src/ops/softmax.cc:53-85 */
int inkq_glue_attention(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev, int T,
                        int nq, int nkv, int max_pos, float scale, float *out_dev);
/* out = silu(gate) * up.  Qwen3SiLuMul, qwen3/src/qwen/QwenOperator.cc:697-722 */
int inkq_glue_silu_mul(inkq_ctx *ctx, const float *gate_dev, const float *up_dev, long long n, float *out_dev);
/* The same on the output of a fused gate_up projection whose columns come in (32 gate, 32 up) groups:
 * gu [T][2F], out[t][k] = SiLU(gu[t][64*(k/32) + k%32]) * gu[t][64*(k/32) + 32 + k%32]. */
int inkq_glue_silu_mul_rows(inkq_ctx *ctx, const float *gu_dev, int T, int F, float *out_dev);
/* One decode-step layer in one launch (no counterpart in the reference, which runs these as separate
 * operators: QwenDecoderLayer.cc:66-105): the M == 1 forward of inkq_linear on
 *   pro 0: x                      pro 1: RMSNorm(x; g, eps)          pro 2: SiLU(gate) * up of a 2K-row in (32 gate, 32 up) groups
 * with the activation quantizer inside the QGEMV's prologue (same arithmetic as inkq_quantize), and
 * accumulate != 0 adding the result onto C (the residual connection) instead of overwriting it. */
int inkq_glue_linear_m1(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int pro, const float *g_dev, float eps, float *C_dev,
                        int accumulate);
/* ---- decode step with the activation work in the producers' epilogues -----------------------
 * No counterpart in the reference (separate operators, QwenDecoderLayer.cc:66-105).  Every matrix-vector
 * product reads a ready quantized row (an activation handle holding M == 1) and the kernel that produces
 * a layer's input also quantizes it:
 *   inkq_glue_decode_gemv, epilogue 0: C = y      1: C += y      2: C += y, then RMSNorm(C; norm_w, eps) of the
 *       whole row quantized into `out` by the CTA that finishes last (xn_out_dev, if not NULL, also receives
 *       the normalized fp32 row)      3: the weight's rows are (32 gate, 32 up) groups - row 64b+e is gate
 *       row 32b+e, row 64b+32+e is up row 32b+e of a fused gate_up projection - and SiLU(gate)*up is quantized
 *       into `out` (C_dev unused)      4: C += y; the CTA's 32 results times norm_w are quantized into `out` at once,
 *       WITHOUT the row's RMS factor, which stays pending in the handle (sums of squares per 32 results) and is applied
 *       to the finished sums by the inkq_glue_decode_gemv call that reads `out` (W (f v) = f (W v)): same result as
 *       epilogue 2 up to a last-bit difference before the rounding to int8, without any whole-row pass.  Such a handle
 *       is only valid as the `in` of inkq_glue_decode_gemv (inkq_act_export shows its raw, unscaled content)
 *   inkq_glue_rmsnorm_quant: the same RMSNorm + quantizer for a row that no product made (after the embedding)
 *   inkq_glue_attention_quant: inkq_glue_attention for one token with its output quantized into `out`
 * `out` must have been created with inkq_act_create(ctx, 1, K_of_the_produced_row); out_qmode is the mode
 * the consuming layer's M == 1 path uses (INKQ_Q8_1_F16 for A81W41, INKQ_Q8_0_F16 for the A80 schemes).
 * Results equal the separate operators' except for the summation order inside RMSNorm. */
int inkq_glue_decode_gemv(inkq_ctx *ctx, const inkq_weight *w, const inkq_act *in, float *C_dev, int epilogue, const float *norm_w_dev, float eps,
                          inkq_act *out, int out_qmode, float *xn_out_dev);
int inkq_glue_rmsnorm_quant(inkq_ctx *ctx, const float *x_dev, const float *norm_w_dev, float eps, int K, inkq_act *out, int out_qmode,
                            float *xn_out_dev);
int inkq_glue_attention_quant(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev,
                              int nq, int nkv, int max_pos, float scale, inkq_act *out, int out_qmode);
/* ---- prompt path with the element-wise operators folded into the quantizer ------------------
 * No counterpart in the reference (separate operators on host matrices, QwenDecoderLayer.cc:57-105).  They write the
 * quantized rows straight into an activation handle (inkq_act_create(ctx, rows >= M, K)) that inkq_gemm then
 * consumes; the bits equal those of the separate operators followed by inkq_quantize.
 *   inkq_glue_add_rmsnorm_quant_rows: x[M][K] += delta[M][K] (skipped when delta_dev is NULL; x is updated in place),
 *       then RMSNorm(x; norm_w, eps) quantized into `out` (xn_out_dev, if not NULL, also receives the normalized rows)
 *   inkq_glue_silu_mul_quant_rows: gu [M][2F] in (32 gate, 32 up) column groups -> SiLU(gate) * up quantized into `out`
 * out_qmode: INKQ_Q8_1_F32 for an A81W41 layer with M > 1 (what inkq_linear uses), INKQ_Q8_0_F16 for the A80 schemes. */
int inkq_glue_add_rmsnorm_quant_rows(inkq_ctx *ctx, float *x_dev, const float *delta_dev, const float *norm_w_dev, float eps, int M, int K,
                                     inkq_act *out, int out_qmode, float *xn_out_dev);
int inkq_glue_silu_mul_quant_rows(inkq_ctx *ctx, const float *gu_dev, int M, int F, inkq_act *out, int out_qmode);
/* inkq_glue_attention for T tokens of one prompt with its output quantized into rows row0 .. row0 + T - 1 of `out`
 * (created for K = nq * 128 and at least total_rows rows; a batch of prompts calls it once per prompt with the same
 * total_rows, and the handle is complete when every row has been written). */
int inkq_glue_attention_quant_rows(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev,
                                   int T, int nq, int nkv, int max_pos, float scale, inkq_act *out, int out_qmode, int row0, int total_rows);
/* One token: inkq_glue_qknorm_rope_cache and inkq_glue_attention_quant in one kernel.  Starts from the fused qkv
 * projection's output row [(nq + 2 nkv) * 128]: per-head RMSNorm + RoPE of the query heads and of the new key, the new
 * key and value appended to the caches at position *pos0, attention over positions 0 .. *pos0, output quantized into
 * `out`.  Same arithmetic as the two calls; nq * 4 must not exceed twice the SM count. */
int inkq_glue_qkv_attention_quant(inkq_ctx *ctx, const float *qkv_dev, const float *q_norm_w, const float *k_norm_w, const float *cos_dev,
                                  const float *sin_dev, const int *pos0_dev, int nq, int nkv, int max_pos, float eps, float scale,
                                  uint16_t *k_cache_dev, uint16_t *v_cache_dev, inkq_act *out, int out_qmode);
/* a += b (residual).  qwen3/src/qwen/QwenDecoderLayer.cc:73,105 */
int inkq_glue_add_inplace(inkq_ctx *ctx, float *a_dev, const float *b_dev, long long n);
/* Greedy sampling: *token_out = argmax(logits) (first index on ties), appended to generated
 * (generated[0] = count, tokens follow; may be NULL), then *pos += advance.
 * qwen3/src/qwen/Pipeline.cc:54-62 */
int inkq_glue_argmax_advance(inkq_ctx *ctx, const float *logits_dev, int n, int *token_out_dev, int *pos_dev, int advance, int *generated_dev,
                             int gen_cap);

#ifdef __cplusplus
}
#endif
#endif /* INKQ_GLUE_H */
