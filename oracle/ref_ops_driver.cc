// TEST INFRASTRUCTURE ONLY.  C entry points that drive the REFERENCE's own operators around the quantized linear
// layer - compiled unmodified from a checkout of the reference project and linked into oracle/_ref/libinkref_<isa>.so
// (oracle/Makefile, target `ref`) - so that the GPU glue kernels can be compared with them operator by operator.
// Each function only builds the reference's matrix objects around the caller's buffers and calls the reference:
//   refop_rmsnorm     Qwen3RMSNorm::forward                         qwen3/src/qwen/QwenOperator.cc:24-53
//   refop_silu_mul    Qwen3SiLuMul                                  qwen3/src/qwen/QwenOperator.cc:697-712
//   refop_add         add                                           qwen3/src/qwen/QwenOperator.cc:714-721
//   refop_rope        RotaryPosEmb::apply                           qwen3/src/ops/RotaryPosEmb.cc:6-79
//   refop_attention   the attention core of Qwen3Attention::forward qwen3/src/qwen/QwenAttention.cc:122-190 with the
//                     causal mask of Qwen3Model::prepare_decoder_attention_mask (qwen3/src/qwen/QwenDecoder.cc:6-20):
//                     bgemxGQA::forward_ink_kernel_qk, batch_Add, the -inf clamp, softmax, forward_ink_kernel_pv
#include <cmath>
#include <cstring>
#include <limits>

#include "QwenOperator.h"
#include "operators.h"

extern "C" {

void refop_rmsnorm(const float *x, const float *w, int rows, int heads, int dim, float eps, float *out)
{
    Qwen3RMSNorm norm(dim);
    std::memcpy(norm.weight.data(), w, sizeof(float) * dim);
    norm.eps = eps;
    Matrix3D<float> in(x, rows, heads, dim);
    Matrix3D<float> y = norm.forward(in);
    std::memcpy(out, y.data(), sizeof(float) * static_cast<size_t>(rows) * heads * dim);
}

void refop_silu_mul(const float *a, const float *b, int rows, int dim, float *out)
{
    Matrix3D<float> ma(a, 1, rows, dim), mb(b, 1, rows, dim);
    Matrix3D<float> y = Qwen3SiLuMul(ma, mb);
    std::memcpy(out, y.data(), sizeof(float) * static_cast<size_t>(rows) * dim);
}

void refop_add(const float *a, const float *b, int rows, int dim, float *out)
{
    Matrix3D<float> ma(a, 1, rows, dim), mb(b, 1, rows, dim);
    Matrix3D<float> y = add(ma, mb);
    std::memcpy(out, y.data(), sizeof(float) * static_cast<size_t>(rows) * dim);
}

// q [nq][len][head_dim], k [nk][len][head_dim], rotated in place at positions start .. start + len - 1;
// cos / sin tables [max_len][head_dim] (the reference asserts max_len > start + len)
void refop_rope(float *q, float *k, int nq, int nk, int len, int head_dim, int start, const float *cos_t, const float *sin_t, int max_len)
{
    RotaryPosEmb rope;
    rope.cos = Matrix3D<float>(cos_t, 1, max_len, head_dim);
    rope.sin = Matrix3D<float>(sin_t, 1, max_len, head_dim);
    Matrix3D<float> mq(q, nq, len, head_dim), mk(k, nk, len, head_dim);
    rope.apply(mq, mk, start, len);
    std::memcpy(q, mq.data(), sizeof(float) * static_cast<size_t>(nq) * len * head_dim);
    std::memcpy(k, mk.data(), sizeof(float) * static_cast<size_t>(nk) * len * head_dim);
}

// q [nq][sq][hd] (after norm and RoPE), caches [nkv][max_len][hd] already holding past + sq positions;
// out [sq][nq * hd], the layout the output projection consumes
void refop_attention(const float *q, float *k_cache, float *v_cache, int nq, int nkv, int sq, int past, int hd, int max_len, float alpha, float *out)
{
    const int total = past + sq;
    Matrix3D<float> query(q, nq, sq, hd);
    MatrixView<float> kview(k_cache, nkv, total, hd, max_len * hd, hd, 1);
    MatrixView<float> vview(v_cache, nkv, total, hd, max_len * hd, hd, 1);
    Matrix3D<float> mask(1, sq, total);
    const float lowest = std::numeric_limits<float>::lowest();
    for (int i = 0; i < sq; i++)
        for (int j = 0; j < total; j++) mask(0, i, j) = (j <= i + past) ? 0.0f : lowest;
    bgemxGQA qk(alpha, nq, nkv), pv(1.0f, nq, nkv);
    Matrix3D<float> weights(nq, sq, total);
    qk.forward_ink_kernel_qk(query, kview, weights);
    batch_Add(weights, mask, weights);
    for (int i = 0; i < weights.length(); i++)
        if (std::isinf(weights.data()[i])) weights.data()[i] = lowest;
    Matrix3D<float> probs(nq, sq, total);
    softmax(weights, probs);
    Matrix3D<float> o(nq, sq, hd);
    pv.forward_ink_kernel_pv(probs, vview, o);
    Matrix3D<float> r = o.permute01();   // [sq][nq][hd]
    std::memcpy(out, r.data(), sizeof(float) * static_cast<size_t>(sq) * nq * hd);
}

}  // extern "C"
