// The element arithmetic of the operators around the quantized linears, written once with explicit
// roundings so that every kernel that folds one of them into its prologue or epilogue produces the same bits as
// the stand-alone operator kernel.
#pragma once

namespace inkq {

// SiLU(a) * b  (Qwen3SiLuMul, qwen3/src/qwen/QwenOperator.cc:697-722)
__device__ __forceinline__ float silu_mul(float a, float b)
{
    return __fmul_rn(__fdiv_rn(a, __fadd_rn(1.0f, __expf(-a))), b);
}

// ss + |v|^2 of four values, fixed order
__device__ __forceinline__ float add_sumsq4(float ss, const float4 v)
{
    return __fadd_rn(ss, __fmaf_rn(v.w, v.w, __fmaf_rn(v.z, v.z, __fmaf_rn(v.y, v.y, __fmul_rn(v.x, v.x)))));
}

// 1 / sqrt(mean of squares + eps)  (Qwen3RMSNorm::forward, qwen3/src/qwen/QwenOperator.cc:24-53)
__device__ __forceinline__ float rms_inv(float sumsq, int dim, float eps)
{
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, static_cast<float>(dim)), eps)));
}

// (x * inv) * g for four values
__device__ __forceinline__ float4 rms_scale4(const float4 v, float inv, const float4 g)
{
    return make_float4(__fmul_rn(__fmul_rn(v.x, inv), g.x), __fmul_rn(__fmul_rn(v.y, inv), g.y), __fmul_rn(__fmul_rn(v.z, inv), g.z),
                       __fmul_rn(__fmul_rn(v.w, inv), g.w));
}

// Per-head RMSNorm (weights nw) and rotate-half RoPE (tables cs / sn of the token's position) of a 128-element head that
// one warp holds as v[i] = x[lane + 32 i]  (qwen3/src/qwen/QwenAttention.cc:85-92, qwen3/src/ops/RotaryPosEmb.cc:6-79):
// out[j] = x[j] cos[j] + rot[j] sin[j], rot[j] = -x[j + 64] for j < 64, x[j - 64] otherwise; the partners sit in one lane.
__device__ __forceinline__ void head_norm_rope(float (&v)[4], int lane, const float *__restrict__ nw, const float *__restrict__ cs,
                                               const float *__restrict__ sn, float eps, float (&r)[4])
{
    float ss = __fmaf_rn(v[3], v[3], __fmaf_rn(v[2], v[2], __fmaf_rn(v[1], v[1], __fmul_rn(v[0], v[0]))));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    const float inv = rms_inv(ss, 128, eps);
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = __fmul_rn(__fmul_rn(v[i], inv), nw[lane + 32 * i]);
    r[0] = __fmaf_rn(v[0], cs[lane], -__fmul_rn(v[2], sn[lane]));
    r[1] = __fmaf_rn(v[1], cs[lane + 32], -__fmul_rn(v[3], sn[lane + 32]));
    r[2] = __fmaf_rn(v[2], cs[lane + 64], __fmul_rn(v[0], sn[lane + 64]));
    r[3] = __fmaf_rn(v[3], cs[lane + 96], __fmul_rn(v[1], sn[lane + 96]));
}

}  // namespace inkq
