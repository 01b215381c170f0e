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

}  // namespace inkq
