// Offline weight quantizers on the GPU: fp32 weights [N][K] -> the reference's on-disk format
// (packed nibbles u8 [N][K/2] in the AWQ-interleaved order, scales and minima f32 [N][K/32],
// zero points i8 [N][K/32]), so that a checkpoint can be packed without the export notebooks.
//
// Restates notebooks/quantize_methods.py of the reference, operation for operation in fp32:
//   quantize_row_q41_tinyml (:68-125)  d = (max - min) / 15, m = min, id = d != 0 ? 1 / d : 0,
//                                      q = clip(rint((x - m) * id), 0, 15)      (np.round: ties to even), zp = 0
//   quantize_row_q40_tinyml (:13-66)   d = x[argmax |x|] / -8 (first index on ties), id likewise,
//                                      q = (uint8) clip(x * id + 8.5, 0, 15)    (truncation), m = 0, zp = 8
//   both: byte[32 g + e] = q[64 g + e] | q[64 g + 32 + e] << 4                  (:61-64, :120-123)
// One warp per pair of blocks (64 weights): lane e owns element e of both blocks and writes byte e.
#include "inkq_internal.h"

namespace inkq {

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_min(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// value of the element with the largest magnitude, lowest index on ties (np.argmax)
__device__ __forceinline__ float warp_first_absmax_value(float x, int lane)
{
    float best = fabsf(x), val = x;
    int idx = lane;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o), ov = __shfl_xor_sync(0xffffffffu, val, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi < idx)) {
            best = ob;
            val = ov;
            idx = oi;
        }
    }
    return val;
}

template <int FORMAT>   // 0: Q4_0, 1: Q4_1
__device__ __forceinline__ uint32_t quantize_block(float x, int lane, float &d_out, float &m_out)
{
    float dd, mm, v;
    if (FORMAT == 1) {
        const float mx = warp_max(x);
        mm = warp_min(x);
        dd = __fdiv_rn(__fsub_rn(mx, mm), 15.0f);
        const float id = (dd != 0.0f) ? __fdiv_rn(1.0f, dd) : 0.0f;
        v = rintf(__fmul_rn(__fsub_rn(x, mm), id));
    } else {
        dd = __fdiv_rn(warp_first_absmax_value(x, lane), -8.0f);
        mm = 0.0f;
        const float id = (dd != 0.0f) ? __fdiv_rn(1.0f, dd) : 0.0f;
        v = __fadd_rn(__fmul_rn(x, id), 8.5f);
    }
    v = fminf(fmaxf(v, 0.0f), 15.0f);
    d_out = dd;
    m_out = mm;
    return static_cast<uint32_t>(v);   // truncation, as astype(np.uint8) of a value in [0, 15]
}

template <int FORMAT>
__global__ void __launch_bounds__(256) k_quantize_weight_q4(const float *__restrict__ w, int N, int K, uint8_t *__restrict__ nib,
                                                            float *__restrict__ d, float *__restrict__ m, int8_t *__restrict__ zp)
{
    const long long pair = static_cast<long long>(blockIdx.x) * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    const int pairs_per_row = K / 64;
    if (pair >= static_cast<long long>(N) * pairs_per_row) return;
    const long long n = pair / pairs_per_row;
    const int g = static_cast<int>(pair % pairs_per_row);
    const float *src = w + n * K + static_cast<long long>(g) * 64;
    float d_lo, m_lo, d_hi, m_hi;
    const uint32_t q_lo = quantize_block<FORMAT>(src[lane], lane, d_lo, m_lo);
    const uint32_t q_hi = quantize_block<FORMAT>(src[32 + lane], lane, d_hi, m_hi);
    nib[n * (K / 2) + static_cast<long long>(g) * 32 + lane] = static_cast<uint8_t>(q_lo | (q_hi << 4));
    if (lane == 0) {
        const long long b = n * (K / QK) + 2 * g;
        d[b] = d_lo;
        d[b + 1] = d_hi;
        m[b] = m_lo;
        m[b + 1] = m_hi;
        if (zp != nullptr) zp[b] = zp[b + 1] = (FORMAT == 0) ? 8 : 0;
    }
}

}  // namespace inkq

using namespace inkq;

extern "C" int inkq_weight_quantize_dev(inkq_ctx *ctx, int format, int N, int K, const float *w_dev, uint8_t *nib_dev, float *d_dev, float *m_dev,
                                        int8_t *zp_dev)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    INKQ_REQUIRE(ctx, format == 0 || format == 1, "format must be 0 (Q4_0) or 1 (Q4_1)");
    INKQ_REQUIRE(ctx, N >= 1 && K >= 64 && K % 64 == 0, "K must be a positive multiple of 64");
    INKQ_REQUIRE(ctx, w_dev && nib_dev && d_dev && m_dev, "null pointer");
    const long long pairs = static_cast<long long>(N) * (K / 64);
    const unsigned grid = static_cast<unsigned>((pairs + 7) / 8);
    if (format == 1) k_quantize_weight_q4<1><<<grid, 256, 0, ctx->stream>>>(w_dev, N, K, nib_dev, d_dev, m_dev, zp_dev);
    else k_quantize_weight_q4<0><<<grid, 256, 0, ctx->stream>>>(w_dev, N, K, nib_dev, d_dev, m_dev, zp_dev);
    return after_launch(ctx, "k_quantize_weight_q4");
}
