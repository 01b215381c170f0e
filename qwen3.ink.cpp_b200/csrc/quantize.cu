// Fused Q8_0 / Q8_1 activation quantizer.
//
// Reference behaviour reproduced bit-for-bit (qwen3/src/qwen/quantized_gemx_kernels.cc):
//   quantize_row_q8_0_repack       :584-691   (mode 0: fp16 scale, no sum)
//   quantize_row_q8_1_repack_fp16  :693-801   (mode 1: fp16 scale and sum)
//   quantize_row_q8_1_repack_fp32  :803-911   (mode 2: fp32 scale and sum)
// per 32-element block: mx = max|x|, d = mx / 127, id = mx != 0 ? 127 / mx : 0,
// q = sat_s8(rne(x * id)), s = d * (float)sum(q) with the unrounded fp32 d.
// Both divisions are IEEE round-to-nearest, the product x*id is a plain fp32
// multiply (never contracted), the rounding is to nearest-even.
//
// Mapping: 8 lanes own one block (one float4 each, 128 contiguous bytes), so a
// warp covers 4 consecutive blocks with one coalesced 512-byte read; max and sum
// are 3-step xor-shuffles inside the 8-lane group.  HBM-bound: 4 bytes read and
// 1.375 bytes written per element.
#include <cuda_fp16.h>

#include "inkq_internal.h"

namespace inkq {

__global__ void __launch_bounds__(256) k_quantize_q8(const float4 *__restrict__ x, int M, int K, int M_ld, int mode,
                                                     int8_t *__restrict__ q, float *__restrict__ d, float *__restrict__ s,
                                                     int32_t *__restrict__ isum)
{
    // lets a dependent kernel launched with programmatic stream serialization (the decode QGEMV) start
    // its weight prefetch while this grid runs; it still waits for this grid's completion before reading
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nb = K / QK;
    const long long gthread = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long blk = gthread >> 3;  // global block index over [M_ld][nb]
    const int sub = threadIdx.x & 7;
    const unsigned gmask = 0xffu << (threadIdx.x & 24);  // the 8 lanes of this block
    if (blk >= static_cast<long long>(M_ld) * nb) return;  // whole 8-lane groups leave together
    const int m = static_cast<int>(blk / nb);
    const int b = static_cast<int>(blk % nb);
    const size_t plane = static_cast<size_t>(b) * M_ld + m;
    if (m >= M) {  // padding rows of the scale planes read as zero
        if (sub == 0) {
            d[plane] = 0.0f;
            s[plane] = 0.0f;
            isum[plane] = 0;
        }
        return;
    }
    const float4 v = x[(static_cast<size_t>(m) * K + static_cast<size_t>(b) * QK) / 4 + sub];
    float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    // the 8 lanes of a block are aligned inside the warp: xor 1, 2, 4 stays in the group,
    // and a group always takes the same branches, so the group mask is exact
    mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 2));
    mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 4));
    const float dd = __fdiv_rn(mx, 127.0f);
    const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
    const int i0 = __float2int_rn(__fmul_rn(v.x, id));
    const int i1 = __float2int_rn(__fmul_rn(v.y, id));
    const int i2 = __float2int_rn(__fmul_rn(v.z, id));
    const int i3 = __float2int_rn(__fmul_rn(v.w, id));
    int sum = (i0 + i1) + (i2 + i3);
    sum += __shfl_xor_sync(gmask, sum, 1);
    sum += __shfl_xor_sync(gmask, sum, 2);
    sum += __shfl_xor_sync(gmask, sum, 4);
    const int c0 = max(-128, min(127, i0)), c1 = max(-128, min(127, i1));
    const int c2 = max(-128, min(127, i2)), c3 = max(-128, min(127, i3));
    const uint32_t packed = (static_cast<uint32_t>(c0) & 0xffu) | ((static_cast<uint32_t>(c1) & 0xffu) << 8) |
                            ((static_cast<uint32_t>(c2) & 0xffu) << 16) | ((static_cast<uint32_t>(c3) & 0xffu) << 24);
    reinterpret_cast<uint32_t *>(q)[(static_cast<size_t>(m) * K + static_cast<size_t>(b) * QK) / 4 + sub] = packed;
    if (sub == 0) {
        const float ss = __fmul_rn(dd, static_cast<float>(sum));
        if (mode == INKQ_Q8_1_F32) {
            d[plane] = dd;
            s[plane] = ss;
        } else {
            d[plane] = __half2float(__float2half_rn(dd));
            s[plane] = (mode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(ss)) : 0.0f;
        }
        isum[plane] = sum;
    }
}

// Integer block sums of an imported (already quantized) activation matrix: isum[b][m] = sum_e q[m][32b+e].
__global__ void __launch_bounds__(256) k_block_isum(const int8_t *__restrict__ q, int M, int K, int M_ld, int32_t *__restrict__ isum)
{
    const int nb = K / QK;
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(M_ld) * nb) return;
    const int m = static_cast<int>(idx / nb), b = static_cast<int>(idx % nb);
    int acc = 0;
    if (m < M) {
        const int *src = reinterpret_cast<const int *>(q + static_cast<size_t>(m) * K + static_cast<size_t>(b) * QK);
#pragma unroll
        for (int i = 0; i < 8; i++) acc = __dp4a(src[i], 0x01010101, acc);
    }
    isum[static_cast<size_t>(b) * M_ld + m] = acc;
}

int launch_block_isum(inkq_ctx *ctx, Act *a, int M, int M_ld)
{
    const long long total = static_cast<long long>(M_ld) * (a->K / QK);
    k_block_isum<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(a->q, M, a->K, M_ld, a->isum);
    return after_launch(ctx, "k_block_isum");
}

int launch_quantize(inkq_ctx *ctx, int qmode, const float *x, int M, int K, Act *a)
{
    const int M_ld = (M + 3) & ~3;
    const long long threads = static_cast<long long>(M_ld) * (K / QK) * 8;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    k_quantize_q8<<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(x), M, K, M_ld, qmode, a->q, a->d, a->s, a->isum);
    a->M = M;
    a->M_ld = M_ld;
    a->qmode = qmode;
    return after_launch(ctx, "k_quantize_q8");
}

}  // namespace inkq
