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
// Mapping: 2 lanes own one block (four interleaved float4 each), so the two IEEE
// divisions are done twice per block, not eight times, four 128-bit loads are in
// flight per lane and every load instruction of a warp touches whole 32-byte
// sectors; max and sum need one xor-shuffle, and the pair trades its packed words so that each lane
// stores 16 contiguous bytes.  HBM-bound: 4 bytes read and 1.375 bytes written per element.
#include <cuda_fp16.h>

#include "glue_math.cuh"
#include "inkq_internal.h"

namespace inkq {

__device__ __forceinline__ uint32_t pack_sat_s8x4(int a, int b, int c, int d)
{
    // two cvt.pack instructions: saturate four s32 to s8 and pack them into one word (a in the low byte).
    // cvt.pack d, x, y, z gives (z << 16) | (sat(x) << 8) | sat(y).
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
    return out;
}

// SILU_MUL: x is the output of a fused gate_up projection, [M][2K] in (32 gate, 32 up) column groups, and the
// quantized row is SiLU(gate) * up (Qwen3SiLuMul, qwen3/src/qwen/QwenOperator.cc:697-722) - the same bits as
// k_silu_mul_rows followed by the plain quantizer, without the fp32 round trip through memory.
template <bool SILU_MUL>
__global__ void __launch_bounds__(256) k_quantize_q8(const float4 *__restrict__ x, int M, int K, int M_ld, int mode,
                                                     int8_t *__restrict__ q, float *__restrict__ d, float *__restrict__ s,
                                                     int32_t *__restrict__ isum, int ld)
{
    // x, q and the planes point at the first of the M rows this launch quantizes; M_ld = M rounded up to 4 (the padding
    // rows of the planes are zeroed), ld = distance between two blocks' entries in the planes (>= M_ld: a launch may fill
    // a window of rows of a larger matrix)
    // lets a dependent kernel launched with programmatic stream serialization (the decode QGEMV) start
    // its weight prefetch while this grid runs; it still waits for this grid's completion before reading
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int nb = K / QK;
    const long long gthread = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long blk = gthread >> 1;  // global block index over [M_ld][nb]; two lanes per block
    const int half = threadIdx.x & 1;
    const unsigned gmask = 0x3u << (threadIdx.x & 30);  // the two lanes of this block
    if (blk >= static_cast<long long>(M_ld) * nb) return;  // both lanes of a block leave together
    // consecutive lane pairs take consecutive rows m of the same block column b: the scale planes are
    // [nb][M_ld], so a warp writes 16 consecutive entries of each plane (64 contiguous bytes) instead of
    // 16 scattered words, and still reads one full 128-byte line of x per pair
    const int b = static_cast<int>(blk / M_ld);
    const int m = static_cast<int>(blk % M_ld);
    const size_t plane = static_cast<size_t>(b) * ld + m;
    if (m >= M) {  // padding rows of the scale planes read as zero
        if (half == 0) {
            d[plane] = 0.0f;
            s[plane] = 0.0f;
            isum[plane] = 0;
        }
        return;
    }
    // lane `half` takes the float4s 2j + half of the block: each load instruction of the warp touches
    // 16 blocks x 32 contiguous bytes (whole sectors), four loads in flight per lane
    float4 v[4];
    if (SILU_MUL) {
        const float4 *src = x + (static_cast<size_t>(m) * 2 * K + static_cast<size_t>(b) * 2 * QK) / 4 + half;
        float4 g[4], u[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            g[j] = src[2 * j];
            u[j] = src[2 * j + QK / 4];
        }
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = make_float4(silu_mul(g[j].x, u[j].x), silu_mul(g[j].y, u[j].y), silu_mul(g[j].z, u[j].z), silu_mul(g[j].w, u[j].w));
    } else {
        const float4 *src = x + (static_cast<size_t>(m) * K + static_cast<size_t>(b) * QK) / 4 + half;
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = src[2 * j];
    }
    float mx = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; j++) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
    // the two lanes of a block always take the same branches, so the pair mask is exact
    mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
    const float dd = __fdiv_rn(mx, 127.0f);
    const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
    int sum = 0;
    uint32_t wq[4];   // this lane's words 2j + half of the block's eight
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int i0 = __float2int_rn(__fmul_rn(v[j].x, id));
        const int i1 = __float2int_rn(__fmul_rn(v[j].y, id));
        const int i2 = __float2int_rn(__fmul_rn(v[j].z, id));
        const int i3 = __float2int_rn(__fmul_rn(v[j].w, id));
        sum += (i0 + i1) + (i2 + i3);   // the unsaturated values, as the reference sums them before packing
        wq[j] = pack_sat_s8x4(i0, i1, i2, i3);
    }
    sum += __shfl_xor_sync(gmask, sum, 1);
    // the pair trades words so that lane 0 holds words 0..3 and lane 1 words 4..7: one 16-byte store each, the block's 32
    // bytes leave as a whole sector (four scattered 4-byte stores per lane cost a quarter of the kernel at M = 8192)
    const uint32_t xa = __shfl_xor_sync(gmask, half ? wq[0] : wq[2], 1);
    const uint32_t xb = __shfl_xor_sync(gmask, half ? wq[1] : wq[3], 1);
    reinterpret_cast<uint4 *>(q)[(static_cast<size_t>(m) * K + static_cast<size_t>(b) * QK) / 16 + half] =
        half ? make_uint4(xa, wq[2], xb, wq[3]) : make_uint4(wq[0], xa, wq[1], xb);
    if (half == 0) {
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
    const long long threads = static_cast<long long>(M_ld) * (K / QK) * 2;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    k_quantize_q8<false><<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(x), M, K, M_ld, qmode, a->q, a->d, a->s, a->isum, M_ld);
    a->M = M;
    a->M_ld = M_ld;
    a->qmode = qmode;
    a->ssq_parts = 0;
    return after_launch(ctx, "k_quantize_q8");
}

// Rows [m0, m0 + rows) of a matrix of M_total rows whose other rows are quantized by other launches into the same handle
// (m0 a multiple of 4).  x points at row m0.
int launch_quantize_rows(inkq_ctx *ctx, int qmode, const float *x, int m0, int rows, int M_total, int K, Act *a)
{
    const int ld = (M_total + 3) & ~3, rows_ld = (rows + 3) & ~3;
    const long long threads = static_cast<long long>(rows_ld) * (K / QK) * 2;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    k_quantize_q8<false><<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(x), rows, K, rows_ld, qmode, a->q + static_cast<size_t>(m0) * K,
                                                         a->d + m0, a->s + m0, a->isum + m0, ld);
    a->M = M_total;
    a->M_ld = ld;
    a->qmode = qmode;
    a->ssq_parts = 0;
    return after_launch(ctx, "k_quantize_q8 (row window)");
}

int launch_silu_mul_quantize(inkq_ctx *ctx, int qmode, const float *gu, int M, int K, Act *a)
{
    const int M_ld = (M + 3) & ~3;
    const long long threads = static_cast<long long>(M_ld) * (K / QK) * 2;
    const unsigned grid = static_cast<unsigned>((threads + 255) / 256);
    k_quantize_q8<true><<<grid, 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(gu), M, K, M_ld, qmode, a->q, a->d, a->s, a->isum, M_ld);
    a->M = M;
    a->M_ld = M_ld;
    a->qmode = qmode;
    a->ssq_parts = 0;
    return after_launch(ctx, "k_quantize_q8<silu_mul>");
}

}  // namespace inkq
