// CUDA-core QGEMM and the int32 block-dot dump.
//
// k_qgemm_simt computes one output per thread in exactly the reference's operation
// order (gemm_repack_A81W41_fp32, qwen3/src/qwen/quantized_gemx_kernels.cc:495-512;
// gemm_repack_A80W40, :323-330), from the same device layouts the tensor-core
// kernel reads.  It is the on-device cross-check of that kernel, not a fast path.
// k_block_dots writes every int32 block dot, [M][rows][K/32].
#include <cuda_fp16.h>

#include "inkq_internal.h"

namespace inkq {

__device__ __forceinline__ float4 load_scales(const Weight &w, size_t rec)
{
    if (w.sc32 != nullptr) return w.sc32[rec];
    const uint2 pk = w.sc16[rec];
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&pk.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&pk.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

__device__ __forceinline__ void pair_dots(const Weight &w, int t, int p, int r, const int8_t *__restrict__ arow, int &ilo, int &ihi)
{
    const uint4 c0 = *reinterpret_cast<const uint4 *>(w.nibT + nib_offset(w.pairs, t, p, r, 0));
    const uint4 c1 = *reinterpret_cast<const uint4 *>(w.nibT + nib_offset(w.pairs, t, p, r, 1));
    const uchar2 z = w.zpT[(static_cast<size_t>(t) * w.pairs + p) * TILE_N + r];
    const uint32_t wd[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const uint32_t *a32 = reinterpret_cast<const uint32_t *>(arow + static_cast<size_t>(p) * 64);
    ilo = 0;
    ihi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t al = a32[i], ah = a32[8 + i];
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int ql = static_cast<int>((wd[i] >> (8 * e)) & 0xf) - z.x;
            const int qh = static_cast<int>((wd[i] >> (8 * e + 4)) & 0xf) - z.y;
            ilo += ql * static_cast<int>(static_cast<int8_t>((al >> (8 * e)) & 0xff));
            ihi += qh * static_cast<int>(static_cast<int8_t>((ah >> (8 * e)) & 0xff));
        }
    }
}

__global__ void __launch_bounds__(256) k_qgemm_simt(Weight w, const int8_t *__restrict__ q, const float *__restrict__ d,
                                                    const float *__restrict__ s, int M, int M_ld, float *__restrict__ C, int ldc)
{
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (n >= w.rows || m >= M) return;
    const int t = n / TILE_N, r = n % TILE_N;
    const int8_t *arow = q + static_cast<size_t>(m) * w.K;
    float acc = 0.0f;
    for (int p = 0; p < w.pairs; p++) {
        int ilo, ihi;
        pair_dots(w, t, p, r, arow, ilo, ihi);
        const float4 sc = load_scales(w, (static_cast<size_t>(t) * w.pairs + p) * TILE_N + r);
        const size_t ab = static_cast<size_t>(2 * p) * M_ld + m;
        acc = fmaf(static_cast<float>(ilo), __fmul_rn(d[ab], sc.x), acc);
        acc = fmaf(static_cast<float>(ihi), __fmul_rn(d[ab + M_ld], sc.y), acc);
        if (w.scheme == INKQ_A81W41) {
            acc = fmaf(sc.z, s[ab], acc);
            acc = fmaf(sc.w, s[ab + M_ld], acc);
        }
    }
    C[static_cast<size_t>(m) * ldc + n] = acc;
}

__global__ void __launch_bounds__(256) k_block_dots(Weight w, const int8_t *__restrict__ q, int M, int32_t *__restrict__ dots)
{
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (n >= w.rows || m >= M) return;
    const int t = n / TILE_N, r = n % TILE_N;
    const int8_t *arow = q + static_cast<size_t>(m) * w.K;
    int32_t *out = dots + (static_cast<size_t>(m) * w.rows + n) * (w.K / QK);
    for (int p = 0; p < w.pairs; p++) {
        int ilo, ihi;
        pair_dots(w, t, p, r, arow, ilo, ihi);
        out[2 * p] = ilo;
        out[2 * p + 1] = ihi;
    }
}

int launch_gemm_simt(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, int ldc)
{
    dim3 grid((w->rows + 31) / 32, (a->M + 7) / 8);
    k_qgemm_simt<<<grid, 256, 0, ctx->stream>>>(*w, a->q, a->d, a->s, a->M, a->M_ld, C, ldc);
    return after_launch(ctx, "k_qgemm_simt");
}

int launch_block_dots(inkq_ctx *ctx, const Act *a, const Weight *w, int32_t *dots)
{
    dim3 grid((w->rows + 31) / 32, (a->M + 7) / 8);
    k_block_dots<<<grid, 256, 0, ctx->stream>>>(*w, a->q, a->M, dots);
    return after_launch(ctx, "k_block_dots");
}

}  // namespace inkq
