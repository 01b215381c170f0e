// fp16-weight matmul (lm_head: fp32 activations x fp16 weights, fp32 accumulate) and
// the CUDA-core weight-only W41 matmul (fp16 activations x dequantised Q4_1 weights).
//
// Neither has a C++ kernel in the reference.  lm_head follows the arithmetic of
// gemv_fp32_rcr_mt_impl_1 (qwen3/src/qwen/fp32_gemx_kernels_rcr.cc:494-507):
// logits[n] = sum_k x[k] * w[n][k].  Weight-only W41 follows
// notebooks/evaluate-qwen3_8b_W4.ipynb cell 13: the weight is replaced by
// w16 = fp16(q*d + m) and a stock fp16 linear with fp32 accumulation runs.
//
// k_f16w_gemv is bandwidth-bound: one warp per weight row, 128-bit streaming loads,
// eight loads in flight per lane, activations staged once per CTA in shared memory.
// Reduction order (fixed): lane l accumulates the 8-element chunks c with
// c % 32 == l in ascending order, then a 5-step xor-shuffle tree combines the lanes.
// Algorithmic bytes per launch: rows*K*2 weight bytes + M*K*4 activation bytes +
// M*rows*4 output bytes.
#include <cuda_fp16.h>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

#ifndef INKQ_F16W_UNROLL
#define INKQ_F16W_UNROLL 8   // 16-byte loads in flight per lane (4: 5.3 TB/s, 8: 6.4 TB/s, 16: 6.0 TB/s on the 1.2 GB lm_head)
#endif
constexpr int F16W_UNROLL = INKQ_F16W_UNROLL;

template <int MT>
__global__ void __launch_bounds__(256) k_f16w_gemv(const uint16_t *__restrict__ w, const float *__restrict__ x, int m0, int M, int rows, int K,
                                                   float *__restrict__ C, int ldc, const ExtraDst extra)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *xs = reinterpret_cast<float *>(smem_raw);  // [MT][K]
    const int mt = min(MT, M - m0);
    for (int i = threadIdx.x; i < MT * K / 4; i += blockDim.x) {
        const int r = (i * 4) / K;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < mt) v = reinterpret_cast<const float4 *>(x + static_cast<size_t>(m0) * K)[i];
        reinterpret_cast<float4 *>(xs)[i] = v;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = K / 8;
    for (int n = blockIdx.x * 8 + warp; n < rows; n += gridDim.x * 8) {
        const uint16_t *wrow = w + static_cast<size_t>(n) * K;
        float acc[MT];
#pragma unroll
        for (int j = 0; j < MT; j++) acc[j] = 0.0f;
        for (int c0 = lane; c0 < chunks; c0 += 32 * F16W_UNROLL) {
            uint4 v[F16W_UNROLL];
#pragma unroll
            for (int u = 0; u < F16W_UNROLL; u++) {
                const int c = c0 + u * 32;
                v[u] = (c < chunks) ? ldg_stream_v4(wrow + static_cast<size_t>(c) * 8) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < F16W_UNROLL; u++) {
                const int c = c0 + u * 32;
                if (c < chunks) {
                    const uint32_t wd[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                    float wf[8];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&wd[i]));
                        wf[2 * i] = f.x;
                        wf[2 * i + 1] = f.y;
                    }
#pragma unroll
                    for (int j = 0; j < MT; j++) {
                        const float4 xa = *reinterpret_cast<const float4 *>(xs + j * K + c * 8);
                        const float4 xb = *reinterpret_cast<const float4 *>(xs + j * K + c * 8 + 4);
                        acc[j] = fmaf(xa.x, wf[0], acc[j]);
                        acc[j] = fmaf(xa.y, wf[1], acc[j]);
                        acc[j] = fmaf(xa.z, wf[2], acc[j]);
                        acc[j] = fmaf(xa.w, wf[3], acc[j]);
                        acc[j] = fmaf(xb.x, wf[4], acc[j]);
                        acc[j] = fmaf(xb.y, wf[5], acc[j]);
                        acc[j] = fmaf(xb.z, wf[6], acc[j]);
                        acc[j] = fmaf(xb.w, wf[7], acc[j]);
                    }
                }
            }
        }
#pragma unroll
        for (int j = 0; j < MT; j++) {
            float v = acc[j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0 && j < mt) {
                const size_t off = static_cast<size_t>(m0 + j) * ldc + n;
                C[off] = v;
#pragma unroll
                for (int e = 0; e < MAX_PEERS - 1; e++)   // further destinations (peers of a row-sharded matrix)
                    if (e < extra.n) extra.p[e][off] = v;
            }
        }
    }
}

int launch_f16w_matmul(inkq_ctx *ctx, const F16W *w, const float *x, int M, float *C, int ldc, const ExtraDst *extra_in)
{
    ExtraDst extra = {};
    if (extra_in != nullptr) extra = *extra_in;
    const int grid = min((w->rows + 7) / 8, ctx->num_sms * 8);
    if (M == 1) {
        const size_t smem = static_cast<size_t>(w->K) * sizeof(float);
        if (smem > 48 * 1024) cudaFuncSetAttribute(k_f16w_gemv<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        k_f16w_gemv<1><<<grid, 256, smem, ctx->stream>>>(w->w, x, 0, M, w->rows, w->K, C, ldc, extra);
        return after_launch(ctx, "k_f16w_gemv");
    }
    const size_t smem = 4 * static_cast<size_t>(w->K) * sizeof(float);
    if (smem > 200 * 1024) return fail(ctx, INKQ_ERR_UNSUPPORTED, "K too large for the fp16-weight matmul");
    if (smem > 48 * 1024) cudaFuncSetAttribute(k_f16w_gemv<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    for (int m0 = 0; m0 < M; m0 += 4) {
        k_f16w_gemv<4><<<grid, 256, smem, ctx->stream>>>(w->w, x, m0, M, w->rows, w->K, C, ldc, extra);
        int rc = after_launch(ctx, "k_f16w_gemv");
        if (rc) return rc;
    }
    return INKQ_OK;
}

// Weight-only W41 on the CUDA cores (cross-check of the tensor-core kernel): one output per thread,
// k ascending, fp32 accumulate: acc = fma(a16[k], w16, acc) with w16 = the half-precision fma q*d + m
// (one rounding), d and m the layer's fp16 scales.
__global__ void __launch_bounds__(256) k_gemm_w41_f16act(Weight w, const __half *__restrict__ a, int M, float *__restrict__ C, int ldc)
{
    const int n = blockIdx.x * 32 + (threadIdx.x & 31);
    const int m = blockIdx.y * 8 + (threadIdx.x >> 5);
    if (n >= w.rows || m >= M) return;
    const int t = n / TILE_N, r = n % TILE_N;
    const __half *arow = a + static_cast<size_t>(m) * w.K;
    float acc = 0.0f;
    for (int p = 0; p < w.pairs; p++) {
        const uint4 c0 = *reinterpret_cast<const uint4 *>(w.nibT + nib_offset(w.pairs, t, p, r, 0));
        const uint4 c1 = *reinterpret_cast<const uint4 *>(w.nibT + nib_offset(w.pairs, t, p, r, 1));
        const size_t rec = (static_cast<size_t>(t) * w.pairs + p) * TILE_N + r;
        const uint2 pk = w.sc16[rec];
        const __half2 d2 = *reinterpret_cast<const __half2 *>(&pk.x), m2 = *reinterpret_cast<const __half2 *>(&pk.y);
        const uint32_t wd[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int hi = 0; hi < 2; hi++) {
            const __half dd = hi ? __high2half(d2) : __low2half(d2), mm = hi ? __high2half(m2) : __low2half(m2);
#pragma unroll
            for (int e = 0; e < 32; e++) {
                const uint32_t nibble = (wd[e >> 2] >> (8 * (e & 3) + 4 * hi)) & 0xf;
                const float wv = __half2float(__hfma(__ushort2half_rn(static_cast<unsigned short>(nibble)), dd, mm));
                acc = fmaf(__half2float(arow[p * 64 + hi * 32 + e]), wv, acc);
            }
        }
    }
    C[static_cast<size_t>(m) * ldc + n] = acc;
}

int launch_gemm_w41_f16(inkq_ctx *ctx, const uint16_t *a16, int M, const Weight *w, float *C, int ldc)
{
    dim3 grid((w->rows + 31) / 32, (M + 7) / 8);
    k_gemm_w41_f16act<<<grid, 256, 0, ctx->stream>>>(*w, reinterpret_cast<const __half *>(a16), M, C, ldc);
    return after_launch(ctx, "k_gemm_w41_f16act");
}

}  // namespace inkq
