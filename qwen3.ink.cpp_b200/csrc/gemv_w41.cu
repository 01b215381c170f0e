// Weight-only W41 for one token (M == 1): C[n] = sum_k a16[k] * w16[n][k], w16 = fp16(q*d + m) (one rounding:
// a half-precision fma), fp32 accumulate.  Same semantic as k_gemm_w41_tc (notebooks/evaluate-qwen3_8b_W4.ipynb
// cell 13 of the reference; no C++ kernel exists there); a tensor-core tile wastes 15/16 of its columns on a
// single row and only offers N/128 work items, so the decode case streams the weights like the A8W4 QGEMV:
// lane = weight row, 8 or 16 warps = K-slices, two batches of two pairs (128-bit loads) in flight per lane.
// Per 4 weights: 2 prmt + 2 sub.f16x2 + 2 fma.f16x2 (dequantise), 4 conversions to fp32, 4 fma with the fp32
// activation values (one 128-bit shared load, broadcast): ~4 instructions per weight, about the HBM time of the layer.
// Reduction order (fixed): k ascending inside a slice, slice partials added in ascending order.
#include <cuda_fp16.h>

#include "inkq_internal.h"
#include "ptx.cuh"
#include "qgemv_common.cuh"

namespace inkq {

// 4 nibbles (one per byte of v, already masked) times 4 activations, accumulated in k order
__device__ __forceinline__ float w41_fma4(uint32_t v, __half2 d2, __half2 m2, const float4 a, float acc)
{
    const uint32_t h01 = __byte_perm(v, 0x64646464u, 0x4140), h23 = __byte_perm(v, 0x64646464u, 0x4342);   // 1024 + q as fp16 bits
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const float2 w01 = __half22float2(__hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&h01), k1024), d2, m2));
    const float2 w23 = __half22float2(__hfma2(__hsub2(*reinterpret_cast<const __half2 *>(&h23), k1024), d2, m2));
    acc = fmaf(a.x, w01.x, acc);
    acc = fmaf(a.y, w01.y, acc);
    acc = fmaf(a.z, w23.x, acc);
    acc = fmaf(a.w, w23.y, acc);
    return acc;
}

template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 3 : 2) k_gemv_w41(const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16,
                                                             const __half *__restrict__ a16, float *__restrict__ C, int rows, int K, int pairs)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *af = reinterpret_cast<float *>(smem_raw);   // K activations widened to fp32 (exact)
    float *part = af + K;                              // [WARPS][32]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x >> 2;
    const int r = ((blockIdx.x & 3) << 5) + lane;
    const bool swz = ((r >> 2) & 1) != 0;
    const int p_begin = (warp * pairs) / WARPS, p_end = ((warp + 1) * pairs) / WARPS;
    const size_t slab = static_cast<size_t>(t) * pairs;
    PairBatch b0, b1;
    if (p_begin < p_end) load_batch<true, false>(b0, nibT, sc16, nullptr, slab, r, p_begin, p_end);
    if (p_begin + GEMV_UNROLL < p_end) load_batch<true, false>(b1, nibT, sc16, nullptr, slab, r, p_begin + GEMV_UNROLL, p_end);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.x; i < K / 2; i += blockDim.x) {
        const float2 f = __half22float2(reinterpret_cast<const __half2 *>(a16)[i]);
        reinterpret_cast<float2 *>(af)[i] = f;
    }
    __syncthreads();

    auto consume = [&](const PairBatch &b, float acc, int p0) {
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; u++) {
            const int p = p0 + u;
            if (p < p_end) {
                const uint4 c0 = swz ? b.cb[u] : b.ca[u], c1 = swz ? b.ca[u] : b.cb[u];   // logical chunks 0 and 1
                const uint32_t wd[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                const __half2 dd = *reinterpret_cast<const __half2 *>(&b.sc[u].x), mm = *reinterpret_cast<const __half2 *>(&b.sc[u].y);
                const __half2 d_lo = __low2half2(dd), d_hi = __high2half2(dd), m_lo = __low2half2(mm), m_hi = __high2half2(mm);
                const float4 *a_lo = reinterpret_cast<const float4 *>(af + p * 64), *a_hi = a_lo + 8;
                // k ascending: the low block (elements 0..31 of the pair), then the high block (32..63)
#pragma unroll
                for (int i = 0; i < 8; i++) acc = w41_fma4(wd[i] & 0x0F0F0F0Fu, d_lo, m_lo, a_lo[i], acc);
#pragma unroll
                for (int i = 0; i < 8; i++) acc = w41_fma4((wd[i] >> 4) & 0x0F0F0F0Fu, d_hi, m_hi, a_hi[i], acc);
            }
        }
        return acc;
    };
    float acc = 0.0f;
    for (int p0 = p_begin; p0 < p_end; p0 += 2 * GEMV_UNROLL) {
        acc = consume(b0, acc, p0);
        if (p0 + 2 * GEMV_UNROLL < p_end) load_batch<true, false>(b0, nibT, sc16, nullptr, slab, r, p0 + 2 * GEMV_UNROLL, p_end);
        if (p0 + GEMV_UNROLL < p_end) {
            acc = consume(b1, acc, p0 + GEMV_UNROLL);
            if (p0 + 3 * GEMV_UNROLL < p_end) load_batch<true, false>(b1, nibT, sc16, nullptr, slab, r, p0 + 3 * GEMV_UNROLL, p_end);
        }
    }
    part[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float tot = part[lane];
#pragma unroll
        for (int w2 = 1; w2 < WARPS; w2++) tot = __fadd_rn(tot, part[w2 * 32 + lane]);
        const int n = t * TILE_N + r;
        if (n < rows) C[n] = tot;
    }
}

template <int WARPS>
static void launch_variant(inkq_ctx *ctx, const uint16_t *a16, const Weight *w, float *C)
{
    const size_t smem = sizeof(float) * (static_cast<size_t>(w->K) + WARPS * 32);
    if (smem > 48 * 1024) cudaFuncSetAttribute(k_gemv_w41<WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_pdl(k_gemv_w41<WARPS>, dim3(static_cast<unsigned>(w->tiles) * 4), dim3(WARPS * 32), smem, ctx->stream, static_cast<const uint8_t *>(w->nibT),
               static_cast<const uint2 *>(w->sc16), reinterpret_cast<const __half *>(a16), C, w->rows, w->K, w->pairs);
}

int launch_gemv_w41(inkq_ctx *ctx, const uint16_t *a16, const Weight *w, float *C)
{
    const bool wide_cta = (w->tiles * 4 <= 2 * ctx->num_sms) || (w->pairs >= 128);
    if (wide_cta) launch_variant<16>(ctx, a16, w, C);
    else launch_variant<8>(ctx, a16, w, C);
    return after_launch(ctx, "k_gemv_w41");
}

}  // namespace inkq
