// Decode QGEMV (M == 1): bandwidth-bound streaming of the 4-bit weights.
//
// Stands in for gemv_repack_A81W41_fp16 (qwen3/src/qwen/quantized_gemx_kernels.cc:111-193)
// and gemv_repack_A80W40 (:39-108); the zero-point scheme has no reference kernel and
// follows the same order with q_w = nibble - zp.  Scales are the fp16-rounded ones,
// as in those reference kernels.
//
// Work split: a CTA owns 32 consecutive weight rows (lane = row) and its 8 warps
// own 8 contiguous K-slices.  For one pair (64 K-elements) a warp reads 32 rows x
// 32 bytes = 1 KB contiguous with two 128-bit loads per lane, plus 8 bytes of
// fp16 {d_lo, d_hi, m_lo, m_hi} per lane.  Four pairs are in flight per lane
// (8 x 128-bit loads) before any is consumed.  The activation row (int8 + block
// scales) is staged once per CTA in shared memory and read as broadcasts.
//
// Reduction order (fixed, documented): inside a K-slice the reference's order is
// kept exactly - per pair fma(I_lo, d_a*d_w), fma(I_hi, ...), fma(m_lo, s_lo),
// fma(m_hi, s_hi), pairs ascending from a zero accumulator; the 8 slice partials
// are then added in ascending slice order ((p0 + p1) + p2) ... + p7.  Every int32
// block dot is exact.
//
// Algorithmic bytes per launch: rows*K/2 nibbles + rows*(K/32)*4 scale bytes
// (+ rows*(K/32) zero-point bytes for the A80 schemes) + K + (K/32)*8 activation
// bytes + rows*4 output bytes, i.e. 0.625 B per weight for A81W41.
#include <cuda_fp16.h>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

constexpr int GEMV_WARPS = 8;
constexpr int GEMV_UNROLL = 4;

__device__ __forceinline__ void dots_of_pair(const uint4 c0, const uint4 c1, const uint32_t *__restrict__ a_lo,
                                             const uint32_t *__restrict__ a_hi, int &ilo, int &ihi)
{
    const uint32_t w[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    ilo = 0;
    ihi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        ilo = __dp4a(static_cast<int>(w[i] & 0x0F0F0F0Fu), static_cast<int>(a_lo[i]), ilo);
        ihi = __dp4a(static_cast<int>((w[i] >> 4) & 0x0F0F0F0Fu), static_cast<int>(a_hi[i]), ihi);
    }
}

template <bool HAS_MIN>
__global__ void __launch_bounds__(GEMV_WARPS * 32) k_qgemv_a8w4(const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16,
                                                               const uchar2 *__restrict__ zpT, const int8_t *__restrict__ q,
                                                               const float *__restrict__ d, const float *__restrict__ s,
                                                               const int32_t *__restrict__ isum, int M_ld, float *__restrict__ C,
                                                               int rows, int K, int pairs)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nb = K / QK;
    uint32_t *qa = reinterpret_cast<uint32_t *>(smem_raw);          // K/4 words
    float *da = reinterpret_cast<float *>(smem_raw + K);            // nb
    float *sa = da + nb;                                            // nb (sums, or integer sums for the A80 schemes)
    float *part = sa + nb;                                          // [GEMV_WARPS][32]

    for (int i = threadIdx.x; i < K / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(qa)[i] = reinterpret_cast<const uint4 *>(q)[i];
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        da[b] = d[static_cast<size_t>(b) * M_ld];
        if (HAS_MIN) sa[b] = s[static_cast<size_t>(b) * M_ld];
        else reinterpret_cast<int32_t *>(sa)[b] = isum[static_cast<size_t>(b) * M_ld];
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x >> 2;
    const int r = ((blockIdx.x & 3) << 5) + lane;
    const bool swz = ((r >> 2) & 1) != 0;
    const int p_begin = (warp * pairs) / GEMV_WARPS, p_end = ((warp + 1) * pairs) / GEMV_WARPS;
    const size_t slab = static_cast<size_t>(t) * pairs;
    float acc = 0.0f;

    for (int p0 = p_begin; p0 < p_end; p0 += GEMV_UNROLL) {
        uint4 ca[GEMV_UNROLL], cb[GEMV_UNROLL];
        uint2 sc[GEMV_UNROLL];
        uchar2 z[GEMV_UNROLL];
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; u++) {
            const int p = min(p0 + u, p_end - 1);  // clamped duplicates are loaded but never used
            const size_t rec = (slab + p) * TILE_N + r;
            const uint8_t *src = nibT + rec * 32;
            ca[u] = ldg_stream_v4(src);
            cb[u] = ldg_stream_v4(src + 16);
            sc[u] = ldg_stream_v2(sc16 + rec);
            if (!HAS_MIN) z[u] = zpT[rec];
        }
#pragma unroll
        for (int u = 0; u < GEMV_UNROLL; u++) {
            const int p = p0 + u;
            if (p < p_end) {
                int ilo, ihi;
                dots_of_pair(swz ? cb[u] : ca[u], swz ? ca[u] : cb[u], qa + p * 16, qa + p * 16 + 8, ilo, ihi);
                const float2 dw = __half22float2(*reinterpret_cast<const __half2 *>(&sc[u].x));
                const float da_lo = da[2 * p], da_hi = da[2 * p + 1];
                if (HAS_MIN) {
                    const float2 mw = __half22float2(*reinterpret_cast<const __half2 *>(&sc[u].y));
                    acc = fmaf(static_cast<float>(ilo), __fmul_rn(da_lo, dw.x), acc);
                    acc = fmaf(static_cast<float>(ihi), __fmul_rn(da_hi, dw.y), acc);
                    acc = fmaf(mw.x, sa[2 * p], acc);
                    acc = fmaf(mw.y, sa[2 * p + 1], acc);
                } else {
                    const int32_t *is = reinterpret_cast<const int32_t *>(sa);
                    ilo -= static_cast<int>(z[u].x) * is[2 * p];
                    ihi -= static_cast<int>(z[u].y) * is[2 * p + 1];
                    acc = fmaf(static_cast<float>(ilo), __fmul_rn(da_lo, dw.x), acc);
                    acc = fmaf(static_cast<float>(ihi), __fmul_rn(da_hi, dw.y), acc);
                }
            }
        }
    }
    part[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float tot = part[lane];
#pragma unroll
        for (int w2 = 1; w2 < GEMV_WARPS; w2++) tot = __fadd_rn(tot, part[w2 * 32 + lane]);
        const int n = t * TILE_N + r;
        if (n < rows) C[n] = tot;
    }
}

int launch_gemv(inkq_ctx *ctx, const Act *a, const Weight *w, float *C)
{
    const size_t smem = static_cast<size_t>(w->K) + 2 * sizeof(float) * (w->K / QK) + sizeof(float) * GEMV_WARPS * 32;
    const unsigned grid = static_cast<unsigned>(w->tiles) * 4;
    if (w->scheme == INKQ_A81W41) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(k_qgemv_a8w4<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        k_qgemv_a8w4<true><<<grid, GEMV_WARPS * 32, smem, ctx->stream>>>(w->nibT, w->sc16, w->zpT, a->q, a->d, a->s, a->isum, a->M_ld, C,
                                                                          w->rows, w->K, w->pairs);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(k_qgemv_a8w4<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        k_qgemv_a8w4<false><<<grid, GEMV_WARPS * 32, smem, ctx->stream>>>(w->nibT, w->sc16, w->zpT, a->q, a->d, a->s, a->isum, a->M_ld, C,
                                                                           w->rows, w->K, w->pairs);
    }
    return after_launch(ctx, "k_qgemv_a8w4");
}

}  // namespace inkq
