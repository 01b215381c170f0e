// Device pieces shared by the decode matrix-vector kernels (qgemv.cu, qgemv_decode.cu): one lane owns one
// weight row, a batch is GEMV_UNROLL pairs (64 K-elements each) of that row as loaded, and the per-pair
// arithmetic is the reference's (qwen3/src/qwen/quantized_gemx_kernels.cc:171-188, :39-108).
#pragma once
#include <cuda_fp16.h>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

constexpr int GEMV_UNROLL = 2;   // pairs per batch; two batches are in flight per lane

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

// One batch of GEMV_UNROLL pairs of this lane's row, as loaded.
struct PairBatch {
    uint4 ca[GEMV_UNROLL], cb[GEMV_UNROLL];
    uint2 sc[GEMV_UNROLL];
    uchar2 z[GEMV_UNROLL];
};

// WIDE: the row's 32 bytes of a pair as one 256-bit request instead of two 128-bit ones (measured per kernel variant:
// better for the 16-warp variants with two batches in flight, worse for the others)
template <bool HAS_MIN, bool WIDE>
__device__ __forceinline__ void load_batch(PairBatch &b, const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16,
                                           const uchar2 *__restrict__ zpT, size_t slab, int r, int p0, int p_end)
{
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; u++) {
        const int p = min(p0 + u, p_end - 1);  // clamped duplicates are loaded but never used
        const size_t rec = (slab + p) * TILE_N + r;
        const uint8_t *src = nibT + rec * 32;
        if (WIDE) {
            ldg_stream_v8(src, b.ca[u], b.cb[u]);
        } else {
            b.ca[u] = ldg_stream_v4(src);
            b.cb[u] = ldg_stream_v4(src + 16);
        }
        b.sc[u] = ldg_stream_v2(sc16 + rec);
        if (!HAS_MIN) b.z[u] = zpT[rec];
    }
}

template <bool HAS_MIN>
__device__ __forceinline__ float consume_batch(const PairBatch &b, float acc, bool swz, const uint32_t *__restrict__ qa, const float *__restrict__ da,
                                               const float *__restrict__ sa, int p0, int p_end)
{
#pragma unroll
    for (int u = 0; u < GEMV_UNROLL; u++) {
        const int p = p0 + u;
        if (p < p_end) {
            int ilo, ihi;
            dots_of_pair(swz ? b.cb[u] : b.ca[u], swz ? b.ca[u] : b.cb[u], qa + p * 16, qa + p * 16 + 8, ilo, ihi);
            const float2 dw = __half22float2(*reinterpret_cast<const __half2 *>(&b.sc[u].x));
            const float da_lo = da[2 * p], da_hi = da[2 * p + 1];
            if (HAS_MIN) {
                const float2 mw = __half22float2(*reinterpret_cast<const __half2 *>(&b.sc[u].y));
                acc = fmaf(static_cast<float>(ilo), __fmul_rn(da_lo, dw.x), acc);
                acc = fmaf(static_cast<float>(ihi), __fmul_rn(da_hi, dw.y), acc);
                acc = fmaf(mw.x, sa[2 * p], acc);
                acc = fmaf(mw.y, sa[2 * p + 1], acc);
            } else {
                const int32_t *is = reinterpret_cast<const int32_t *>(sa);
                ilo -= static_cast<int>(b.z[u].x) * is[2 * p];
                ihi -= static_cast<int>(b.z[u].y) * is[2 * p + 1];
                acc = fmaf(static_cast<float>(ilo), __fmul_rn(da_lo, dw.x), acc);
                acc = fmaf(static_cast<float>(ihi), __fmul_rn(da_hi, dw.y), acc);
            }
        }
    }
    return acc;
}

// A lane's walk over its K-slice [p_begin, p_end) of one weight row with DEPTH batches in flight: prime() issues the
// first DEPTH batches (they do not depend on the activations), run() consumes the pairs in ascending order - the
// accumulation order never depends on DEPTH - and refills each batch as soon as it is consumed.
template <bool HAS_MIN, int DEPTH, bool WIDE>
struct RowStream {
    PairBatch b[DEPTH];
    __device__ __forceinline__ void prime(const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16, const uchar2 *__restrict__ zpT, size_t slab,
                                          int r, int p_begin, int p_end)
    {
#pragma unroll
        for (int i = 0; i < DEPTH; i++)
            if (p_begin + i * GEMV_UNROLL < p_end) load_batch<HAS_MIN, WIDE>(b[i], nibT, sc16, zpT, slab, r, p_begin + i * GEMV_UNROLL, p_end);
    }
    __device__ __forceinline__ float run(float acc, bool swz, const uint32_t *__restrict__ qa, const float *__restrict__ da, const float *__restrict__ sa,
                                         const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16, const uchar2 *__restrict__ zpT, size_t slab,
                                         int r, int p_begin, int p_end)
    {
        for (int p0 = p_begin; p0 < p_end; p0 += DEPTH * GEMV_UNROLL) {
#pragma unroll
            for (int i = 0; i < DEPTH; i++) {
                const int pi = p0 + i * GEMV_UNROLL;
                if (pi < p_end) {
                    acc = consume_batch<HAS_MIN>(b[i], acc, swz, qa, da, sa, pi, p_end);
                    if (pi + DEPTH * GEMV_UNROLL < p_end) load_batch<HAS_MIN, WIDE>(b[i], nibT, sc16, zpT, slab, r, pi + DEPTH * GEMV_UNROLL, p_end);
                }
            }
        }
        return acc;
    }
};

// Batches in flight per lane and CTAs per SM of a kernel variant: 8 warps x 3 CTAs and 16 warps x 2 CTAs keep two
// batches in flight; DEEP (16 warps, one CTA per SM: layers with no more 32-row groups than SMs and long rows) four.
template <int WARPS, bool DEEP> struct GemvShape {
    static constexpr int DEPTH = DEEP ? 4 : 2;
    static constexpr int CTAS_PER_SM = DEEP ? 1 : (WARPS == 8 ? 3 : 2);
    static constexpr bool WIDE = (WARPS == 16) && !DEEP;   // measured in the decode step: +1.2 % there, -1 % in the other variants
};
// the rule both matrix-vector kernels use (so that they stay bit-identical): few CTAs and at least three batches per lane
inline bool gemv_deep(int ctas, int pairs, int warps, int num_sms) { return ctas <= num_sms && pairs / warps >= 3 * GEMV_UNROLL; }

// Saturating pack of four s32 to s8 (a in the low byte): two cvt.pack instructions.
__device__ __forceinline__ uint32_t pack_sat_s8x4_m1(int a, int b, int c, int d)
{
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
    return out;
}

// One quantized activation row (M == 1) in the device layout of an activation handle, as an output.
struct QuantOut {     // one quantized activation row (M == 1) in the device layout of an activation handle
    int8_t *q;
    float *d, *s;
    int32_t *isum;
    int M_ld, qmode;
};


// Writes block `blk` of a quantized row from the 32 values held one per lane (whole warp).
__device__ __forceinline__ void quantize_block_lanes(float v, int blk, int lane, const QuantOut &o)
{
    float mx = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    const float dd = __fdiv_rn(mx, 127.0f);
    const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
    const int qi = __float2int_rn(__fmul_rn(v, id));
    int sum = qi;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    o.q[blk * QK + lane] = static_cast<int8_t>(max(-128, min(127, qi)));
    if (lane == 0) {
        const size_t pl = static_cast<size_t>(blk) * o.M_ld;
        const float ss = __fmul_rn(dd, static_cast<float>(sum));
        if (o.qmode == INKQ_Q8_1_F32) {
            o.d[pl] = dd;
            o.s[pl] = ss;
        } else {
            o.d[pl] = __half2float(__float2half_rn(dd));
            o.s[pl] = (o.qmode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(ss)) : 0.0f;
        }
        o.isum[pl] = sum;
    }
}

// Points a QuantOut at an activation handle and marks the handle as holding one row quantized in `qmode`.
inline QuantOut quant_out_of(Act *a, int K, int qmode)
{
    QuantOut o;
    o.q = a->q;
    o.d = a->d;
    o.s = a->s;
    o.isum = a->isum;
    o.M_ld = 4;
    o.qmode = qmode;
    a->K = K;
    a->M = 1;
    a->M_ld = 4;
    a->qmode = qmode;
    a->ssq_parts = 0;
    return o;
}

}  // namespace inkq
