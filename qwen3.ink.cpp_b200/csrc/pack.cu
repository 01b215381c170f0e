// Load-time weight re-tiler: logical on-disk format -> sm_100a device layout, and
// its inverse (used by round-trip checks).
//
// Stands in for repack_w80_weight / repack_w81_weight_fp16 / repack_w81_weight_fp32
// (qwen3/src/qwen/QwenOperator.cc:757-892).  The reference builds 64(K) x 8(N)
// superblocks for 256-bit AVX loads; here the unit is a 128-row tile whose
// (tile, pair) slab is 4096 contiguous bytes so that one untiled bulk (TMA) copy
// feeds a pipeline stage, with the two 16-byte chunks of each row swizzled by row
// so that shared-memory reads by 8 consecutive rows are conflict-free.
// The nibble pairing of the disk format (low nibble = block 2p, high nibble =
// block 2p+1, notebooks/quantize_methods.py:120-123) is kept: one AND and one
// shift+AND split a 32-bit word into four int8 of each block.
#include <cuda_fp16.h>

#include "inkq_internal.h"

namespace inkq {

// one thread per 16-byte chunk of nibT
__global__ void __launch_bounds__(256) k_retile_nibbles(const uint8_t *__restrict__ nib, int rows, int K, int tiles, int pairs,
                                                        uint8_t *__restrict__ nibT)
{
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long total = static_cast<long long>(tiles) * pairs * TILE_N * 2;
    if (idx >= total) return;
    const int chunk = static_cast<int>(idx & 1);
    const int r = static_cast<int>((idx >> 1) % TILE_N);
    const long long tp = (idx >> 1) / TILE_N;
    const int p = static_cast<int>(tp % pairs);
    const int t = static_cast<int>(tp / pairs);
    const int n = t * TILE_N + r;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (n < rows) v = *reinterpret_cast<const uint4 *>(nib + static_cast<size_t>(n) * (K / 2) + p * 32 + chunk * 16);
    *reinterpret_cast<uint4 *>(nibT + nib_offset(pairs, t, p, r, chunk)) = v;
}

// one thread per (tile, pair, row)
__global__ void __launch_bounds__(256) k_retile_scales(const float *__restrict__ d, const float *__restrict__ m,
                                                       const uint8_t *__restrict__ zp, int scheme, int rows, int K, int tiles,
                                                       int pairs, float4 *__restrict__ sc32, int round16, uint2 *__restrict__ sc16,
                                                       uchar2 *__restrict__ zpT)
{
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long total = static_cast<long long>(tiles) * pairs * TILE_N;
    if (idx >= total) return;
    const int r = static_cast<int>(idx % TILE_N);
    const int p = static_cast<int>((idx / TILE_N) % pairs);
    const int t = static_cast<int>(idx / TILE_N / pairs);
    const int n = t * TILE_N + r;
    float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
    uchar2 z = make_uchar2(0, 0);
    if (n < rows) {
        const size_t b = static_cast<size_t>(n) * (K / QK) + 2 * p;
        sc.x = d[b];
        sc.y = d[b + 1];
        if (m != nullptr) {
            sc.z = m[b];
            sc.w = m[b + 1];
        }
        if (scheme == INKQ_A80W40) z = make_uchar2(8, 8);
        if (scheme == INKQ_A80W4Z) z = make_uchar2(zp[b], zp[b + 1]);
    }
    const __half2 h0 = __floats2half2_rn(sc.x, sc.y);
    const __half2 h1 = __floats2half2_rn(sc.z, sc.w);
    if (sc32 != nullptr) {
        // the prefill kernel reads fp32 records either way (widening fp16 in its inner loop costs more than the
        // extra bytes): the values as given, or the fp16-rounded ones widened again
        if (round16) {
            const float2 a = __half22float2(h0), b = __half22float2(h1);
            sc = make_float4(a.x, a.y, b.x, b.y);
        }
        sc32[idx] = sc;
    }
    uint2 packed;
    packed.x = *reinterpret_cast<const uint32_t *>(&h0);
    packed.y = *reinterpret_cast<const uint32_t *>(&h1);
    sc16[idx] = packed;
    zpT[idx] = z;
}

__global__ void __launch_bounds__(256) k_export_nibbles(const uint8_t *__restrict__ nibT, int rows, int K, int pairs,
                                                        uint8_t *__restrict__ nib)
{
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long total = static_cast<long long>(rows) * pairs * 2;
    if (idx >= total) return;
    const int chunk = static_cast<int>(idx & 1);
    const int p = static_cast<int>((idx >> 1) % pairs);
    const int n = static_cast<int>((idx >> 1) / pairs);
    const uint4 v = *reinterpret_cast<const uint4 *>(nibT + nib_offset(pairs, n / TILE_N, p, n % TILE_N, chunk));
    *reinterpret_cast<uint4 *>(nib + static_cast<size_t>(n) * (K / 2) + p * 32 + chunk * 16) = v;
}

__global__ void __launch_bounds__(256) k_export_scales(const float4 *__restrict__ sc32, const uint2 *__restrict__ sc16,
                                                       const uchar2 *__restrict__ zpT, int rows, int K, int pairs,
                                                       float *__restrict__ d, float *__restrict__ m, uint8_t *__restrict__ zp)
{
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long total = static_cast<long long>(rows) * pairs;
    if (idx >= total) return;
    const int p = static_cast<int>(idx % pairs);
    const int n = static_cast<int>(idx / pairs);
    const size_t src = (static_cast<size_t>(n / TILE_N) * pairs + p) * TILE_N + (n % TILE_N);
    float4 sc;
    if (sc32 != nullptr) {
        sc = sc32[src];
    } else {
        const uint2 pk = sc16[src];
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&pk.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&pk.y));
        sc = make_float4(a.x, a.y, b.x, b.y);
    }
    const size_t b = static_cast<size_t>(n) * (K / QK) + 2 * p;
    if (d != nullptr) {
        d[b] = sc.x;
        d[b + 1] = sc.y;
    }
    if (m != nullptr) {
        m[b] = sc.z;
        m[b + 1] = sc.w;
    }
    if (zp != nullptr) {
        const uchar2 z = zpT[src];
        zp[b] = z.x;
        zp[b + 1] = z.y;
    }
}

int launch_retile(inkq_ctx *ctx, Weight *w, const uint8_t *nib, const float *d, const float *m, const uint8_t *zp, int n_begin)
{
    const size_t row_nib = static_cast<size_t>(w->K) / 2, row_sc = static_cast<size_t>(w->K) / QK;
    const uint8_t *nib0 = nib + static_cast<size_t>(n_begin) * row_nib;
    const float *d0 = d + static_cast<size_t>(n_begin) * row_sc;
    const float *m0 = m ? m + static_cast<size_t>(n_begin) * row_sc : nullptr;
    const uint8_t *zp0 = zp ? zp + static_cast<size_t>(n_begin) * row_sc : nullptr;
    {
        const long long total = static_cast<long long>(w->tiles) * w->pairs * TILE_N * 2;
        k_retile_nibbles<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(nib0, w->rows, w->K, w->tiles, w->pairs,
                                                                                            w->nibT);
        int rc = after_launch(ctx, "k_retile_nibbles");
        if (rc) return rc;
    }
    {
        const long long total = static_cast<long long>(w->tiles) * w->pairs * TILE_N;
        k_retile_scales<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(d0, m0, zp0, w->scheme, w->rows, w->K, w->tiles,
                                                                                           w->pairs, w->sc32, w->scale_mode == INKQ_SCALES_F16 ? 1 : 0, w->sc16, w->zpT);
        return after_launch(ctx, "k_retile_scales");
    }
}

int launch_export(inkq_ctx *ctx, const Weight *w, uint8_t *nib, float *d, float *m, uint8_t *zp)
{
    if (nib != nullptr) {
        const long long total = static_cast<long long>(w->rows) * w->pairs * 2;
        k_export_nibbles<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(w->nibT, w->rows, w->K, w->pairs, nib);
        int rc = after_launch(ctx, "k_export_nibbles");
        if (rc) return rc;
    }
    if (d != nullptr || m != nullptr || zp != nullptr) {
        const long long total = static_cast<long long>(w->rows) * w->pairs;
        k_export_scales<<<static_cast<unsigned>((total + 255) / 256), 256, 0, ctx->stream>>>(w->sc32, w->sc16, w->zpT, w->rows, w->K, w->pairs,
                                                                                           d, m, zp);
        return after_launch(ctx, "k_export_scales");
    }
    return INKQ_OK;
}

}  // namespace inkq
