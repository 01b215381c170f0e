// Prompt attention on the tensor cores (glue around the quantized linears, not the hot path itself).
//
// Causal grouped-query attention of T query tokens over cache positions 0 .. pos0 + t, as the reference's attention
// core computes it (qwen3/src/qwen/QwenAttention.cc:122-190: q k^T scaled, causal mask, softmax, p v), for head
// dimension 128 and fp16 key / value caches.  One CTA = 64 query tokens of one query head, 4 warps of 16 tokens each;
// keys and values pass through shared memory in tiles of 64 positions; scores and outputs are warp-level
// m16n8k16 fp16 matrix products with fp32 accumulation, online softmax in registers.
//
// Precision: the fp32 queries (already scaled) and the softmax weights are each split into an fp16 value and an fp16
// remainder and both parts are multiplied (the keys and values are fp16 in the cache, so those products are exact),
// which keeps the result within ~1e-6 of an fp32 evaluation; exponentials with the fast fp32 exponential.
//
// The epilogue writes the fp32 output and / or quantizes it for the output projection: a head's 128 outputs are four
// quantization blocks, each held by the four lanes that share a row of the accumulator fragment; same arithmetic as the
// stand-alone quantizer (quantized_gemx_kernels.cc:693-911), so attention followed by the quantizer gives the same bits.
#include <cuda_fp16.h>
#include <math.h>

#include "inkq_internal.h"
#include "ptx.cuh"
#include "qgemv_common.cuh"

namespace inkq {

constexpr int AM_HD = 128, AM_ROWS = 64, AM_KEYS = 64, AM_STRIDE = AM_HD + 8;   // padded rows: conflict-free ldmatrix

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem_row)));
}
// x = hi + lo with hi = fp16(x), lo = fp16(x - hi), for two values packed as half2 words
__device__ __forceinline__ void split_f16x2(float x, float y, uint32_t &hi, uint32_t &lo)
{
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

__global__ void __launch_bounds__(128) k_attention_prefill_mma(const float *__restrict__ q, const __half *__restrict__ k_cache,
                                                               const __half *__restrict__ v_cache, const int *__restrict__ pos0_dev, int T, int nq,
                                                               int nkv, int max_pos, float scale, float *__restrict__ out, const QuantOut qo,
                                                               int qrow0)
{
    __shared__ __align__(16) __half ks[AM_KEYS][AM_STRIDE];
    __shared__ __align__(16) __half vs[AM_KEYS][AM_STRIDE];
    // the last row blocks see the most keys: they get the lowest CTA indices, so that they start first
    const int t0 = (gridDim.x - 1 - blockIdx.x) * AM_ROWS, h = blockIdx.y;
    const int kvh = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, tq = lane & 3;
    const int pos0 = *pos0_dev;
    const int r0 = t0 + warp * 16 + g, r1 = r0 + 8;                      // this thread's two query rows
    const int lim0 = min(pos0 + min(r0, T - 1), max_pos - 1), lim1 = min(pos0 + min(r1, T - 1), max_pos - 1);   // last visible key
    const int warp_lim = min(pos0 + min(t0 + warp * 16 + 15, T - 1), max_pos - 1);
    const int cta_keys = min(pos0 + min(t0 + AM_ROWS, T), max_pos);

    // ---- the warp's 16 x 128 query tile as A fragments (hi and lo halves), scaled
    uint32_t qh[8][4], ql[8][4];
    {
        const float *q0 = q + (static_cast<size_t>(min(r0, T - 1)) * nq + h) * AM_HD;
        const float *q1 = q + (static_cast<size_t>(min(r1, T - 1)) * nq + h) * AM_HD;
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
            const int c = kk * 16 + 2 * tq;
            const float2 a0 = *reinterpret_cast<const float2 *>(q0 + c), a1 = *reinterpret_cast<const float2 *>(q1 + c);
            const float2 a2 = *reinterpret_cast<const float2 *>(q0 + c + 8), a3 = *reinterpret_cast<const float2 *>(q1 + c + 8);
            split_f16x2(a0.x * scale, a0.y * scale, qh[kk][0], ql[kk][0]);
            split_f16x2(a1.x * scale, a1.y * scale, qh[kk][1], ql[kk][1]);
            split_f16x2(a2.x * scale, a2.y * scale, qh[kk][2], ql[kk][2]);
            split_f16x2(a3.x * scale, a3.y * scale, qh[kk][3], ql[kk][3]);
        }
    }
    float o[16][4];
#pragma unroll
    for (int nt = 0; nt < 16; nt++) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.0f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    const __half *kb = k_cache + static_cast<size_t>(kvh) * max_pos * AM_HD;
    const __half *vb = v_cache + static_cast<size_t>(kvh) * max_pos * AM_HD;

    for (int k0 = 0; k0 < cta_keys; k0 += AM_KEYS) {
        __syncthreads();   // the previous tile is consumed
#pragma unroll
        for (int u = 0; u < AM_KEYS * (AM_HD / 8) / 128; u++) {
            const int i = threadIdx.x + u * 128;
            const int r = i / (AM_HD / 8), c = i % (AM_HD / 8);
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (k0 + r < cta_keys) {
                kv = reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(k0 + r) * AM_HD)[c];
                vv = reinterpret_cast<const uint4 *>(vb + static_cast<size_t>(k0 + r) * AM_HD)[c];
            }
            *reinterpret_cast<uint4 *>(&ks[r][c * 8]) = kv;
            *reinterpret_cast<uint4 *>(&vs[r][c * 8]) = vv;
        }
        __syncthreads();
        if (k0 > warp_lim) continue;   // warp-uniform: none of this warp's rows sees a key of the tile

        // ---- scores: s[nt] = this warp's 16 rows x keys k0 + 8 nt .. + 7
        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
#pragma unroll
            for (int np = 0; np < 4; np++) {
                // four 8x8 matrices: keys 16 np .. + 7 and + 8 .. + 15, dims 16 kk .. + 7 and + 8 .. + 15
                uint32_t b[4];
                ldmatrix_x4(b, &ks[np * 16 + (lane & 7) + ((lane >> 4) << 3)][kk * 16 + (((lane >> 3) & 1) << 3)]);
                mma_f16(s[2 * np], qh[kk], b[0], b[1]);
                mma_f16(s[2 * np], ql[kk], b[0], b[1]);
                mma_f16(s[2 * np + 1], qh[kk], b[2], b[3]);
                mma_f16(s[2 * np + 1], ql[kk], b[2], b[3]);
            }
        }
        // ---- causal mask, online softmax (rows r0: s[.][0..1], r1: s[.][2..3]; a row lives in the 4 lanes of a quad)
        float tm0 = -INFINITY, tm1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const int key = k0 + nt * 8 + 2 * tq;
            if (key > lim0) s[nt][0] = -INFINITY;
            if (key + 1 > lim0) s[nt][1] = -INFINITY;
            if (key > lim1) s[nt][2] = -INFINITY;
            if (key + 1 > lim1) s[nt][3] = -INFINITY;
            tm0 = fmaxf(tm0, fmaxf(s[nt][0], s[nt][1]));
            tm1 = fmaxf(tm1, fmaxf(s[nt][2], s[nt][3]));
        }
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1));
        tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1));
        tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
        const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);
        // (a row that sees no key of this tile keeps its state: mn == m; key 0 is visible to every row, so mn is finite
        //  from the first tile on)
        const float c0 = (mn0 == -INFINITY) ? 1.0f : __expf(m0 - mn0), c1 = (mn1 == -INFINITY) ? 1.0f : __expf(m1 - mn1);
        m0 = mn0;
        m1 = mn1;
        l0 *= c0;
        l1 *= c1;
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
            o[nt][0] *= c0;
            o[nt][1] *= c0;
            o[nt][2] *= c1;
            o[nt][3] *= c1;
        }
        uint32_t ph[4][4], pl[4][4];   // the probabilities as A fragments of the 4 key sub-tiles of 16
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            const float p0 = (s[nt][0] == -INFINITY) ? 0.0f : __expf(s[nt][0] - mn0), p1 = (s[nt][1] == -INFINITY) ? 0.0f : __expf(s[nt][1] - mn0);
            const float p2 = (s[nt][2] == -INFINITY) ? 0.0f : __expf(s[nt][2] - mn1), p3 = (s[nt][3] == -INFINITY) ? 0.0f : __expf(s[nt][3] - mn1);
            l0 += p0 + p1;
            l1 += p2 + p3;
            split_f16x2(p0, p1, ph[nt >> 1][(nt & 1) * 2], pl[nt >> 1][(nt & 1) * 2]);
            split_f16x2(p2, p3, ph[nt >> 1][(nt & 1) * 2 + 1], pl[nt >> 1][(nt & 1) * 2 + 1]);
        }
        // ---- o += p v: B fragments of v (keys x dims, dims contiguous) through transposing matrix loads
#pragma unroll
        for (int kt = 0; kt < 4; kt++) {
#pragma unroll
            for (int np = 0; np < 8; np++) {
                // four 8x8 matrices: keys 16 kt .. + 7 and + 8 .. + 15 of dims 16 np .. + 7, then the same keys of dims + 8 .. + 15
                uint32_t b[4];
                ldmatrix_x4_trans(b, &vs[kt * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)][np * 16 + ((lane >> 4) << 3)]);
                mma_f16(o[2 * np], ph[kt], b[0], b[1]);
                mma_f16(o[2 * np], pl[kt], b[0], b[1]);
                mma_f16(o[2 * np + 1], ph[kt], b[2], b[3]);
                mma_f16(o[2 * np + 1], pl[kt], b[2], b[3]);
            }
        }
    }
    // ---- epilogue
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.0f / l0, inv1 = 1.0f / l1;
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int row = half ? r1 : r0;
        const float inv = half ? inv1 : inv0;
        const bool live = row < T;       // (whole quads agree: a row belongs to one quad)
        float v[16][2];
#pragma unroll
        for (int nt = 0; nt < 16; nt++) {
            v[nt][0] = o[nt][2 * half] * inv;
            v[nt][1] = o[nt][2 * half + 1] * inv;
        }
        if (live && out != nullptr) {
            float *dst = out + (static_cast<size_t>(row) * nq + h) * AM_HD + 2 * tq;
#pragma unroll
            for (int nt = 0; nt < 16; nt++) *reinterpret_cast<float2 *>(dst + nt * 8) = make_float2(v[nt][0], v[nt][1]);
        }
        if (qo.q != nullptr) {   // (warp-uniform; the shuffles below are executed by every lane, only the stores are per row)
            const int qrow = qrow0 + row;
#pragma unroll
            for (int blk = 0; blk < 4; blk++) {   // dims 32 blk .. + 31 = accumulator tiles 4 blk .. + 3, eight values per lane
                float mx = 0.0f;
#pragma unroll
                for (int u = 0; u < 4; u++) mx = fmaxf(mx, fmaxf(fabsf(v[4 * blk + u][0]), fabsf(v[4 * blk + u][1])));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float dd = __fdiv_rn(mx, 127.0f);
                const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
                int sum = 0;
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int i0 = __float2int_rn(__fmul_rn(v[4 * blk + u][0], id)), i1 = __float2int_rn(__fmul_rn(v[4 * blk + u][1], id));
                    sum += i0 + i1;
                    const int c0s = max(-128, min(127, i0)), c1s = max(-128, min(127, i1));
                    if (live)
                        *reinterpret_cast<uint16_t *>(qo.q + (static_cast<size_t>(qrow) * nq + h) * AM_HD + (4 * blk + u) * 8 + 2 * tq) =
                            static_cast<uint16_t>((c0s & 0xff) | ((c1s & 0xff) << 8));
                }
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                if (tq == 0 && (live || qrow < qo.M_ld)) {
                    // (rows past T inside the padded planes - only the call that holds the last rows reaches them - read as zero)
                    const size_t pl = static_cast<size_t>(h * (AM_HD / QK) + blk) * qo.M_ld + qrow;
                    const float sv = __fmul_rn(dd, static_cast<float>(sum));
                    float dw = 0.0f, sw = 0.0f;
                    if (live) {
                        if (qo.qmode == INKQ_Q8_1_F32) {
                            dw = dd;
                            sw = sv;
                        } else {
                            dw = __half2float(__float2half_rn(dd));
                            sw = (qo.qmode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(sv)) : 0.0f;
                        }
                    }
                    qo.d[pl] = dw;
                    qo.s[pl] = sw;
                    qo.isum[pl] = live ? sum : 0;
                }
            }
        }
    }
}

int launch_attention_prefill_mma(inkq_ctx *ctx, const float *q, const uint16_t *k_cache, const uint16_t *v_cache, const int *pos0_dev, int T, int nq,
                                 int nkv, int max_pos, float scale, float *out, const QuantOut &qo, int qrow0)
{
    k_attention_prefill_mma<<<dim3((T + AM_ROWS - 1) / AM_ROWS, nq), 128, 0, ctx->stream>>>(q, reinterpret_cast<const __half *>(k_cache),
                                                                                            reinterpret_cast<const __half *>(v_cache), pos0_dev, T, nq,
                                                                                            nkv, max_pos, scale, out, qo, qrow0);
    return after_launch(ctx, "k_attention_prefill_mma");
}

}  // namespace inkq
