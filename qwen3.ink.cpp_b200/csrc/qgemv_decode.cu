// Decode-step QGEMV whose epilogue prepares the NEXT layer's quantized activations.
//
// In a decode step (one token) the time between two matrix-vector products - residual add, RMSNorm,
// SiLU*up, activation quantizer - costs as much as the products themselves when every CTA of the next
// product redoes it in its prologue, or when it runs as separate tiny kernels.  Here the producer does it
// once, in its epilogue, and every product reads a ready Q8 row (the short staging path of k_qgemv_a8w4):
//   EPI_STORE       C[n] = y[n]
//   EPI_ACC         C[n] += y[n]                                  (residual connection)
//   EPI_ACC_NORMQ   C[n] += y[n]; the CTA that finishes last (a device counter) then applies
//                   RMSNorm(C; g, eps) to the whole row and quantizes it into `out` (and, optionally,
//                   also writes the normalized fp32 row): input of the next qkv / gate_up / lm_head
//   EPI_PAIR_SILUQ  the weight's rows come in (32 gate rows, 32 up rows) groups (an interleaved fused
//                   gate_up projection); a CTA computes both groups, SiLU(gate)*up of its 32 results is
//                   exactly one quantization block, quantized into `out`: input of down_proj
//   EPI_ACC_QUANT_PENDING  C[n] += y[n]; the CTA's 32 results times the norm weights are one quantization block,
//                   quantized on the spot WITHOUT the row's RMS factor, and the CTA leaves the sum of squares of its
//                   32 results; the factor 1 / sqrt(mean(C^2) + eps) is a scalar of the whole row, so the consuming
//                   product applies it to its finished sums (W (f v) = f (W v)): no CTA has to see the whole row and
//                   the serial last-CTA pass of EPI_ACC_NORMQ disappears.  The quantized values differ from
//                   EPI_ACC_NORMQ's in the last bit at most (x * g against (x * f) * g before rounding to int8); the
//                   block scales stay fp32 (an fp16 scale of an un-normalized row could overflow).
// The matrix-vector arithmetic and its fixed reduction order are those of k_qgemv_a8w4 (per K-slice the
// reference's per-pair order, qwen3/src/qwen/quantized_gemx_kernels.cc:171-188; slice partials ascending);
// the quantization arithmetic is k_quantize_q8's (quantized_gemx_kernels.cc:693-801), operation for
// operation, so the row written here equals RMSNorm / SiLU*up followed by the stand-alone quantizer.
// The reference runs all of these as separate operators (qwen3/src/qwen/QwenDecoderLayer.cc:66-105).
//
// Last-CTA hand-over: every CTA stores its 32 outputs, fences (device scope) and takes a ticket from a
// counter in the context; the CTA drawing the last ticket fences again, reads the row through L2 and
// resets the counter.  No CTA ever waits for another one.
#include <cuda_fp16.h>

#include "inkq_glue.h"
#include "glue_math.cuh"
#include "inkq_internal.h"
#include "ptx.cuh"
#include "qgemv_common.cuh"

namespace inkq {

enum { EPI_STORE = 0, EPI_ACC = 1, EPI_ACC_NORMQ = 2, EPI_PAIR_SILUQ = 3, EPI_ACC_QUANT_PENDING = 4 };

struct DecodeEpi {
    int mode;
    const float *g;      // EPI_ACC_NORMQ: norm weights [rows]
    float eps;
    float *xn;           // EPI_ACC_NORMQ: optional fp32 copy of the normalized row
    unsigned *counter;   // EPI_ACC_NORMQ: ticket counter (zero between launches)
    float *ssq_out;      // EPI_ACC_QUANT_PENDING: sums of squares, one per 32-row group
    QuantOut out;
};

// RMS factor still to be applied to the input row (the producer ran EPI_ACC_QUANT_PENDING); parts == 0: none
struct PendingNorm {
    const float *ssq;
    int parts, n;
    float eps;
};

// RMSNorm of the fp32 row x[0..n) (read through L2) by the whole CTA, then quantization, two lanes per block.
__device__ __forceinline__ void cta_rmsnorm_quant(const float *x, const float *g, float eps, int n, float *xn, const QuantOut &o, float *red)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int nb = n / QK;
    const int half = threadIdx.x & 1;
    const unsigned gmask = 0x3u << (threadIdx.x & 30);
    // rows of up to 16 * blockDim.x elements are read once and kept in registers between the two passes
    const bool single_trip = nb <= static_cast<int>(blockDim.x >> 1);
    float4 keep[4], gkeep[4];   // the norm weights are fetched together with the row: their latency hides under the reduction
    float ss = 0.0f;
    if (single_trip) {
        const int blk = threadIdx.x >> 1;
        if (blk < nb) {
#pragma unroll
            for (int j = 0; j < 4; j++) {
                keep[j] = __ldcg(reinterpret_cast<const float4 *>(x) + blk * 8 + 2 * j + half);
                gkeep[j] = reinterpret_cast<const float4 *>(g)[blk * 8 + 2 * j + half];
            }
#pragma unroll
            for (int j = 0; j < 4; j++) ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
        }
    } else {
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(x) + i);
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
    for (int w2 = 0; w2 < nwarps; w2++) tot += red[w2];
    const float inv = rms_inv(tot, n, eps);
    for (int blk = threadIdx.x >> 1; blk < nb; blk += blockDim.x >> 1) {
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i4 = blk * 8 + 2 * j + half;
            const float4 t = single_trip ? keep[j] : __ldcg(reinterpret_cast<const float4 *>(x) + i4);
            const float4 gg = single_trip ? gkeep[j] : reinterpret_cast<const float4 *>(g)[i4];
            v[j] = rms_scale4(t, inv, gg);
            if (xn != nullptr) reinterpret_cast<float4 *>(xn)[i4] = v[j];
        }
        float mx = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
        mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
        const float dd = __fdiv_rn(mx, 127.0f);
        const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
        int sum = 0;
        uint32_t *dst = reinterpret_cast<uint32_t *>(o.q);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i0 = __float2int_rn(__fmul_rn(v[j].x, id));
            const int i1 = __float2int_rn(__fmul_rn(v[j].y, id));
            const int i2 = __float2int_rn(__fmul_rn(v[j].z, id));
            const int i3 = __float2int_rn(__fmul_rn(v[j].w, id));
            sum += (i0 + i1) + (i2 + i3);
            dst[blk * 8 + 2 * j + half] = pack_sat_s8x4_m1(i0, i1, i2, i3);
        }
        sum += __shfl_xor_sync(gmask, sum, 1);
        if (half == 0) {
            const size_t pl = static_cast<size_t>(blk) * o.M_ld;
            const float sv = __fmul_rn(dd, static_cast<float>(sum));
            if (o.qmode == INKQ_Q8_1_F32) {
                o.d[pl] = dd;
                o.s[pl] = sv;
            } else {
                o.d[pl] = __half2float(__float2half_rn(dd));
                o.s[pl] = (o.qmode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(sv)) : 0.0f;
            }
            o.isum[pl] = sum;
        }
    }
}

template <bool HAS_MIN, int WARPS, bool DEEP>
__global__ void __launch_bounds__(WARPS * 32, GemvShape<WARPS, DEEP>::CTAS_PER_SM) k_qgemv_decode(const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16,
                                                                 const uchar2 *__restrict__ zpT, const int8_t *__restrict__ q,
                                                                 const float *__restrict__ d, const float *__restrict__ s,
                                                                 const int32_t *__restrict__ isum, int M_ld, float *C, int rows, int K,
                                                                 int pairs, const DecodeEpi epi, const PendingNorm pend)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nb = K / QK;
    uint32_t *qa = reinterpret_cast<uint32_t *>(smem_raw);          // K/4 words
    float *da = reinterpret_cast<float *>(smem_raw + K);            // nb
    float *sa = da + nb;                                            // nb (sums, or integer sums for the A80 schemes)
    float *part = sa + nb;                                          // [WARPS][32]
    __shared__ unsigned ticket_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int groups = (epi.mode == EPI_PAIR_SILUQ) ? 2 : 1;         // 32-row groups per CTA
    const int per_tile = 4 / groups;
    const int t = blockIdx.x / per_tile;
    const int g0 = (blockIdx.x % per_tile) * groups;
    const int p_begin = (warp * pairs) / WARPS, p_end = ((warp + 1) * pairs) / WARPS;
    const size_t slab = static_cast<size_t>(t) * pairs;

    int r = (g0 << 5) + lane;
    RowStream<HAS_MIN, GemvShape<WARPS, DEEP>::DEPTH, GemvShape<WARPS, DEEP>::WIDE> rs;
    rs.prime(nibT, sc16, zpT, slab, r, p_begin, p_end);
    // the weights do not depend on the predecessor in the stream; everything below does
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // A pending RMS factor f of the input row multiplies the finished sums (W (f v) = f (W v)), so only the warp that
    // finishes them needs it: warp 0 requests the group sums now (the first 128: a row of 4096 values; four loads in
    // flight per lane) and adds them up after the product, when they have long arrived.
    float pv[4] = {0.f, 0.f, 0.f, 0.f};
    if (pend.parts > 0 && warp == 0) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = u * 32 + lane;
            pv[u] = (i < pend.parts) ? __ldcg(pend.ssq + i) : 0.0f;
        }
    }
    // the residual value and the norm weight this lane's result meets in the epilogue are requested now as well (nobody
    // else touches them while this grid runs), so their latency passes under the product
    const int n_early = t * TILE_N + (g0 << 5) + lane;
    float c_early = 0.0f, g_early = 0.0f;
    if (warp == 0 && n_early < rows && groups == 1) {
        if (epi.mode != EPI_STORE) c_early = C[n_early];
        if (epi.mode == EPI_ACC_QUANT_PENDING) g_early = epi.g[n_early];
    }
    for (int i = threadIdx.x; i < K / 16; i += blockDim.x) reinterpret_cast<uint4 *>(qa)[i] = reinterpret_cast<const uint4 *>(q)[i];
    for (int b = threadIdx.x; b < nb; b += blockDim.x) {
        da[b] = d[static_cast<size_t>(b) * M_ld];
        if (HAS_MIN) sa[b] = s[static_cast<size_t>(b) * M_ld];
        else reinterpret_cast<int32_t *>(sa)[b] = isum[static_cast<size_t>(b) * M_ld];
    }
    __syncthreads();

    float tot[2] = {0.0f, 0.0f};
    for (int gi = 0; gi < groups; gi++) {
        const bool swz = ((r >> 2) & 1) != 0;
        const float acc = rs.run(0.0f, swz, qa, da, sa, nibT, sc16, zpT, slab, r, p_begin, p_end);
        if (gi + 1 < groups) {   // the second group's first batches fly while the first group is reduced
            r += 32;
            rs.prime(nibT, sc16, zpT, slab, r, p_begin, p_end);
        }
        part[warp * 32 + lane] = acc;
        __syncthreads();
        if (warp == 0) {
            float sum = part[lane];
#pragma unroll
            for (int w2 = 1; w2 < WARPS; w2++) sum = __fadd_rn(sum, part[w2 * 32 + lane]);
            tot[gi] = sum;
        }
        __syncthreads();   // part is rewritten by the next group
    }
    if (pend.parts > 0 && warp == 0) {
        // every CTA adds the group sums in the same order (lane-strided ascending, then an xor tree): one factor for all
        float ss = 0.0f;
#pragma unroll
        for (int u = 0; u < 4; u++) ss = __fadd_rn(ss, pv[u]);
        for (int i = 128 + lane; i < pend.parts; i += 32) ss = __fadd_rn(ss, __ldcg(pend.ssq + i));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
        const float f = rms_inv(ss, pend.n, pend.eps);
        tot[0] = __fmul_rn(tot[0], f);
        tot[1] = __fmul_rn(tot[1], f);
    }

    if (epi.mode == EPI_PAIR_SILUQ) {
        if (warp == 0) {
            const int blk = blockIdx.x;                           // output block = CTA index: rows come in (gate32, up32) groups
            const float a = silu_mul(tot[0], tot[1]);
            quantize_block_lanes(a, blk, lane, epi.out);
        }
        return;
    }
    const int n = t * TILE_N + (g0 << 5) + lane;
    if (epi.mode == EPI_ACC_QUANT_PENDING) {
        if (warp == 0) {   // rows is a multiple of 32 here: the whole warp holds results
            const float y = __fadd_rn(c_early, tot[0]);
            C[n] = y;
            float ss = __fmul_rn(y, y);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, off));
            if (lane == 0) epi.ssq_out[n >> 5] = ss;
            quantize_block_lanes(__fmul_rn(y, g_early), n >> 5, lane, epi.out);
        }
        return;
    }
    if (warp == 0 && n < rows) {
        float y = tot[0];
        if (epi.mode != EPI_STORE) y = __fadd_rn(c_early, y);
        C[n] = y;
    }
    if (epi.mode != EPI_ACC_NORMQ) return;
    // ---- last CTA: RMSNorm + quantizer over the finished row
    if (warp == 0) {
        __threadfence();                                           // every storing lane: its store before the ticket
        __syncwarp();
        if (lane == 0) ticket_s = atomicAdd(epi.counter, 1u);
    }
    __syncthreads();
    if (ticket_s != gridDim.x - 1) return;
    __threadfence();                                               // every other CTA's stores before the reads below
    cta_rmsnorm_quant(C, epi.g, epi.eps, rows, epi.xn, epi.out, part);
    if (threadIdx.x == 0) *epi.counter = 0u;                       // ready for the next launch
}

__global__ void __launch_bounds__(512) k_rmsnorm_quant_row(const float *x, const float *g, float eps, int n, float *xn, const QuantOut o)
{
    __shared__ float red[16];
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    cta_rmsnorm_quant(x, g, eps, n, xn, o, red);
}

template <bool HAS_MIN, int WARPS, bool DEEP = false>
static void launch_decode_variant(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, const DecodeEpi &epi, const PendingNorm &pend)
{
    const size_t smem = static_cast<size_t>(w->K) + 2 * sizeof(float) * (w->K / QK) + sizeof(float) * WARPS * 32;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k_qgemv_decode<HAS_MIN, WARPS, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(w->tiles) * (epi.mode == EPI_PAIR_SILUQ ? 2 : 4));
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // weight prefetch may overlap the predecessor's tail
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, k_qgemv_decode<HAS_MIN, WARPS, DEEP>, static_cast<const uint8_t *>(w->nibT), static_cast<const uint2 *>(w->sc16),
                       static_cast<const uchar2 *>(w->zpT), static_cast<const int8_t *>(a->q), static_cast<const float *>(a->d),
                       static_cast<const float *>(a->s), static_cast<const int32_t *>(a->isum), a->M_ld, C, w->rows, w->K, w->pairs, epi, pend);
}

}  // namespace inkq

using namespace inkq;

static int decode_use(inkq_ctx *ctx)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    return INKQ_OK;
}

extern "C" {

int inkq_glue_decode_gemv(inkq_ctx *ctx, const inkq_weight *w, const inkq_act *in, float *C_dev, int epilogue, const float *norm_w_dev, float eps,
                          inkq_act *out, int out_qmode, float *xn_out_dev)
{
    int rc = decode_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && in != nullptr, "null weight or activation handle");
    INKQ_REQUIRE(ctx, epilogue >= EPI_STORE && epilogue <= EPI_ACC_QUANT_PENDING, "epilogue must be 0..4");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations");
    INKQ_REQUIRE(ctx, in->M == 1 && in->K == w->K, "the input must be one quantized row of the layer's K");
    const int expect = (w->scheme == INKQ_A81W41) ? INKQ_Q8_1_F16 : INKQ_Q8_0_F16;
    // (a row whose RMS factor is pending carries fp32 block scales and sums whatever the scheme)
    INKQ_REQUIRE(ctx, in->qmode == expect || in->ssq_parts > 0, "the input row was quantized in another mode than this layer's M == 1 path uses");
    PendingNorm pend = {};
    if (in->ssq_parts > 0) {
        pend.ssq = in->ssq;
        pend.parts = in->ssq_parts;
        pend.n = in->norm_n;
        pend.eps = in->norm_eps;
    }
    INKQ_REQUIRE(ctx, epilogue == EPI_PAIR_SILUQ || C_dev != nullptr, "null output");
    DecodeEpi epi = {};
    epi.mode = epilogue;
    if (epilogue == EPI_ACC_QUANT_PENDING) {
        INKQ_REQUIRE(ctx, out != nullptr && out != in && out->K == w->rows, "out must be another handle created for K = the layer's row count");
        INKQ_REQUIRE(ctx, norm_w_dev != nullptr && w->rows % 128 == 0 && w->rows / 32 <= ACT_SSQ_CAP && out->ssq != nullptr,
                     "the pending-norm epilogue needs the norm weights and a row count that is a multiple of 128, at most 16384");
        epi.g = norm_w_dev;
        epi.ssq_out = out->ssq;
        epi.out = quant_out_of(out, w->rows, INKQ_Q8_1_F32);
        out->ssq_parts = w->rows / 32;
        out->norm_n = w->rows;
        out->norm_eps = eps;
    }
    if (epilogue == EPI_ACC_NORMQ || epilogue == EPI_PAIR_SILUQ) {
        INKQ_REQUIRE(ctx, out != nullptr, "this epilogue writes a quantized row: out is required");
        INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
        const int out_K = (epilogue == EPI_PAIR_SILUQ) ? w->rows / 2 : w->rows;
        // gate/up pairs: one CTA per 64 rows writes output block blockIdx.x, and the grid covers whole 128-row tiles
        INKQ_REQUIRE(ctx, w->rows % (epilogue == EPI_PAIR_SILUQ ? 128 : 32) == 0, "the row count must be a multiple of 32 (128 for gate/up pairs)");
        INKQ_REQUIRE(ctx, out->K == out_K && out != in, "the output activation handle must have been created for K = the produced row length, and differ from the input");
        epi.out = quant_out_of(out, out_K, out_qmode);
    }
    if (epilogue == EPI_ACC_NORMQ) {
        INKQ_REQUIRE(ctx, norm_w_dev != nullptr && (reinterpret_cast<uintptr_t>(norm_w_dev) & 15) == 0 && (reinterpret_cast<uintptr_t>(C_dev) & 15) == 0,
                     "the norm weights and C must be 16-byte aligned");
        INKQ_REQUIRE(ctx, w->rows % 128 == 0, "the row count must be a multiple of 128 for the fused RMSNorm");
        epi.g = norm_w_dev;
        epi.eps = eps;
        epi.xn = xn_out_dev;
        epi.counter = reinterpret_cast<unsigned *>(ctx->dev_flag) + 1;
    }
    const bool wide_cta = (w->tiles * 4 <= 2 * ctx->num_sms) || (w->pairs >= 128);
    const int ctas = w->tiles * (epilogue == EPI_PAIR_SILUQ ? 2 : 4);
    const bool deep = wide_cta && gemv_deep(ctas, w->pairs, 16, ctx->num_sms);
    if (w->scheme == INKQ_A81W41) {
        if (deep) launch_decode_variant<true, 16, true>(ctx, in, w, C_dev, epi, pend);
        else if (wide_cta) launch_decode_variant<true, 16>(ctx, in, w, C_dev, epi, pend);
        else launch_decode_variant<true, 8>(ctx, in, w, C_dev, epi, pend);
    } else {
        if (deep) launch_decode_variant<false, 16, true>(ctx, in, w, C_dev, epi, pend);
        else if (wide_cta) launch_decode_variant<false, 16>(ctx, in, w, C_dev, epi, pend);
        else launch_decode_variant<false, 8>(ctx, in, w, C_dev, epi, pend);
    }
    return after_launch(ctx, "k_qgemv_decode");
}

int inkq_glue_rmsnorm_quant(inkq_ctx *ctx, const float *x_dev, const float *norm_w_dev, float eps, int K, inkq_act *out, int out_qmode,
                            float *xn_out_dev)
{
    int rc = decode_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, x_dev != nullptr && norm_w_dev != nullptr && out != nullptr && K >= 32 && K % 32 == 0, "bad rmsnorm_quant arguments");
    INKQ_REQUIRE(ctx, out->K == K, "the output activation handle must have been created for this K");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0 && (reinterpret_cast<uintptr_t>(norm_w_dev) & 15) == 0, "x and the weights must be 16-byte aligned");
    launch_pdl(k_rmsnorm_quant_row, dim3(1), dim3(512), 0, ctx->stream, x_dev, norm_w_dev, eps, K, xn_out_dev, quant_out_of(out, K, out_qmode));
    return after_launch(ctx, "k_rmsnorm_quant_row");
}

}  // extern "C"
