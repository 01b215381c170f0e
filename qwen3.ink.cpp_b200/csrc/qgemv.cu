// Decode QGEMV (M == 1): bandwidth-bound streaming of the 4-bit weights.
//
// Stands in for gemv_repack_A81W41_fp16 (qwen3/src/qwen/quantized_gemx_kernels.cc:111-193)
// and gemv_repack_A80W40 (:39-108); the zero-point scheme has no reference kernel and
// follows the same order with q_w = nibble - zp.  Scales are the fp16-rounded ones,
// as in those reference kernels.
//
// Work split: a CTA owns 32 consecutive weight rows (lane = row) and its 8 or 16 warps
// own as many contiguous K-slices.  For one pair (64 K-elements) a warp reads 32 rows x
// 32 bytes = 1 KB contiguous with two 128-bit loads per lane, plus 8 bytes of
// fp16 {d_lo, d_hi, m_lo, m_hi} per lane.  Two batches of two pairs (8 x 128-bit loads)
// are in flight per lane, the first two issued before the activation row (int8 + block
// scales) is staged in shared memory, so that staging hides behind the weight latency.
//
// Reduction order (fixed, documented): inside a K-slice the reference's order is
// kept exactly - per pair fma(I_lo, d_a*d_w), fma(I_hi, ...), fma(m_lo, s_lo),
// fma(m_hi, s_hi), pairs ascending from a zero accumulator; the slice partials
// are then added in ascending slice order ((p0 + p1) + p2) + ...  (8 slices, or 16 for
// narrow or long-row layers: the choice depends only on the layer's shape).  Every int32
// block dot is exact.
//
// Algorithmic bytes per launch: rows*K/2 nibbles + rows*(K/32)*4 scale bytes
// (+ rows*(K/32) zero-point bytes for the A80 schemes) + K + (K/32)*8 activation
// bytes + rows*4 output bytes, i.e. 0.625 B per weight for A81W41.
#include <cuda_fp16.h>

#include "glue_math.cuh"
#include "inkq_internal.h"
#include "ptx.cuh"
#include "qgemv_common.cuh"

namespace inkq {

// What a fused launch does around the matrix-vector product (decode step of a model: one launch per layer
// instead of norm + quantizer + QGEMV + residual add).  The quantization arithmetic is the quantizer's own,
// operation for operation, so the result equals quantize + QGEMV on the same fp32 row.
struct FusedM1 {
    const float *x;      // fp32 input row: K values (PRO_SILU_MUL: 2K values in (32 gate, 32 up) groups)
    const float *g;      // PRO_RMSNORM: the norm's weight vector
    float eps;
    int pro;             // PRO_*
    int qmode;           // INKQ_Q8_1_F16 or INKQ_Q8_0_F16
    int accumulate;      // 1: C[n] += result (residual connection), 0: C[n] = result
};
enum { PRO_PLAIN = 0, PRO_RMSNORM = 1, PRO_SILU_MUL = 2 };

// Builds the quantized activation row in shared memory from fp32 input (two lanes per 32-element block, as
// k_quantize_q8): optional RMSNorm (x * 1/sqrt(mean(x^2) + eps) * g) or SiLU(gate) * up first.
template <bool HAS_MIN>
__device__ __forceinline__ void fused_prologue(const FusedM1 &f, int K, uint32_t *qa, float *da, float *sa, float *red)
{
    const int nb = K / QK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int half = threadIdx.x & 1;
    const unsigned gmask = 0x3u << (threadIdx.x & 30);                     // the two lanes of a block
    // When the row fits one trip of the block loop (K <= 16 * blockDim.x) the values read for the sum of squares
    // stay in registers for the quantization: every CTA of the grid reads the row, so a second read doubles the
    // L2 traffic of the prologue.
    const bool single_trip = nb <= static_cast<int>(blockDim.x >> 1);
    float4 keep[4];
    float inv = 1.0f;
    if (f.pro == PRO_RMSNORM) {
        float ss = 0.0f;
        if (single_trip) {
            const int blk = threadIdx.x >> 1;
            if (blk < nb) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    keep[j] = reinterpret_cast<const float4 *>(f.x)[blk * 8 + 2 * j + half];
                    ss += keep[j].x * keep[j].x + keep[j].y * keep[j].y + keep[j].z * keep[j].z + keep[j].w * keep[j].w;
                }
            }
        } else {
            for (int i = threadIdx.x; i < K / 4; i += blockDim.x) {
                const float4 v = reinterpret_cast<const float4 *>(f.x)[i];
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        float tot = 0.0f;
        for (int w2 = 0; w2 < nwarps; w2++) tot += red[w2];
        inv = rms_inv(tot, K, f.eps);
        __syncthreads();   // red is reused for the slice partials
    }
    for (int blk = threadIdx.x >> 1; blk < nb; blk += blockDim.x >> 1) {   // both lanes of a pair run the same trip count
        float4 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i4 = blk * 8 + 2 * j + half;
            float4 t;
            if (f.pro == PRO_RMSNORM && single_trip) t = keep[j];
            else if (f.pro == PRO_SILU_MUL) t = reinterpret_cast<const float4 *>(f.x)[blk * 16 + 2 * j + half];   // gate half of the group
            else t = reinterpret_cast<const float4 *>(f.x)[i4];
            if (f.pro == PRO_RMSNORM) {
                const float4 gg = reinterpret_cast<const float4 *>(f.g)[i4];
                t = rms_scale4(t, inv, gg);
            } else if (f.pro == PRO_SILU_MUL) {
                const float4 u = reinterpret_cast<const float4 *>(f.x)[blk * 16 + 8 + 2 * j + half];                   // up half
                t = make_float4(silu_mul(t.x, u.x), silu_mul(t.y, u.y), silu_mul(t.z, u.z), silu_mul(t.w, u.w));
            }
            v[j] = t;
        }
        float mx = 0.0f;
#pragma unroll
        for (int j = 0; j < 4; j++) mx = fmaxf(mx, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
        mx = fmaxf(mx, __shfl_xor_sync(gmask, mx, 1));
        const float dd = __fdiv_rn(mx, 127.0f);
        const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int i0 = __float2int_rn(__fmul_rn(v[j].x, id));
            const int i1 = __float2int_rn(__fmul_rn(v[j].y, id));
            const int i2 = __float2int_rn(__fmul_rn(v[j].z, id));
            const int i3 = __float2int_rn(__fmul_rn(v[j].w, id));
            sum += (i0 + i1) + (i2 + i3);
            qa[blk * 8 + 2 * j + half] = pack_sat_s8x4_m1(i0, i1, i2, i3);
        }
        sum += __shfl_xor_sync(gmask, sum, 1);
        if (half == 0) {
            da[blk] = __half2float(__float2half_rn(dd));
            if (HAS_MIN) sa[blk] = (f.qmode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(__fmul_rn(dd, static_cast<float>(sum)))) : 0.0f;
            else reinterpret_cast<int32_t *>(sa)[blk] = sum;
        }
    }
}

// WARPS = K-slices per CTA: 8 for wide layers, 16 for narrow ones (more bytes in flight per SM when
// the grid alone cannot fill the machine).  The register budget keeps 3 (resp. 2) CTAs per SM resident so
// that every Qwen3-8B shape runs as a single wave.  FUSED: the activation row is built from fp32 input in
// the prologue (FusedM1) instead of being read from a quantizer's output.
template <bool HAS_MIN, int WARPS, bool FUSED, bool DEEP>
__global__ void __launch_bounds__(WARPS * 32, GemvShape<WARPS, DEEP>::CTAS_PER_SM) k_qgemv_a8w4(const uint8_t *__restrict__ nibT, const uint2 *__restrict__ sc16,
                                                               const uchar2 *__restrict__ zpT, const int8_t *__restrict__ q,
                                                               const float *__restrict__ d, const float *__restrict__ s,
                                                               const int32_t *__restrict__ isum, int M_ld, float *__restrict__ C,
                                                               int rows, int K, int pairs, const ExtraDst extra, const FusedM1 fused)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nb = K / QK;
    uint32_t *qa = reinterpret_cast<uint32_t *>(smem_raw);          // K/4 words
    float *da = reinterpret_cast<float *>(smem_raw + K);            // nb
    float *sa = da + nb;                                            // nb (sums, or integer sums for the A80 schemes)
    float *part = sa + nb;                                          // [WARPS][32]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x >> 2;
    const int r = ((blockIdx.x & 3) << 5) + lane;
    const bool swz = ((r >> 2) & 1) != 0;
    const int p_begin = (warp * pairs) / WARPS, p_end = ((warp + 1) * pairs) / WARPS;
    const size_t slab = static_cast<size_t>(t) * pairs;

    // The weight stream does not depend on the activations: put the first two batches in flight
    // before anything else, so the staging of the activation row hides behind their latency.
    RowStream<HAS_MIN, GemvShape<WARPS, DEEP>::DEPTH, GemvShape<WARPS, DEEP>::WIDE> rs;
    rs.prime(nibT, sc16, zpT, slab, r, p_begin, p_end);
    // Programmatic dependent launch: this grid may have started while its predecessor in the stream
    // (normally the quantizer that produces q, d, s) was still running.  The weights above are
    // independent of it; everything below is not, so wait for the predecessor to complete here, and
    // let the successor start its own weight prefetch right away.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (FUSED) {
        fused_prologue<HAS_MIN>(fused, K, qa, da, sa, part);
    } else {
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x)
            reinterpret_cast<uint4 *>(qa)[i] = reinterpret_cast<const uint4 *>(q)[i];
        for (int b = threadIdx.x; b < nb; b += blockDim.x) {
            da[b] = d[static_cast<size_t>(b) * M_ld];
            if (HAS_MIN) sa[b] = s[static_cast<size_t>(b) * M_ld];
            else reinterpret_cast<int32_t *>(sa)[b] = isum[static_cast<size_t>(b) * M_ld];
        }
    }
    __syncthreads();

    const float acc = rs.run(0.0f, swz, qa, da, sa, nibT, sc16, zpT, slab, r, p_begin, p_end);
    part[warp * 32 + lane] = acc;
    __syncthreads();
    if (warp == 0) {
        float tot = part[lane];
#pragma unroll
        for (int w2 = 1; w2 < WARPS; w2++) tot = __fadd_rn(tot, part[w2 * 32 + lane]);
        const int n = t * TILE_N + r;
        if (n < rows) {
            if (FUSED && fused.accumulate) tot = __fadd_rn(C[n], tot);
            C[n] = tot;
#pragma unroll
            for (int e = 0; e < MAX_PEERS - 1; e++)                  // column-sharded layer: the same element in every peer's buffer
                if (e < extra.n) extra.p[e][n] = tot;                // (static indices: the parameter array stays out of local memory)
        }
    }
}

template <bool HAS_MIN, int WARPS, bool FUSED, bool DEEP = false>
static void launch_gemv_variant(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, const ExtraDst &extra, const FusedM1 &fused)
{
    const size_t smem = static_cast<size_t>(w->K) + 2 * sizeof(float) * (w->K / QK) + sizeof(float) * WARPS * 32;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(k_qgemv_a8w4<HAS_MIN, WARPS, FUSED, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    // launched with programmatic stream serialization: the grid may begin (and prefetch weights) before the
    // previous kernel in the stream has finished; it waits for that kernel inside (griddepcontrol.wait)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(w->tiles) * 4);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, k_qgemv_a8w4<HAS_MIN, WARPS, FUSED, DEEP>, static_cast<const uint8_t *>(w->nibT), static_cast<const uint2 *>(w->sc16),
                       static_cast<const uchar2 *>(w->zpT), static_cast<const int8_t *>(a ? a->q : nullptr),
                       static_cast<const float *>(a ? a->d : nullptr), static_cast<const float *>(a ? a->s : nullptr),
                       static_cast<const int32_t *>(a ? a->isum : nullptr), a ? a->M_ld : 0, C, w->rows, w->K, w->pairs, extra, fused);
}

template <bool FUSED>
static void launch_gemv_any(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, const ExtraDst &extra, const FusedM1 &fused)
{
    // narrow layers (few CTAs) or long rows: 16 K-slices per CTA
    const bool wide_cta = (w->tiles * 4 <= 2 * ctx->num_sms) || (w->pairs >= 128);
    // no more CTAs than SMs and long rows: one CTA per SM with four batches in flight per lane (same accumulation order)
    const bool deep = wide_cta && gemv_deep(w->tiles * 4, w->pairs, 16, ctx->num_sms);
    if (w->scheme == INKQ_A81W41) {
        if (deep) launch_gemv_variant<true, 16, FUSED, true>(ctx, a, w, C, extra, fused);
        else if (wide_cta) launch_gemv_variant<true, 16, FUSED>(ctx, a, w, C, extra, fused);
        else launch_gemv_variant<true, 8, FUSED>(ctx, a, w, C, extra, fused);
    } else {
        if (deep) launch_gemv_variant<false, 16, FUSED, true>(ctx, a, w, C, extra, fused);
        else if (wide_cta) launch_gemv_variant<false, 16, FUSED>(ctx, a, w, C, extra, fused);
        else launch_gemv_variant<false, 8, FUSED>(ctx, a, w, C, extra, fused);
    }
}

int launch_gemv(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, const ExtraDst *extra_in)
{
    ExtraDst extra = {};
    if (extra_in != nullptr) extra = *extra_in;
    launch_gemv_any<false>(ctx, a, w, C, extra, FusedM1{});
    return after_launch(ctx, "k_qgemv_a8w4");
}

int launch_gemv_fused(inkq_ctx *ctx, const Weight *w, const float *x, int pro, const float *g, float eps, float *C, int accumulate)
{
    FusedM1 f;
    f.x = x;
    f.g = g;
    f.eps = eps;
    f.pro = pro;
    f.qmode = (w->scheme == INKQ_A81W41) ? INKQ_Q8_1_F16 : INKQ_Q8_0_F16;   // as inkq_linear chooses for M == 1
    f.accumulate = accumulate;
    launch_gemv_any<true>(ctx, nullptr, w, C, ExtraDst{}, f);
    return after_launch(ctx, "k_qgemv_a8w4 (fused prologue)");
}

}  // namespace inkq
