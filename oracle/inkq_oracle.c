/*
 * CPU oracle for the A8W4 quantized-matmul path of Qwen3.Ink.Cpp.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the shipped library links, loads or calls it.
 *
 * It restates, in plain scalar C, the arithmetic of the reference's AVX2/VNNI
 * kernels (paths are relative to the reference project root):
 *   quantizers   qwen3/src/qwen/quantized_gemx_kernels.cc:584-911
 *   matmuls      qwen3/src/qwen/quantized_gemx_kernels.cc:39-582
 *   re-tilers    qwen3/src/qwen/QwenOperator.cc:757-892
 *   tile structs qwen3/include/qwen/QwenOperator.h:46-80
 * and, for the schemes the reference has no C++ kernel for, the notebook math
 *   A80W4z       notebooks/evaluate-qwen3_8b_A8W4.ipynb cell 16
 *   W41 w-only   notebooks/evaluate-qwen3_8b_W4.ipynb cell 13
 *
 * Parity pin: every function that has a reference counterpart is compared
 * bit-for-bit against the reference's own objects (compiled unmodified by
 * oracle/Makefile into oracle/_ref/) and against the committed fixtures under
 * tests/golden/, which were produced by those objects.  The restatement-only
 * schemes (A80W4z, weight-only W41, fp16 lm_head) have no reference kernel:
 * parity unpinned for those three, they follow the cited notebook formulas.
 *
 * fp16 conversion: the reference uses ggml's GGML_FP32_TO_FP16, whose contract
 * is IEEE-754 binary16 round-to-nearest-even; ggml is an un-vendored submodule
 * of the reference (no pinned commit visible), so the conversion is restated
 * here from the IEEE definition and cross-checked against F16C and NumPy.
 *
 * Build: gcc -O2 -mfma -ffp-contract=off -fopenmp -fPIC -shared (oracle/Makefile).
 * Every fused multiply-add the reference performs is written as fmaf(); with
 * contraction off nothing else is fused.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK 32

/* ------------------------------------------------------------------------- */
/* IEEE binary16 <-> binary32, round-to-nearest-even                          */
/* ------------------------------------------------------------------------- */
uint16_t ink_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) { /* inf / nan */
        if (absx > 0x7f800000u) return (uint16_t)(sign | 0x7e00u | ((absx >> 13) & 0x3ffu));
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u); /* rounds to inf (>= 65520) */
    if (absx < 0x33000001u) return (uint16_t)sign;              /* <= 2^-25 rounds to zero */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x7fffffu) | 0x800000u; /* 24-bit significand */
    int shift;
    uint32_t half_exp;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        half_exp = 0;
    } else {
        shift = 13;
        half_exp = (uint32_t)(e + 15);
    }
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    uint32_t out;
    if (half_exp == 0) {
        out = q; /* may carry into the exponent field: that is the correct normal */
    } else {
        out = ((half_exp - 1) << 10) + q; /* q carries the implicit bit (0x400) */
    }
    return (uint16_t)(sign | out);
}

float ink_f16_to_f32(uint16_t h)
{
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t x;
    if (e == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int sh = 0;
            while (!(man & 0x400u)) { man <<= 1; sh++; }
            man &= 0x3ffu;
            x = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (man << 13);
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (man << 13);
    } else {
        x = sign | ((e + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

static inline float round_f16(float f) { return ink_f16_to_f32(ink_f32_to_f16(f)); }

/* ------------------------------------------------------------------------- */
/* Activation quantizer (Q8_0 / Q8_1), planar output                          */
/* ------------------------------------------------------------------------- */
/*
 * mode 0: Q8_0, fp16 scale            quantized_gemx_kernels.cc:584-691
 * mode 1: Q8_1, fp16 scale and sum    quantized_gemx_kernels.cc:693-801
 * mode 2: Q8_1, fp32 scale and sum    quantized_gemx_kernels.cc:803-911
 *
 * Per block of 32: mx = max|x|; d = mx / 127; id = mx != 0 ? 127 / mx : 0;
 * q = saturate_s8(rne(x * id)); s = d * (float)sum(q), with d the UNROUNDED
 * fp32 value even in mode 1 (:777,:779).  d and s are returned as fp32 numbers
 * that hold the (possibly fp16-rounded) stored value.  In mode 0 the reference
 * leaves the sum fields unwritten; here s is set to 0.
 *
 * The reference rounds with _mm256_round_ps(NEAREST) then cvtps_epi32, then
 * packs with signed saturation (:893-900): |x*id| <= 127 up to one rounding, so
 * saturation can only matter for non-finite input; it is kept for fidelity.
 */
void ink_quantize_q8(const float *x, int64_t n_elems, int mode, int8_t *q, float *d, float *s)
{
    const int64_t nb = n_elems / QK;
    for (int64_t b = 0; b < nb; b++) {
        const float *xb = x + b * QK;
        float mx = 0.0f;
        for (int e = 0; e < QK; e++) {
            const float a = fabsf(xb[e]);
            if (a > mx) mx = a; /* maxps semantics: NaN operands never win */
        }
        const float dd = mx / 127.0f;
        const float id = (mx != 0.0f) ? 127.0f / mx : 0.0f;
        int32_t sum = 0;
        for (int e = 0; e < QK; e++) {
            const float v = nearbyintf(xb[e] * id); /* default rounding mode: nearest-even */
            int32_t iv;
            if (!(v >= -2147483648.0f && v < 2147483648.0f)) iv = INT32_MIN; /* cvtps2dq indefinite */
            else iv = (int32_t)v;
            sum += iv;
            if (iv > 127) iv = 127;
            if (iv < -128) iv = -128;
            q[b * QK + e] = (int8_t)iv;
        }
        const float ss = dd * (float)sum;
        if (mode == 2) {
            d[b] = dd;
            s[b] = ss;
        } else {
            d[b] = round_f16(dd);
            s[b] = (mode == 1) ? round_f16(ss) : 0.0f;
        }
    }
}

/* Reference activation tile structs, QwenOperator.h:56-63 and :73-80. */
typedef struct {
    uint16_t s_low, s_high, scaled_sum_low, scaled_sum_high;
    int8_t q_low[32], q_high[32];
} ink_q8_1x2_fp16;
typedef struct {
    float s_low, s_high, scaled_sum_low, scaled_sum_high;
    int8_t q_low[32], q_high[32];
} ink_q8_1x2_fp32;

/*
 * The three reference entry points, writing the reference's own byte layout so
 * the result can be memcmp'd with what the reference writes.  For Q8_0 the sum
 * fields are left untouched, as the reference does.
 */
static void quantize_struct(const float *x, void *vy, int64_t k, int mode)
{
    const int64_t npair = k / (2 * QK);
    int8_t q[2 * QK];
    float d[2], s[2];
    for (int64_t i = 0; i < npair; i++) {
        ink_quantize_q8(x + i * 2 * QK, 2 * QK, mode, q, d, s);
        if (mode == 2) {
            ink_q8_1x2_fp32 *y = (ink_q8_1x2_fp32 *)vy + i;
            y->s_low = d[0];
            y->s_high = d[1];
            y->scaled_sum_low = s[0];
            y->scaled_sum_high = s[1];
            memcpy(y->q_low, q, QK);
            memcpy(y->q_high, q + QK, QK);
        } else {
            ink_q8_1x2_fp16 *y = (ink_q8_1x2_fp16 *)vy + i;
            y->s_low = ink_f32_to_f16(d[0]);
            y->s_high = ink_f32_to_f16(d[1]);
            if (mode == 1) {
                y->scaled_sum_low = ink_f32_to_f16(s[0]);
                y->scaled_sum_high = ink_f32_to_f16(s[1]);
            }
            memcpy(y->q_low, q, QK);
            memcpy(y->q_high, q + QK, QK);
        }
    }
}
void ink_quantize_row_q8_0_repack(const float *x, void *vy, int64_t k) { quantize_struct(x, vy, k, 0); }
void ink_quantize_row_q8_1_repack_fp16(const float *x, void *vy, int64_t k) { quantize_struct(x, vy, k, 1); }
void ink_quantize_row_q8_1_repack_fp32(const float *x, void *vy, int64_t k) { quantize_struct(x, vy, k, 2); }

/* ------------------------------------------------------------------------- */
/* Load-time weight re-tilers into the reference's CPU superblocks            */
/* ------------------------------------------------------------------------- */
/* QwenOperator.h:48-54 and :65-71 */
typedef struct {
    uint16_t s_low[8], s_high[8], min_low[8], min_high[8];
    uint8_t q_coupled[256];
} ink_q4_2x8_fp16;
typedef struct {
    float s_low[8], s_high[8], min_low[8], min_high[8];
    uint8_t q_coupled[256];
} ink_q4_2x8_fp32;

/*
 * Superblock (j = n/8, i = k/64) sits at index j*(K/64)+i; within it
 * q_coupled[p*32 + jj*4 + ii] = disk_byte[n = 8j+jj][32i + 4p + ii]
 * (QwenOperator.cc:862,879-888).  SB / MinB are [N][K/32] fp32.
 * variant 0: w80 (fp16 scales, mins untouched)   :757-799
 * variant 1: w81 fp16                             :801-850
 * variant 2: w81 fp32                             :852-892
 */
static void repack(int K, int N, void *out, const float *SB, const float *MinB, const uint8_t *B, int variant)
{
    const int nbk = K / 64, nbn = N / 8, ldb = K / 2, lds = K / QK;
    for (int j = 0; j < nbn; j++)
        for (int i = 0; i < nbk; i++) {
            uint8_t *qc;
            if (variant == 2) {
                ink_q4_2x8_fp32 *t = (ink_q4_2x8_fp32 *)out + (size_t)j * nbk + i;
                for (int jj = 0; jj < 8; jj++) {
                    const size_t r = (size_t)(j * 8 + jj) * lds;
                    t->s_low[jj] = SB[r + 2 * i];
                    t->s_high[jj] = SB[r + 2 * i + 1];
                    t->min_low[jj] = MinB[r + 2 * i];
                    t->min_high[jj] = MinB[r + 2 * i + 1];
                }
                qc = t->q_coupled;
            } else {
                ink_q4_2x8_fp16 *t = (ink_q4_2x8_fp16 *)out + (size_t)j * nbk + i;
                for (int jj = 0; jj < 8; jj++) {
                    const size_t r = (size_t)(j * 8 + jj) * lds;
                    t->s_low[jj] = ink_f32_to_f16(SB[r + 2 * i]);
                    t->s_high[jj] = ink_f32_to_f16(SB[r + 2 * i + 1]);
                    if (variant == 1) {
                        t->min_low[jj] = ink_f32_to_f16(MinB[r + 2 * i]);
                        t->min_high[jj] = ink_f32_to_f16(MinB[r + 2 * i + 1]);
                    }
                }
                qc = t->q_coupled;
            }
            for (int p = 0; p < 8; p++)
                for (int jj = 0; jj < 8; jj++)
                    for (int ii = 0; ii < 4; ii++)
                        qc[p * 32 + jj * 4 + ii] = B[(size_t)(j * 8 + jj) * ldb + i * 32 + p * 4 + ii];
        }
}
void ink_repack_w80_weight(int K, int N, void *out, const float *SB, const uint8_t *B) { repack(K, N, out, SB, NULL, B, 0); }
void ink_repack_w81_weight_fp16(int K, int N, void *out, const float *SB, const float *MinB, const uint8_t *B) { repack(K, N, out, SB, MinB, B, 1); }
void ink_repack_w81_weight_fp32(int K, int N, void *out, const float *SB, const float *MinB, const uint8_t *B) { repack(K, N, out, SB, MinB, B, 2); }

/* ------------------------------------------------------------------------- */
/* A8W4 matmuls from the logical (planar) formats                             */
/* ------------------------------------------------------------------------- */
/*
 * Logical inputs
 *   activations: q_a s8 [M][K], d_a f32 [M][K/32], s_a f32 [M][K/32]
 *   weights    : nib u8 [N][K/2] in the on-disk AWQ-interleaved order
 *                (byte[32g+e] = q[64g+e] | q[64g+32+e] << 4,
 *                 notebooks/quantize_methods.py:61-64,120-123),
 *                d_w f32 [N][K/32], m_w f32 [N][K/32], zp u8 [N][K/32]
 * The caller passes scales already rounded the way the reference kernel under
 * test sees them (fp32 as stored for gemm_repack_A81W41_fp32; fp16-rounded for
 * the three fp16 kernels), so one routine per scheme covers GEMM and GEMV: the
 * reference's GEMM and GEMV use the same per-output operation order.
 *
 * scheme 0  A81W41: acc = fma((float)I_lo, d_a_lo*d_w_lo, acc);
 *                   acc = fma((float)I_hi, d_a_hi*d_w_hi, acc);
 *                   acc = fma(m_lo, s_a_lo, acc); acc = fma(m_hi, s_a_hi, acc)
 *           per 64-element pair, pairs ascending
 *           (quantized_gemx_kernels.cc:495-512 and :181-188); I = sum q_a*q_w,
 *           q_w in [0,15].
 * scheme 1  A80W40: acc = fma((float)I_lo, d_a_lo*d_w_lo, acc); same for hi;
 *           q_w = nibble - 8 (:246-248,:323-330 and :72-74,:99-102).
 * scheme 2  A80W4z: as scheme 1 with q_w = nibble - zp[n][block]
 *           (w ~ (q - zp) * s, evaluate-qwen3_8b_A8W4.ipynb cell 16); there is
 *           no reference kernel for it, the order is chosen to match scheme 1.
 *
 * dots (nullable) receives every int32 block dot, [rows][N][K/32].
 * The routine computes rows listed in row_idx (nullable = all M rows) and
 * columns [n0, n1).
 */
void ink_gemm_a8w4(int scheme, int M, int N, int K,
                   const int8_t *q_a, const float *d_a, const float *s_a,
                   const uint8_t *nib, const float *d_w, const float *m_w, const uint8_t *zp,
                   float *C, int ldc, int32_t *dots,
                   int n0, int n1)
{
    const int nbk = K / QK, npair = K / 64;
#pragma omp parallel for schedule(static)
    for (int n = n0; n < n1; n++) {
        const uint8_t *wrow = nib + (size_t)n * (K / 2);
        for (int i = 0; i < M; i++) {
            const int8_t *arow = q_a + (size_t)i * K;
            float acc = 0.0f;
            for (int g = 0; g < npair; g++) {
                int zlo = 0, zhi = 0;
                if (scheme == 1) zlo = zhi = 8;
                if (scheme == 2) {
                    zlo = zp[(size_t)n * nbk + 2 * g];
                    zhi = zp[(size_t)n * nbk + 2 * g + 1];
                }
                int32_t ilo = 0, ihi = 0;
                for (int e = 0; e < 32; e++) {
                    const uint8_t byte = wrow[g * 32 + e];
                    ilo += (int32_t)arow[g * 64 + e] * ((int32_t)(byte & 0x0f) - zlo);
                    ihi += (int32_t)arow[g * 64 + 32 + e] * ((int32_t)(byte >> 4) - zhi);
                }
                if (dots) {
                    dots[((size_t)i * N + n) * nbk + 2 * g] = ilo;
                    dots[((size_t)i * N + n) * nbk + 2 * g + 1] = ihi;
                }
                const size_t ab = (size_t)i * nbk + 2 * g, wb = (size_t)n * nbk + 2 * g;
                const float slo = d_a[ab] * d_w[wb];
                const float shi = d_a[ab + 1] * d_w[wb + 1];
                acc = fmaf((float)ilo, slo, acc);
                acc = fmaf((float)ihi, shi, acc);
                if (scheme == 0) {
                    acc = fmaf(m_w[wb], s_a[ab], acc);
                    acc = fmaf(m_w[wb + 1], s_a[ab + 1], acc);
                }
            }
            C[(size_t)i * ldc + n] = acc;
        }
    }
}

/* Same arithmetic for a list of (row, col) samples; out[t] = C[rows[t]][cols[t]]. */
void ink_gemm_a8w4_samples(int scheme, int N, int K,
                           const int8_t *q_a, const float *d_a, const float *s_a,
                           const uint8_t *nib, const float *d_w, const float *m_w, const uint8_t *zp,
                           const int32_t *rows, const int32_t *cols, int nsamples, float *out)
{
#pragma omp parallel for schedule(static)
    for (int t = 0; t < nsamples; t++) {
        const int i = rows[t], n = cols[t];
        (void)N;
        ink_gemm_a8w4(scheme, 1, n + 1, K, q_a + (size_t)i * K, d_a + (size_t)i * (K / QK),
                      s_a ? s_a + (size_t)i * (K / QK) : NULL, nib, d_w, m_w, zp,
                      out + t - n, 0, NULL, n, n + 1);
    }
}

/* ------------------------------------------------------------------------- */
/* Weight-only W41 and fp16 lm_head (restatements; no reference C++ kernel)   */
/* ------------------------------------------------------------------------- */
/*
 * Weight-only W41 (evaluate-qwen3_8b_W4.ipynb cell 13): the fp16 model's weight
 * is replaced by the dequantised value w = q*d + m held in fp16, then a stock
 * fp16 linear runs.  Restated as: w16 = fp16(q*d + m) with d, m the fp16-rounded
 * block scale and minimum and ONE rounding of the exact value (what a half-precision
 * fused multiply-add returns); C = sum_k a16*w16 accumulated in fp32, k ascending.
 * a is given as fp16 bit patterns.
 */
/* Nearest fp16 (ties to even) of a double that holds an exact value, returned as float. */
static float round_f16_exact(double v)
{
    if (v == 0.0) return 0.0f;
    int e;
    (void)frexp(fabs(v), &e);                /* |v| = f * 2^e, f in [0.5, 1) */
    int ulp_exp = (e - 1) - 10;              /* fp16 keeps 11 significant bits */
    if (ulp_exp < -24) ulp_exp = -24;        /* subnormal grid */
    const double r = nearbyint(ldexp(v, -ulp_exp));   /* exact scaling; default rounding mode = ties to even */
    double out = ldexp(r, ulp_exp);
    if (fabs(out) > 65504.0) out = copysign(INFINITY, v);
    return (float)out;
}

void ink_gemm_w41_f16act(int M, int N, int K, const uint16_t *a16,
                         const uint8_t *nib, const float *d_w, const float *m_w,
                         float *C, int ldc)
{
    const int nbk = K / QK;
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; n++) {
        float *w = (float *)malloc(sizeof(float) * (size_t)K);
        for (int g = 0; g < K / 64; g++)
            for (int e = 0; e < 32; e++) {
                const uint8_t byte = nib[(size_t)n * (K / 2) + g * 32 + e];
                const size_t wb = (size_t)n * nbk + 2 * g;
                /* q*d + m is exact in double (4 + 11 + 11 significant bits within fp16's exponent range) */
                w[g * 64 + e] = round_f16_exact((double)(byte & 0x0f) * (double)round_f16(d_w[wb]) + (double)round_f16(m_w[wb]));
                w[g * 64 + 32 + e] = round_f16_exact((double)(byte >> 4) * (double)round_f16(d_w[wb + 1]) + (double)round_f16(m_w[wb + 1]));
            }
        for (int i = 0; i < M; i++) {
            float acc = 0.0f;
            for (int k = 0; k < K; k++) acc = fmaf(ink_f16_to_f32(a16[(size_t)i * K + k]), w[k], acc);
            C[(size_t)i * ldc + n] = acc;
        }
        free(w);
    }
}

/*
 * lm_head with fp16 weights and fp32 activations: logits[n] = sum_k x[k]*w[n][k].
 * Nearest reference arithmetic: gemv_fp32_rcr_mt_impl_1,
 * qwen3/src/qwen/fp32_gemx_kernels_rcr.cc:494-507 (the reference's own lm_head is
 * an int4 A81W41 linear, QwenForCausalLM.cc:121).  There is no reference kernel
 * to be bit-compatible with, so the oracle accumulates in double and rounds once:
 * it is the exact value any fp32 summation order is compared against.
 */
void ink_lmhead_f16w(int M, int N, int K, const float *x, const uint16_t *w16, float *C, int ldc,
                     int n0, int n1)
{
#pragma omp parallel for schedule(static)
    for (int n = n0; n < n1; n++)
        for (int i = 0; i < M; i++) {
            double acc = 0.0;
            for (int k = 0; k < K; k++)
                acc += (double)x[(size_t)i * K + k] * (double)ink_f16_to_f32(w16[(size_t)n * K + k]);
            C[(size_t)i * ldc + n] = (float)acc;
        }
}

/* ------------------------------------------------------------------------- */
/* Offline weight quantizers (format definition)                              */
/* ------------------------------------------------------------------------- */
/*
 * Q4_1: notebooks/quantize_methods.py:68-125.  Per block: d = (max-min)/15,
 * m = min, id = d != 0 ? 1/d : 0, q = clip(rint((x-m)*id), 0, 15) (np.round is
 * round-half-even).  Output in the disk layout: nib [N][K/2], d/m [N][K/32].
 * Q4_0: notebooks/quantize_methods.py:13-66.  d = x[argmax|x|] / -8 (first
 * index on ties, as np.argmax), id = d != 0 ? 1/d : 0,
 * q = (uint8)clip(x*id + 8.5, 0, 15) (truncation), m = 0.
 */
void ink_quantize_weight_q4(int which /*0: Q4_0, 1: Q4_1*/, int N, int K, const float *w,
                            uint8_t *nib, float *d, float *m)
{
    const int nbk = K / QK;
    for (int n = 0; n < N; n++)
        for (int b = 0; b < nbk; b++) {
            const float *x = w + (size_t)n * K + (size_t)b * QK;
            uint8_t q[QK];
            float dd, mm;
            if (which == 1) {
                float mx = x[0], mn = x[0];
                for (int e = 1; e < QK; e++) {
                    if (x[e] > mx) mx = x[e];
                    if (x[e] < mn) mn = x[e];
                }
                dd = (mx - mn) / 15.0f;
                mm = mn;
                const float id = (dd != 0.0f) ? 1.0f / dd : 0.0f;
                for (int e = 0; e < QK; e++) {
                    float v = nearbyintf((x[e] - mm) * id);
                    if (v < 0.0f) v = 0.0f;
                    if (v > 15.0f) v = 15.0f;
                    q[e] = (uint8_t)v;
                }
            } else {
                int arg = 0;
                float best = fabsf(x[0]);
                for (int e = 1; e < QK; e++)
                    if (fabsf(x[e]) > best) { best = fabsf(x[e]); arg = e; }
                dd = x[arg] / -8.0f;
                mm = 0.0f;
                const float id = (dd != 0.0f) ? 1.0f / dd : 0.0f;
                for (int e = 0; e < QK; e++) {
                    float v = x[e] * id + 8.5f;
                    if (v < 0.0f) v = 0.0f;
                    if (v > 15.0f) v = 15.0f;
                    q[e] = (uint8_t)v;
                }
            }
            d[(size_t)n * nbk + b] = dd;
            m[(size_t)n * nbk + b] = mm;
            uint8_t *dst = nib + (size_t)n * (K / 2) + (size_t)(b / 2) * 32;
            for (int e = 0; e < QK; e++) {
                if (b % 2 == 0) dst[e] = (uint8_t)((dst[e] & 0xf0) | q[e]);
                else dst[e] = (uint8_t)((dst[e] & 0x0f) | (q[e] << 4));
            }
        }
}
