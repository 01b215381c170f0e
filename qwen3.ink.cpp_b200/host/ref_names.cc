// The reference's kernel-level functions, by their own names and signatures
// (qwen3/include/qwen/QwenOperator.h:82-84,276-304), running on the GPU.
//
// A caller that already links against the reference's free functions - its tests
// (qwen3/tests/test_linear*.cc) or Qwen_Linear_with_bias_Int4::forward itself - can link
// this object instead: host pointers in, host pointers out, the reference's own struct
// layouts (q8_repack_1x2_fp16/_fp32, q4_repack_2x8_fp16/_fp32, QwenOperator.h:46-80) on both
// sides.  The arithmetic runs in the CUDA library; what happens here is only the
// re-arrangement between the reference's CPU tile structs and the logical arrays the C ABI
// takes.  C++ linkage on purpose: these are drop-ins for C++ functions.
//
// Weights: repack_* writes the reference's superblock layout into the caller's buffer (so a
// copied buffer still works, the reference deep-copies its layers) and uploads the re-tiled
// weights once, remembered by buffer address; the matmuls look the buffer up and fall back
// to rebuilding the upload from the superblocks when the address is unknown.  The cache is
// keyed by address: a buffer that is refilled with other weights must go through repack_*
// again (or inkq_refshim_forget), and a freed buffer should be forgotten; one lock is held from
// the look-up to the end of the matmul, so a concurrent re-registration cannot free an entry
// in use.
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "inkq.h"

typedef uint16_t fp16_t;
namespace {

struct q4_2x8_f16 { fp16_t s_low[8], s_high[8], min_low[8], min_high[8]; uint8_t q_coupled[256]; };
struct q4_2x8_f32 { float s_low[8], s_high[8], min_low[8], min_high[8]; uint8_t q_coupled[256]; };
struct q8_1x2_f16 { fp16_t s_low, s_high, scaled_sum_low, scaled_sum_high; int8_t q_low[32], q_high[32]; };
struct q8_1x2_f32 { float s_low, s_high, scaled_sum_low, scaled_sum_high; int8_t q_low[32], q_high[32]; };
static_assert(sizeof(q4_2x8_f16) == 320 && sizeof(q4_2x8_f32) == 384 && sizeof(q8_1x2_f16) == 72 && sizeof(q8_1x2_f32) == 80, "layout");

// IEEE binary16 <-> binary32, round to nearest even (the contract of the reference's GGML_FP32_TO_FP16).
fp16_t f32_to_f16(float f)
{
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, a = x & 0x7fffffffu;
    if (a >= 0x7f800000u) return static_cast<fp16_t>(sign | (a > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (a >= 0x477ff000u) return static_cast<fp16_t>(sign | 0x7c00u);
    if (a < 0x33000001u) return static_cast<fp16_t>(sign);
    const int e = static_cast<int>(a >> 23) - 127;
    const uint32_t man = (a & 0x7fffffu) | 0x800000u;
    const int shift = e < -14 ? 13 + (-14 - e) : 13;
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    const uint32_t out = e < -14 ? q : ((static_cast<uint32_t>(e + 15) - 1u) << 10) + q;
    return static_cast<fp16_t>(sign | out);
}
float f16_to_f32(fp16_t h)
{
    const uint32_t sign = (static_cast<uint32_t>(h) & 0x8000u) << 16, e = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu, x;
    if (e == 0) {
        if (man == 0) x = sign;
        else {
            int sh = 0;
            while (!(man & 0x400u)) { man <<= 1; sh++; }
            x = sign | (static_cast<uint32_t>(113 - sh) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (e == 31) x = sign | 0x7f800000u | (man << 13);
    else x = sign | ((e + 112) << 23) | (man << 13);
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

struct Entry {
    inkq_weight *w;
    int scale_mode;
};
struct Gpu {
    inkq_ctx *ctx = nullptr;
    std::recursive_mutex mu;
    std::map<const void *, Entry> weights;   // by B_repack address
    inkq_act *act = nullptr;
    int act_rows = 0, act_k = 0;
    Gpu()
    {
        if (inkq_ctx_create(0, nullptr, &ctx) != INKQ_OK) throw std::runtime_error(std::string("inkq: ") + inkq_last_error(nullptr));
    }
    void check(int rc) { if (rc != INKQ_OK) throw std::runtime_error(std::string("inkq: ") + inkq_last_error(ctx)); }
    inkq_act *activation(int rows, int k)
    {
        if (act == nullptr || act_k != k || act_rows < rows) {
            if (act) inkq_act_destroy(act);
            act = nullptr;
            check(inkq_act_create(ctx, rows, k, &act));
            act_rows = rows;
            act_k = k;
        }
        return act;
    }
};
Gpu &gpu()
{
    static Gpu g;
    return g;
}

// ---- activations: x -> reference struct array ---------------------------------------------
void quantize_to_structs(const float *x, void *vy, int64_t k, int qmode)
{
    Gpu &g = gpu();
    std::lock_guard<std::recursive_mutex> lk(g.mu);
    // blocks are independent, so the whole [m*k] vector is quantized as one row of k elements
    const int K = static_cast<int>(k);
    inkq_act *a = g.activation(1, K);
    std::vector<int8_t> q(k);
    std::vector<float> d(k / 32), s(k / 32);
    g.check(inkq_quantize_host(g.ctx, qmode, x, 1, K, a));
    g.check(inkq_act_export(g.ctx, a, q.data(), d.data(), s.data(), nullptr));
    const int64_t npair = k / 64;
    for (int64_t i = 0; i < npair; i++) {
        if (qmode == INKQ_Q8_1_F32) {
            q8_1x2_f32 *y = static_cast<q8_1x2_f32 *>(vy) + i;
            y->s_low = d[2 * i];
            y->s_high = d[2 * i + 1];
            y->scaled_sum_low = s[2 * i];
            y->scaled_sum_high = s[2 * i + 1];
            std::memcpy(y->q_low, &q[64 * i], 32);
            std::memcpy(y->q_high, &q[64 * i + 32], 32);
        } else {
            q8_1x2_f16 *y = static_cast<q8_1x2_f16 *>(vy) + i;
            y->s_low = f32_to_f16(d[2 * i]);
            y->s_high = f32_to_f16(d[2 * i + 1]);
            if (qmode == INKQ_Q8_1_F16) {   // the Q8_0 entry point leaves the sum fields untouched, as the reference does
                y->scaled_sum_low = f32_to_f16(s[2 * i]);
                y->scaled_sum_high = f32_to_f16(s[2 * i + 1]);
            }
            std::memcpy(y->q_low, &q[64 * i], 32);
            std::memcpy(y->q_high, &q[64 * i + 32], 32);
        }
    }
}

// ---- weights: logical arrays <-> reference superblocks ---------------------------------------
template <typename SB>
void write_superblocks(int K, int N, SB *out, const float *scales, const float *mins, const uint8_t *nib, bool fp16)
{
    const int nbk = K / 64, ldb = K / 2, lds = K / 32;
    for (int n = 0; n < N; n++) {
        const int j = n >> 3, jj = n & 7;
        for (int i = 0; i < nbk; i++) {
            SB &t = out[static_cast<size_t>(j) * nbk + i];
            const float sl = scales[static_cast<size_t>(n) * lds + 2 * i], sh = scales[static_cast<size_t>(n) * lds + 2 * i + 1];
            if constexpr (sizeof(t.s_low[0]) == 2) {
                t.s_low[jj] = f32_to_f16(sl);
                t.s_high[jj] = f32_to_f16(sh);
                if (mins) {
                    t.min_low[jj] = f32_to_f16(mins[static_cast<size_t>(n) * lds + 2 * i]);
                    t.min_high[jj] = f32_to_f16(mins[static_cast<size_t>(n) * lds + 2 * i + 1]);
                }
            } else {
                t.s_low[jj] = sl;
                t.s_high[jj] = sh;
                t.min_low[jj] = mins[static_cast<size_t>(n) * lds + 2 * i];
                t.min_high[jj] = mins[static_cast<size_t>(n) * lds + 2 * i + 1];
            }
            (void)fp16;
            // byte e of the pair's 32 disk bytes goes to pack e/4, lane jj, position e%4
            const uint8_t *src = nib + static_cast<size_t>(n) * ldb + i * 32;
            for (int e = 0; e < 32; e++) t.q_coupled[(e >> 2) * 32 + jj * 4 + (e & 3)] = src[e];
        }
    }
}

template <typename SB>
void read_superblocks(int K, int N, const SB *in, std::vector<uint8_t> &nib, std::vector<float> &d, std::vector<float> &m)
{
    const int nbk = K / 64, ldb = K / 2, lds = K / 32;
    nib.resize(static_cast<size_t>(N) * ldb);
    d.resize(static_cast<size_t>(N) * lds);
    m.assign(static_cast<size_t>(N) * lds, 0.0f);
    for (int n = 0; n < N; n++) {
        const int j = n >> 3, jj = n & 7;
        for (int i = 0; i < nbk; i++) {
            const SB &t = in[static_cast<size_t>(j) * nbk + i];
            const size_t b = static_cast<size_t>(n) * lds + 2 * i;
            if constexpr (sizeof(t.s_low[0]) == 2) {
                d[b] = f16_to_f32(t.s_low[jj]);
                d[b + 1] = f16_to_f32(t.s_high[jj]);
                m[b] = f16_to_f32(t.min_low[jj]);
                m[b + 1] = f16_to_f32(t.min_high[jj]);
            } else {
                d[b] = t.s_low[jj];
                d[b + 1] = t.s_high[jj];
                m[b] = t.min_low[jj];
                m[b + 1] = t.min_high[jj];
            }
            uint8_t *dst = nib.data() + static_cast<size_t>(n) * ldb + i * 32;
            for (int e = 0; e < 32; e++) dst[e] = t.q_coupled[(e >> 2) * 32 + jj * 4 + (e & 3)];
        }
    }
}

void remember(const void *key, int scheme, int scale_mode, int N, int K, const uint8_t *nib, const float *d, const float *m)
{
    Gpu &g = gpu();
    std::lock_guard<std::recursive_mutex> lk(g.mu);
    auto it = g.weights.find(key);
    if (it != g.weights.end()) {
        inkq_weight_destroy(it->second.w);
        g.weights.erase(it);
    }
    inkq_weight *w = nullptr;
    g.check(inkq_weight_create(g.ctx, scheme, scale_mode, N, K, nib, d, m, nullptr, 0, N, &w));
    g.weights[key] = Entry{w, scale_mode};
}

// Call with g.mu held (the caller keeps it until the matmul that uses the handle has returned).
template <typename SB>
inkq_weight *lookup(const void *B_repack, int scheme, int scale_mode, int N, int K)
{
    Gpu &g = gpu();
    auto it = g.weights.find(B_repack);
    if (it != g.weights.end()) {
        int rows = 0, k = 0, sch = 0;
        inkq_weight_info(it->second.w, &rows, &k, &sch, nullptr);
        if (rows == N && k == K && sch == scheme && it->second.scale_mode == scale_mode) return it->second.w;
    }
    std::vector<uint8_t> nib;
    std::vector<float> d, m;
    read_superblocks(K, N, static_cast<const SB *>(B_repack), nib, d, m);
    remember(B_repack, scheme, scale_mode, N, K, nib.data(), d.data(), scheme == INKQ_A81W41 ? m.data() : nullptr);
    return g.weights[B_repack].w;
}

template <typename AS, typename SB>
void matmul(int scheme, int scale_mode, int qmode, const void *A_repack, const void *B_repack, float *C, int M, int N, int K, bool gemv)
{
    Gpu &g = gpu();
    std::lock_guard<std::recursive_mutex> lk(g.mu);
    inkq_weight *w = lookup<SB>(B_repack, scheme, scale_mode, N, K);
    const int nb = K / 32, npair = K / 64;
    std::vector<int8_t> q(static_cast<size_t>(M) * K);
    std::vector<float> d(static_cast<size_t>(M) * nb), s(static_cast<size_t>(M) * nb, 0.0f);
    const AS *A = static_cast<const AS *>(A_repack);
    for (int i = 0; i < M; i++)
        for (int p = 0; p < npair; p++) {
            const AS &t = A[static_cast<size_t>(i) * npair + p];
            std::memcpy(&q[static_cast<size_t>(i) * K + 64 * p], t.q_low, 32);
            std::memcpy(&q[static_cast<size_t>(i) * K + 64 * p + 32], t.q_high, 32);
            const size_t b = static_cast<size_t>(i) * nb + 2 * p;
            if constexpr (sizeof(t.s_low) == 2) {
                d[b] = f16_to_f32(t.s_low);
                d[b + 1] = f16_to_f32(t.s_high);
                if (qmode != INKQ_Q8_0_F16) {
                    s[b] = f16_to_f32(t.scaled_sum_low);
                    s[b + 1] = f16_to_f32(t.scaled_sum_high);
                }
            } else {
                d[b] = t.s_low;
                d[b + 1] = t.s_high;
                s[b] = t.scaled_sum_low;
                s[b + 1] = t.scaled_sum_high;
            }
        }
    inkq_act *a = g.activation(M, K);
    g.check(inkq_act_import(g.ctx, a, qmode, M, q.data(), d.data(), qmode == INKQ_Q8_0_F16 ? nullptr : s.data()));
    g.check(gemv ? inkq_gemv_host(g.ctx, a, w, C) : inkq_gemm_host(g.ctx, a, w, C, N));
    (void)scheme;
}

}  // namespace

// ---- the reference's names ----------------------------------------------------------------------
void quantize_row_q8_0_repack(const float *x, void *vy, int64_t k) { quantize_to_structs(x, vy, k, INKQ_Q8_0_F16); }
void quantize_row_q8_1_repack_fp16(const float *x, void *vy, int64_t k) { quantize_to_structs(x, vy, k, INKQ_Q8_1_F16); }
void quantize_row_q8_1_repack_fp32(const float *x, void *vy, int64_t k) { quantize_to_structs(x, vy, k, INKQ_Q8_1_F32); }

void repack_w80_weight(const int K, const int N, const int /*Q_BLK_SIZE*/, void *B_repack, const float *SB, const uint8_t *B)
{
    write_superblocks(K, N, static_cast<q4_2x8_f16 *>(B_repack), SB, nullptr, B, true);
    remember(B_repack, INKQ_A80W40, INKQ_SCALES_F16, N, K, B, SB, nullptr);
}
void repack_w81_weight_fp16(const int K, const int N, const int /*Q_BLK_SIZE*/, void *B_repack, const float *SB, const float *MinB, const uint8_t *B)
{
    write_superblocks(K, N, static_cast<q4_2x8_f16 *>(B_repack), SB, MinB, B, true);
    remember(B_repack, INKQ_A81W41, INKQ_SCALES_F16, N, K, B, SB, MinB);
}
void repack_w81_weight_fp32(const int K, const int N, const int /*Q_BLK_SIZE*/, void *B_repack, const float *SB, const float *MinB, const uint8_t *B)
{
    write_superblocks(K, N, static_cast<q4_2x8_f32 *>(B_repack), SB, MinB, B, false);
    remember(B_repack, INKQ_A81W41, INKQ_SCALES_F32, N, K, B, SB, MinB);
}

void gemm_repack_A81W41_fp32(void *A_repack, void *B_repack, float *C, const int M, const int N, const int K)
{
    matmul<q8_1x2_f32, q4_2x8_f32>(INKQ_A81W41, INKQ_SCALES_F32, INKQ_Q8_1_F32, A_repack, B_repack, C, M, N, K, false);
}
void gemv_repack_A81W41_fp16(void *A_repack, void *B_repack, float *C, const int M, const int N, const int K)
{
    matmul<q8_1x2_f16, q4_2x8_f16>(INKQ_A81W41, INKQ_SCALES_F16, INKQ_Q8_1_F16, A_repack, B_repack, C, M, N, K, true);
}
void gemm_repack_A80W40(void *A_repack, void *B_repack, float *C, const int M, const int N, const int K)
{
    matmul<q8_1x2_f16, q4_2x8_f16>(INKQ_A80W40, INKQ_SCALES_F16, INKQ_Q8_0_F16, A_repack, B_repack, C, M, N, K, false);
}
void gemv_repack_A80W40(void *A_repack, void *B_repack, float *C, const int M, const int N, const int K)
{
    matmul<q8_1x2_f16, q4_2x8_f16>(INKQ_A80W40, INKQ_SCALES_F16, INKQ_Q8_0_F16, A_repack, B_repack, C, M, N, K, true);
}

// Drops the device copy remembered for a weight buffer (call before freeing or refilling the buffer outside repack_*).
void inkq_refshim_forget(const void *B_repack)
{
    Gpu &g = gpu();
    std::lock_guard<std::recursive_mutex> lk(g.mu);
    auto it = g.weights.find(B_repack);
    if (it != g.weights.end()) {
        inkq_weight_destroy(it->second.w);
        g.weights.erase(it);
    }
}
