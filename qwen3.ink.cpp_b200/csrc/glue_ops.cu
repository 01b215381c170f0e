// Thin device-resident stand-ins for the non-GEMM operators around the quantized linear layers
// of a Qwen3 decoder, so that a whole synthetic forward (prompt prefill + greedy decode) can keep
// its activations on the GPU between the 181 quantized linears of a token.  Correct and simple,
// not tuned: the named hot path is the quantized matmul, these only connect its calls.
//
// Reference behaviour followed (paths inside the reference project):
//   embedding gather           qwen3/src/ops/embedding.cc:11-26
//   RMSNorm (eps 1e-6)         qwen3/src/qwen/QwenOperator.cc:24-53
//   per-head q/k RMSNorm, RoPE qwen3/src/qwen/QwenAttention.cc:85-92, qwen3/src/ops/RotaryPosEmb.cc:6-79
//                              (rotate_half form: x*cos + rotate_half(x)*sin, tables [pos][head_dim])
//   KV cache append            qwen3/src/qwen/QwenAttention.cc:105-121   (fp16 here, fp32 there)
//   causal GQA attention       qwen3/src/qwen/QwenAttention.cc:154-190, qwen3/src/ops/softmax.cc:53-85
//   SiLU(gate) * up            qwen3/src/qwen/QwenOperator.cc:697-722
//   residual add               qwen3/src/qwen/QwenDecoderLayer.cc:73,105
//   greedy argmax              qwen3/src/qwen/Pipeline.cc:54-62
// Activations are fp32 row-major [tokens][features].  The position of the first token of a call
// is read from device memory so that one captured CUDA graph serves every decode step.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <math.h>

#include <mutex>

#include "glue_math.cuh"
#include "inkq_glue.h"
#include "inkq_internal.h"
#include "qgemv_common.cuh"

namespace inkq {

constexpr int HEAD_DIM = 128;

__global__ void __launch_bounds__(256) k_embedding(const __half *__restrict__ table, const int *__restrict__ tokens, int T, int dim, int vocab,
                                                   float *__restrict__ out)
{
    const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx >= static_cast<long long>(T) * dim / 2) return;
    const int t = static_cast<int>(idx / (dim / 2)), c = static_cast<int>(idx % (dim / 2));
    const int tok = min(max(tokens[t], 0), vocab - 1);   // a token id outside the table (e.g. from NaN logits) must not become an address
    const float2 v = __half22float2(reinterpret_cast<const __half2 *>(table + static_cast<size_t>(tok) * dim)[c]);
    reinterpret_cast<float2 *>(out + static_cast<size_t>(t) * dim)[c] = v;
}

// one CTA per row
__global__ void __launch_bounds__(256) k_rmsnorm(const float *__restrict__ x, const float *__restrict__ w, int rows, int dim, float eps,
                                                 float *__restrict__ y)
{
    __shared__ float red[8];
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float4 *xr = reinterpret_cast<const float4 *>(x + static_cast<size_t>(row) * dim);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < dim / 4; i += 256) {
        ss = add_sumsq4(ss, xr[i]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float inv = rms_inv(tot, dim, eps);
    float4 *yr = reinterpret_cast<float4 *>(y + static_cast<size_t>(row) * dim);
    const float4 *wr = reinterpret_cast<const float4 *>(w);
    for (int i = threadIdx.x; i < dim / 4; i += 256) yr[i] = rms_scale4(xr[i], inv, wr[i]);
}

// Prompt path, one CTA per row: x += delta (the residual connection, optional), RMSNorm of the row, and the
// activation quantizer of the layer that consumes it, in one pass: the row is read once, kept in shared memory
// between the sum of squares and the scaling, and leaves as int8 + block scales.  Element arithmetic, summation
// order and quantizer are those of k_add_inplace, k_rmsnorm and k_quantize_q8, so the quantized row is the one the
// three kernels would produce.  Eight consecutive threads share a 32-element quantization block.
__global__ void __launch_bounds__(256) k_add_rmsnorm_quant_rows(float *__restrict__ x, const float *__restrict__ delta, const float *__restrict__ w,
                                                                int M, int dim, float eps, int M_ld, int mode, int8_t *__restrict__ q,
                                                                float *__restrict__ d, float *__restrict__ s, int32_t *__restrict__ isum,
                                                                float *__restrict__ xn_out)
{
    extern __shared__ __align__(16) float4 rowbuf[];
    __shared__ float red[8];
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n4 = dim / 4, nb = dim / QK;
    if (row >= M) {   // padding rows of the scale planes read as zero
        for (int b = threadIdx.x; b < nb; b += 256) {
            const size_t pl = static_cast<size_t>(b) * M_ld + row;
            d[pl] = 0.0f;
            s[pl] = 0.0f;
            isum[pl] = 0;
        }
        return;
    }
    float4 *xr = reinterpret_cast<float4 *>(x + static_cast<size_t>(row) * dim);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < n4; i += 256) {
        float4 v = xr[i];
        if (delta != nullptr) {
            const float4 y = reinterpret_cast<const float4 *>(delta + static_cast<size_t>(row) * dim)[i];
            v = make_float4(v.x + y.x, v.y + y.y, v.z + y.z, v.w + y.w);
            xr[i] = v;
        }
        rowbuf[i] = v;
        ss = add_sumsq4(ss, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) tot += red[i];
    const float inv = rms_inv(tot, dim, eps);
    const float4 *wr = reinterpret_cast<const float4 *>(w);
    for (int base = 0; base < n4; base += 256) {   // trip count is the same for every thread: the shuffles below see whole warps
        const int i = base + threadIdx.x;
        const bool live = i < n4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            v = rms_scale4(rowbuf[i], inv, wr[i]);
            if (xn_out != nullptr) reinterpret_cast<float4 *>(xn_out + static_cast<size_t>(row) * dim)[i] = v;
        }
        float mx = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float dd = __fdiv_rn(mx, 127.0f);
        const float id = (mx != 0.0f) ? __fdiv_rn(127.0f, mx) : 0.0f;
        const int i0 = __float2int_rn(__fmul_rn(v.x, id)), i1 = __float2int_rn(__fmul_rn(v.y, id));
        const int i2 = __float2int_rn(__fmul_rn(v.z, id)), i3 = __float2int_rn(__fmul_rn(v.w, id));
        int sum = (i0 + i1) + (i2 + i3);
#pragma unroll
        for (int o = 1; o < 8; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (live) {
            reinterpret_cast<uint32_t *>(q)[static_cast<size_t>(row) * n4 + i] = pack_sat_s8x4_m1(i0, i1, i2, i3);
            if ((i & 7) == 0) {
                const size_t pl = static_cast<size_t>(i >> 3) * M_ld + row;
                const float sv = __fmul_rn(dd, static_cast<float>(sum));
                if (mode == INKQ_Q8_1_F32) {
                    d[pl] = dd;
                    s[pl] = sv;
                } else {
                    d[pl] = __half2float(__float2half_rn(dd));
                    s[pl] = (mode == INKQ_Q8_1_F16) ? __half2float(__float2half_rn(sv)) : 0.0f;
                }
                isum[pl] = sum;
            }
        }
    }
}

// One warp per (token, head) of the fused qkv output [T][(nq + 2*nkv) * 128]:
//   q heads : per-head RMSNorm, RoPE, written to q_out [T][nq][128] fp32
//   k heads : per-head RMSNorm, RoPE, written to k_cache [nkv][max_pos][128] fp16 at position pos0 + t
//   v heads : copied to v_cache likewise
// Lane l holds elements l, l+32, l+64, l+96: the rotate_half partners (j, j+64) sit in one lane.
__global__ void __launch_bounds__(256) k_qknorm_rope_cache(const float *__restrict__ qkv, const float *__restrict__ q_norm_w,
                                                           const float *__restrict__ k_norm_w, const float *__restrict__ cos_t,
                                                           const float *__restrict__ sin_t, const int *__restrict__ pos0_dev, int T, int nq,
                                                           int nkv, int max_pos, float eps, float *__restrict__ q_out,
                                                           __half *__restrict__ k_cache, __half *__restrict__ v_cache)
{
    // launched with programmatic stream serialization in the decode step: wait for the producer of the inputs,
    // then let the next kernel (a QGEMV) start its weight prefetch while this grid runs
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int heads = nq + 2 * nkv;
    const int item = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const int t = item / heads, h = item % heads;
    const int pos = *pos0_dev + t;
    if (pos >= max_pos) return;
    const float *src = qkv + static_cast<size_t>(t) * heads * HEAD_DIM + static_cast<size_t>(h) * HEAD_DIM;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = src[lane + 32 * i];
    if (h >= nq + nkv) {  // value head: straight to the cache
        __half *dst = v_cache + (static_cast<size_t>(h - nq - nkv) * max_pos + pos) * HEAD_DIM;
#pragma unroll
        for (int i = 0; i < 4; i++) dst[lane + 32 * i] = __float2half_rn(v[i]);
        return;
    }
    float r[4];
    head_norm_rope(v, lane, (h < nq) ? q_norm_w : k_norm_w, cos_t + static_cast<size_t>(pos) * HEAD_DIM, sin_t + static_cast<size_t>(pos) * HEAD_DIM,
                   eps, r);
    if (h < nq) {
        float *dst = q_out + (static_cast<size_t>(t) * nq + h) * HEAD_DIM;
#pragma unroll
        for (int i = 0; i < 4; i++) dst[lane + 32 * i] = r[i];
    } else {
        __half *dst = k_cache + (static_cast<size_t>(h - nq) * max_pos + pos) * HEAD_DIM;
#pragma unroll
        for (int i = 0; i < 4; i++) dst[lane + 32 * i] = __float2half_rn(r[i]);
    }
}

// One CTA (128 threads) per (query token t, query head h).  Keys 0 .. pos0 + t (causal), the kv
// head is h / (nq / nkv).  Pass 1: one thread per key computes the scaled dot product into shared
// memory; block max and sum; pass 2: warp w accumulates the values of keys j = w mod 4, lanes over
// the 128 dimensions; the four partials are added in warp order.
template <int NT>
__global__ void __launch_bounds__(NT) k_attention(const float *__restrict__ q, const __half *__restrict__ k_cache,
                                                   const __half *__restrict__ v_cache, const int *__restrict__ pos0_dev, int T, int nq, int nkv,
                                                   int max_pos, float scale, float *__restrict__ out, const QuantOut qo)
{
    // launched with programmatic stream serialization in the decode step: wait for the producer of the inputs,
    // then let the next kernel (a QGEMV) start its weight prefetch while this grid runs
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ float sm[];
    float *qs = sm;                  // 128
    constexpr int NW = NT / 32;
    float *part = sm + HEAD_DIM;        // NW * 128
    float *red = part + NW * HEAD_DIM;  // 2 * NW
    float *sc = red + 2 * NW;           // scores, nkeys
    const int t = blockIdx.x / nq, h = blockIdx.x % nq;
    const int kvh = h / (nq / nkv);
    const int nkeys = min(*pos0_dev + t + 1, max_pos);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < HEAD_DIM) qs[tid] = q[(static_cast<size_t>(t) * nq + h) * HEAD_DIM + tid];
    __syncthreads();
    const __half *kb = k_cache + static_cast<size_t>(kvh) * max_pos * HEAD_DIM;
    const __half *vb = v_cache + static_cast<size_t>(kvh) * max_pos * HEAD_DIM;
    float lmax = -INFINITY;
    for (int j = tid; j < nkeys; j += NT) {
        const uint4 *kr = reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(j) * HEAD_DIM);
        float acc = 0.0f;
        // the key's 256 bytes as two groups of eight independent 16-byte loads: the row is latency-bound (a decode step has
        // one CTA per head), so the loads in flight per thread set its speed; summation order: c ascending
#pragma unroll
        for (int c8 = 0; c8 < HEAD_DIM / 8; c8 += 8) {
            uint4 pk[8];
#pragma unroll
            for (int u = 0; u < 8; u++) pk[u] = kr[c8 + u];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int c = c8 + u;
                const uint32_t wd[4] = {pk[u].x, pk[u].y, pk[u].z, pk[u].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&wd[i]));
                    acc = fmaf(qs[c * 8 + 2 * i], f.x, acc);
                    acc = fmaf(qs[c * 8 + 2 * i + 1], f.y, acc);
                }
            }
        }
        acc *= scale;
        sc[j] = acc;
        lmax = fmaxf(lmax, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float gmax = red[0];
#pragma unroll
    for (int i = 1; i < NW; i++) gmax = fmaxf(gmax, red[i]);
    float lsum = 0.0f;
    for (int j = tid; j < nkeys; j += NT) {
        const float e = __expf(sc[j] - gmax);
        sc[j] = e;
        lsum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    if (lane == 0) red[NW + warp] = lsum;
    __syncthreads();
    float den = 0.0f;
#pragma unroll
    for (int i = 0; i < NW; i++) den += red[NW + i];
    const float inv = 1.0f / den;
    float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
    for (int j = warp; j < nkeys; j += NW) {
        const float p = sc[j];
        const uint2 pk = reinterpret_cast<const uint2 *>(vb + static_cast<size_t>(j) * HEAD_DIM)[lane];
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.y));
        a[0] = fmaf(p, f0.x, a[0]);
        a[1] = fmaf(p, f0.y, a[1]);
        a[2] = fmaf(p, f1.x, a[2]);
        a[3] = fmaf(p, f1.y, a[3]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++) part[warp * HEAD_DIM + lane * 4 + i] = a[i];
    __syncthreads();
    if (tid < HEAD_DIM) {
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < NW; i++) o += part[i * HEAD_DIM + tid];
        o *= inv;
        if (out != nullptr) out[(static_cast<size_t>(t) * nq + h) * HEAD_DIM + tid] = o;
        // decode step: the head's 128 outputs are four quantization blocks of the o_proj input row, one per warp
        if (qo.q != nullptr) quantize_block_lanes(o, (t * nq + h) * (HEAD_DIM / QK) + warp, lane, qo);
    }
}

// Decode-step attention split over the keys: ATT_S CTAs per query head, each takes a contiguous share of the
// keys 0 .. pos0 (so a head's 2 x 256 bytes per key come in through ATT_S times as many loads in flight; a decode
// step has one query token and would otherwise run on nq of the SMs).  A CTA produces an unnormalized partial
// (running max, sum of exponentials, 128 weighted value sums); the ATT_S CTAs of a head form a thread-block cluster,
// write their partials into the first one's shared memory and meet at the cluster barrier; the first one merges them
// in ascending share order and writes and/or quantizes the head's output.  Scores: four threads per key (32 dimensions each, xor-shuffle);
// values: warp w takes keys w, w + 16, ... of the share, lane = 4 output dimensions.
#ifndef INKQ_ATT_S
#define INKQ_ATT_S 4   // tuning knob: shares per head
#endif
constexpr int ATT_S = INKQ_ATT_S, ATT_SPLIT_NT = 512, ATT_SPLIT_NW = ATT_SPLIT_NT / 32;
static_assert(ATT_S >= 1 && ATT_S <= 8, "a portable cluster holds at most 8 CTAs");
constexpr int ATT_PART_WORDS = HEAD_DIM + 4;   // a share's partial: 128 sums, running max, sum of exponentials
// When qkv is not NULL the kernel starts from the fused qkv projection's output row [(nq + 2 nkv) * 128] instead of a
// ready query: warp 0 of every CTA normalizes and rotates the query head itself, and the share that holds the newest key
// (position pos0) does the same for the key head and takes the value head, uses both from shared memory (rounded to
// fp16, as the cache holds them) and - for the first query head of a kv group - appends them to the caches.  Same
// arithmetic as k_qknorm_rope_cache (head_norm_rope), one kernel and one pass through L2 less per layer.
struct FusedQkv {
    const float *qkv, *q_norm_w, *k_norm_w, *cos_t, *sin_t;
    float eps;
    __half *k_cache_w, *v_cache_w;
};
__global__ void __cluster_dims__(ATT_S, 1, 1) __launch_bounds__(ATT_SPLIT_NT)
    k_attention_split(const float *__restrict__ q, const __half *__restrict__ k_cache, const __half *__restrict__ v_cache,
                      const int *__restrict__ pos0_dev, int nq, int nkv, int max_pos, float scale, float *__restrict__ out, const QuantOut qo,
                      const FusedQkv fz)
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    extern __shared__ float sm[];
    float *qs = sm;                               // 128
    float *part = sm + HEAD_DIM;                  // NW * 128
    float *red = part + ATT_SPLIT_NW * HEAD_DIM;  // 2 * NW
    float *sc = red + 2 * ATT_SPLIT_NW;           // scores of the share
    const int h = blockIdx.x / ATT_S, sp = blockIdx.x % ATT_S;
    const int kvh = h / (nq / nkv);
    const int pos_raw = *pos0_dev;
    const int nkeys = min(pos_raw + 1, max_pos);
    const int share = (nkeys + ATT_S - 1) / ATT_S;
    const int k0 = min(sp * share, nkeys), n = min(nkeys - k0, share);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const __half *kb = k_cache + (static_cast<size_t>(kvh) * max_pos + k0) * HEAD_DIM;
    const __half *vb = v_cache + (static_cast<size_t>(kvh) * max_pos + k0) * HEAD_DIM;
    const int sub = tid & 3;
    // Everything the share needs from memory is requested up front - the query, the first 128 keys (four threads per
    // key, 64 bytes each) and this warp's first eight value rows - so that one L2 latency covers all of it; a share of
    // more than 128 keys (contexts beyond 512 positions) takes the remaining ones in further, unprefetched passes.
    constexpr int KPASS = ATT_SPLIT_NT / 4, VPRE = 8;
    __shared__ __align__(16) __half knew[HEAD_DIM], vnew[HEAD_DIM];
    const bool fused = fz.qkv != nullptr;
    // the newest key is the last one of the last share that holds any; in the fused form it comes from shared memory
    const int j_new = (fused && pos_raw < max_pos && n > 0 && k0 + n == nkeys) ? n - 1 : -1;   // (a position past the caches is not stored)
    uint4 pk0[4];
    {
        const int j = tid >> 2;
        const uint4 *kr = reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(min(j, max(n - 1, 0))) * HEAD_DIM) + sub * 4;
#pragma unroll
        for (int u = 0; u < 4; u++) pk0[u] = (j < n && j != j_new) ? kr[u] : make_uint4(0, 0, 0, 0);
    }
    uint2 pv0[VPRE];
#pragma unroll
    for (int u = 0; u < VPRE; u++) {
        const int j = warp + u * ATT_SPLIT_NW;
        pv0[u] = (j < n && j != j_new) ? reinterpret_cast<const uint2 *>(vb + static_cast<size_t>(j) * HEAD_DIM)[lane] : make_uint2(0, 0);
    }
    if (!fused) {
        if (tid < HEAD_DIM) qs[tid] = q[static_cast<size_t>(h) * HEAD_DIM + tid];
    } else if (warp < 3) {
        const int pos = nkeys - 1;
        const int G = nq / nkv;
        const float *cs = fz.cos_t + static_cast<size_t>(pos) * HEAD_DIM, *sn = fz.sin_t + static_cast<size_t>(pos) * HEAD_DIM;
        if (warp == 0) {
            float v[4], r[4];
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = fz.qkv[static_cast<size_t>(h) * HEAD_DIM + lane + 32 * i];
            head_norm_rope(v, lane, fz.q_norm_w, cs, sn, fz.eps, r);
#pragma unroll
            for (int i = 0; i < 4; i++) qs[lane + 32 * i] = r[i];
        } else if (j_new >= 0) {
            const bool writer = (h % G) == 0;   // one query head per kv group appends to the caches
            float v[4], r[4];
            const int src_head = (warp == 1) ? nq + kvh : nq + nkv + kvh;
#pragma unroll
            for (int i = 0; i < 4; i++) v[i] = fz.qkv[static_cast<size_t>(src_head) * HEAD_DIM + lane + 32 * i];
            if (warp == 1) head_norm_rope(v, lane, fz.k_norm_w, cs, sn, fz.eps, r);
            __half *sm_dst = (warp == 1) ? knew : vnew;
            __half *gl_dst = ((warp == 1) ? fz.k_cache_w : fz.v_cache_w) + (static_cast<size_t>(kvh) * max_pos + pos) * HEAD_DIM;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const __half hv = __float2half_rn((warp == 1) ? r[i] : v[i]);
                sm_dst[lane + 32 * i] = hv;
                if (writer) gl_dst[lane + 32 * i] = hv;
            }
        }
    }
    __syncthreads();
    float lmax = -INFINITY;
    for (int jb = 0; jb < n; jb += KPASS) {
        const int j = jb + (tid >> 2);
        float acc = 0.0f;
        if (j < n) {
            uint4 pk[4];
            if (j == j_new) {
#pragma unroll
                for (int u = 0; u < 4; u++) pk[u] = reinterpret_cast<const uint4 *>(knew)[sub * 4 + u];
            } else if (jb == 0) {
#pragma unroll
                for (int u = 0; u < 4; u++) pk[u] = pk0[u];
            } else {
                const uint4 *kr = reinterpret_cast<const uint4 *>(kb + static_cast<size_t>(j) * HEAD_DIM) + sub * 4;
#pragma unroll
                for (int u = 0; u < 4; u++) pk[u] = kr[u];
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const uint32_t wd[4] = {pk[u].x, pk[u].y, pk[u].z, pk[u].w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&wd[i]));
                    acc = fmaf(qs[sub * 32 + u * 8 + 2 * i], f.x, acc);
                    acc = fmaf(qs[sub * 32 + u * 8 + 2 * i + 1], f.y, acc);
                }
            }
        }
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        if (j < n) {
            acc *= scale;
            if (sub == 0) sc[j] = acc;
            lmax = fmaxf(lmax, acc);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, o));
    if (lane == 0) red[warp] = lmax;
    __syncthreads();
    float gmax = red[0];
#pragma unroll
    for (int i = 1; i < ATT_SPLIT_NW; i++) gmax = fmaxf(gmax, red[i]);
    float lsum = 0.0f;
    for (int j = tid; j < n; j += ATT_SPLIT_NT) {
        const float e = __expf(sc[j] - gmax);
        sc[j] = e;
        lsum += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
    if (lane == 0) red[ATT_SPLIT_NW + warp] = lsum;
    __syncthreads();
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    auto add_value = [&](float pj, const uint2 pk) {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.y));
        a[0] = fmaf(pj, f0.x, a[0]);
        a[1] = fmaf(pj, f0.y, a[1]);
        a[2] = fmaf(pj, f1.x, a[2]);
        a[3] = fmaf(pj, f1.y, a[3]);
    };
#pragma unroll
    for (int u = 0; u < VPRE; u++) {
        const int j = warp + u * ATT_SPLIT_NW;
        if (j < n) add_value(sc[j], (j == j_new) ? reinterpret_cast<const uint2 *>(vnew)[lane] : pv0[u]);
    }
#pragma unroll 4
    for (int j = warp + VPRE * ATT_SPLIT_NW; j < n; j += ATT_SPLIT_NW)
        add_value(sc[j], (j == j_new) ? reinterpret_cast<const uint2 *>(vnew)[lane]
                                      : reinterpret_cast<const uint2 *>(vb + static_cast<size_t>(j) * HEAD_DIM)[lane]);
#pragma unroll
    for (int i = 0; i < 4; i++) part[warp * HEAD_DIM + lane * 4 + i] = a[i];
    __syncthreads();
    // the head's ATT_S shares are one thread-block cluster: every share writes its partial into share 0's shared memory
    // (distributed shared memory), the cluster meets at its hardware barrier, share 0 merges
    __shared__ float merge[ATT_S][ATT_PART_WORDS];
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    float *mine = cluster.map_shared_rank(&merge[0][0], 0) + sp * ATT_PART_WORDS;
    if (tid < HEAD_DIM) {
        float o = 0.0f;
#pragma unroll
        for (int i = 0; i < ATT_SPLIT_NW; i++) o += part[i * HEAD_DIM + tid];
        mine[tid] = o;
        if (tid == 0) {
            float den = 0.0f;
#pragma unroll
            for (int i = 0; i < ATT_SPLIT_NW; i++) den += red[ATT_SPLIT_NW + i];
            mine[HEAD_DIM] = (n > 0) ? gmax : -INFINITY;
            mine[HEAD_DIM + 1] = den;
        }
    }
    cluster.sync();
    if (sp != 0) return;
    if (tid < HEAD_DIM) {
        float m[ATT_S], l[ATT_S], o[ATT_S];
#pragma unroll
        for (int s2 = 0; s2 < ATT_S; s2++) {
            m[s2] = merge[s2][HEAD_DIM];
            l[s2] = merge[s2][HEAD_DIM + 1];
            o[s2] = merge[s2][tid];
        }
        float mm = m[0];   // share 0 always holds key 0
#pragma unroll
        for (int s2 = 1; s2 < ATT_S; s2++) mm = fmaxf(mm, m[s2]);
        float den = 0.0f, num = 0.0f;
#pragma unroll
        for (int s2 = 0; s2 < ATT_S; s2++) {
            const float w = __expf(m[s2] - mm);   // 0 for an empty share
            den = fmaf(l[s2], w, den);
            num = fmaf(o[s2], w, num);
        }
        const float res = num / den;
        if (out != nullptr) out[static_cast<size_t>(h) * HEAD_DIM + tid] = res;
        if (qo.q != nullptr) quantize_block_lanes(res, h * (HEAD_DIM / QK) + warp, lane, qo);
    }
}


__global__ void __launch_bounds__(256) k_silu_mul(const float4 *__restrict__ gate, const float4 *__restrict__ up, long long n4,
                                                  float4 *__restrict__ out)
{
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 g = gate[i], u = up[i];
    out[i] = make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w));
}

// gu [T][2F] in (32 gate, 32 up) column groups -> out [T][F]: out[k] = SiLU(gu[64*(k/32) + k%32]) * gu[64*(k/32) + 32 + k%32]
__global__ void __launch_bounds__(256) k_silu_mul_rows(const float4 *__restrict__ gu, int T, int F4, float4 *__restrict__ out)
{
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= static_cast<long long>(T) * F4) return;
    const long long t = i / F4, c = i % F4;            // c: float4 index inside the row; 8 float4 per 32-element block
    const long long src = t * 2 * F4 + (c / 8) * 16 + (c % 8);
    const float4 g = gu[src], u = gu[src + 8];
    out[i] = make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w));
}

__global__ void __launch_bounds__(256) k_add_inplace(float4 *__restrict__ a, const float4 *__restrict__ b, long long n4)
{
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 x = a[i], y = b[i];
    a[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
}

// Greedy sampling over the logits by a cluster of 8 CTAs: every CTA scans an eighth of the vector with 128-bit
// loads, the eight (value, index) candidates meet in CTA 0's shared memory (distributed shared memory), and CTA 0
// publishes the token, appends it to the generated list and advances the position.  Ties go to the lowest index.
constexpr int ARGMAX_CTAS = 8;
__device__ __forceinline__ void argmax_take(float v, int i, float &best, int &idx)
{
    if (v > best || (v == best && i < idx)) {
        best = v;
        idx = i;
    }
}
__global__ void __cluster_dims__(ARGMAX_CTAS, 1, 1) __launch_bounds__(1024)
    k_argmax_advance(const float *__restrict__ logits, int n, int *__restrict__ token_out, int *__restrict__ pos_dev, int advance,
                     int *__restrict__ generated, int gen_cap)
{
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ float bv[32];
    __shared__ int bi[32];
    __shared__ float cv[ARGMAX_CTAS];
    __shared__ int ci[ARGMAX_CTAS];
    const int rank = static_cast<int>(cluster.block_rank());
    const int gtid = rank * 1024 + threadIdx.x, gthreads = ARGMAX_CTAS * 1024;
    float best = -INFINITY;
    int idx = n - 1;   // stays a valid index even when every logit is NaN
    const int n4 = n / 4;
    for (int i = gtid; i < n4; i += gthreads) {
        const float4 v = reinterpret_cast<const float4 *>(logits)[i];
        argmax_take(v.x, 4 * i, best, idx);
        argmax_take(v.y, 4 * i + 1, best, idx);
        argmax_take(v.z, 4 * i + 2, best, idx);
        argmax_take(v.w, 4 * i + 3, best, idx);
    }
    for (int i = 4 * n4 + gtid; i < n; i += gthreads) argmax_take(logits[i], i, best, idx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        argmax_take(ov, oi, best, idx);
    }
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 32; w++) argmax_take(bv[w], bi[w], best, idx);
        cluster.map_shared_rank(cv, 0)[rank] = best;   // into CTA 0's shared memory
        cluster.map_shared_rank(ci, 0)[rank] = idx;
    }
    cluster.sync();
    if (rank == 0 && threadIdx.x == 0) {
        best = cv[0];
        idx = ci[0];
        for (int c = 1; c < ARGMAX_CTAS; c++) argmax_take(cv[c], ci[c], best, idx);
        *token_out = idx;
        if (generated != nullptr) {
            const int slot = generated[0];   // generated[0] counts the tokens stored so far, the tokens follow
            if (slot + 1 < gen_cap) {
                generated[slot + 1] = idx;
                generated[0] = slot + 1;
            }
        }
        *pos_dev += advance;
    }
}

}  // namespace inkq

using namespace inkq;

static int glue_use(inkq_ctx *ctx)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    return INKQ_OK;
}

extern "C" {

int inkq_glue_embedding(inkq_ctx *ctx, const uint16_t *table16_dev, const int *tokens_dev, int T, int dim, int vocab, float *out_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, table16_dev && tokens_dev && out_dev && T >= 1 && dim % 2 == 0 && vocab >= 1, "bad embedding arguments");
    const long long n = static_cast<long long>(T) * dim / 2;
    k_embedding<<<static_cast<unsigned>((n + 255) / 256), 256, 0, ctx->stream>>>(reinterpret_cast<const __half *>(table16_dev), tokens_dev, T, dim, vocab, out_dev);
    return after_launch(ctx, "k_embedding");
}

int inkq_glue_rmsnorm(inkq_ctx *ctx, const float *x_dev, const float *w_dev, int rows, int dim, float eps, float *y_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, x_dev && w_dev && y_dev && rows >= 1 && dim % 4 == 0, "bad rmsnorm arguments");
    k_rmsnorm<<<rows, 256, 0, ctx->stream>>>(x_dev, w_dev, rows, dim, eps, y_dev);
    return after_launch(ctx, "k_rmsnorm");
}

int inkq_glue_qknorm_rope_cache(inkq_ctx *ctx, const float *qkv_dev, const float *q_norm_w, const float *k_norm_w, const float *cos_dev,
                                const float *sin_dev, const int *pos0_dev, int T, int nq, int nkv, int max_pos, float eps, float *q_out_dev,
                                uint16_t *k_cache_dev, uint16_t *v_cache_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, qkv_dev && q_norm_w && k_norm_w && cos_dev && sin_dev && pos0_dev && q_out_dev && k_cache_dev && v_cache_dev, "null argument");
    INKQ_REQUIRE(ctx, T >= 1 && nq >= 1 && nkv >= 1 && nq % nkv == 0 && max_pos >= 1, "bad head configuration");
    const int items = T * (nq + 2 * nkv);
    launch_pdl(k_qknorm_rope_cache, dim3((items + 7) / 8), dim3(256), 0, ctx->stream, qkv_dev, q_norm_w, k_norm_w, cos_dev, sin_dev, pos0_dev, T, nq,
               nkv, max_pos, eps, q_out_dev, reinterpret_cast<__half *>(k_cache_dev), reinterpret_cast<__half *>(v_cache_dev));
    return after_launch(ctx, "k_qknorm_rope_cache");
}

static int attention_impl(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev, int T,
                          int nq, int nkv, int max_pos, float scale, float *out_dev, const QuantOut &qo, int qrow0 = 0, const FusedQkv &fz = FusedQkv{});

int inkq_glue_attention(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev, int T,
                        int nq, int nkv, int max_pos, float scale, float *out_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out_dev != nullptr, "null argument");
    return attention_impl(ctx, q_dev, k_cache_dev, v_cache_dev, pos0_dev, T, nq, nkv, max_pos, scale, out_dev, QuantOut{});
}

int inkq_glue_attention_quant(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev,
                              int nq, int nkv, int max_pos, float scale, inkq_act *out, int out_qmode)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr && out->K == nq * HEAD_DIM, "the output activation handle must have been created for K = nq * 128");
    INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
    return attention_impl(ctx, q_dev, k_cache_dev, v_cache_dev, pos0_dev, 1, nq, nkv, max_pos, scale, nullptr, quant_out_of(out, nq * HEAD_DIM, out_qmode));
}

int inkq_glue_qkv_attention_quant(inkq_ctx *ctx, const float *qkv_dev, const float *q_norm_w, const float *k_norm_w, const float *cos_dev,
                                  const float *sin_dev, const int *pos0_dev, int nq, int nkv, int max_pos, float eps, float scale,
                                  uint16_t *k_cache_dev, uint16_t *v_cache_dev, inkq_act *out, int out_qmode)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, qkv_dev && q_norm_w && k_norm_w && cos_dev && sin_dev, "null argument");
    INKQ_REQUIRE(ctx, out != nullptr && out->K == nq * HEAD_DIM, "the output activation handle must have been created for K = nq * 128");
    INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
    FusedQkv fz;
    fz.qkv = qkv_dev;
    fz.q_norm_w = q_norm_w;
    fz.k_norm_w = k_norm_w;
    fz.cos_t = cos_dev;
    fz.sin_t = sin_dev;
    fz.eps = eps;
    fz.k_cache_w = reinterpret_cast<__half *>(k_cache_dev);
    fz.v_cache_w = reinterpret_cast<__half *>(v_cache_dev);
    return attention_impl(ctx, nullptr, k_cache_dev, v_cache_dev, pos0_dev, 1, nq, nkv, max_pos, scale, nullptr, quant_out_of(out, nq * HEAD_DIM, out_qmode), 0,
                          fz);
}

int inkq_glue_attention_quant_rows(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev,
                                   int T, int nq, int nkv, int max_pos, float scale, inkq_act *out, int out_qmode, int row0, int total_rows)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr && out->K == nq * HEAD_DIM, "the output activation handle must have been created for K = nq * 128");
    INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
    INKQ_REQUIRE(ctx, T >= 1 && row0 >= 0 && row0 + T <= total_rows && total_rows <= out->max_rows, "rows outside the activation handle");
    QuantOut qo;
    qo.q = out->q;
    qo.d = out->d;
    qo.s = out->s;
    qo.isum = out->isum;
    qo.M_ld = (total_rows + 3) & ~3;
    qo.qmode = out_qmode;
    out->M = total_rows;
    out->M_ld = qo.M_ld;
    out->qmode = out_qmode;
    out->ssq_parts = 0;
    // a one-row handle keeps the layout of the decode-step kernel; everything else goes through the prompt kernel
    if (total_rows == 1) return attention_impl(ctx, q_dev, k_cache_dev, v_cache_dev, pos0_dev, 1, nq, nkv, max_pos, scale, nullptr, qo);
    return attention_impl(ctx, q_dev, k_cache_dev, v_cache_dev, pos0_dev, T, nq, nkv, max_pos, scale, nullptr, qo, row0);
}

static int attention_impl(inkq_ctx *ctx, const float *q_dev, const uint16_t *k_cache_dev, const uint16_t *v_cache_dev, const int *pos0_dev, int T,
                          int nq, int nkv, int max_pos, float scale, float *out_dev, const QuantOut &qo, int qrow0, const FusedQkv &fz)
{
    int rc = INKQ_OK;
    INKQ_REQUIRE(ctx, (q_dev || fz.qkv) && k_cache_dev && v_cache_dev && pos0_dev, "null argument");
    INKQ_REQUIRE(ctx, T >= 1 && nq % nkv == 0 && max_pos >= 1, "bad head configuration");
    INKQ_REQUIRE(ctx, fz.qkv == nullptr || (T == 1 && nq * ATT_S <= 2 * ctx->num_sms),
                 "the form that starts from the qkv row serves one token and at most SMs / 2 query heads");
    const bool quant_rows = qo.q != nullptr && (T > 1 || qrow0 > 0 || qo.M_ld > 4);
    if (T >= 16 || quant_rows)   // a prompt: tensor-core kernel (attention_prefill_mma.cu), 64 tokens of one query head per CTA
        return launch_attention_prefill_mma(ctx, q_dev, k_cache_dev, v_cache_dev, pos0_dev, T, nq, nkv, max_pos, scale, out_dev, qo, qrow0);
    if (T == 1 && nq * ATT_S <= 2 * ctx->num_sms && !quant_rows) {
        // a decode step: the keys of each head split over a cluster of ATT_S CTAs
        const int share_max = (max_pos + ATT_S - 1) / ATT_S;
        const size_t smem_s = sizeof(float) * (HEAD_DIM + ATT_SPLIT_NW * HEAD_DIM + 2 * ATT_SPLIT_NW + static_cast<size_t>(share_max));
        INKQ_REQUIRE(ctx, smem_s <= 200 * 1024, "context too long for the decode attention kernel");
        if (smem_s > 48 * 1024) cudaFuncSetAttribute(k_attention_split, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_s));
        launch_pdl(k_attention_split, dim3(nq * ATT_S), dim3(ATT_SPLIT_NT), smem_s, ctx->stream, q_dev, reinterpret_cast<const __half *>(k_cache_dev),
                   reinterpret_cast<const __half *>(v_cache_dev), pos0_dev, nq, nkv, max_pos, scale, out_dev, qo, fz);
        return after_launch(ctx, "k_attention_split");
    }
    // few (token, head) items (a decode step): 16 warps per item so that the item's keys are spread over more
    // loads in flight; many items (a prompt): 4 warps per item, the grid fills the machine
    const bool wide = T * nq <= 4 * ctx->num_sms;
    const int nw = wide ? 16 : 4;
    const size_t smem = sizeof(float) * (HEAD_DIM + nw * HEAD_DIM + 2 * nw + static_cast<size_t>(max_pos));
    INKQ_REQUIRE(ctx, smem <= 200 * 1024, "context too long for the simple attention kernel");
    const __half *kc = reinterpret_cast<const __half *>(k_cache_dev), *vc = reinterpret_cast<const __half *>(v_cache_dev);
    if (wide) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(k_attention<512>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        launch_pdl(k_attention<512>, dim3(T * nq), dim3(512), smem, ctx->stream, q_dev, kc, vc, pos0_dev, T, nq, nkv, max_pos, scale, out_dev, qo);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(k_attention<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        k_attention<128><<<T * nq, 128, smem, ctx->stream>>>(q_dev, kc, vc, pos0_dev, T, nq, nkv, max_pos, scale, out_dev, qo);
    }
    return after_launch(ctx, "k_attention");
}

int inkq_glue_silu_mul(inkq_ctx *ctx, const float *gate_dev, const float *up_dev, long long n, float *out_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, gate_dev && up_dev && out_dev && n % 4 == 0, "bad silu_mul arguments");
    k_silu_mul<<<static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(gate_dev),
                                                                                  reinterpret_cast<const float4 *>(up_dev), n / 4,
                                                                                  reinterpret_cast<float4 *>(out_dev));
    return after_launch(ctx, "k_silu_mul");
}

int inkq_glue_silu_mul_rows(inkq_ctx *ctx, const float *gu_dev, int T, int F, float *out_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, gu_dev && out_dev && T >= 1 && F >= 32 && F % 32 == 0, "bad silu_mul_rows arguments (F must be a multiple of 32)");
    const long long n4 = static_cast<long long>(T) * (F / 4);
    k_silu_mul_rows<<<static_cast<unsigned>((n4 + 255) / 256), 256, 0, ctx->stream>>>(reinterpret_cast<const float4 *>(gu_dev), T, F / 4,
                                                                                    reinterpret_cast<float4 *>(out_dev));
    return after_launch(ctx, "k_silu_mul_rows");
}

int inkq_glue_linear_m1(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int pro, const float *g_dev, float eps, float *C_dev, int accumulate)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && x_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, pro >= 0 && pro <= 2, "pro must be 0 (plain), 1 (RMSNorm) or 2 (SiLU * up)");
    INKQ_REQUIRE(ctx, pro != 1 || g_dev != nullptr, "RMSNorm needs its weight vector");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0 && (g_dev == nullptr || (reinterpret_cast<uintptr_t>(g_dev) & 15) == 0),
                 "x and g must be 16-byte aligned");
    return launch_gemv_fused(ctx, w, x_dev, pro, g_dev, eps, C_dev, accumulate);
}

int inkq_glue_add_rmsnorm_quant_rows(inkq_ctx *ctx, float *x_dev, const float *delta_dev, const float *norm_w_dev, float eps, int M, int K,
                                     inkq_act *out, int out_qmode, float *xn_out_dev)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, x_dev != nullptr && norm_w_dev != nullptr && out != nullptr, "null argument");
    INKQ_REQUIRE(ctx, M >= 1 && K >= QK && K % QK == 0 && K <= 32768, "K must be a multiple of 32, at most 32768");
    INKQ_REQUIRE(ctx, out->K == K && M <= out->max_rows, "the activation handle was created for another K or for fewer rows");
    INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
    const int M_ld = (M + 3) & ~3;
    const size_t smem = static_cast<size_t>(K) * sizeof(float);
    if (smem + 64 > 48 * 1024) {   // the kernel also holds 32 bytes of static shared memory
        static std::mutex mu;
        static bool configured[64] = {};
        std::lock_guard<std::mutex> g(mu);
        if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, INKQ_ERR_INVALID, "device index out of range");
        if (!configured[ctx->device]) {
            INKQ_CUDA(ctx, cudaFuncSetAttribute(k_add_rmsnorm_quant_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
            configured[ctx->device] = true;
        }
    }
    k_add_rmsnorm_quant_rows<<<M_ld, 256, smem, ctx->stream>>>(x_dev, delta_dev, norm_w_dev, M, K, eps, M_ld, out_qmode, out->q, out->d, out->s,
                                                                out->isum, xn_out_dev);
    out->M = M;
    out->M_ld = M_ld;
    out->qmode = out_qmode;
    out->ssq_parts = 0;
    return after_launch(ctx, "k_add_rmsnorm_quant_rows");
}

int inkq_glue_silu_mul_quant_rows(inkq_ctx *ctx, const float *gu_dev, int M, int F, inkq_act *out, int out_qmode)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, gu_dev != nullptr && out != nullptr, "null argument");
    INKQ_REQUIRE(ctx, M >= 1 && F >= QK && F % QK == 0, "F must be a multiple of 32");
    INKQ_REQUIRE(ctx, out->K == F && M <= out->max_rows, "the activation handle was created for another K or for fewer rows");
    INKQ_REQUIRE(ctx, out_qmode == INKQ_Q8_1_F16 || out_qmode == INKQ_Q8_0_F16 || out_qmode == INKQ_Q8_1_F32, "bad output quantization mode");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(gu_dev) & 15) == 0, "the input must be 16-byte aligned");
    return launch_silu_mul_quantize(ctx, out_qmode, gu_dev, M, F, out);
}

int inkq_glue_add_inplace(inkq_ctx *ctx, float *a_dev, const float *b_dev, long long n)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, a_dev && b_dev && n % 4 == 0, "bad add arguments");
    k_add_inplace<<<static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, ctx->stream>>>(reinterpret_cast<float4 *>(a_dev),
                                                                                     reinterpret_cast<const float4 *>(b_dev), n / 4);
    return after_launch(ctx, "k_add_inplace");
}

int inkq_glue_argmax_advance(inkq_ctx *ctx, const float *logits_dev, int n, int *token_out_dev, int *pos_dev, int advance, int *generated_dev,
                             int gen_cap)
{
    int rc = glue_use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, logits_dev && token_out_dev && pos_dev && n >= 1, "bad argmax arguments");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(logits_dev) & 15) == 0, "the logits must be 16-byte aligned");
    k_argmax_advance<<<ARGMAX_CTAS, 1024, 0, ctx->stream>>>(logits_dev, n, token_out_dev, pos_dev, advance, generated_dev, gen_cap);
    return after_launch(ctx, "k_argmax_advance");
}

}  // extern "C"
