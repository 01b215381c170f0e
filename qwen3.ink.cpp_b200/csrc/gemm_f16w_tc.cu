// fp16-weight matmul on the 5th-generation tensor cores (lm_head for many rows):
//   C[m][n] = sum_k x[m][k] * w[n][k],  w fp16 [rows][K], x fp32 [M][K], fp32 accumulate.
//
// No C++ kernel exists in the reference for this operand format (its lm_head is an int4 linear applied to the
// last token only, qwen3/src/qwen/QwenForCausalLM.cc:43-46,121); the arithmetic is that of its fp32 row-times-row
// GEMV gemv_fp32_rcr_mt_impl_1 (qwen3/src/qwen/fp32_gemx_kernels_rcr.cc:494-507).  M == 1 stays on the
// bandwidth-bound CUDA-core kernel (k_f16w_gemv); this file serves M >= 16.
//
// Numerics.  The tensor cores take 16-bit operands, so the fp32 activations are first written as fp16:
//   x16[m][k] = fp16(x[m][k] * 2^e_m)      e_m = the power of two that brings the row's largest magnitude to [2^13, 2^14)
// (k_f16w_split; the scaling is exact and is undone on the finished sum, so the row keeps fp16's full 11 significant
// bits whatever its magnitude).  With `passes` == 2 a second operand xlo16 = fp16(x * 2^e_m - x16) holds the next 11
// bits and the K loop runs a second time over it, accumulating sum_k xlo16 * w into the same tensor-memory
// accumulator: the activations then enter with 22 significant bits and the result agrees with an fp32 evaluation to
// ~1e-5 of the output's rms, at twice the tensor-core work.  With `passes` == 1 each activation
// carries a relative rounding error of at most 2^-11, i.e. |error| <= 2^-11 * sum_k |x_k * w_k| (about 3e-4 of the
// output's rms for random data).  Products are exact in fp32; the sum is accumulated in fp32 inside tensor memory in
// the hardware's order.
//
// Kernel: tcgen05.mma.cta_group::1.kind::f16, M = 128 weight rows (TMEM lanes) x N = block_m <= 256 activation rows
// (TMEM columns), K = 16 per instruction; the whole K extent accumulates in tensor memory.  A CTA multiplies TWO
// 128-row weight tiles with one activation stage (accumulators in columns [0,256) and [256,512)), which halves the
// activation bytes read from L2 / shared memory per output.  Persistent, 256 threads:
//   warp 0     TMA producer: per stage (64 K-elements) three tiled 2-D copies with the 128-byte swizzle: the two
//              weight tiles [128 rows][128 B] and the activations [block_m rows][128 B]; rows beyond the matrix are
//              zero-filled by TMA
//   warp 1     MMA issuer (one elected thread): 8 MMAs per stage, one commit per stage
//   warp 2     tensor-memory allocation / release
//   warps 4-7  epilogue: tcgen05.ld of the finished tiles, * 2^-e_m, transposed through a shared-memory staging buffer so
//              that each warp instruction stores 512 contiguous bytes of one output row and a row's 1 KB piece leaves
//              the SM together (the output of the vocabulary-sized matrix is far larger than L2 and its rows are
//              600 KB apart: 128-byte pieces arriving at different times cost most of the DRAM write bandwidth);
//              the same stores go to further destinations (peers of a column-sharded layer)
// No TMA multicast.  Every mbarrier wait is bounded; on expiry a device flag is set, all roles run out their loops
// without further waiting and the host reports INKQ_ERR_TIMEOUT.
//
// Algorithmic work per launch: 2*M*rows*K flop; compulsory bytes rows*K*2 + M*K*2 + M*rows*4.
#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {
namespace f16w {

constexpr int THREADS = 256;
constexpr int NT = 2;                                  // weight tiles per work item
constexpr int MAX_BLOCK_M = 256;
constexpr int A_TILE_BYTES = TILE_N * 128;             // 128 rows x 64 halves
constexpr int B_BYTES = MAX_BLOCK_M * 128;
constexpr int STAGE_BYTES = NT * A_TILE_BYTES + B_BYTES;   // 65536
constexpr int STAGES = 3;
constexpr int OUT_ROWS = 16;                            // activation rows per staging step of the epilogue
constexpr int OUT_BYTES = 2 * OUT_ROWS * NT * TILE_N * 4;  // two buffers of [16 rows][256 columns] fp32
constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * STAGE_BYTES + OUT_BYTES + 256 /*barriers*/;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

struct Params {
    float *C;
    const float *row_scale;   // 2^-e_m per activation row
    ExtraDst extra;
    int *flag;
    int M, rows, k_stages, passes, tiles_n, groups_n, tiles_m, block_m, ldc;
};

__device__ __forceinline__ void wait_bounded(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *dev_flag, uint32_t sleep_ns)
{
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
#pragma unroll 1
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return;
        if (sleep_ns != 0u) __nanosleep(sleep_ns);
        if ((spin & 31u) == 0u) {
            if (*abort_flag != 0) return;
            if (clock64() - t0 > INKQ_SPIN_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicExch(dev_flag, 1);
                return;
            }
        }
    }
}

__global__ void __launch_bounds__(THREADS, 1)
    k_gemm_f16w_tc(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_xlo,
                   const Params prm)
{
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    float *out_stage = reinterpret_cast<float *>(smem + STAGES * STAGE_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + STAGES * STAGE_BYTES + OUT_BYTES);
    uint64_t *full = bars, *empty = full + STAGES, *acc_full = empty + STAGES, *acc_empty = acc_full + 1, *drain = acc_empty + 1;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(drain + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_items = prm.groups_n * prm.tiles_m;   // work item = (pair of weight tiles, activation tile)

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
        mbar_init(drain, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 2) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_w);
            tma_prefetch_desc(&map_x);
            if (prm.passes == 2) tma_prefetch_desc(&map_xlo);
            uint32_t idx = 0, phase = 0;
            const uint32_t tx = NT * A_TILE_BYTES + static_cast<uint32_t>(prm.block_m) * 128u;   // boxes are always full size
            for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
                const int tg = item / prm.tiles_m, tm = item % prm.tiles_m;
                for (int s = 0; s < prm.passes * prm.k_stages; s++) {
                    const int ks = s % prm.k_stages;
                    wait_bounded(&empty[idx], phase ^ 1, abort_flag, prm.flag, 100u);
                    unsigned char *st = smem + idx * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[idx], tx);
#pragma unroll
                    for (int wt = 0; wt < NT; wt++)   // a tile past the end of the matrix arrives as zeros
                        tma_tensor2d_g2s(st + wt * A_TILE_BYTES, &map_w, ks * 64, (tg * NT + wt) * TILE_N, &full[idx]);
                    tma_tensor2d_g2s(st + NT * A_TILE_BYTES, s < prm.k_stages ? &map_x : &map_xlo, ks * 64, tm * prm.block_m, &full[idx]);
                    if (++idx == STAGES) {
                        idx = 0;
                        phase ^= 1;
                    }
                }
            }
            if (*abort_flag != 0) {   // copies nobody consumed may still be in flight: wait (bounded) for each stage's last fill
                for (uint32_t s = 0; s < STAGES; s++) mbar_wait_drain(&full[s], s < idx ? phase : phase ^ 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TILE_N, prm.block_m);
            uint32_t idx = 0, phase = 0, acc_phase = 0;
            for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
                wait_bounded(acc_empty, acc_phase ^ 1, abort_flag, prm.flag, 0u);
                tc_fence_after_sync();
                for (int ks = 0; ks < prm.passes * prm.k_stages; ks++) {
                    wait_bounded(&full[idx], phase, abort_flag, prm.flag, 0u);
                    tc_fence_after_sync();
                    // both operands: 128-byte swizzled rows of 64 halves (the TMA layout); the j-th K=16 slice is the
                    // j-th 32-byte part of a row; 8-row groups are 1024 B apart.  Start addresses count 16-byte units.
                    const uint32_t st = smem_u32(smem + idx * STAGE_BYTES);
                    const uint64_t b_desc0 = umma_smem_desc(st + NT * A_TILE_BYTES, 16, 1024, 2);
#pragma unroll
                    for (int wt = 0; wt < NT; wt++) {
                        const uint64_t a_desc0 = umma_smem_desc(st + wt * A_TILE_BYTES, 16, 1024, 2);
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            umma_f16(tmem_base + wt * MAX_BLOCK_M, a_desc0 + static_cast<uint64_t>(j * 2), b_desc0 + static_cast<uint64_t>(j * 2), idesc,
                                     (ks > 0 || j > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[idx]);   // the only commit of the stage
                    if (++idx == STAGES) {
                        idx = 0;
                        phase ^= 1;
                    }
                }
                umma_commit(acc_full);
                acc_phase ^= 1;
            }
            umma_commit(drain);   // every MMA has completed before tensor memory is released
            mbar_wait_drain(drain, 0u);
        }
        __syncwarp();
    } else if (warp >= 4) {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;          // TMEM lane quadrant this warp may read (warps 4..7 -> 0..3)
        const int row = quad * 32 + lane;
        uint32_t acc_phase = 0, buf = 0;
        for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
            const int tg = item / prm.tiles_m, tm = item % prm.tiles_m;
            const int n_base = tg * NT * TILE_N;                      // first output column of the item's 256
            wait_bounded(acc_full, acc_phase, abort_flag, prm.flag, 50u);
            acc_phase ^= 1;
            tc_fence_after_sync();
#pragma unroll 1
            for (int c0 = 0; c0 < prm.block_m; c0 += OUT_ROWS) {
                float *st = out_stage + buf * (OUT_ROWS * NT * TILE_N);
                // tensor memory -> registers -> staging [16 activation rows][256 columns] (lane = column: conflict-free)
#pragma unroll
                for (int wt = 0; wt < NT; wt++) {
                    uint32_t v[16];
                    tmem_ld_x16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + wt * MAX_BLOCK_M + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; j++) st[j * (NT * TILE_N) + wt * TILE_N + row] = __uint_as_float(v[j]);
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");    // the four epilogue warps
                // staging -> global: warp q stores rows q, q+4, q+8, q+12; a lane stores two float4 (512 B per warp instruction)
#pragma unroll
                for (int jj = 0; jj < OUT_ROWS / 4; jj++) {
                    const int j = jj * 4 + quad;
                    const int m = tm * prm.block_m + c0 + j;
                    if (m < prm.M && c0 + j < prm.block_m) {
                        const float sc = prm.row_scale[m];            // exact: a power of two
                        const size_t off = static_cast<size_t>(m) * prm.ldc + n_base;
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            const int nl = h * 128 + lane * 4;
                            if (n_base + nl < prm.rows) {             // rows is a multiple of 4: a float4 is inside or outside as a whole
                                float4 r = *reinterpret_cast<const float4 *>(st + j * (NT * TILE_N) + nl);
                                r.x *= sc;
                                r.y *= sc;
                                r.z *= sc;
                                r.w *= sc;
                                *reinterpret_cast<float4 *>(prm.C + off + nl) = r;
#pragma unroll
                                for (int e = 0; e < MAX_PEERS - 1; e++)
                                    if (e < prm.extra.n) *reinterpret_cast<float4 *>(prm.extra.p[e] + off + nl) = r;
                            }
                        }
                    }
                }
                buf ^= 1;   // the other buffer is free: its readers passed the barrier above one step ago
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// x fp32 [M][K] -> hi (and lo) fp16 [M][K] scaled by 2^e_m, and 2^-e_m per row.  One warp per row.
__global__ void __launch_bounds__(256) k_f16w_split(const float *__restrict__ x, int M, int K, __half *__restrict__ hi, __half *__restrict__ lo,
                                                    float *__restrict__ inv_scale)
{
    const int m = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (m >= M) return;
    const float4 *row = reinterpret_cast<const float4 *>(x + static_cast<size_t>(m) * K);
    float amax = 0.f;
    for (int i = lane; i < K / 4; i += 32) {
        const float4 v = row[i];
        amax = fmaxf(fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))), amax);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // 2^e with amax * 2^e in [2^13, 2^14); rows of zeros, infinities or NaNs are left unscaled
    int e = 0;
    if (amax > 0.f && amax < 3.0e38f) e = 13 - ilogbf(amax);
    e = max(-100, min(100, e));
    const float s = ldexpf(1.0f, e);
    if (lane == 0) inv_scale[m] = ldexpf(1.0f, -e);
    __half2 *h2 = reinterpret_cast<__half2 *>(hi + static_cast<size_t>(m) * K);
    __half2 *l2 = (lo != nullptr) ? reinterpret_cast<__half2 *>(lo + static_cast<size_t>(m) * K) : nullptr;
    for (int i = lane; i < K / 4; i += 32) {
        const float4 v = row[i];
        const float a[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
        __half h[4];
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __float2half_rn(a[j]);
        h2[2 * i] = __halves2half2(h[0], h[1]);
        h2[2 * i + 1] = __halves2half2(h[2], h[3]);
        if (l2 != nullptr) {
            __half l[4];
#pragma unroll
            for (int j = 0; j < 4; j++) l[j] = __float2half_rn(a[j] - __half2float(h[j]));   // the difference is exact in fp32
            l2[2 * i] = __halves2half2(l[0], l[1]);
            l2[2 * i + 1] = __halves2half2(l[2], l[3]);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int encode_f16_rows(inkq_ctx *ctx, CUtensorMap *map, const void *base, int K, int rows, int box_rows)
{
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(K) * 2};
    const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_rows)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult cr = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(base), gdim, gstride, box,
                                                                     estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(ctx, INKQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(cr)));
    return INKQ_OK;
}

}  // namespace f16w

// x16: M*K halves (hi) followed, when passes == 2, by M*K halves (lo); row_scale: M floats.  Both in the context's scratch.
int launch_f16w_gemm_tc(inkq_ctx *ctx, const F16W *w, const float *x, int M, float *C, int ldc, int passes, uint16_t *x16, float *row_scale,
                        const ExtraDst *extra)
{
    using namespace f16w;
    if (ctx->encode_tiled == nullptr) return fail(ctx, INKQ_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled entry point not available");
    if (w->K % 64 != 0) return fail(ctx, INKQ_ERR_UNSUPPORTED, "the tensor-core fp16-weight matmul needs K to be a multiple of 64");
    if (w->rows % 4 != 0 || ldc % 4 != 0 || (reinterpret_cast<uintptr_t>(C) & 15) != 0)
        return fail(ctx, INKQ_ERR_UNSUPPORTED, "the tensor-core fp16-weight matmul stores 16-byte pieces: rows and ldc must be multiples of 4 and C 16-byte aligned");
    const size_t mk = static_cast<size_t>(M) * w->K;
    __half *hi = reinterpret_cast<__half *>(x16), *lo = (passes == 2) ? hi + mk : nullptr;
    k_f16w_split<<<(M + 7) / 8, 256, 0, ctx->stream>>>(x, M, w->K, hi, lo, row_scale);
    int rc = after_launch(ctx, "k_f16w_split");
    if (rc) return rc;

    const int tiles_m = (M + MAX_BLOCK_M - 1) / MAX_BLOCK_M;
    const int block_m = (((M + tiles_m - 1) / tiles_m) + 15) & ~15;   // even split, multiple of 16
    CUtensorMap map_w, map_x, map_xlo;
    if ((rc = encode_f16_rows(ctx, &map_w, w->w, w->K, w->rows, TILE_N))) return rc;
    if ((rc = encode_f16_rows(ctx, &map_x, hi, w->K, M, block_m))) return rc;
    if ((rc = encode_f16_rows(ctx, &map_xlo, passes == 2 ? lo : hi, w->K, M, block_m))) return rc;

    Params prm;
    prm.C = C;
    prm.row_scale = row_scale;
    prm.extra = ExtraDst{};
    if (extra != nullptr) prm.extra = *extra;
    prm.passes = passes;
    prm.flag = ctx->dev_flag;
    prm.M = M;
    prm.rows = w->rows;
    prm.k_stages = w->K / 64;
    prm.tiles_n = (w->rows + TILE_N - 1) / TILE_N;
    prm.groups_n = (prm.tiles_n + NT - 1) / NT;
    prm.tiles_m = tiles_m;
    prm.block_m = block_m;
    prm.ldc = ldc;
    {
        static std::mutex mu;
        static bool configured[64] = {};
        if (ctx->device < 0 || ctx->device >= 64) return fail(ctx, INKQ_ERR_UNSUPPORTED, "device index beyond the launch table");
        std::lock_guard<std::mutex> lk(mu);
        if (!configured[ctx->device]) {   // the opt-in for large dynamic shared memory is per device
            cudaError_t e = cudaFuncSetAttribute(k_gemm_f16w_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
            if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("cudaFuncSetAttribute(k_gemm_f16w_tc): ") + cudaGetErrorString(e));
            configured[ctx->device] = true;
        }
    }
    const long long total = static_cast<long long>(prm.groups_n) * tiles_m;
    const int grid = static_cast<int>(total < ctx->num_sms ? total : ctx->num_sms);
    k_gemm_f16w_tc<<<grid, THREADS, SMEM_BYTES, ctx->stream>>>(map_w, map_x, map_xlo, prm);
    return after_launch(ctx, "k_gemm_f16w_tc");
}

}  // namespace inkq
