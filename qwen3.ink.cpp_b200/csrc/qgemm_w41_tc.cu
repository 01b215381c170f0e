// Weight-only W41 matmul on the 5th-generation tensor cores: fp16 activations x Q4_1 weights
// dequantised to fp16 on the fly, tcgen05.mma.kind::f16 with fp32 accumulators in tensor memory.
//
// No C++ kernel exists in the reference for this scheme; it follows
// notebooks/evaluate-qwen3_8b_W4.ipynb cell 13: the fp16 model's weight is replaced by the
// dequantised value and a stock fp16 linear with fp32 accumulation runs:
//   w16[n][k] = fp16(q[n][k] * d[n][k/32] + m[n][k/32])      (one rounding: a half-precision fma)
//   C[m][n]   = sum_k a16[m][k] * w16[n][k]                   (fp32 accumulate)
// Unlike the A8W4 schemes there is no per-block epilogue: the whole K extent accumulates inside
// tensor memory and the CUDA cores only dequantise (2.1 instructions per weight, once per tile)
// and store the finished tile, so this kernel is bound by the tensor pipe / shared-memory
// operand bandwidth, not by the epilogue.
//
// "Swap-AB" like the int8 kernel: the 128 weight rows of a tile are the UMMA M side (TMEM lanes),
// block_m = 16..192 activation rows (a multiple of 16, chosen on the host) the UMMA N side (TMEM
// columns).  One stage = one pair of quantization blocks = 64 K-elements = four K=16 MMAs.
//
// Persistent, warp-specialised, one CTA per SM, 512 threads:
//   warp 0       TMA producer: per stage one tiled 2-D copy of the fp16 activations
//                [block_m rows][64 halves = 128 B] (128-byte swizzle, rows beyond M zero-filled)
//                and two untiled bulk copies: the pair's packed nibbles (4096 B) and its fp16
//                scales {d_lo, d_hi, m_lo, m_hi} per row (1024 B)
//   warp 1       MMA issuer (one elected thread), commits free the stages
//   warp 2       tensor-memory allocation / release
//   warps 4-11   dequantise: thread = (row, low or high nibble block): 32 nibbles -> 32 halves with
//                prmt (nibble -> 1024+q as fp16 bits), sub.f16x2, fma.rn.f16x2, written in the
//                canonical no-swizzle K-major core-matrix layout (conflict-free on both sides)
//   warps 12-15  epilogue: tcgen05.ld of the finished fp32 tile, coalesced stores of C
// One ring of stages for all roles (raw operands + dequantised weights per stage), released by one tcgen05.commit
// per stage (back-to-back MMAs with a commit after every one or two run 2-3x slower than with one commit per 4-16;
// measured: 363 / 208 / 128 / 70 cycles per 128x112x32 MMA with 1 / 2 / 4 / 16 MMAs per commit).
// Every mbarrier wait is bounded; on expiry the kernel sets a device flag and all roles drain.
//
// Algorithmic work per launch: 2*M*N*K flop; bytes: N*K*0.625 weights + M*K*2 activations (re-read
// from L2 once per weight tile) + M*N*4 output.
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

namespace w41 {
constexpr int THREADS = 512;
constexpr int DEQ_WARPS = 8, EPI_WARPS = 4;
constexpr int RAW_W_BYTES = TILE_N * 32;                // packed nibbles of one (tile, pair): 4096
constexpr int RAW_S_BYTES = TILE_N * 8;                 // its fp16 scales: 1024
constexpr int U16_TILE_BYTES = TILE_N * 64 * 2;         // one dequantised (tile, pair): 16384
constexpr int ACC_COLS = 256;                          // TMEM columns of one accumulator (block_m <= 256)
// NT = weight tiles (of 128 rows) a CTA multiplies with one activation stage.  NT = 2 halves the activation bytes
// fetched from L2 per output (the limiter of the NT = 1 kernel) at the price of a single accumulator slot:
//   NT = 1: block_m <= 192, 4 stages, two accumulator slots of 256 columns (epilogue overlaps the next tile)
//   NT = 2: block_m <= 256, 3 stages, one slot: tile 0 in columns [0, 256), tile 1 in [256, 512)
template <int NT>
struct Cfg {
    static constexpr int MAX_BLOCK_M = (NT == 1) ? 192 : 256;
    static constexpr int RAW_A_BYTES = MAX_BLOCK_M * 128;
    static constexpr int RAW_STAGE_BYTES = ((RAW_A_BYTES + NT * (RAW_W_BYTES + RAW_S_BYTES)) + 1023) / 1024 * 1024;
    static constexpr int STAGES = (NT == 1) ? 4 : 3;
    static constexpr int U16_STAGE_BYTES = NT * U16_TILE_BYTES;
    static constexpr int ACC_STAGES = (NT == 1) ? 2 : 1;
    static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * (RAW_STAGE_BYTES + U16_STAGE_BYTES) + 256 /*barriers*/;
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

struct Params {
    const uint8_t *nibT;
    const uint2 *sc16;
    float *C;
    int *flag;
    int M, rows, pairs, tiles_n, groups_n, tiles_m, block_m, ldc;   // groups_n = ceil(tiles_n / NT)
};

struct Ring {
    uint32_t idx = 0, phase = 0;
    int n;
    __device__ explicit Ring(int n_) : n(n_) {}
    __device__ void advance()
    {
        if (++idx == static_cast<uint32_t>(n)) {
            idx = 0;
            phase ^= 1;
        }
    }
};

// Four nibbles (one per byte of v, already masked) -> four halves q*d + m, as two packed pairs.
__device__ __forceinline__ void dequant4(uint32_t v, __half2 d2, __half2 m2, uint32_t &out01, uint32_t &out23)
{
    // byte b -> fp16 bits 0x6400 | b = 1024 + b exactly; subtracting 1024 leaves b exactly
    const uint32_t h01 = __byte_perm(v, 0x64646464u, 0x4140);
    const uint32_t h23 = __byte_perm(v, 0x64646464u, 0x4342);
    const __half2 k1024 = __half2half2(__ushort_as_half(0x6400));
    const __half2 q01 = __hsub2(*reinterpret_cast<const __half2 *>(&h01), k1024);
    const __half2 q23 = __hsub2(*reinterpret_cast<const __half2 *>(&h23), k1024);
    const __half2 w01 = __hfma2(q01, d2, m2);
    const __half2 w23 = __hfma2(q23, d2, m2);
    out01 = *reinterpret_cast<const uint32_t *>(&w01);
    out23 = *reinterpret_cast<const uint32_t *>(&w23);
}

template <int NT>
__global__ void __launch_bounds__(THREADS, 1) k_gemm_w41_tc(const __grid_constant__ CUtensorMap map_a, const Params prm)
{
    constexpr int STAGES = Cfg<NT>::STAGES, RAW_STAGE_BYTES = Cfg<NT>::RAW_STAGE_BYTES, RAW_A_BYTES = Cfg<NT>::RAW_A_BYTES;
    constexpr int U16_STAGE_BYTES = Cfg<NT>::U16_STAGE_BYTES, ACC_STAGES = Cfg<NT>::ACC_STAGES;
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char *raw_base = smem;
    unsigned char *u16_base = raw_base + STAGES * RAW_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(u16_base + STAGES * U16_STAGE_BYTES);
    // per stage: raw_full (TMA bytes landed), u16_full (dequantised), consumed (raw operands read by the
    // dequantisers AND every MMA of the stage complete: the stage's two halves are free together)
    uint64_t *raw_full = bars, *u16_full = raw_full + STAGES, *consumed = u16_full + STAGES;
    uint64_t *acc_full = consumed + STAGES, *acc_empty = acc_full + ACC_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + ACC_STAGES);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = prm.groups_n * prm.tiles_m;   // work items: (group of NT weight tiles, activation tile)

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) {
            mbar_init(&raw_full[i], 1);
            mbar_init(&u16_full[i], DEQ_WARPS * 32);
            mbar_init(&consumed[i], DEQ_WARPS + 1);  // the dequantising warps + the MMA commit
        }
        for (int i = 0; i < ACC_STAGES; i++) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
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

#define INKQ_GIVE_UP()            \
    {                             \
        *abort_flag = 1;          \
        atomicExch(prm.flag, 1);  \
        dead = true;              \
        break;                    \
    }

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            Ring raw(STAGES);
            bool dead = false;
            for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
                const int tg = tile / prm.tiles_m, tm = tile % prm.tiles_m;
                const int nvalid = min(NT, prm.tiles_n - tg * NT);   // weight tiles of this group that exist
                const uint32_t tx = static_cast<uint32_t>(prm.block_m) * 128u + nvalid * (RAW_W_BYTES + RAW_S_BYTES);
                for (int p = 0; p < prm.pairs; p++) {
                    if (!mbar_wait_abortable(abort_flag, &consumed[raw.idx], raw.phase ^ 1, 500u)) INKQ_GIVE_UP();
                    unsigned char *st = raw_base + raw.idx * RAW_STAGE_BYTES;
                    mbar_arrive_expect_tx(&raw_full[raw.idx], tx);
                    tma_tensor2d_g2s(st, &map_a, p * 64, tm * prm.block_m, &raw_full[raw.idx]);
                    for (int wt = 0; wt < nvalid; wt++) {
                        const size_t slab = static_cast<size_t>(tg * NT + wt) * prm.pairs + p;
                        tma_bulk_g2s(st + RAW_A_BYTES + wt * RAW_W_BYTES, prm.nibT + slab * RAW_W_BYTES, RAW_W_BYTES, &raw_full[raw.idx]);
                        tma_bulk_g2s(st + RAW_A_BYTES + NT * RAW_W_BYTES + wt * RAW_S_BYTES,
                                     reinterpret_cast<const unsigned char *>(prm.sc16) + slab * RAW_S_BYTES, RAW_S_BYTES, &raw_full[raw.idx]);
                    }
                    raw.advance();
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_f16(TILE_N, prm.block_m);
            Ring raw(STAGES), acc(ACC_STAGES);
            bool dead = false;
            for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
                const int nvalid = min(NT, prm.tiles_n - (tile / prm.tiles_m) * NT);
                if (!mbar_wait_abortable(abort_flag, &acc_empty[acc.idx], acc.phase ^ 1, 0u)) INKQ_GIVE_UP();
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + ((NT == 1) ? acc.idx * ACC_COLS : 0);
                for (int p = 0; p < prm.pairs; p++) {
                    if (!mbar_wait_abortable(abort_flag, &raw_full[raw.idx], raw.phase, 0u)) INKQ_GIVE_UP();
                    if (!mbar_wait_abortable(abort_flag, &u16_full[raw.idx], raw.phase, 0u)) INKQ_GIVE_UP();
                    tc_fence_after_sync();
                    // A: dequantised weights, no swizzle: element (row r, k) at (k / 8) * 2048 + r * 16 + (k % 8) * 2:
                    //    K-adjacent 8x8 core matrices 2048 B apart (leading offset), 8-row groups 128 B apart (stride
                    //    offset); the j-th K=16 slice starts 4096 B further.
                    // B: activations, 128-byte swizzled rows of 64 halves; slice j is the j-th 32-byte part of the
                    //    row; 8-row groups are 1024 B apart.  The start-address field counts 16-byte units.
                    const uint64_t a_desc0 = umma_smem_desc(smem_u32(u16_base + raw.idx * U16_STAGE_BYTES), 2048, 128, 0);
                    const uint64_t b_desc0 = umma_smem_desc(smem_u32(raw_base + raw.idx * RAW_STAGE_BYTES), 16, 1024, 2);
#pragma unroll
                    for (int wt = 0; wt < NT; wt++) {
                        if (wt < nvalid) {
#pragma unroll
                            for (int j = 0; j < 4; j++)
                                umma_f16(d_tmem + wt * ACC_COLS, a_desc0 + static_cast<uint64_t>((wt * U16_TILE_BYTES + j * 4096) >> 4),
                                         b_desc0 + static_cast<uint64_t>(j * (32 >> 4)), idesc, (p > 0 || j > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&consumed[raw.idx]);   // the only commit of the stage
                    raw.advance();
                }
                if (dead) break;
                umma_commit(&acc_full[acc.idx]);
                acc.advance();
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 4 + DEQ_WARPS) {
        // ------------------------------ dequantise ------------------------------
        const int t = threadIdx.x - 128;
        const int r = t & 127;          // weight row inside the tile (32 consecutive rows per warp)
        const int hi = t >> 7;          // 0: low nibbles = block 2p (k 0..31), 1: high nibbles = block 2p+1 (k 32..63)
        const int swz = (r >> 2) & 1;   // chunk swizzle of the packed layout
        Ring raw(STAGES);
        bool dead = false;
        for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
            const int nvalid = min(NT, prm.tiles_n - (tile / prm.tiles_m) * NT);
            for (int p = 0; p < prm.pairs; p++) {
                // fresh operands in the stage imply that its previous round is consumed (the producer refills a stage
                // only then), so the dequantised half of the stage is free as well
                if (!mbar_wait_abortable(abort_flag, &raw_full[raw.idx], raw.phase, 100u)) INKQ_GIVE_UP();
#pragma unroll
                for (int wt = 0; wt < NT; wt++) {
                if (wt >= nvalid) continue;
                const unsigned char *wsrc = raw_base + raw.idx * RAW_STAGE_BYTES + RAW_A_BYTES + wt * RAW_W_BYTES;
                const unsigned char *ssrc = raw_base + raw.idx * RAW_STAGE_BYTES + RAW_A_BYTES + NT * RAW_W_BYTES + wt * RAW_S_BYTES;
                unsigned char *stage = u16_base + raw.idx * U16_STAGE_BYTES + wt * U16_TILE_BYTES;
                unsigned char *dst = stage + (4 * hi) * 2048 + r * 16;
                const uint2 sc = *reinterpret_cast<const uint2 *>(ssrc + r * 8);   // {d_lo, d_hi | m_lo, m_hi}
                const uint32_t dbits = hi ? (sc.x >> 16) : (sc.x & 0xFFFFu), mbits = hi ? (sc.y >> 16) : (sc.y & 0xFFFFu);
                const __half2 d2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(dbits)));
                const __half2 m2 = __half2half2(__ushort_as_half(static_cast<unsigned short>(mbits)));
#pragma unroll
                for (int c = 0; c < 2; c++) {   // logical 16-byte chunk c holds elements 16c..16c+15 of both blocks
                    const uint4 v = *reinterpret_cast<const uint4 *>(wsrc + r * 32 + ((c ^ swz) * 16));
                    const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                    uint32_t o[8];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const uint32_t nib = (hi ? (in[i] >> 4) : in[i]) & 0x0F0F0F0Fu;
                        dequant4(nib, d2, m2, o[2 * i], o[2 * i + 1]);
                    }
                    // elements 16c..16c+7 -> core matrix 2c, 16c+8..16c+15 -> core matrix 2c+1 of this block's four
                    *reinterpret_cast<uint4 *>(dst + (2 * c) * 2048) = make_uint4(o[0], o[1], o[2], o[3]);
                    *reinterpret_cast<uint4 *>(dst + (2 * c + 1) * 2048) = make_uint4(o[4], o[5], o[6], o[7]);
                }
                }   // weight tiles of the group
                fence_proxy_async_smem();
                mbar_arrive(&u16_full[raw.idx]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&consumed[raw.idx]);
                raw.advance();
            }
        }
    } else if (warp >= 4 + DEQ_WARPS) {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;          // TMEM lane quadrant this warp may read (warps 12..15 -> 0..3)
        const int row = quad * 32 + lane;
        Ring acc(ACC_STAGES);
        bool dead = false;
        for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
            const int tg = tile / prm.tiles_m, tm = tile % prm.tiles_m;
            const int nvalid = min(NT, prm.tiles_n - tg * NT);
            if (!mbar_wait_abortable(abort_flag, &acc_full[acc.idx], acc.phase, 50u)) INKQ_GIVE_UP();
            tc_fence_after_sync();
            for (int wt = 0; wt < nvalid; wt++) {
                const int n = (tg * NT + wt) * TILE_N + row;
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + ((NT == 1) ? acc.idx * ACC_COLS : wt * ACC_COLS);
                for (int c0 = 0; c0 < prm.block_m; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld_x16(taddr + c0, v);
                    tmem_ld_wait();
                    if (n < prm.rows) {
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            const int m = tm * prm.block_m + c0 + j;
                            if (m < prm.M) prm.C[static_cast<size_t>(m) * prm.ldc + n] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc.idx]);
            acc.advance();
        }
    }
#undef INKQ_GIVE_UP
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 2) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
}  // namespace w41

template <int NT>
static int launch_w41(inkq_ctx *ctx, const uint16_t *a16, int M, const Weight *w, float *C, int ldc)
{
    using namespace w41;
    const int tiles_m = (M + Cfg<NT>::MAX_BLOCK_M - 1) / Cfg<NT>::MAX_BLOCK_M;
    const int block_m = (((M + tiles_m - 1) / tiles_m) + 15) & ~15;   // even split, multiple of 16

    CUtensorMap map;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(w->K), static_cast<cuuint64_t>(M)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(w->K) * 2};
    const cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(block_m)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult cr = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<uint16_t *>(a16), gdim, gstride,
                                                                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(ctx, INKQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(cr)));

    Params prm;
    prm.nibT = w->nibT;
    prm.sc16 = w->sc16;
    prm.C = C;
    prm.flag = ctx->dev_flag;
    prm.M = M;
    prm.rows = w->rows;
    prm.pairs = w->pairs;
    prm.tiles_n = w->tiles;
    prm.groups_n = (w->tiles + NT - 1) / NT;
    prm.tiles_m = tiles_m;
    prm.block_m = block_m;
    prm.ldc = ldc;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_gemm_w41_tc<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<NT>::SMEM_BYTES);
        if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("cudaFuncSetAttribute(k_gemm_w41_tc): ") + cudaGetErrorString(e));
        configured = true;
    }
    const int total = prm.groups_n * prm.tiles_m;
    const int grid = total < ctx->num_sms ? total : ctx->num_sms;
    k_gemm_w41_tc<NT><<<grid, THREADS, Cfg<NT>::SMEM_BYTES, ctx->stream>>>(map, prm);
    return after_launch(ctx, "k_gemm_w41_tc");
}

int launch_gemm_w41_tc(inkq_ctx *ctx, const uint16_t *a16, int M, const Weight *w, float *C, int ldc)
{
    if (ctx->encode_tiled == nullptr) return fail(ctx, INKQ_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(a16) & 15) != 0) return fail(ctx, INKQ_ERR_INVALID, "the fp16 activations must be 16-byte aligned");
    // two weight tiles per CTA (half the activation bytes fetched per output: 1.10-1.15 vs 0.89-0.92 PFLOP/s at
    // M >= 2048, 52 vs 63 us at M = 322) unless that leaves more than half of the SMs without a work item
    const long long items2 = static_cast<long long>((w->tiles + 1) / 2) * ((M + 255) / 256);
    const bool two = 2 * items2 >= ctx->num_sms;
    return two ? launch_w41<2>(ctx, a16, M, w, C, ldc) : launch_w41<1>(ctx, a16, M, w, C, ldc);
}

}  // namespace inkq
