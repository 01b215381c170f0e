// Prefill QGEMM on the 5th-generation tensor cores: tcgen05.mma.kind::i8 with int32
// accumulators in tensor memory, operands staged by TMA, per-block fp32 epilogue.
//
// Stands in for gemm_repack_A81W41_fp32 (qwen3/src/qwen/quantized_gemx_kernels.cc:349-582)
// and gemm_repack_A80W40 (:195-347); A80W4Z has no reference kernel and shares the
// A80W40 code with q_w = nibble - zp.
//
//   C[m][n] = sum over 32-element blocks b of  d_a[m,b]*d_w[n,b]*I[m,n,b] + m_w[n,b]*s_a[m,b]
//   I[m,n,b] = sum_e q_a[m,32b+e] * q_w[n,32b+e]                       (exact int32)
//
// One tcgen05.mma has K = 32 for 8-bit operands, i.e. exactly one quantization
// block, so every MMA produces a fresh int32 tile that must be scaled on the CUDA
// cores before the next block may be added.  The kernel is "swap-AB": the 128
// weight rows of a tile are the UMMA M side (TMEM lanes), the activation rows are
// the UMMA N side (TMEM columns, BLOCK_M = 16..128 in steps of 16), which keeps
// the padding of a ragged M small and makes the store of C[m][n0..n0+127] coalesced.
//
// Persistent, warp-specialised, one CTA per SM, 512 threads:
//   warp 0      TMA producer: per stage (4 blocks = 128 K-bytes) one tiled 2-D copy of the
//               int8 activations [BLOCK_M rows][128 B] (128-byte swizzle, rows beyond M are
//               zero-filled by TMA) and two untiled bulk copies of the packed weights
//               (2 pairs x 4096 B) and their zero points
//   warp 1      MMA issuer: one elected thread issues the K=32 MMAs and commits
//   warp 2      tensor-memory allocation / release
//   warps 4-7   unpack: packed nibbles (smem) -> signed int8 (q - z) in the canonical
//               no-swizzle K-major core-matrix layout the MMA reads
//   warps 8-15  epilogue: tcgen05.ld of a block's int32 tile, s32->f32, scale, accumulate
//               in registers in exactly the reference's order; at the end of a tile the
//               fp32 accumulators are stored to C
// Rings: 4 raw stages, 2 unpacked stages, 4 TMEM accumulators of 128 columns.
// Every mbarrier wait is bounded; on expiry the kernel sets a device flag and all
// roles drain and leave (the context stays usable, the host reports INKQ_ERR_TIMEOUT).
//
// Operation order per output (bit-identical to the reference): for each pair of
// blocks ascending: acc = fma((float)I_lo, d_a_lo*d_w_lo, acc); fma((float)I_hi, ...);
// acc = fma(m_lo, s_a_lo, acc); acc = fma(m_hi, s_a_hi, acc).
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

constexpr int TC_THREADS = 512;
constexpr int STAGE_PAIRS = 2;                         // pairs per stage
constexpr int STAGE_BLOCKS = 2 * STAGE_PAIRS;          // 4 MMAs per stage
constexpr int RAW_STAGES = 4;
constexpr int U8_STAGES = 2;
constexpr int ACC_STAGES = 4;
constexpr int ACC_COLS = 128;                          // TMEM columns per accumulator
constexpr int RAW_A_BYTES = 128 * 128;                 // activations: up to 128 rows x 128 B
constexpr int RAW_W_BYTES = STAGE_PAIRS * TILE_N * 32; // packed weights: 8192
constexpr int RAW_Z_BYTES = STAGE_PAIRS * TILE_N * 2;  // zero points: 512
constexpr int RAW_STAGE_BYTES = 25600;                 // 16384 + 8192 + 512, rounded to 1024
constexpr int U8_BLOCK_BYTES = TILE_N * 32;            // one unpacked block: 4096
constexpr int U8_STAGE_BYTES = STAGE_BLOCKS * U8_BLOCK_BYTES;
constexpr int TC_SMEM_BYTES = 1024 /*align slack*/ + RAW_STAGES * RAW_STAGE_BYTES + U8_STAGES * U8_STAGE_BYTES + 256 /*barriers*/;

struct TcParams {
    const uint8_t *nibT;
    const float4 *sc32;
    const uint2 *sc16;
    const uchar2 *zpT;
    const float *d_a, *s_a;
    float *C;
    int32_t *dots;   // non-null: dump raw int32 block dots [M][rows][K/32] instead of computing C
    int *flag;
    int M, M_ld, rows, K, pairs, tiles_n, tiles_m, block_m, ldc;
    int desc_swap;   // debug: exchange the two offsets of the no-swizzle descriptor
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

// CW = columns of the accumulator handled by one epilogue warpgroup (BLOCK_M / 2).
template <int CW, bool HAS_MIN>
__global__ void __launch_bounds__(TC_THREADS, 1) k_qgemm_tc(const __grid_constant__ CUtensorMap map_a, const TcParams prm)
{
    constexpr int BLOCK_M = 2 * CW;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~static_cast<uintptr_t>(1023));
    unsigned char *raw_base = smem;
    unsigned char *u8_base = smem + RAW_STAGES * RAW_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(u8_base + U8_STAGES * U8_STAGE_BYTES);
    uint64_t *raw_full = bars, *raw_empty = bars + RAW_STAGES;
    uint64_t *u8_full = bars + 2 * RAW_STAGES, *u8_empty = u8_full + U8_STAGES;
    uint64_t *acc_full = u8_empty + U8_STAGES, *acc_empty = acc_full + ACC_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + ACC_STAGES);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = prm.tiles_n * prm.tiles_m;
    const int k_stages = (prm.pairs + STAGE_PAIRS - 1) / STAGE_PAIRS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RAW_STAGES; i++) {
            mbar_init(&raw_full[i], 1);
            mbar_init(&raw_empty[i], 4 + 1);  // 4 unpack warps + the MMA commit
        }
        for (int i = 0; i < U8_STAGES; i++) {
            mbar_init(&u8_full[i], 128);
            mbar_init(&u8_empty[i], 1);
        }
        for (int i = 0; i < ACC_STAGES; i++) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 8);  // one arrive per epilogue warp
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

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            Ring raw(RAW_STAGES);
            bool dead = false;
            for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
                const int tn = tile / prm.tiles_m, tm = tile % prm.tiles_m;
                for (int ks = 0; ks < k_stages; ks++) {
                    if (*abort_flag) { dead = true; break; }
                    if (!mbar_wait_abortable(abort_flag, &raw_empty[raw.idx], raw.phase ^ 1)) {
                        *abort_flag = 1;
                        atomicExch(prm.flag, 1);
                        dead = true;
                        break;
                    }
                    const int np = min(STAGE_PAIRS, prm.pairs - ks * STAGE_PAIRS);
                    unsigned char *st = raw_base + raw.idx * RAW_STAGE_BYTES;
                    const uint32_t tx = BLOCK_M * 128 + np * (TILE_N * 32) + np * (TILE_N * 2);
                    mbar_arrive_expect_tx(&raw_full[raw.idx], tx);
                    tma_tensor2d_g2s(st, &map_a, ks * 128, tm * BLOCK_M, &raw_full[raw.idx]);
                    const size_t slab = static_cast<size_t>(tn) * prm.pairs + static_cast<size_t>(ks) * STAGE_PAIRS;
                    tma_bulk_g2s(st + RAW_A_BYTES, prm.nibT + slab * (TILE_N * 32), np * (TILE_N * 32), &raw_full[raw.idx]);
                    tma_bulk_g2s(st + RAW_A_BYTES + RAW_W_BYTES, reinterpret_cast<const unsigned char *>(prm.zpT) + slab * (TILE_N * 2),
                                 np * (TILE_N * 2), &raw_full[raw.idx]);
                    raw.advance();
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(TILE_N, BLOCK_M);
            Ring raw(RAW_STAGES), u8(U8_STAGES), acc(ACC_STAGES);
            bool dead = false;
            for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
                for (int ks = 0; ks < k_stages && !dead; ks++) {
                    if (*abort_flag) { dead = true; break; }
                    if (!mbar_wait_abortable(abort_flag, &raw_full[raw.idx], raw.phase) || !mbar_wait_abortable(abort_flag, &u8_full[u8.idx], u8.phase)) {
                        *abort_flag = 1;
                        atomicExch(prm.flag, 1);
                        dead = true;
                        break;
                    }
                    tc_fence_after_sync();
                    const int nblk = 2 * min(STAGE_PAIRS, prm.pairs - ks * STAGE_PAIRS);
                    const uint32_t a_smem = smem_u32(u8_base + u8.idx * U8_STAGE_BYTES);
                    const uint32_t b_smem = smem_u32(raw_base + raw.idx * RAW_STAGE_BYTES);
                    for (int j = 0; j < nblk; j++) {
                        if (!mbar_wait_abortable(abort_flag, &acc_empty[acc.idx], acc.phase ^ 1)) {
                            *abort_flag = 1;
                            atomicExch(prm.flag, 1);
                            dead = true;
                            break;
                        }
                        tc_fence_after_sync();
                        // A: unpacked weights of block j, no swizzle: element (row r, k) at
                        //    (k / 16) * 2048 + r * 16 + (k % 16): 8-row core matrices 128 B apart
                        //    along rows, the two K halves 2048 B apart.
                        const uint64_t a_desc = prm.desc_swap ? umma_smem_desc(a_smem + j * U8_BLOCK_BYTES, 128, 2048, 0)
                                                              : umma_smem_desc(a_smem + j * U8_BLOCK_BYTES, 2048, 128, 0);
                        // B: activations, 128-byte swizzled rows of 128 B; block j is the j-th
                        //    32-byte slice of the row; 8-row groups are 1024 B apart.
                        const uint64_t b_desc = umma_smem_desc(b_smem + j * 32, 16, 1024, 2);
                        umma_i8(tmem_base + acc.idx * ACC_COLS, a_desc, b_desc, idesc, 0u);
                        umma_commit(&acc_full[acc.idx]);
                        acc.advance();
                    }
                    umma_commit(&raw_empty[raw.idx]);
                    umma_commit(&u8_empty[u8.idx]);
                    raw.advance();
                    u8.advance();
                }
            }
        }
        __syncwarp();
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------ unpack ------------------------------
        // lane -> 16 rows x 2 chunks per warp step; 8 consecutive lanes = 8 consecutive rows of
        // one logical chunk: conflict-free 16-byte reads (thanks to the row swizzle of the packed
        // layout) and one contiguous 128-byte core matrix per 8 lanes on the write side.
        const int uw = warp - 4;
        const int rr = (lane & 7) + 8 * (lane >> 4);
        const int chunk = (lane >> 3) & 1;
        Ring raw(RAW_STAGES), u8(U8_STAGES);
        bool dead = false;
        for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
            for (int ks = 0; ks < k_stages; ks++) {
                if (*abort_flag) { dead = true; break; }
                if (!mbar_wait_abortable(abort_flag, &raw_full[raw.idx], raw.phase) || !mbar_wait_abortable(abort_flag, &u8_empty[u8.idx], u8.phase ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(prm.flag, 1);
                    dead = true;
                    break;
                }
                const int np = min(STAGE_PAIRS, prm.pairs - ks * STAGE_PAIRS);
                const unsigned char *wsrc = raw_base + raw.idx * RAW_STAGE_BYTES + RAW_A_BYTES;
                const unsigned char *zsrc = wsrc + RAW_W_BYTES;
                unsigned char *dst = u8_base + u8.idx * U8_STAGE_BYTES;
                for (int pp = 0; pp < np; pp++) {
#pragma unroll
                    for (int it = 0; it < 2; it++) {
                        const int r = (it * 4 + uw) * 16 + rr;
                        const uint4 v = *reinterpret_cast<const uint4 *>(wsrc + pp * (TILE_N * 32) + r * 32 + ((chunk ^ ((r >> 2) & 1)) * 16));
                        const uchar2 z = *reinterpret_cast<const uchar2 *>(zsrc + pp * (TILE_N * 2) + r * 2);
                        const uint32_t zl = static_cast<uint32_t>(z.x) * 0x01010101u, zh = static_cast<uint32_t>(z.y) * 0x01010101u;
                        const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                        uint32_t lo[4], hi[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            // byte-wise (nibble - z) without borrows between bytes: set bit 7, subtract, clear
                            lo[i] = (((in[i] & 0x0F0F0F0Fu) | 0x80808080u) - zl) ^ 0x80808080u;
                            hi[i] = ((((in[i] >> 4) & 0x0F0F0F0Fu) | 0x80808080u) - zh) ^ 0x80808080u;
                        }
                        unsigned char *o = dst + chunk * 2048 + r * 16;
                        *reinterpret_cast<uint4 *>(o + (2 * pp) * U8_BLOCK_BYTES) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                        *reinterpret_cast<uint4 *>(o + (2 * pp + 1) * U8_BLOCK_BYTES) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(&u8_full[u8.idx]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[raw.idx]);
                raw.advance();
                u8.advance();
            }
        }
    } else if (warp >= 8) {
        // ------------------------------ epilogue ------------------------------
        const int quad = warp & 3;            // TMEM lane quadrant this warp may read
        const int half = (warp - 8) >> 2;     // which half of the accumulator columns
        const int row = quad * 32 + lane;     // weight row inside the tile = TMEM lane
        const int nbk = 2 * prm.pairs;
        Ring acc(ACC_STAGES);
        bool dead = false;
        for (int tile = blockIdx.x; tile < total_tiles && !dead; tile += gridDim.x) {
            const int tn = tile / prm.tiles_m, tm = tile % prm.tiles_m;
            const int n = tn * TILE_N + row;
            const int m_base = tm * BLOCK_M + half * CW;
            float accf[CW];
#pragma unroll
            for (int j = 0; j < CW; j++) accf[j] = 0.0f;
            float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int b = 0; b < nbk; b++) {
                if ((b & 1) == 0) {
                    const size_t rec = (static_cast<size_t>(tn) * prm.pairs + (b >> 1)) * TILE_N + row;
                    if (prm.sc32 != nullptr) {
                        sc = prm.sc32[rec];
                    } else {
                        const uint2 pk = prm.sc16[rec];
                        const float2 x0 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.x));
                        const float2 x1 = __half22float2(*reinterpret_cast<const __half2 *>(&pk.y));
                        sc = make_float4(x0.x, x0.y, x1.x, x1.y);
                    }
                }
                if (*abort_flag) { dead = true; break; }
                if (!mbar_wait_abortable(abort_flag, &acc_full[acc.idx], acc.phase)) {
                    *abort_flag = 1;
                    atomicExch(prm.flag, 1);
                    dead = true;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc.idx * ACC_COLS + half * CW;
                const float dw = (b & 1) ? sc.y : sc.x;
                const float *da_row = prm.d_a + static_cast<size_t>(b) * prm.M_ld;
                const float *sa_row = prm.s_a + static_cast<size_t>(b) * prm.M_ld;
#pragma unroll
                for (int c8 = 0; c8 < CW / 8; c8++) {
                    uint32_t raw[8];
                    tmem_ld_x8(taddr + c8 * 8, raw);
                    tmem_ld_wait();
                    if (c8 == CW / 8 - 1) {
                        // the whole accumulator is in registers: hand the TMEM buffer back
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&acc_empty[acc.idx]);
                    }
                    const int m0 = m_base + c8 * 8;
                    if (prm.dots != nullptr) {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            if (m0 + j < prm.M && n < prm.rows)
                                prm.dots[(static_cast<size_t>(m0 + j) * prm.rows + n) * nbk + b] = static_cast<int32_t>(raw[j]);
                        continue;
                    }
#pragma unroll
                    for (int j4 = 0; j4 < 8; j4 += 4) {
                        const int m = m0 + j4;
                        float4 da = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (m < prm.M_ld) da = *reinterpret_cast<const float4 *>(da_row + m);
                        const float dav[4] = {da.x, da.y, da.z, da.w};
#pragma unroll
                        for (int j = 0; j < 4; j++)
                            accf[c8 * 8 + j4 + j] = fmaf(static_cast<float>(static_cast<int32_t>(raw[j4 + j])), __fmul_rn(dav[j], dw), accf[c8 * 8 + j4 + j]);
                        if (HAS_MIN && (b & 1)) {
                            float4 s0 = make_float4(0.f, 0.f, 0.f, 0.f), s1 = s0;
                            if (m < prm.M_ld) {
                                s0 = *reinterpret_cast<const float4 *>(sa_row - prm.M_ld + m);
                                s1 = *reinterpret_cast<const float4 *>(sa_row + m);
                            }
                            const float s0v[4] = {s0.x, s0.y, s0.z, s0.w}, s1v[4] = {s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                accf[c8 * 8 + j4 + j] = fmaf(sc.z, s0v[j], accf[c8 * 8 + j4 + j]);
                                accf[c8 * 8 + j4 + j] = fmaf(sc.w, s1v[j], accf[c8 * 8 + j4 + j]);
                            }
                        }
                    }
                }
                acc.advance();
            }
            if (!dead && prm.dots == nullptr && n < prm.rows) {
#pragma unroll
                for (int j = 0; j < CW; j++) {
                    const int m = m_base + j;
                    if (m < prm.M) prm.C[static_cast<size_t>(m) * prm.ldc + n] = accf[j];
                }
            }
        }
    }
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

template <int CW, bool HAS_MIN>
static int launch_one(inkq_ctx *ctx, const CUtensorMap &map, const TcParams &prm, int grid)
{
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(k_qgemm_tc<CW, HAS_MIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
        if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("cudaFuncSetAttribute(k_qgemm_tc): ") + cudaGetErrorString(e));
        configured = true;
    }
    k_qgemm_tc<CW, HAS_MIN><<<grid, TC_THREADS, TC_SMEM_BYTES, ctx->stream>>>(map, prm);
    return after_launch(ctx, "k_qgemm_tc");
}

template <bool HAS_MIN>
static int launch_cw(inkq_ctx *ctx, int cw, const CUtensorMap &map, const TcParams &prm, int grid)
{
    switch (cw) {
        case 8: return launch_one<8, HAS_MIN>(ctx, map, prm, grid);
        case 16: return launch_one<16, HAS_MIN>(ctx, map, prm, grid);
        case 24: return launch_one<24, HAS_MIN>(ctx, map, prm, grid);
        case 32: return launch_one<32, HAS_MIN>(ctx, map, prm, grid);
        case 40: return launch_one<40, HAS_MIN>(ctx, map, prm, grid);
        case 48: return launch_one<48, HAS_MIN>(ctx, map, prm, grid);
        case 56: return launch_one<56, HAS_MIN>(ctx, map, prm, grid);
        case 64: return launch_one<64, HAS_MIN>(ctx, map, prm, grid);
    }
    return fail(ctx, INKQ_ERR_INVALID, "internal: bad column width");
}

int launch_gemm_tc(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, int ldc, int32_t *dots)
{
    if (ctx->encode_tiled == nullptr) return fail(ctx, INKQ_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled entry point not available");
    const int M = a->M;
    const int tiles_m = (M + 127) / 128;
    const int block_m = (((M + tiles_m - 1) / tiles_m) + 15) & ~15;  // even split, multiple of 16, <= 128

    CUtensorMap map;
    const cuuint64_t gdim[2] = {static_cast<cuuint64_t>(a->K), static_cast<cuuint64_t>(M)};
    const cuuint64_t gstride[1] = {static_cast<cuuint64_t>(a->K)};
    const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(block_m)};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult cr = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->q, gdim, gstride, box, estr,
                                                                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(ctx, INKQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(cr)));

    TcParams prm;
    prm.nibT = w->nibT;
    prm.sc32 = w->sc32;
    prm.sc16 = w->sc16;
    prm.zpT = w->zpT;
    prm.d_a = a->d;
    prm.s_a = a->s;
    prm.C = C;
    prm.dots = dots;
    prm.flag = ctx->dev_flag;
    prm.M = M;
    prm.M_ld = a->M_ld;
    prm.rows = w->rows;
    prm.K = w->K;
    prm.pairs = w->pairs;
    prm.tiles_n = w->tiles;
    prm.tiles_m = tiles_m;
    prm.block_m = block_m;
    prm.ldc = ldc;
    const char *dbg = getenv("INKQ_TC_DESC_SWAP");
    prm.desc_swap = (dbg != nullptr && dbg[0] == '1') ? 1 : 0;
    const int total = prm.tiles_n * prm.tiles_m;
    const int grid = total < ctx->num_sms ? total : ctx->num_sms;
    if (w->scheme == INKQ_A81W41) return launch_cw<true>(ctx, block_m / 2, map, prm, grid);
    return launch_cw<false>(ctx, block_m / 2, map, prm, grid);
}

}  // namespace inkq
