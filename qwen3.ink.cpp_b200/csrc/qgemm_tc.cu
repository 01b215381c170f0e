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
// Persistent, warp-specialised, one CTA per SM, 768 threads:
//   warp 0      operand TMA producer: per stage (4 blocks = 128 K-bytes) one tiled 2-D copy of
//               the int8 activations [BLOCK_M rows][128 B] (128-byte swizzle, rows beyond M
//               are zero-filled by TMA) and two untiled bulk copies of the packed weights
//               (2 pairs x 4096 B) and their zero points
//   warp 1      MMA issuer: one elected thread issues the K=32 MMAs and commits
//   warp 2      tensor-memory allocation / release
//   warp 3      scale TMA producer: per stage the activation block scales d_a and sums s_a of
//               the tile's rows ([4 blocks][BLOCK_M] fp32 each, tiled 2-D copies, zero-filled
//               past the end) and the weight rows' {d_lo, d_hi, m_lo, m_hi} records (one bulk
//               copy), into their own ring because the epilogue consumes them later than the
//               MMA consumes the operands
//   warps 4-7   unpack: packed nibbles (smem) -> signed int8 (q - z) in the canonical
//               no-swizzle K-major core-matrix layout the MMA reads
//   warps 8-23  epilogue (the binding resource: it owns all four schedulers): tcgen05.ld of a
//               block's int32 tile, s32->f32, scale, accumulate in registers in exactly the
//               reference's order; at the end of a tile the fp32 accumulators are stored to C.
//               Warp w reads TMEM lanes 32*(w%4).. and a quarter of the columns.
// Rings: 5 raw stages, 3 unpacked stages (both freed by one "stage done" commit), 4 scale stages, and as many tensor-memory accumulator
// slots as fit into the 512 columns (a slot = one pair of blocks = 2*BLOCK_M columns: two MMAs,
// one commit, one hand-shake), so that narrow tiles keep many pairs in flight.
// Every mbarrier wait is bounded; when one runs out the kernel sets a device flag, every later
// wait of every role returns at once, all roles run to the end of their loops (on garbage,
// inside their buffers) and leave; the host reports INKQ_ERR_TIMEOUT and the context stays usable.
//
// Operation order per output (bit-identical to the reference): for each pair of
// blocks ascending: acc = fma((float)I_lo, d_a_lo*d_w_lo, acc); fma((float)I_hi, ...);
// acc = fma(m_lo, s_a_lo, acc); acc = fma(m_hi, s_a_hi, acc).
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdlib.h>

#include <mutex>

#include "inkq_internal.h"
#include "ptx.cuh"

namespace inkq {

constexpr int TC_THREADS = 768;
constexpr int EPI_WARPS = 16;
// Register re-balancing after the roles split (setmaxnreg).  The kernel is launched with LAUNCH_REGS per
// thread (checked on the host before the first launch); the two non-epilogue warpgroups release registers,
// the four epilogue warpgroups take them.  A request larger than what was released would block forever,
// hence the static check.
#ifndef INKQ_TC_CTRL_REGS
#define INKQ_TC_CTRL_REGS 40
#endif
#ifndef INKQ_TC_UNPACK_REGS
#define INKQ_TC_UNPACK_REGS 48
#endif
#ifndef INKQ_TC_EPI_REGS
#define INKQ_TC_EPI_REGS 96
#endif
// columns per tcgen05.ld chunk of the epilogue's software pipeline (8 or 16)
#ifndef INKQ_TC_CHUNK
#define INKQ_TC_CHUNK 16
#endif
constexpr int LAUNCH_REGS = 80, CTRL_REGS = INKQ_TC_CTRL_REGS, UNPACK_REGS = INKQ_TC_UNPACK_REGS, EPI_REGS = INKQ_TC_EPI_REGS;
static_assert(128 * (LAUNCH_REGS - CTRL_REGS) + 128 * (LAUNCH_REGS - UNPACK_REGS) >= 512 * (EPI_REGS - LAUNCH_REGS), "setmaxnreg budget");
constexpr int STAGE_PAIRS = 2;                         // pairs per stage
constexpr int STAGE_BLOCKS = 2 * STAGE_PAIRS;          // 4 MMAs per stage
constexpr int RAW_STAGES = 5;
constexpr int U8_STAGES = 3;
constexpr int MAX_ACC_SLOTS = 8;
constexpr int DONE_RING = 8;   // "the MMAs of K-stage g have completed" barriers, indexed by g % DONE_RING (deeper than both smem rings)
constexpr int SC_STAGES = 4;
constexpr int SC_PLANE_BYTES = STAGE_BLOCKS * 128 * 4;    // one plane of a scale stage: [4 blocks][128 rows] fp32
constexpr int SC_W_BYTES = STAGE_PAIRS * TILE_N * 16;    // the weight rows' float4 records of the stage's pairs
constexpr int SC_STAGE_BYTES = 2 * SC_PLANE_BYTES + SC_W_BYTES;   // d_a, s_a, weight scales
constexpr int RAW_A_BYTES = 128 * 128;                 // activations: up to 128 rows x 128 B
constexpr int RAW_W_BYTES = STAGE_PAIRS * TILE_N * 32; // packed weights: 8192
constexpr int RAW_Z_BYTES = STAGE_PAIRS * TILE_N * 2;  // zero points: 512
constexpr int RAW_STAGE_BYTES = 25600;                 // 16384 + 8192 + 512, rounded to 1024
constexpr int U8_BLOCK_BYTES = TILE_N * 32;            // one unpacked block: 4096
constexpr int U8_STAGE_BYTES = STAGE_BLOCKS * U8_BLOCK_BYTES;
constexpr int TC_SMEM_BYTES =
    1024 /*align slack*/ + RAW_STAGES * RAW_STAGE_BYTES + U8_STAGES * U8_STAGE_BYTES + SC_STAGES * SC_STAGE_BYTES + 512 /*barriers*/;
static_assert(TC_SMEM_BYTES <= 227 * 1024, "shared memory budget");

__host__ __device__ constexpr int acc_slots_for(int block_m)
{
    return (512 / (2 * block_m)) < MAX_ACC_SLOTS ? (512 / (2 * block_m)) : MAX_ACC_SLOTS;
}

struct TcParams {
    const uint8_t *nibT;
    const float4 *sc32;
    const uchar2 *zpT;
    float *C;
    ExtraDst extra;  // further destinations of every C element (peers of a column-sharded layer)
    int32_t *dots;   // non-null: dump raw int32 block dots [M][rows][K/32] instead of computing C
    int *flag;
    int M, rows, pairs, tn0, tiles_n, tiles_m, ldc;   // this launch covers weight tiles tn0 .. tn0 + tiles_n - 1
};

struct Ring {
    uint32_t idx = 0, phase = 0;
    int n;
    __device__ explicit Ring(int n_) : n(n_) {}
    __device__ __forceinline__ void advance()
    {
        if (++idx == static_cast<uint32_t>(n)) {
            idx = 0;
            phase ^= 1;
        }
    }
};

// Bounded wait of this kernel.  The common case (phase already complete) is one probe and one
// untaken branch.  Otherwise the thread probes until the phase completes, the CTA's abort word is
// set by another role, or the cycle limit runs out; in the last case it sets the abort word and the
// device flag.  It always returns: after an abort the roles finish their loops without waiting.
__device__ __forceinline__ void tc_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *dev_flag, uint32_t sleep_ns)
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

// One arrival per warp without a divergent branch: the elected lane arrives, predicated.
__device__ __forceinline__ void mbar_arrive_elect(uint64_t *bar)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 st;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "@p mbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
        : "memory");
}

// Two fp32 values in one 64-bit register and the IEEE (round-to-nearest) packed
// multiply / fused multiply-add of sm_100: each half rounds exactly like the scalar
// instruction, so results stay bit-identical while the issue slots are halved.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long mul2(unsigned long long a, unsigned long long b)
{
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c)
{
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// Two block dots -> packed fp32 pair, exactly (a block dot is at most 32 * 128 * 15 = 61440 in magnitude).
__device__ __forceinline__ unsigned long long cvt2_exact(uint32_t v0, uint32_t v1)
{
    return pack2(static_cast<float>(static_cast<int32_t>(v0)), static_cast<float>(static_cast<int32_t>(v1)));
}

// Loads N consecutive TMEM columns of this thread's lane; N a multiple of 4 up to 16.
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t *r)
{
    if constexpr (N == 16) {
        tmem_ld_x16(taddr, r);
    } else if constexpr (N == 12) {
        tmem_ld_x8(taddr, r);
        tmem_ld_x4(taddr + 8, r + 8);
    } else if constexpr (N == 8) {
        tmem_ld_x8(taddr, r);
    } else {
        static_assert(N == 4, "column chunk must be 4, 8, 12 or 16");
        tmem_ld_x4(taddr, r);
    }
}

// CW = columns of the accumulator handled by one epilogue warp (BLOCK_M / 4).
template <int CW, bool HAS_MIN, bool DUMP>
__global__ void __launch_bounds__(TC_THREADS, 1)
    k_qgemm_tc(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_d, const __grid_constant__ CUtensorMap map_s,
               const TcParams prm)
{
    constexpr int BLOCK_M = 4 * CW;
    constexpr int ACC_SLOTS = acc_slots_for(BLOCK_M);
    constexpr int SLOT_COLS = 2 * BLOCK_M;   // low block at +0, high block at +BLOCK_M
    // 1024-byte alignment (128-byte swizzle atoms) by an offset from the shared array itself, so
    // that every access below stays a shared-space (not generic) load or store
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    unsigned char *smem = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char *raw_base = smem;
    unsigned char *u8_base = raw_base + RAW_STAGES * RAW_STAGE_BYTES;
    unsigned char *sc_base = u8_base + U8_STAGES * U8_STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sc_base + SC_STAGES * SC_STAGE_BYTES);
    uint64_t *raw_full = bars, *stage_done = raw_full + RAW_STAGES;
    uint64_t *u8_full = stage_done + DONE_RING;
    uint64_t *acc_full = u8_full + U8_STAGES, *acc_empty = acc_full + MAX_ACC_SLOTS;
    uint64_t *sc_full = acc_empty + MAX_ACC_SLOTS, *sc_empty = sc_full + SC_STAGES;
    uint64_t *drain_bar = sc_empty + SC_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(drain_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = prm.tiles_n * prm.tiles_m;
    const int k_stages = (prm.pairs + STAGE_PAIRS - 1) / STAGE_PAIRS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < RAW_STAGES; i++) mbar_init(&raw_full[i], 1);
        for (int i = 0; i < DONE_RING; i++) mbar_init(&stage_done[i], 1);   // one tcgen05.commit per K-stage
        for (int i = 0; i < U8_STAGES; i++) mbar_init(&u8_full[i], 4);      // one arrival per unpack warp
        for (int i = 0; i < MAX_ACC_SLOTS; i++) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], EPI_WARPS);
        }
        for (int i = 0; i < SC_STAGES; i++) {
            mbar_init(&sc_full[i], 1);
            mbar_init(&sc_empty[i], EPI_WARPS);
        }
        mbar_init(drain_bar, 1);
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
    // Launched with programmatic stream serialization: everything above (barriers, tensor-memory allocation) may overlap
    // the tail of the kernel before this one in the stream (normally the quantizer that writes the activations); nothing
    // below may, and a dependent kernel launched the same way may begin its own set-up from here on.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp < 4) setmaxnreg_dec<CTRL_REGS>();
    if (warp >= 4 && warp < 8) setmaxnreg_dec<UNPACK_REGS>();
    if (warp == 0) {
        // ------------------------------ operand TMA producer ------------------------------
        if (lane == 0) {
            tma_prefetch_desc(&map_a);
            Ring raw(RAW_STAGES);
            uint32_t g = 0;   // K-stages issued so far (over all tiles of this CTA)
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int tn = prm.tn0 + tile / prm.tiles_m, tm = tile % prm.tiles_m;
                for (int ks = 0; ks < k_stages; ks++, g++) {
                    // the slot last held stage g - RAW_STAGES: free once that stage's MMAs have completed (which also
                    // means the unpack warps are done with its packed weights)
                    if (g >= RAW_STAGES) {
                        const uint32_t h = g - RAW_STAGES;
                        tc_wait(&stage_done[h % DONE_RING], (h / DONE_RING) & 1u, abort_flag, prm.flag, 200u);
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
            if (*abort_flag != 0) {
                // copies of stages nobody consumed may still be in flight: wait (bounded) for each stage's last fill
                for (int s = 0; s < RAW_STAGES; s++) mbar_wait_drain(&raw_full[s], static_cast<uint32_t>(s) < raw.idx ? raw.phase : raw.phase ^ 1);
            }
        }
        __syncwarp();
    } else if (warp == 3) {
        // ------------------------------ scale TMA producer ------------------------------
        if (lane == 0 && !DUMP) {  // the block-dot dump applies no scales
            tma_prefetch_desc(&map_d);
            if (HAS_MIN) tma_prefetch_desc(&map_s);
            Ring sc(SC_STAGES);
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                const int tn = prm.tn0 + tile / prm.tiles_m, tm = tile % prm.tiles_m;
                for (int ks = 0; ks < k_stages; ks++) {
                    tc_wait(&sc_empty[sc.idx], sc.phase ^ 1, abort_flag, prm.flag, 200u);
                    const int np = min(STAGE_PAIRS, prm.pairs - ks * STAGE_PAIRS);
                    unsigned char *st = sc_base + sc.idx * SC_STAGE_BYTES;
                    const uint32_t plane = STAGE_BLOCKS * BLOCK_M * 4;  // the box is always full size; out-of-range parts arrive as zeros
                    mbar_arrive_expect_tx(&sc_full[sc.idx], (HAS_MIN ? 2 * plane : plane) + np * (TILE_N * 16));
                    tma_tensor2d_g2s(st, &map_d, tm * BLOCK_M, ks * STAGE_BLOCKS, &sc_full[sc.idx]);
                    if (HAS_MIN) tma_tensor2d_g2s(st + SC_PLANE_BYTES, &map_s, tm * BLOCK_M, ks * STAGE_BLOCKS, &sc_full[sc.idx]);
                    const size_t slab = static_cast<size_t>(tn) * prm.pairs + static_cast<size_t>(ks) * STAGE_PAIRS;
                    tma_bulk_g2s(st + 2 * SC_PLANE_BYTES, prm.sc32 + slab * TILE_N, np * (TILE_N * 16), &sc_full[sc.idx]);
                    sc.advance();
                }
            }
            if (*abort_flag != 0) {
                for (int s = 0; s < SC_STAGES; s++) mbar_wait_drain(&sc_full[s], static_cast<uint32_t>(s) < sc.idx ? sc.phase : sc.phase ^ 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc_i8(TILE_N, BLOCK_M);
            Ring raw(RAW_STAGES), u8(U8_STAGES), acc(ACC_SLOTS);
            uint32_t g = 0;
            for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
                for (int ks = 0; ks < k_stages; ks++, g++) {
                    tc_wait(&raw_full[raw.idx], raw.phase, abort_flag, prm.flag, 0u);
                    tc_wait(&u8_full[u8.idx], u8.phase, abort_flag, prm.flag, 0u);
                    tc_fence_after_sync();
                    const int np = min(STAGE_PAIRS, prm.pairs - ks * STAGE_PAIRS);
                    // A: unpacked weights, no swizzle: element (row r, k) of a block at (k / 16) * 2048 + r * 16 + (k % 16):
                    //    the two K halves 2048 B apart (leading offset), 8-row core matrices 128 B apart (stride offset);
                    //    consecutive blocks of the stage are 4096 B apart.
                    // B: activations, 128-byte swizzled rows of 128 B; block j is the j-th 32-byte slice of the row; 8-row
                    //    groups are 1024 B apart.  The start-address field counts 16-byte units.
                    const uint64_t a_desc0 = umma_smem_desc(smem_u32(u8_base + u8.idx * U8_STAGE_BYTES), 2048, 128, 0);
                    const uint64_t b_desc0 = umma_smem_desc(smem_u32(raw_base + raw.idx * RAW_STAGE_BYTES), 16, 1024, 2);
#pragma unroll
                    for (int pp = 0; pp < STAGE_PAIRS; pp++) {
                        if (pp < np) {
                            tc_wait(&acc_empty[acc.idx], acc.phase ^ 1, abort_flag, prm.flag, 0u);
                            tc_fence_after_sync();
#pragma unroll
                            for (int hi = 0; hi < 2; hi++) {
                                const int j = 2 * pp + hi;
                                umma_i8(tmem_base + acc.idx * SLOT_COLS + hi * BLOCK_M, a_desc0 + static_cast<uint64_t>(j * (U8_BLOCK_BYTES >> 4)),
                                        b_desc0 + static_cast<uint64_t>(j * (32 >> 4)), idesc, 0u);
                            }
                            umma_commit(&acc_full[acc.idx]);
                            acc.advance();
                        }
                    }
                    umma_commit(&stage_done[g % DONE_RING]);   // frees the stage's raw and unpacked buffers (one commit: each costs tensor-pipe time)
                    raw.advance();
                    u8.advance();
                }
            }
            // every MMA issued above has completed before tensor memory is released
            umma_commit(drain_bar);
            mbar_wait_drain(drain_bar, 0u);
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
        uint32_t g = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            for (int ks = 0; ks < k_stages; ks++, g++) {
                tc_wait(&raw_full[raw.idx], raw.phase, abort_flag, prm.flag, 100u);
                if (g >= U8_STAGES) {   // the unpacked slot last held stage g - U8_STAGES
                    const uint32_t h = g - U8_STAGES;
                    tc_wait(&stage_done[h % DONE_RING], (h / DONE_RING) & 1u, abort_flag, prm.flag, 100u);
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
                __syncwarp();
                mbar_arrive_elect(&u8_full[u8.idx]);
                raw.advance();
                u8.advance();
            }
        }
    } else if (warp >= 8) {
        // ------------------------------ epilogue ------------------------------
        // Software pipeline: a pair's accumulator columns are read in items (low block: chunks of CH
        // columns, then the high block's); while the arithmetic of one item runs, the tcgen05.ld of
        // the next item (of this pair or of the next one) is in flight into the other register
        // buffer, so the TMEM round trip and the probe of the accumulator barrier are off the
        // critical path.  The number of items per pair is even, so a given item always uses the
        // same buffer.
        setmaxnreg_inc<EPI_REGS>();
        constexpr int CH = (CW > INKQ_TC_CHUNK) ? INKQ_TC_CHUNK : CW;    // columns per item
        constexpr int NCH = (CW + CH - 1) / CH;
        constexpr int CH_LAST = CW - (NCH - 1) * CH;
        constexpr int ITEMS = 2 * NCH;
        const int quad = warp & 3;             // TMEM lane quadrant this warp may read
        const int cq = (warp - 8) >> 2;        // which quarter of the accumulator columns
        const int row = quad * 32 + lane;      // weight row inside the tile = TMEM lane
        const int nbk = 2 * prm.pairs;
        const int col0 = cq * CW;              // first column of this warp inside the tile
        const uint32_t tmem_warp = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + col0;
        Ring acc(ACC_SLOTS), sc(SC_STAGES);
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
            const int tn = prm.tn0 + tile / prm.tiles_m, tm = tile % prm.tiles_m;
            const int n = tn * TILE_N + row;
            unsigned long long accp[CW / 2];
#pragma unroll
            for (int j = 0; j < CW / 2; j++) accp[j] = 0ull;
            uint32_t rbuf[2][CH];                 // the two item buffers

            // pipeline prologue: first item of the tile's first pair
            tc_wait(&acc_full[acc.idx], acc.phase, abort_flag, prm.flag, 0u);
            tc_fence_after_sync();
            uint32_t taddr_cur = tmem_warp + acc.idx * SLOT_COLS;   // pair being consumed
            uint32_t slot_cur = acc.idx;
            acc.advance();
            tmem_ld_cols<(NCH == 1) ? CH_LAST : CH>(taddr_cur, rbuf[0]);

#pragma unroll 1
            for (int p = 0; p < prm.pairs; p++) {
                const int pj = p & (STAGE_PAIRS - 1);
                if (pj == 0 && !DUMP) tc_wait(&sc_full[sc.idx], sc.phase, abort_flag, prm.flag, 0u);
                const unsigned char *scst = sc_base + sc.idx * SC_STAGE_BYTES;
                const float *sd_lo = reinterpret_cast<const float *>(scst) + (2 * pj) * BLOCK_M + col0;   // d_a of the low block; the high block's follows
                const float *ss_lo = sd_lo + SC_PLANE_BYTES / 4;                                         // s_a likewise
                float4 wsc = make_float4(0.f, 0.f, 0.f, 0.f);
                if (!DUMP) wsc = *reinterpret_cast<const float4 *>(scst + 2 * SC_PLANE_BYTES + (pj * TILE_N + row) * 16);
                const unsigned long long mlo = pack2(wsc.z, wsc.z), mhi = pack2(wsc.w, wsc.w);
                uint32_t taddr_next = taddr_cur, slot_next = slot_cur;
#pragma unroll
                for (int it = 0; it < ITEMS; it++) {   // items of the pair: (low, chunks...), (high, chunks...)
                    const int hi = it / NCH, c = it % NCH;
                    const int cur = it & 1, nxt = cur ^ 1;
                    tmem_ld_wait();   // item `it` has arrived in rbuf[cur]
                    if (it == ITEMS - 1) {
                        // that was the pair's last load: hand the TMEM slot back
                        tc_fence_before_sync();
                        mbar_arrive_elect(&acc_empty[slot_cur]);
                    }
                    // start the load of the item after it into the other buffer
                    if (it + 1 < ITEMS) {
                        const int nhi = (it + 1) / NCH, nc = (it + 1) % NCH;
                        if (nc == NCH - 1) tmem_ld_cols<CH_LAST>(taddr_cur + nhi * BLOCK_M + nc * CH, rbuf[nxt]);
                        else tmem_ld_cols<CH>(taddr_cur + nhi * BLOCK_M + nc * CH, rbuf[nxt]);
                    } else if (p + 1 < prm.pairs) {   // first item of the next pair
                        tc_wait(&acc_full[acc.idx], acc.phase, abort_flag, prm.flag, 0u);
                        tc_fence_after_sync();
                        taddr_next = tmem_warp + acc.idx * SLOT_COLS;
                        slot_next = acc.idx;
                        acc.advance();
                        tmem_ld_cols<(NCH == 1) ? CH_LAST : CH>(taddr_next, rbuf[nxt]);
                    }
                    const uint32_t *raw = rbuf[cur];
                    const int ncols = (c == NCH - 1) ? CH_LAST : CH;
                    if (DUMP) {
                        const int b = 2 * p + hi;
#pragma unroll
                        for (int j = 0; j < CH; j++) {
                            const int m = tm * BLOCK_M + col0 + c * CH + j;
                            if (j < ncols && m < prm.M && n < prm.rows)
                                prm.dots[(static_cast<size_t>(m) * prm.rows + n) * nbk + b] = static_cast<int32_t>(raw[j]);
                        }
                    } else {
                        const float dw = hi ? wsc.y : wsc.x;
                        const unsigned long long dw2 = pack2(dw, dw);
                        const float *sd = sd_lo + hi * BLOCK_M + c * CH;   // d_a of this block, this item's columns
#pragma unroll
                        for (int j4 = 0; j4 < CH; j4 += 4) {
                            if (j4 < ncols) {
                                // 128-bit shared loads straight into 64-bit register pairs: (d_a[m], d_a[m+1]) is already the
                                // packed operand of the f32x2 instructions
                                const ulonglong2 da = *reinterpret_cast<const ulonglong2 *>(sd + j4);
                                const int a0 = (c * CH + j4) / 2;
                                accp[a0] = fma2(cvt2_exact(raw[j4], raw[j4 + 1]), mul2(da.x, dw2), accp[a0]);
                                accp[a0 + 1] = fma2(cvt2_exact(raw[j4 + 2], raw[j4 + 3]), mul2(da.y, dw2), accp[a0 + 1]);
                                if (HAS_MIN && hi) {
                                    const ulonglong2 s0 = *reinterpret_cast<const ulonglong2 *>(ss_lo + c * CH + j4);
                                    const ulonglong2 s1 = *reinterpret_cast<const ulonglong2 *>(ss_lo + BLOCK_M + c * CH + j4);
                                    accp[a0] = fma2(mlo, s0.x, accp[a0]);
                                    accp[a0] = fma2(mhi, s1.x, accp[a0]);
                                    accp[a0 + 1] = fma2(mlo, s0.y, accp[a0 + 1]);
                                    accp[a0 + 1] = fma2(mhi, s1.y, accp[a0 + 1]);
                                }
                            }
                        }
                    }
                }
                taddr_cur = taddr_next;
                slot_cur = slot_next;
                if (!DUMP && (pj == STAGE_PAIRS - 1 || p == prm.pairs - 1)) {
                    // this warp is done with the stage's scales
                    __syncwarp();
                    mbar_arrive_elect(&sc_empty[sc.idx]);
                    sc.advance();
                }
            }
            if (!DUMP && n < prm.rows) {
                float accf[CW];
#pragma unroll
                for (int j = 0; j < CW / 2; j++) unpack2(accp[j], accf[2 * j], accf[2 * j + 1]);
#pragma unroll
                for (int j = 0; j < CW; j++) {
                    const int m = tm * BLOCK_M + col0 + j;
                    if (m < prm.M) prm.C[static_cast<size_t>(m) * prm.ldc + n] = accf[j];
                }
#pragma unroll
                for (int e = 0; e < MAX_PEERS - 1; e++) {   // static indices: the parameter array stays out of local memory
                    if (e < prm.extra.n) {
                        float *__restrict__ Ce = prm.extra.p[e];
#pragma unroll
                        for (int j = 0; j < CW; j++) {
                            const int m = tm * BLOCK_M + col0 + j;
                            if (m < prm.M) Ce[static_cast<size_t>(m) * prm.ldc + n] = accf[j];
                        }
                    }
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

// The opt-in for large dynamic shared memory is a per-device function attribute: remember per device
// (and per instantiation, through the template's own statics) whether it has been set.
constexpr int MAX_DEVICES = 64;

template <int CW, bool HAS_MIN, bool DUMP>
static int launch_one(inkq_ctx *ctx, const CUtensorMap *maps, const TcParams &prm, int grid)
{
    static std::mutex mu;
    static bool configured[MAX_DEVICES] = {};
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return fail(ctx, INKQ_ERR_UNSUPPORTED, "device index beyond the launch table");
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!configured[ctx->device]) {
            cudaFuncAttributes attr;
            cudaError_t e = cudaFuncGetAttributes(&attr, k_qgemm_tc<CW, HAS_MIN, DUMP>);
            if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("cudaFuncGetAttributes(k_qgemm_tc): ") + cudaGetErrorString(e));
            if (attr.numRegs != LAUNCH_REGS)   // the in-kernel register re-balancing is sized for exactly this launch value
                return fail(ctx, INKQ_ERR_UNSUPPORTED, "k_qgemm_tc was compiled to " + std::to_string(attr.numRegs) + " registers per thread, expected " +
                                                           std::to_string(LAUNCH_REGS));
            e = cudaFuncSetAttribute(k_qgemm_tc<CW, HAS_MIN, DUMP>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
            if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("cudaFuncSetAttribute(k_qgemm_tc): ") + cudaGetErrorString(e));
            configured[ctx->device] = true;
        }
    }
    cudaError_t le = launch_pdl(k_qgemm_tc<CW, HAS_MIN, DUMP>, dim3(grid), dim3(TC_THREADS), TC_SMEM_BYTES, ctx->stream, maps[0], maps[1], maps[2], prm);
    if (le != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string("k_qgemm_tc launch: ") + cudaGetErrorString(le));
    return after_launch(ctx, "k_qgemm_tc");
}

template <bool HAS_MIN, bool DUMP>
static int launch_cw(inkq_ctx *ctx, int cw, const CUtensorMap *maps, const TcParams &prm, int grid)
{
    switch (cw) {
        case 4: return launch_one<4, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 8: return launch_one<8, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 12: return launch_one<12, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 16: return launch_one<16, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 20: return launch_one<20, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 24: return launch_one<24, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 28: return launch_one<28, HAS_MIN, DUMP>(ctx, maps, prm, grid);
        case 32: return launch_one<32, HAS_MIN, DUMP>(ctx, maps, prm, grid);
    }
    return fail(ctx, INKQ_ERR_INVALID, "internal: bad column width");
}

static int encode2d(inkq_ctx *ctx, CUtensorMap *map, CUtensorMapDataType dt, int elem_bytes, const void *base, uint64_t dim0, uint64_t dim1,
                    uint32_t box0, uint32_t box1, CUtensorMapSwizzle swz, uint64_t pitch_elems = 0)
{
    const cuuint64_t gdim[2] = {dim0, dim1};
    const cuuint64_t gstride[1] = {(pitch_elems ? pitch_elems : dim0) * static_cast<uint64_t>(elem_bytes)};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1u, 1u};
    CUresult cr = reinterpret_cast<EncodeTiledFn>(ctx->encode_tiled)(map, dt, 2, const_cast<void *>(base), gdim, gstride, box, estr,
                                                                     CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                                                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) return fail(ctx, INKQ_ERR_CUDA, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(cr)));
    return INKQ_OK;
}

// Relative cost of one tile by its width block_m = 16 * index (any common factor cancels; measured on a B200 with
// one tile per SM at K = 4096: 32.2, 35.4, 39.3, 45.7, 51.7, 58.4, 66.0, 76.6 us): narrow tiles are bounded by the chain of
// K=32 MMAs and their commits, wide ones by the epilogue arithmetic.  The ratios hardly depend on K (both terms are per block).
static const float tile_cost[9] = {0.f, 1.00f, 1.10f, 1.22f, 1.42f, 1.61f, 1.81f, 2.05f, 2.38f};

int launch_gemm_tc(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, int ldc, int32_t *dots, const ExtraDst *extra, int tn_begin, int tn_count,
                   int m_begin, int m_count)
{
    if (tn_count < 0) tn_count = w->tiles - tn_begin;   // default: every tile from tn_begin on
    if (m_count < 0) m_count = a->M - m_begin;          // default: every row from m_begin on
    if (m_begin < 0 || (m_begin & 3) != 0 || m_count < 1 || m_begin + m_count > a->M || (m_begin != 0 && dots != nullptr))
        return fail(ctx, INKQ_ERR_INVALID, "bad activation row window");
    if (ctx->encode_tiled == nullptr) return fail(ctx, INKQ_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled entry point not available");
    if (w->sc32 == nullptr) return fail(ctx, INKQ_ERR_INVALID, "this weight holds no fp32 scale records (weight-only layers use inkq_gemm_w41_f16act)");
    const int M = m_count;
    // Split of the M activation rows into tiles of block_m columns (a multiple of 16, at most 128).  With few
    // weight tiles (a shard of a column-sharded layer) narrower tiles fill more SMs; the choice minimises
    // waves x tile cost.  It depends on the shapes and the SM count only, and every choice gives the same bits
    // (the per-output operation order never changes).
    int tiles_m = (M + 127) / 128, block_m = 128;
    {
        float best = 0.f;
        for (int tm = (M + 127) / 128; tm <= (M + 15) / 16; tm++) {
            const int bm = (((M + tm - 1) / tm) + 15) & ~15;
            const long long total = static_cast<long long>(tn_count) * tm;
            const float cost = static_cast<float>((total + ctx->num_sms - 1) / ctx->num_sms) * tile_cost[bm / 16];
            if (best == 0.f || cost < best * 0.999f) {
                best = cost;
                tiles_m = tm;
                block_m = bm;
            }
            if (total > 64LL * ctx->num_sms) break;   // many waves already: finer splits only add padding
        }
    }
    const int nb = a->K / QK;

    CUtensorMap maps[3];
    // a row window starts m_begin rows into q and m_begin entries into every block's line of the planes
    int rc = encode2d(ctx, &maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->q + static_cast<size_t>(m_begin) * a->K, a->K, M, 128u, block_m,
                      CU_TENSOR_MAP_SWIZZLE_128B);
    if (!rc) rc = encode2d(ctx, &maps[1], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->d + m_begin, a->M_ld - m_begin, nb, block_m, STAGE_BLOCKS,
                           CU_TENSOR_MAP_SWIZZLE_NONE, a->M_ld);
    if (!rc) rc = encode2d(ctx, &maps[2], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a->s + m_begin, a->M_ld - m_begin, nb, block_m, STAGE_BLOCKS,
                           CU_TENSOR_MAP_SWIZZLE_NONE, a->M_ld);
    if (rc) return rc;

    TcParams prm;
    prm.nibT = w->nibT;
    prm.sc32 = w->sc32;
    prm.zpT = w->zpT;
    const size_t c_off = static_cast<size_t>(m_begin) * ldc;
    prm.C = (C != nullptr) ? C + c_off : nullptr;
    prm.extra = ExtraDst{};
    if (extra != nullptr) {
        prm.extra = *extra;
        for (int e = 0; e < prm.extra.n; e++) prm.extra.p[e] += c_off;
    }
    prm.dots = dots;
    prm.flag = ctx->dev_flag;
    prm.M = M;
    prm.rows = w->rows;
    prm.pairs = w->pairs;
    prm.tn0 = tn_begin;
    prm.tiles_n = tn_count;
    prm.tiles_m = tiles_m;
    prm.ldc = ldc;
    const int total = prm.tiles_n * prm.tiles_m;
    const int grid = total < ctx->num_sms ? total : ctx->num_sms;
    if (dots != nullptr) return launch_cw<false, true>(ctx, block_m / 4, maps, prm, grid);
    if (w->scheme == INKQ_A81W41) return launch_cw<true, false>(ctx, block_m / 4, maps, prm, grid);
    return launch_cw<false, false>(ctx, block_m / 4, maps, prm, grid);
}

}  // namespace inkq
