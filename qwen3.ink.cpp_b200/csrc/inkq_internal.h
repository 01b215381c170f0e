// Internal definitions shared by the .cu files: handle structs, device layouts,
// error plumbing.  Nothing here is part of the public ABI (see include/inkq.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <string>

#include "inkq.h"

namespace inkq {

constexpr int QK = 32;       // quantization block (reference: QK, qwen3/include/qwen/QwenConfig.h:8)
constexpr int TILE_N = 128;  // weight rows per device tile (one UMMA M=128 operand)

// ---------------------------------------------------------------------------
// Device layouts
//
// Weights of one layer (rows R = n_end - n_begin, T = ceil(R/128) tiles, P = K/64 pairs):
//   nibT  u8     [T][P][128][32]   row r of a tile holds the layer's 32 disk bytes of pair p
//                                  (low nibble = element e of block 2p, high nibble = element e
//                                  of block 2p+1); its two 16-byte chunks are stored at chunk
//                                  position c ^ ((r >> 2) & 1) so that 8 consecutive rows read
//                                  the same logical chunk from 8 distinct bank groups.
//   sc32  float4 [T][P][128]       {d_lo, d_hi, m_lo, m_hi}, only when scales are kept in fp32
//   sc16  half x4[T][P][128]       the same rounded to fp16 (always present)
//   zpT   u8 x2  [T][P][128]       {z_lo, z_hi}: 0 (Q4_1), 8 (Q4_0) or the block zero point
// Rows beyond R inside the last tile hold zero nibbles, zero scales, zero z.
// One (tile, pair) is 4096 contiguous bytes of nibbles: a pipeline stage is one
// untiled bulk copy.
//
// Quantized activations (M rows, NB = K/32 blocks, M_ld = round_up(M, 4)):
//   q     s8  [M][K]      row-major (K-major operand for the MMA, TMA-tiled with 128B swizzle)
//   d, s  f32 [NB][M_ld]  block scale and scaled block sum, block-major so that one
//                         tile's columns of one block are contiguous
//   isum  s32 [NB][M_ld]  integer block sums of q
// ---------------------------------------------------------------------------
__host__ __device__ inline size_t nib_offset(int P, int t, int p, int r, int chunk)
{
    return ((static_cast<size_t>(t) * P + p) * TILE_N + r) * 32 + static_cast<size_t>((chunk ^ ((r >> 2) & 1)) * 16);
}

struct Weight {
    inkq_ctx *ctx;
    int scheme, scale_mode;
    int rows, K, tiles, pairs;
    uint8_t *nibT;
    float4 *sc32;   // may be null
    uint2 *sc16;    // 4 x fp16
    uchar2 *zpT;
    size_t bytes;
};

struct Act {
    inkq_ctx *ctx;
    int max_rows, K;
    int M, M_ld, qmode;  // of the last quantize call
    int8_t *q;
    float *d, *s;
    int32_t *isum;
    // Pending RMS scale (decode step only, inkq_glue_decode_gemv epilogue 4): the row was quantized as x * g WITHOUT
    // the factor 1 / sqrt(mean(x^2) + eps), and ssq[0 .. ssq_parts) holds the sums of squares of its 32-element groups;
    // the consuming matrix-vector product derives the factor from them and applies it to its finished sums.
    // ssq_parts == 0: nothing pending (every other producer resets it).
    float *ssq = nullptr;
    int ssq_parts = 0, norm_n = 0;
    float norm_eps = 0.0f;
};
constexpr int ACT_SSQ_CAP = 512;   // groups of 32: rows of up to 16384 values

// Further destinations of an output matrix: the same element offset is stored through every pointer
// (other GPUs' mapped buffers of a column-sharded layer, or other local buffers).
constexpr int MAX_PEERS = 8;
struct ExtraDst {
    float *p[MAX_PEERS - 1];
    int n;
};

struct PeerSet {
    inkq_ctx *ctx;
    int world, rank;
    size_t bytes;
    char *ptr[MAX_PEERS];    // every rank's buffer as mapped into this process (ptr[rank] = the local one)
    void *opened[MAX_PEERS]; // base addresses returned by cudaIpcOpenMemHandle (null for local / caller-mapped)
};

struct F16W {
    inkq_ctx *ctx;
    int rows, K;
    uint16_t *w;
    size_t bytes;
};

}  // namespace inkq

struct inkq_ctx {
    int device;
    cudaStream_t stream;
    std::string err;
    uint64_t launches;
    int num_sms;
    int *dev_flag;        // device word set by a kernel whose bounded wait ran out (word 0), a ticket counter behind it
    int *host_flag;       // page-locked host word the flag is copied to at the end of the stream in inkq_ctx_synchronize
    inkq::Act *scratch_act;  // activation scratch of inkq_linear (grown on demand)
    size_t scratch_elems;    // its capacity in activation elements (M * K)
    size_t scratch_planes;   // capacity of each of its per-block planes, in entries
    float *lin_x, *lin_c;    // device staging of inkq_linear_host
    size_t lin_x_cap, lin_c_cap;
    float *pin_x, *pin_c;    // pinned host staging of inkq_linear_host
    size_t pin_x_cap, pin_c_cap;
    uint16_t *f16_x;         // fp16 (hi, lo) form of the activations of inkq_f16w_matmul's tensor-core path (grown on demand)
    size_t f16_x_cap;        // in halves
    float *f16_scale;        // its per-row power-of-two factors
    size_t f16_scale_cap;
    void *encode_tiled;      // cuTensorMapEncodeTiled entry point
    cudaStream_t copy_stream;   // inkq_linear_host: device-to-host copies of finished row chunks (created on first use)
    cudaStream_t h2d_stream;    // inkq_linear_host: host-to-device copies of the row chunks
    cudaEvent_t chunk_ev[8], h2d_ev[8], start_ev;
};
// dev_flag points to four 4-byte words: [0] time-out flag, [1] ticket counter of the decode GEMV's last-CTA epilogue
namespace inkq {
constexpr size_t CTX_FLAG_WORDS = 4;
}
struct inkq_weight : inkq::Weight {};
struct inkq_act : inkq::Act {};
struct inkq_f16w : inkq::F16W {};
struct inkq_peerset : inkq::PeerSet {};

namespace inkq {

void set_global_error(const std::string &msg);
int fail(inkq_ctx *ctx, int code, const std::string &msg);

#define INKQ_CUDA(ctx, call)                                                                         \
    do {                                                                                             \
        cudaError_t e__ = (call);                                                                    \
        if (e__ != cudaSuccess)                                                                      \
            return ::inkq::fail((ctx), INKQ_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
    } while (0)

#define INKQ_REQUIRE(ctx, cond, msg)                                            \
    do {                                                                        \
        if (!(cond)) return ::inkq::fail((ctx), INKQ_ERR_INVALID, (msg));       \
    } while (0)

// Launch with programmatic stream serialization: the grid may be scheduled while its predecessor in the stream is
// still running; the kernel must execute griddepcontrol.wait before it touches anything the predecessor writes
// (everything before that instruction overlaps the predecessor's tail).
template <typename... KArgs, typename... Args>
static inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Checks the launch, counts it.
int after_launch(inkq_ctx *ctx, const char *what);

// kernels' host launchers (defined in the respective .cu files)
int launch_quantize(inkq_ctx *ctx, int qmode, const float *x, int M, int K, Act *a);
struct QuantOut;
// prompt attention on the tensor cores (attention_prefill_mma.cu); out and / or qo.q receive the result
int launch_attention_prefill_mma(inkq_ctx *ctx, const float *q, const uint16_t *k_cache, const uint16_t *v_cache, const int *pos0_dev, int T, int nq,
                                 int nkv, int max_pos, float scale, float *out, const QuantOut &qo, int qrow0);
int launch_quantize_rows(inkq_ctx *ctx, int qmode, const float *x, int m0, int rows, int M_total, int K, Act *a);
// gu [M][2K] in (32 gate, 32 up) column groups -> the quantized rows of SiLU(gate) * up
int launch_silu_mul_quantize(inkq_ctx *ctx, int qmode, const float *gu, int M, int K, Act *a);
int launch_block_isum(inkq_ctx *ctx, Act *a, int M, int M_ld);
int launch_retile(inkq_ctx *ctx, Weight *w, const uint8_t *nib, const float *d, const float *m, const uint8_t *zp, int n_begin);
int launch_export(inkq_ctx *ctx, const Weight *w, uint8_t *nib, float *d, float *m, uint8_t *zp);
int launch_gemv(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, const ExtraDst *extra = nullptr);
// decode QGEMV that builds its quantized activation row itself: pro 0 = x as is, 1 = RMSNorm(x; g, eps), 2 = SiLU(x[0..K)) * x[K..2K)
int launch_gemv_fused(inkq_ctx *ctx, const Weight *w, const float *x, int pro, const float *g, float eps, float *C, int accumulate);
int launch_gemm_simt(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, int ldc);
int launch_block_dots(inkq_ctx *ctx, const Act *a, const Weight *w, int32_t *dots);
// tn_begin / tn_count: the launch covers the weight tiles (of 128 rows) tn_begin .. tn_begin + tn_count - 1 (default: all)
// tn_begin / tn_count: a range of the weight's 128-row tiles; m_begin / m_count: a window of the activation rows (m_begin a
// multiple of 4; C and the extra destinations still point at row 0)
int launch_gemm_tc(inkq_ctx *ctx, const Act *a, const Weight *w, float *C, int ldc, int32_t *dots, const ExtraDst *extra = nullptr,
                   int tn_begin = 0, int tn_count = -1, int m_begin = 0, int m_count = -1);
int launch_gemm_w41_f16(inkq_ctx *ctx, const uint16_t *a16, int M, const Weight *w, float *C, int ldc);   // CUDA cores
int launch_gemm_w41_tc(inkq_ctx *ctx, const uint16_t *a16, int M, const Weight *w, float *C, int ldc);    // tcgen05 kind::f16
int launch_gemv_w41(inkq_ctx *ctx, const uint16_t *a16, const Weight *w, float *C);                        // M == 1, bandwidth-bound
// inkq_linear with further destinations for every output element (defined in inkq_api.cu)
int linear_impl(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, float *C_dev, int ldc, const ExtraDst *extra);
int launch_f16w_matmul(inkq_ctx *ctx, const F16W *w, const float *x, int M, float *C, int ldc, const ExtraDst *extra = nullptr);   // CUDA cores (bandwidth-bound, M small)
// inkq_f16w_matmul_prec with further destinations for every output element (defined in inkq_api.cu)
int f16w_matmul_impl(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc, int precision, const ExtraDst *extra);
// tensor cores, M >= 16; passes 2: activations as fp16 hi + lo (22 significant bits), 1: hi only
int launch_f16w_gemm_tc(inkq_ctx *ctx, const F16W *w, const float *x, int M, float *C, int ldc, int passes, uint16_t *x16, float *row_scale,
                        const ExtraDst *extra = nullptr);

}  // namespace inkq
