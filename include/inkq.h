/*
 * inkq.h - C ABI of the B200 (sm_100a) A8W4 quantized-matmul path.
 *
 * This is the one boundary between host code (the C++ linear layer that mirrors
 * Qwen3.Ink.Cpp's Qwen_Linear_with_bias_Int4, a test driver, a model runtime) and
 * the CUDA kernels.  Plain pointers and sizes only.  Every entry point returns an
 * inkq_status (0 = ok), never throws and never aborts; inkq_last_error() gives
 * the message of the last failure.  There is no CPU fallback: without a CUDA
 * device inkq_ctx_create() fails.
 *
 * Each declaration cites the reference interface it stands in for, as
 * file:line inside the reference project.
 *
 * Logical ("on-disk") weight format accepted by inkq_weight_create, exactly what
 * the reference linear layer loads (qwen3/include/qwen/QwenOperator.h:128-140):
 *   nib  u8  [N][K/2]  byte[32g+e] = q[64g+e] | q[64g+32+e] << 4   (AWQ interleave)
 *   d    f32 [N][K/32] block scales
 *   m    f32 [N][K/32] block mins        (A81W41 / W41; NULL otherwise)
 *   zp   u8  [N][K/32] block zero points (A80W4Z; NULL otherwise)
 * N % 8 == 0 and K % 64 == 0, as the reference requires
 * (qwen3/src/qwen/quantized_gemx_kernels.cc:359-361).
 */
#ifndef INKQ_H
#define INKQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    INKQ_OK = 0,
    INKQ_ERR_INVALID = 1,     /* bad argument (shape, null pointer, handle) */
    INKQ_ERR_CUDA = 2,        /* a CUDA runtime/driver call failed */
    INKQ_ERR_ALLOC = 3,       /* device or host allocation failed */
    INKQ_ERR_UNSUPPORTED = 4, /* valid request this build cannot serve */
    INKQ_ERR_TIMEOUT = 5      /* a bounded device-side wait ran out; the context stays usable */
} inkq_status;

/* Quantization schemes (reference: enum LinearKernelType, qwen3/include/qwen/QwenConfig.h:13). */
typedef enum {
    INKQ_A81W41 = 0, /* Q8_1 activations x Q4_1 weights: sum_b d_a*d_w*I + m_w*s_a */
    INKQ_A80W40 = 1, /* Q8_0 activations x Q4_0 weights (q-8) */
    INKQ_A80W4Z = 2, /* Q8_0 activations x zero-point int4 weights (q-zp) */
    INKQ_W41 = 3     /* weight-only Q4_1, fp16 activations, fp32 accumulate */
} inkq_scheme;

/* Activation quantizer variants. */
typedef enum {
    INKQ_Q8_0_F16 = 0, /* quantize_row_q8_0_repack        quantized_gemx_kernels.cc:584-691 */
    INKQ_Q8_1_F16 = 1, /* quantize_row_q8_1_repack_fp16   quantized_gemx_kernels.cc:693-801 */
    INKQ_Q8_1_F32 = 2  /* quantize_row_q8_1_repack_fp32   quantized_gemx_kernels.cc:803-911 */
} inkq_qmode;

/* How a weight's block scales are held on the device. */
typedef enum {
    INKQ_SCALES_F32 = 0, /* as given (what gemm_repack_A81W41_fp32 sees; repack_w81_weight_fp32, QwenOperator.cc:852-892) */
    INKQ_SCALES_F16 = 1  /* rounded to fp16 (what the three fp16 kernels see; repack_w81_weight_fp16 / repack_w80_weight, QwenOperator.cc:757-850) */
} inkq_scale_mode;

typedef struct inkq_ctx inkq_ctx;       /* device, stream, scratch; stands in for ModelContext, QwenOperator.h:34-43 */
typedef struct inkq_weight inkq_weight; /* one linear layer's re-tiled weights; stands in for weight_repack_fp16/_fp32, QwenOperator.h:102-103 */
typedef struct inkq_act inkq_act;       /* quantized activations; stands in for ModelContext::activation_buffer */
typedef struct inkq_f16w inkq_f16w;     /* fp16 weight matrix (lm_head) */

/* ---- context ------------------------------------------------------------ */
/* stream: a cudaStream_t cast to void*, or NULL for the default stream. */
int inkq_ctx_create(int device, void *stream, inkq_ctx **out);
int inkq_ctx_destroy(inkq_ctx *ctx);
int inkq_ctx_set_stream(inkq_ctx *ctx, void *stream);
int inkq_ctx_synchronize(inkq_ctx *ctx);
/* Message of the last error on this context (or of the last context-less error when ctx is NULL). */
const char *inkq_last_error(const inkq_ctx *ctx);
/* Number of kernels this library has launched on the context since creation. */
uint64_t inkq_launch_count(const inkq_ctx *ctx);

/* ---- load-time weight re-tiling ------------------------------------------
 * Replaces repack_w80_weight / repack_w81_weight_fp16 / repack_w81_weight_fp32
 * (qwen3/include/qwen/QwenOperator.h:82-84; QwenOperator.cc:757-892) and the
 * constructor's load (QwenOperator.h:112-157).  Host pointers in the logical
 * format; rows [n_begin, n_end) are uploaded and re-tiled on the device into the
 * 128-row, chunk-swizzled sm_100a layout (n_begin = 0, n_end = N for the whole
 * matrix; a sub-range is one tensor-parallel column shard).  *_dev takes device
 * pointers instead. */
int inkq_weight_create(inkq_ctx *ctx, int scheme, int scale_mode, int N, int K,
                       const uint8_t *nib, const float *d, const float *m, const uint8_t *zp,
                       int n_begin, int n_end, inkq_weight **out);
int inkq_weight_create_dev(inkq_ctx *ctx, int scheme, int scale_mode, int N, int K,
                           const uint8_t *nib_dev, const float *d_dev, const float *m_dev, const uint8_t *zp_dev,
                           int n_begin, int n_end, inkq_weight **out);
int inkq_weight_destroy(inkq_weight *w);
/* rows = n_end - n_begin, device bytes held. */
int inkq_weight_info(const inkq_weight *w, int *rows, int *K, int *scheme, size_t *device_bytes);
/* Inverse of the re-tiling, for round-trip checks: writes the logical format of
 * the held rows to host buffers (any of the outputs may be NULL). d/m come back as
 * the values the kernels see (fp16-rounded when scale_mode is F16). */
int inkq_weight_export(inkq_ctx *ctx, const inkq_weight *w, uint8_t *nib, float *d, float *m, uint8_t *zp);

/* ---- offline weight quantizers -----------------------------------------------
 * fp32 weights [N][K] on the device -> the on-disk format inkq_weight_create takes
 * (nibbles u8 [N][K/2] AWQ-interleaved, scales and minima f32 [N][K/32], zero points
 * i8 [N][K/32], may be NULL), all on the device.  format 0: Q4_0, 1: Q4_1.
 * Replaces quantize_row_q40_tinyml / quantize_row_q41_tinyml
 * (notebooks/quantize_methods.py:13-66, :68-125), bit for bit. */
int inkq_weight_quantize_dev(inkq_ctx *ctx, int format, int N, int K, const float *w_dev, uint8_t *nib_dev, float *d_dev, float *m_dev,
                             int8_t *zp_dev);

/* ---- activation quantizer -------------------------------------------------
 * Replaces quantize_row_q8_0_repack / quantize_row_q8_1_repack_fp16 / _fp32
 * (QwenOperator.h:276-278).  x_dev: fp32 [M][K] on the device. */
int inkq_act_create(inkq_ctx *ctx, int max_rows, int K, inkq_act **out);
int inkq_act_destroy(inkq_act *a);
int inkq_quantize(inkq_ctx *ctx, int qmode, const float *x_dev, int M, int K, inkq_act *act);
/* Copies the quantized form to host: q s8 [M][K], d f32 [M][K/32], s f32 [M][K/32]
 * (s = 0 for Q8_0), isum s32 [M][K/32] (block sums of q).  Any output may be NULL. */
int inkq_act_export(inkq_ctx *ctx, const inkq_act *act, int8_t *q, float *d, float *s, int32_t *isum);

/* inkq_quantize with x in host memory (copied to the device inside the call). */
int inkq_quantize_host(inkq_ctx *ctx, int qmode, const float *x_host, int M, int K, inkq_act *act);
/* Uploads an already quantized activation matrix (host arrays: q s8 [M][K], d f32 [M][K/32],
 * s f32 [M][K/32] or NULL for Q8_0) into the handle, as if inkq_quantize had produced it.  Used
 * by the reference-named host entry points, whose callers hand over the reference's own
 * quantized structs (q8_repack_1x2_fp16/_fp32, QwenOperator.h:56-80). */
int inkq_act_import(inkq_ctx *ctx, inkq_act *act, int qmode, int M, const int8_t *q, const float *d, const float *s);

/* ---- matmuls ---------------------------------------------------------------
 * inkq_gemm  : tcgen05 int8 tensor-core path, any M >= 1. Replaces
 *              gemm_repack_A81W41_fp32 / gemm_repack_A80W40 (QwenOperator.h:280-298).
 * inkq_gemv  : bandwidth path, M == 1. Replaces gemv_repack_A81W41_fp16 /
 *              gemv_repack_A80W40 (QwenOperator.h:286-304).
 * inkq_gemm_simt : plain CUDA-core path kept as an on-device cross-check of the
 *              tensor-core kernel (same layouts, same per-output operation order).
 * C_dev: fp32 [M][ldc] on the device; columns [0, rows) of each row are written. */
int inkq_gemm(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev, int ldc);
int inkq_gemv(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev);
int inkq_gemm_simt(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev, int ldc);
/* inkq_gemm / inkq_gemv with the result delivered to host memory (C_host fp32 [M][ldc]); the
 * call returns when the copy is complete.  These are what the reference-named host functions
 * gemm_repack_* / gemv_repack_* (QwenOperator.h:280-304) are built on. */
int inkq_gemm_host(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_host, int ldc);
int inkq_gemv_host(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_host);
/* Every int32 block dot, dots_dev s32 [M][rows][K/32]; for bit-exactness checks. */
int inkq_debug_block_dots(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, int32_t *dots_dev);
/* As inkq_debug_block_dots but produced by the tensor-core kernel's own MMA path. */
int inkq_debug_block_dots_tc(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, int32_t *dots_dev);

/* ---- the linear layer's forward ---------------------------------------------
 * Replaces Qwen_Linear_with_bias_Int4::forward (QwenOperator.h:224,
 * QwenOperator.cc:80-124): quantize, then M > 1 -> QGEMM, M == 1 -> QGEMV.  As
 * in the reference, an A81W41 layer quantizes with Q8_1/fp32 scales for M > 1
 * and Q8_1/fp16 scales for M == 1; A80 schemes use Q8_0/fp16.
 * inkq_linear       : x and C on the device (uses the context's activation scratch).
 * inkq_linear_host  : x and C in host memory; the copies are part of the call. */
int inkq_linear(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, float *C_dev, int ldc);
int inkq_linear_host(inkq_ctx *ctx, const inkq_weight *w, const float *x_host, int M, float *C_host, int ldc);

/* ---- decode forward without any allocation ---------------------------------------
 * No counterpart in the reference.  For hosts that may not call cudaMalloc while
 * serving (a latency-bound decode loop, a process whose device heap belongs to
 * another allocator): the M == 1 forward of inkq_linear with its scratch - one
 * quantized activation row - in a fixed 40 KiB device array inside the library
 * instead of the context's growable buffer.  K <= 16384, else INKQ_ERR_UNSUPPORTED.
 * The first call on a device resolves the array's address; make it before any
 * stream capture.  All calls on a device share the array: calls that overlap on
 * the GPU race, order them.  Never allocates or frees device memory. */
int inkq_linear_m1_static(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, float *C_dev);

/* ---- column-sharded layer with the exchange step inside the matmul ------------------
 * No counterpart in the reference (one process, CPU threads; its kernels parallelise
 * over 8-column groups, qwen3/src/qwen/quantized_gemx_kernels.cc:364-365, which is the
 * independence this sharding uses).  Rank r of P holds the weight rows [r*N/P, (r+1)*N/P)
 * (inkq_weight_create with that range); inkq_linear_scatter runs the forward of
 * inkq_linear and stores every output element into the buffer of EVERY rank of a peer
 * set at the same byte offset, straight from the kernel's epilogue over NVLink;
 * inkq_peer_barrier then tells every peer that this rank's stores are complete and waits
 * for the same from each of them (bounded: after timeout_ms the kernel gives up and the
 * next inkq_ctx_synchronize returns INKQ_ERR_TIMEOUT).  After the barrier every rank
 * holds the full [M][N] matrix; no collective library call is involved.
 *
 * A peer set is world <= 8 device buffers of equal size, one per rank, 256-byte aligned.
 * Their first INKQ_PEER_RESERVED_BYTES belong to the barrier and must be zero when the set
 * is made.  With one process per GPU: inkq_peer_export writes an INKQ_PEER_HANDLE_BYTES
 * blob for the local buffer (CUDA IPC; the buffer must come from cudaMalloc, directly or
 * through a caching allocator that does not use virtual-memory segments), the host
 * gathers all ranks' blobs in rank order and inkq_peerset_open maps them.  With one
 * process for all GPUs (peer access enabled) or several buffers on one GPU:
 * inkq_peerset_from_pointers.  Use two offsets alternately when steps follow each other
 * without any other synchronisation: a rank may start step i+1 while a peer still reads
 * the result of step i. */
#define INKQ_PEER_RESERVED_BYTES 256
#define INKQ_PEER_HANDLE_BYTES 80
typedef struct inkq_peerset inkq_peerset;
int inkq_peer_export(inkq_ctx *ctx, void *dev_ptr, size_t bytes, void *blob_out);
int inkq_peerset_open(inkq_ctx *ctx, int world, int rank, void *local_ptr, const void *blobs, inkq_peerset **out);
int inkq_peerset_from_pointers(inkq_ctx *ctx, int world, int rank, void *const *ptrs, size_t bytes, inkq_peerset **out);
int inkq_peerset_destroy(inkq_peerset *ps);
int inkq_linear_scatter(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, inkq_peerset *ps, size_t byte_offset, int ldc);
/* inkq_gemm (rows already quantized into `act`, M > 1) with the same multi-destination epilogue. */
int inkq_gemm_scatter(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, inkq_peerset *ps, size_t byte_offset, int ldc);
int inkq_peer_barrier(inkq_ctx *ctx, inkq_peerset *ps, int timeout_ms);
/* inkq_f16w_matmul_prec of a row shard of the fp16 matrix (inkq_f16w_create with [n_begin, n_end)), the output columns
 * stored into every rank's buffer like inkq_linear_scatter (lm_head of QwenForCausalLM.cc:43-46, column-sharded). */
int inkq_f16w_matmul_scatter(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, inkq_peerset *ps, size_t byte_offset, int ldc, int precision);

/* ---- weight-only W41 (fp16 activations) and fp16 lm_head ---------------------
 * No C++ kernel exists in the reference for these two; they follow
 * notebooks/evaluate-qwen3_8b_W4.ipynb cell 13 and, for lm_head, the fp32 GEMV
 * gemv_fp32_rcr_mt_impl_1 (qwen3/src/qwen/fp32_gemx_kernels_rcr.cc:494-507). */
int inkq_gemm_w41_f16act(inkq_ctx *ctx, const uint16_t *a16_dev, int M, const inkq_weight *w, float *C_dev, int ldc);
/* The same matmul on the CUDA cores, k ascending (cross-check of the tensor-core kernel above; slow). */
int inkq_gemm_w41_f16act_simt(inkq_ctx *ctx, const uint16_t *a16_dev, int M, const inkq_weight *w, float *C_dev, int ldc);
int inkq_f16w_create(inkq_ctx *ctx, int N, int K, const uint16_t *w16_host, int n_begin, int n_end, inkq_f16w **out);
int inkq_f16w_create_dev(inkq_ctx *ctx, int N, int K, const uint16_t *w16_dev, int n_begin, int n_end, inkq_f16w **out);
int inkq_f16w_destroy(inkq_f16w *w);
/* C[m][n] = sum_k x[m][k] * w[n][k].  M < 16: bandwidth-bound CUDA-core kernel, fp32 activations, exact products.
 * M >= 16 (and K % 64 == 0): tensor cores; the fp32 activations enter as fp16 hi + lo parts (22 significant bits, the
 * K loop runs over both; result within ~1e-5 of the output's rms of an fp32 evaluation) or, with INKQ_F16W_ACT_FP16,
 * as one fp16 value (half the work; each activation rounded with relative error <= 2^-11, about 1e-3 of the
 * output's rms).  inkq_f16w_matmul = INKQ_F16W_ACT_FP32. */
typedef enum { INKQ_F16W_ACT_FP32 = 0, INKQ_F16W_ACT_FP16 = 1 } inkq_f16w_precision;
int inkq_f16w_matmul(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc);
int inkq_f16w_matmul_prec(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc, int precision);

#ifdef __cplusplus
}
#endif
#endif /* INKQ_H */
