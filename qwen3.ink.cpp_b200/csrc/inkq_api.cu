// The C ABI (include/inkq.h): contexts, handles, argument validation, dispatch.
// All device work is launched on the context's stream; nothing here computes on
// the CPU.  Errors are returned as status codes with a message, never thrown.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>
#include <new>
#include <vector>

#include "inkq_internal.h"

namespace inkq {

static std::mutex g_err_mu;
static std::string g_err;

void set_global_error(const std::string &msg)
{
    std::lock_guard<std::mutex> lk(g_err_mu);
    g_err = msg;
}

int fail(inkq_ctx *ctx, int code, const std::string &msg)
{
    if (ctx != nullptr) ctx->err = msg;
    set_global_error(msg);
    return code;
}

int after_launch(inkq_ctx *ctx, const char *what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ctx, INKQ_ERR_CUDA, std::string(what) + " launch: " + cudaGetErrorString(e));
    ctx->launches++;
    return INKQ_OK;
}

static int use(inkq_ctx *ctx)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    return INKQ_OK;
}

template <typename T>
static int dev_alloc(inkq_ctx *ctx, T **p, size_t count)
{
    *p = nullptr;
    if (count == 0) return INKQ_OK;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(p), count * sizeof(T));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, INKQ_ERR_ALLOC, std::string("cudaMalloc of ") + std::to_string(count * sizeof(T)) + " bytes: " + cudaGetErrorString(e));
    }
    return INKQ_OK;
}

static void free_weight(Weight *w)
{
    cudaFree(w->nibT);
    cudaFree(w->sc32);
    cudaFree(w->sc16);
    cudaFree(w->zpT);
}

static void free_act(Act *a)
{
    cudaFree(a->q);
    cudaFree(a->d);
    cudaFree(a->s);
    cudaFree(a->isum);
    cudaFree(a->ssq);
}

static int check_weight_args(inkq_ctx *ctx, int scheme, int scale_mode, int N, int K, const void *nib, const void *d, const void *m,
                             const void *zp, int n_begin, int n_end)
{
    INKQ_REQUIRE(ctx, scheme >= INKQ_A81W41 && scheme <= INKQ_W41, "unknown scheme");
    INKQ_REQUIRE(ctx, scale_mode == INKQ_SCALES_F32 || scale_mode == INKQ_SCALES_F16, "unknown scale mode");
    INKQ_REQUIRE(ctx, N > 0 && K > 0, "N and K must be positive");
    INKQ_REQUIRE(ctx, K % 64 == 0, "K must be a multiple of 64 (two 32-element blocks per nibble pair)");
    INKQ_REQUIRE(ctx, N % 8 == 0, "N must be a multiple of 8");
    INKQ_REQUIRE(ctx, 0 <= n_begin && n_begin < n_end && n_end <= N, "row range [n_begin, n_end) out of bounds");
    INKQ_REQUIRE(ctx, nib != nullptr && d != nullptr, "nibbles and scales are required");
    INKQ_REQUIRE(ctx, (scheme != INKQ_A81W41 && scheme != INKQ_W41) || m != nullptr, "block mins are required for Q4_1 weights");
    INKQ_REQUIRE(ctx, scheme != INKQ_A80W4Z || zp != nullptr, "zero points are required for A80W4Z");
    return INKQ_OK;
}

static int build_weight(inkq_ctx *ctx, int scheme, int scale_mode, int K, const uint8_t *nib_dev, const float *d_dev, const float *m_dev,
                        const uint8_t *zp_dev, int n_begin, int n_end, inkq_weight **out)
{
    inkq_weight *w = new (std::nothrow) inkq_weight();
    if (w == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
    w->ctx = ctx;
    w->scheme = scheme;
    w->scale_mode = scale_mode;
    w->rows = n_end - n_begin;
    w->K = K;
    w->tiles = (w->rows + TILE_N - 1) / TILE_N;
    w->pairs = K / 64;
    w->nibT = nullptr;
    w->sc32 = nullptr;
    w->sc16 = nullptr;
    w->zpT = nullptr;
    const size_t recs = static_cast<size_t>(w->tiles) * w->pairs * TILE_N;
    int rc = dev_alloc(ctx, &w->nibT, recs * 32);
    if (!rc) rc = dev_alloc(ctx, &w->sc16, recs);
    if (!rc) rc = dev_alloc(ctx, &w->zpT, recs);
    const bool want32 = scheme != INKQ_W41;   // fp32 scale records for the prefill QGEMM (the weight-only kernel reads fp16)
    if (!rc && want32) rc = dev_alloc(ctx, &w->sc32, recs);
    w->bytes = recs * (32 + 8 + 2 + (want32 ? 16 : 0));
    if (!rc) rc = launch_retile(ctx, w, nib_dev, d_dev, (scheme == INKQ_A81W41 || scheme == INKQ_W41) ? m_dev : nullptr,
                                scheme == INKQ_A80W4Z ? zp_dev : nullptr, n_begin);
    if (rc) {
        free_weight(w);
        delete w;
        return rc;
    }
    *out = w;
    return INKQ_OK;
}

}  // namespace inkq

using namespace inkq;

extern "C" {

int inkq_ctx_create(int device, void *stream, inkq_ctx **out)
{
    if (out == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null output pointer");
    *out = nullptr;
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) {
        cudaGetLastError();
        return fail(nullptr, INKQ_ERR_CUDA, std::string("no CUDA device available: ") + cudaGetErrorString(e));
    }
    if (device < 0 || device >= ndev) return fail(nullptr, INKQ_ERR_INVALID, "device index out of range");
    inkq_ctx *ctx = new (std::nothrow) inkq_ctx();
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_ALLOC, "host allocation failed");
    ctx->device = device;
    ctx->stream = static_cast<cudaStream_t>(stream);
    ctx->launches = 0;
    ctx->scratch_act = nullptr;
    ctx->scratch_planes = 0;
    ctx->scratch_elems = 0;
    ctx->f16_x = nullptr;
    ctx->f16_scale = nullptr;
    ctx->f16_x_cap = ctx->f16_scale_cap = 0;
    ctx->lin_x = ctx->lin_c = nullptr;
    ctx->lin_x_cap = ctx->lin_c_cap = 0;
    ctx->pin_x = ctx->pin_c = nullptr;
    ctx->pin_x_cap = ctx->pin_c_cap = 0;
    ctx->dev_flag = nullptr;
    ctx->host_flag = nullptr;
    ctx->encode_tiled = nullptr;
    ctx->copy_stream = nullptr;
    ctx->h2d_stream = nullptr;
    ctx->start_ev = nullptr;
    for (int i = 0; i < 8; i++) ctx->chunk_ev[i] = ctx->h2d_ev[i] = nullptr;
    cudaDeviceProp prop;
    if ((e = cudaSetDevice(device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) {
        delete ctx;
        return fail(nullptr, INKQ_ERR_CUDA, std::string("cudaSetDevice/Properties: ") + cudaGetErrorString(e));
    }
    if (prop.major != 10) {
        delete ctx;
        return fail(nullptr, INKQ_ERR_UNSUPPORTED, "this library is built for sm_100a (B200) only; found compute capability " +
                                                        std::to_string(prop.major) + "." + std::to_string(prop.minor));
    }
    ctx->num_sms = prop.multiProcessorCount;
    // word 0: set by a kernel whose bounded wait ran out; word 1: ticket counter of the decode GEMV's last-CTA epilogue
    if ((e = cudaMalloc(reinterpret_cast<void **>(&ctx->dev_flag), CTX_FLAG_WORDS * sizeof(int))) != cudaSuccess ||
        (e = cudaMemset(ctx->dev_flag, 0, CTX_FLAG_WORDS * sizeof(int))) != cudaSuccess ||
        (e = cudaHostAlloc(reinterpret_cast<void **>(&ctx->host_flag), sizeof(int), cudaHostAllocDefault)) != cudaSuccess) {
        cudaFree(ctx->dev_flag);
        delete ctx;
        return fail(nullptr, INKQ_ERR_ALLOC, std::string("context allocation: ") + cudaGetErrorString(e));
    }
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
        ctx->encode_tiled = fn;
    else
        cudaGetLastError();
    *out = ctx;
    return INKQ_OK;
}

int inkq_ctx_destroy(inkq_ctx *ctx)
{
    if (ctx == nullptr) return INKQ_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch_act != nullptr) {
        free_act(ctx->scratch_act);
        delete static_cast<inkq_act *>(ctx->scratch_act);
    }
    cudaFree(ctx->f16_x);
    cudaFree(ctx->f16_scale);
    cudaFree(ctx->lin_x);
    cudaFree(ctx->lin_c);
    cudaFree(ctx->dev_flag);
    cudaFreeHost(ctx->host_flag);
    if (ctx->copy_stream != nullptr) cudaStreamDestroy(ctx->copy_stream);
    if (ctx->h2d_stream != nullptr) cudaStreamDestroy(ctx->h2d_stream);
    if (ctx->start_ev != nullptr) cudaEventDestroy(ctx->start_ev);
    for (int i = 0; i < 8; i++) {
        if (ctx->chunk_ev[i] != nullptr) cudaEventDestroy(ctx->chunk_ev[i]);
        if (ctx->h2d_ev[i] != nullptr) cudaEventDestroy(ctx->h2d_ev[i]);
    }
    delete ctx;
    return INKQ_OK;
}

int inkq_ctx_set_stream(inkq_ctx *ctx, void *stream)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    ctx->stream = static_cast<cudaStream_t>(stream);
    return INKQ_OK;
}

int inkq_ctx_synchronize(inkq_ctx *ctx)
{
    int rc = use(ctx);
    if (rc) return rc;
    // the time-out word travels to a page-locked host word at the end of the stream: one wait covers the work and the flag
    INKQ_CUDA(ctx, cudaMemcpyAsync(ctx->host_flag, ctx->dev_flag, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const int flag = *static_cast<volatile int *>(ctx->host_flag);
    if (flag != 0) {
        cudaMemset(ctx->dev_flag, 0, sizeof(int));
        return fail(ctx, INKQ_ERR_TIMEOUT, "a bounded device-side wait ran out inside a kernel; its output is invalid");
    }
    return INKQ_OK;
}

const char *inkq_last_error(const inkq_ctx *ctx)
{
    if (ctx != nullptr) return ctx->err.c_str();
    static thread_local std::string copy;
    std::lock_guard<std::mutex> lk(g_err_mu);
    copy = g_err;
    return copy.c_str();
}

uint64_t inkq_launch_count(const inkq_ctx *ctx) { return ctx != nullptr ? ctx->launches : 0; }

// ---- weights -------------------------------------------------------------------
int inkq_weight_create_dev(inkq_ctx *ctx, int scheme, int scale_mode, int N, int K, const uint8_t *nib_dev, const float *d_dev,
                           const float *m_dev, const uint8_t *zp_dev, int n_begin, int n_end, inkq_weight **out)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    rc = check_weight_args(ctx, scheme, scale_mode, N, K, nib_dev, d_dev, m_dev, zp_dev, n_begin, n_end);
    if (rc) return rc;
    return build_weight(ctx, scheme, scale_mode, K, nib_dev, d_dev, m_dev, zp_dev, n_begin, n_end, out);
}

int inkq_weight_create(inkq_ctx *ctx, int scheme, int scale_mode, int N, int K, const uint8_t *nib, const float *d, const float *m,
                       const uint8_t *zp, int n_begin, int n_end, inkq_weight **out)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    rc = check_weight_args(ctx, scheme, scale_mode, N, K, nib, d, m, zp, n_begin, n_end);
    if (rc) return rc;
    // stage only the requested rows on the device, re-tile there, drop the staging copy
    const size_t rows = static_cast<size_t>(n_end - n_begin), row_nib = static_cast<size_t>(K) / 2, row_sc = static_cast<size_t>(K) / QK;
    uint8_t *nib_dev = nullptr, *zp_dev = nullptr;
    float *d_dev = nullptr, *m_dev = nullptr;
    const bool need_m = (scheme == INKQ_A81W41 || scheme == INKQ_W41), need_z = (scheme == INKQ_A80W4Z);
    rc = dev_alloc(ctx, &nib_dev, rows * row_nib);
    if (!rc) rc = dev_alloc(ctx, &d_dev, rows * row_sc);
    if (!rc && need_m) rc = dev_alloc(ctx, &m_dev, rows * row_sc);
    if (!rc && need_z) rc = dev_alloc(ctx, &zp_dev, rows * row_sc);
    cudaError_t e = cudaSuccess;
    if (!rc) e = cudaMemcpyAsync(nib_dev, nib + n_begin * row_nib, rows * row_nib, cudaMemcpyHostToDevice, ctx->stream);
    if (!rc && e == cudaSuccess)
        e = cudaMemcpyAsync(d_dev, d + n_begin * row_sc, rows * row_sc * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (!rc && e == cudaSuccess && need_m)
        e = cudaMemcpyAsync(m_dev, m + n_begin * row_sc, rows * row_sc * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (!rc && e == cudaSuccess && need_z)
        e = cudaMemcpyAsync(zp_dev, zp + n_begin * row_sc, rows * row_sc, cudaMemcpyHostToDevice, ctx->stream);
    if (!rc && e != cudaSuccess) rc = fail(ctx, INKQ_ERR_CUDA, std::string("weight upload: ") + cudaGetErrorString(e));
    if (!rc) rc = build_weight(ctx, scheme, scale_mode, K, nib_dev, d_dev, m_dev, zp_dev, 0, static_cast<int>(rows), out);
    cudaStreamSynchronize(ctx->stream);
    cudaFree(nib_dev);
    cudaFree(d_dev);
    cudaFree(m_dev);
    cudaFree(zp_dev);
    return rc;
}

int inkq_weight_destroy(inkq_weight *w)
{
    if (w == nullptr) return INKQ_OK;
    cudaSetDevice(w->ctx->device);
    free_weight(w);
    delete w;
    return INKQ_OK;
}

int inkq_weight_info(const inkq_weight *w, int *rows, int *K, int *scheme, size_t *device_bytes)
{
    if (w == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null weight handle");
    if (rows) *rows = w->rows;
    if (K) *K = w->K;
    if (scheme) *scheme = w->scheme;
    if (device_bytes) *device_bytes = w->bytes;
    return INKQ_OK;
}

int inkq_weight_export(inkq_ctx *ctx, const inkq_weight *w, uint8_t *nib, float *d, float *m, uint8_t *zp)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr, "null weight handle");
    const size_t rows = w->rows, row_nib = static_cast<size_t>(w->K) / 2, row_sc = static_cast<size_t>(w->K) / QK;
    uint8_t *nib_dev = nullptr, *zp_dev = nullptr;
    float *d_dev = nullptr, *m_dev = nullptr;
    if (nib) rc = dev_alloc(ctx, &nib_dev, rows * row_nib);
    if (!rc && d) rc = dev_alloc(ctx, &d_dev, rows * row_sc);
    if (!rc && m) rc = dev_alloc(ctx, &m_dev, rows * row_sc);
    if (!rc && zp) rc = dev_alloc(ctx, &zp_dev, rows * row_sc);
    if (!rc) rc = launch_export(ctx, w, nib_dev, d_dev, m_dev, zp_dev);
    cudaError_t e = cudaSuccess;
    if (!rc && nib) e = cudaMemcpyAsync(nib, nib_dev, rows * row_nib, cudaMemcpyDeviceToHost, ctx->stream);
    if (!rc && e == cudaSuccess && d) e = cudaMemcpyAsync(d, d_dev, rows * row_sc * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
    if (!rc && e == cudaSuccess && m) e = cudaMemcpyAsync(m, m_dev, rows * row_sc * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
    if (!rc && e == cudaSuccess && zp) e = cudaMemcpyAsync(zp, zp_dev, rows * row_sc, cudaMemcpyDeviceToHost, ctx->stream);
    if (!rc && e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (!rc && e != cudaSuccess) rc = fail(ctx, INKQ_ERR_CUDA, std::string("weight export: ") + cudaGetErrorString(e));
    cudaFree(nib_dev);
    cudaFree(d_dev);
    cudaFree(m_dev);
    cudaFree(zp_dev);
    return rc;
}

// ---- activations -----------------------------------------------------------------
int inkq_act_create(inkq_ctx *ctx, int max_rows, int K, inkq_act **out)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    INKQ_REQUIRE(ctx, max_rows > 0 && K > 0 && K % 64 == 0, "max_rows must be positive and K a positive multiple of 64");
    inkq_act *a = new (std::nothrow) inkq_act();
    if (a == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
    a->ctx = ctx;
    a->max_rows = max_rows;
    a->K = K;
    a->M = 0;
    a->M_ld = 0;
    a->qmode = -1;
    a->q = nullptr;
    a->d = a->s = nullptr;
    a->isum = nullptr;
    const size_t ld = (static_cast<size_t>(max_rows) + 3) & ~static_cast<size_t>(3), nb = static_cast<size_t>(K) / QK;
    rc = dev_alloc(ctx, &a->q, static_cast<size_t>(max_rows) * K);
    if (!rc) rc = dev_alloc(ctx, &a->d, ld * nb);
    if (!rc) rc = dev_alloc(ctx, &a->s, ld * nb);
    if (!rc) rc = dev_alloc(ctx, &a->isum, ld * nb);
    if (!rc) rc = dev_alloc(ctx, &a->ssq, static_cast<size_t>(ACT_SSQ_CAP));
    if (rc) {
        free_act(a);
        delete a;
        return rc;
    }
    *out = a;
    return INKQ_OK;
}

int inkq_act_destroy(inkq_act *a)
{
    if (a == nullptr) return INKQ_OK;
    cudaSetDevice(a->ctx->device);
    free_act(a);
    delete a;
    return INKQ_OK;
}

int inkq_quantize(inkq_ctx *ctx, int qmode, const float *x_dev, int M, int K, inkq_act *act)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && x_dev != nullptr, "null activation handle or input");
    INKQ_REQUIRE(ctx, qmode >= INKQ_Q8_0_F16 && qmode <= INKQ_Q8_1_F32, "unknown quantizer mode");
    INKQ_REQUIRE(ctx, K == act->K, "K differs from the activation handle's K");
    INKQ_REQUIRE(ctx, M >= 1 && M <= act->max_rows, "M exceeds the activation handle's capacity");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0, "x must be 16-byte aligned");
    return launch_quantize(ctx, qmode, x_dev, M, K, act);
}

int inkq_act_export(inkq_ctx *ctx, const inkq_act *act, int8_t *q, float *d, float *s, int32_t *isum)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && act->M > 0, "activation handle holds no quantized data");
    const size_t M = act->M, nb = static_cast<size_t>(act->K) / QK, ld = act->M_ld;
    INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (q) INKQ_CUDA(ctx, cudaMemcpy(q, act->q, M * act->K, cudaMemcpyDeviceToHost));
    // planes are [nb][M_ld] on the device, [M][nb] for the caller: transpose on the host side of the copy
    const void *planes[3] = {act->d, act->s, act->isum};
    void *outs[3] = {d, s, isum};
    for (int i = 0; i < 3; i++) {
        if (outs[i] == nullptr) continue;
        uint32_t *tmp = new (std::nothrow) uint32_t[nb * ld];
        if (tmp == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
        cudaError_t e = cudaMemcpy(tmp, planes[i], nb * ld * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) {
            delete[] tmp;
            return fail(ctx, INKQ_ERR_CUDA, std::string("activation export: ") + cudaGetErrorString(e));
        }
        uint32_t *o = static_cast<uint32_t *>(outs[i]);
        for (size_t m = 0; m < M; m++)
            for (size_t b = 0; b < nb; b++) o[m * nb + b] = tmp[b * ld + m];
        delete[] tmp;
    }
    return INKQ_OK;
}

static int ensure_staging(inkq_ctx *ctx, size_t xn, size_t cn)
{
    int rc;
    if (ctx->lin_x_cap < xn) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->lin_x);
        ctx->lin_x_cap = 0;
        if ((rc = dev_alloc(ctx, &ctx->lin_x, xn))) return rc;
        ctx->lin_x_cap = xn;
    }
    if (ctx->lin_c_cap < cn) {
        cudaStreamSynchronize(ctx->stream);
        cudaFree(ctx->lin_c);
        ctx->lin_c_cap = 0;
        if ((rc = dev_alloc(ctx, &ctx->lin_c, cn))) return rc;
        ctx->lin_c_cap = cn;
    }
    return INKQ_OK;
}

int inkq_quantize_host(inkq_ctx *ctx, int qmode, const float *x_host, int M, int K, inkq_act *act)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, x_host != nullptr && M >= 1 && K >= 1, "null input or bad shape");
    const size_t xn = static_cast<size_t>(M) * K;
    if ((rc = ensure_staging(ctx, xn, 0))) return rc;
    INKQ_CUDA(ctx, cudaMemcpyAsync(ctx->lin_x, x_host, xn * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    return inkq_quantize(ctx, qmode, ctx->lin_x, M, K, act);
}

int inkq_act_import(inkq_ctx *ctx, inkq_act *act, int qmode, int M, const int8_t *q, const float *d, const float *s)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && q != nullptr && d != nullptr, "null activation handle or input");
    INKQ_REQUIRE(ctx, qmode >= INKQ_Q8_0_F16 && qmode <= INKQ_Q8_1_F32, "unknown quantizer mode");
    INKQ_REQUIRE(ctx, qmode == INKQ_Q8_0_F16 || s != nullptr, "Q8_1 activations need the scaled sums");
    INKQ_REQUIRE(ctx, M >= 1 && M <= act->max_rows, "M exceeds the activation handle's capacity");
    const size_t nb = static_cast<size_t>(act->K) / QK, ld = (static_cast<size_t>(M) + 3) & ~static_cast<size_t>(3);
    // planes are block-major [nb][M_ld] on the device: transpose while staging (a layout change, no arithmetic);
    // the integer block sums are recomputed from q on the device
    std::vector<float> dp(nb * ld, 0.0f), sp(nb * ld, 0.0f);
    for (size_t m = 0; m < static_cast<size_t>(M); m++)
        for (size_t b = 0; b < nb; b++) {
            dp[b * ld + m] = d[m * nb + b];
            if (s != nullptr) sp[b * ld + m] = s[m * nb + b];
        }
    INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    INKQ_CUDA(ctx, cudaMemcpy(act->q, q, static_cast<size_t>(M) * act->K, cudaMemcpyHostToDevice));
    INKQ_CUDA(ctx, cudaMemcpy(act->d, dp.data(), nb * ld * sizeof(float), cudaMemcpyHostToDevice));
    INKQ_CUDA(ctx, cudaMemcpy(act->s, sp.data(), nb * ld * sizeof(float), cudaMemcpyHostToDevice));
    if ((rc = launch_block_isum(ctx, act, M, static_cast<int>(ld)))) return rc;
    act->M = M;
    act->M_ld = static_cast<int>(ld);
    act->qmode = qmode;
    act->ssq_parts = 0;
    return INKQ_OK;
}

// ---- matmuls -----------------------------------------------------------------------
static int check_mm(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, const void *C)
{
    INKQ_REQUIRE(ctx, act != nullptr && w != nullptr && C != nullptr, "null handle or output");
    INKQ_REQUIRE(ctx, act->M > 0, "activation handle holds no quantized data");
    INKQ_REQUIRE(ctx, act->ssq_parts == 0, "the handle holds a row whose RMS scale is pending: only inkq_glue_decode_gemv consumes it");
    INKQ_REQUIRE(ctx, act->K == w->K, "activation and weight K differ");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations: use inkq_gemm_w41_f16act");
    const bool want_q81 = (w->scheme == INKQ_A81W41);
    const bool have_q81 = (act->qmode != INKQ_Q8_0_F16);
    INKQ_REQUIRE(ctx, want_q81 == have_q81, "activation quantizer mode does not match the weight scheme (Q8_1 for A81W41, Q8_0 otherwise)");
    return INKQ_OK;
}

int inkq_gemm(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev, int ldc)
{
    int rc = use(ctx);
    if (rc) return rc;
    if ((rc = check_mm(ctx, act, w, C_dev))) return rc;
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    return launch_gemm_tc(ctx, act, w, C_dev, ldc, nullptr);
}

int inkq_gemm_simt(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev, int ldc)
{
    int rc = use(ctx);
    if (rc) return rc;
    if ((rc = check_mm(ctx, act, w, C_dev))) return rc;
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    return launch_gemm_simt(ctx, act, w, C_dev, ldc);
}

int inkq_gemv(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_dev)
{
    int rc = use(ctx);
    if (rc) return rc;
    if ((rc = check_mm(ctx, act, w, C_dev))) return rc;
    INKQ_REQUIRE(ctx, act->M == 1, "inkq_gemv takes a single activation row");
    return launch_gemv(ctx, act, w, C_dev);
}

static int matmul_host(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_host, int ldc, bool gemv)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && w != nullptr && C_host != nullptr, "null handle or output");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    const size_t cn = static_cast<size_t>(act->M) * w->rows;
    if ((rc = ensure_staging(ctx, 0, cn))) return rc;
    rc = gemv ? inkq_gemv(ctx, act, w, ctx->lin_c) : inkq_gemm(ctx, act, w, ctx->lin_c, w->rows);
    if (rc) return rc;
    INKQ_CUDA(ctx, cudaMemcpy2DAsync(C_host, static_cast<size_t>(ldc) * sizeof(float), ctx->lin_c, static_cast<size_t>(w->rows) * sizeof(float),
                                     static_cast<size_t>(w->rows) * sizeof(float), act->M, cudaMemcpyDeviceToHost, ctx->stream));
    return inkq_ctx_synchronize(ctx);
}

int inkq_gemm_host(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_host, int ldc) { return matmul_host(ctx, act, w, C_host, ldc, false); }
int inkq_gemv_host(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, float *C_host)
{
    return matmul_host(ctx, act, w, C_host, w != nullptr ? w->rows : 0, true);
}

int inkq_debug_block_dots(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, int32_t *dots_dev)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && w != nullptr && dots_dev != nullptr, "null handle or output");
    INKQ_REQUIRE(ctx, act->M > 0 && act->K == w->K, "activation handle empty or K mismatch");
    return launch_block_dots(ctx, act, w, dots_dev);
}

int inkq_debug_block_dots_tc(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, int32_t *dots_dev)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && w != nullptr && dots_dev != nullptr, "null handle or output");
    INKQ_REQUIRE(ctx, act->M > 0 && act->K == w->K, "activation handle empty or K mismatch");
    return launch_gemm_tc(ctx, act, w, nullptr, 0, dots_dev);
}

// ---- linear forward ---------------------------------------------------------------------
// The context's activation scratch (the reference's ModelContext::activation_buffer, sized once for the
// largest layer, QwenForCausalLM.cc:101-113): one allocation that serves every (M, K) whose M*K fits.  It
// only grows, so a model's layers with different K (4096 / 12288) share it without re-allocating, and a
// warmed-up context allocates nothing more (which also keeps inkq_linear capturable in a CUDA graph).
static int ensure_scratch_act(inkq_ctx *ctx, int M, int K)
{
    const size_t need = static_cast<size_t>(M) * K;
    const size_t need_planes = static_cast<size_t>(K / QK) * ((static_cast<size_t>(M) + 3) & ~static_cast<size_t>(3));   // [K/32][round_up(M, 4)]
    Act *a = ctx->scratch_act;
    if (a == nullptr || ctx->scratch_elems < need || ctx->scratch_planes < need_planes) {
        if (a != nullptr) {
            cudaStreamSynchronize(ctx->stream);
            free_act(a);
            delete static_cast<inkq_act *>(a);
            ctx->scratch_act = nullptr;
            ctx->scratch_elems = 0;
            ctx->scratch_planes = 0;
        }
        size_t elems = need < (static_cast<size_t>(512) * 12288) ? static_cast<size_t>(512) * 12288 : need;
        inkq_act *na = new (std::nothrow) inkq_act();
        if (na == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
        na->ctx = ctx;
        na->q = nullptr;
        na->d = na->s = nullptr;
        na->isum = nullptr;
        size_t planes = elems / QK + 65536;   // room for the row padding of every shape with M*K <= elems and K <= 2^19
        if (planes < need_planes) planes = need_planes;   // longer rows: the exact need of this shape (checked on every call)
        int rc = dev_alloc(ctx, &na->q, elems);
        if (!rc) rc = dev_alloc(ctx, &na->d, planes);
        if (!rc) rc = dev_alloc(ctx, &na->s, planes);
        if (!rc) rc = dev_alloc(ctx, &na->isum, planes);
        if (rc) {
            free_act(na);
            delete na;
            return rc;
        }
        ctx->scratch_act = na;
        ctx->scratch_elems = elems;
        ctx->scratch_planes = planes;
        a = na;
    }
    a->K = K;
    a->max_rows = static_cast<int>(ctx->scratch_elems / K);
    a->M = 0;
    return INKQ_OK;
}

int inkq_linear(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, float *C_dev, int ldc)
{
    return inkq::linear_impl(ctx, w, x_dev, M, C_dev, ldc, nullptr);
}

}  // extern "C"

int inkq::linear_impl(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, float *C_dev, int ldc, const ExtraDst *extra)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && x_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, M >= 1, "M must be at least 1");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations: use inkq_gemm_w41_f16act");
    if (M == 1 && extra == nullptr && (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0) {
        // one token: the QGEMV quantizes the row in its own prologue (same arithmetic, same result bits as the
        // stand-alone quantizer followed by the QGEMV, one launch less)
        return launch_gemv_fused(ctx, w, x_dev, 0, nullptr, 0.0f, C_dev, 0);
    }
    if ((rc = ensure_scratch_act(ctx, M, w->K))) return rc;
    inkq_act *act = static_cast<inkq_act *>(ctx->scratch_act);
    int qmode;
    if (w->scheme == INKQ_A81W41) qmode = (M > 1) ? INKQ_Q8_1_F32 : INKQ_Q8_1_F16;  // QwenOperator.cc:96-120
    else qmode = INKQ_Q8_0_F16;
    if ((rc = inkq_quantize(ctx, qmode, x_dev, M, w->K, act))) return rc;
    if (M > 1) return launch_gemm_tc(ctx, act, w, C_dev, ldc, nullptr, extra);
    return launch_gemv(ctx, act, w, C_dev, extra);
}

extern "C" {

int inkq_linear_host(inkq_ctx *ctx, const inkq_weight *w, const float *x_host, int M, float *C_host, int ldc)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && x_host != nullptr && C_host != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, M >= 1, "M must be at least 1");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    const size_t xn = static_cast<size_t>(M) * w->K, cn = static_cast<size_t>(M) * w->rows;
    if ((rc = ensure_staging(ctx, xn, cn))) return rc;
    if (M >= 96 && w->scheme != INKQ_W41) {
        // Both copies (M*K*4 bytes in, M*N*4 bytes out over PCIe) take longer than the arithmetic, so the call works on
        // windows of rows: window i's activations travel to the device on one stream while window i-1 is quantized and
        // multiplied on the context's stream and window i-2's finished rows (contiguous in the result) travel back on
        // a third.  The first windows are small, so that the device-to-host link, which carries the most bytes, starts
        // early and then never waits: a window's product is ready before its predecessor's rows have left.
        constexpr int MAXC = 8;
        int m0[MAXC + 1], nch = 0, at = 0;
        const int lead[3] = {48, 80, 96};
        m0[0] = 0;
        while (nch < 3 && M - at >= lead[nch] + 32) {
            at += lead[nch];
            m0[++nch] = at;
        }
        if (at < M) {
            const int left = M - at, parts = (left + 127) / 128 < MAXC - nch ? (left + 127) / 128 : MAXC - nch;
            const int step = ((left + parts - 1) / parts + 15) & ~15;
            while (at < M) {
                at = (at + step < M) ? at + step : M;
                m0[++nch] = at;
            }
        }
        if (ctx->copy_stream == nullptr) {
            INKQ_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
            INKQ_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
            INKQ_CUDA(ctx, cudaEventCreateWithFlags(&ctx->start_ev, cudaEventDisableTiming));
            for (int i = 0; i < MAXC; i++) {
                INKQ_CUDA(ctx, cudaEventCreateWithFlags(&ctx->chunk_ev[i], cudaEventDisableTiming));
                INKQ_CUDA(ctx, cudaEventCreateWithFlags(&ctx->h2d_ev[i], cudaEventDisableTiming));
            }
        }
        if ((rc = ensure_scratch_act(ctx, M, w->K))) return rc;
        inkq_act *act = static_cast<inkq_act *>(ctx->scratch_act);
        const int qmode = (w->scheme == INKQ_A81W41) ? INKQ_Q8_1_F32 : INKQ_Q8_0_F16;
        // whatever the context's stream still does with the staging buffers finishes before they are overwritten
        INKQ_CUDA(ctx, cudaEventRecord(ctx->start_ev, ctx->stream));
        INKQ_CUDA(ctx, cudaStreamWaitEvent(ctx->h2d_stream, ctx->start_ev, 0));
        INKQ_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->start_ev, 0));
        for (int c = 0; c < nch; c++) {
            const size_t off = static_cast<size_t>(m0[c]) * w->K, cnt = static_cast<size_t>(m0[c + 1] - m0[c]) * w->K;
            INKQ_CUDA(ctx, cudaMemcpyAsync(ctx->lin_x + off, x_host + off, cnt * sizeof(float), cudaMemcpyHostToDevice, ctx->h2d_stream));
            INKQ_CUDA(ctx, cudaEventRecord(ctx->h2d_ev[c], ctx->h2d_stream));
        }
        for (int c = 0; c < nch; c++) {
            const int rows = m0[c + 1] - m0[c];
            INKQ_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->h2d_ev[c], 0));
            if ((rc = launch_quantize_rows(ctx, qmode, ctx->lin_x + static_cast<size_t>(m0[c]) * w->K, m0[c], rows, M, w->K, act))) return rc;
            if ((rc = launch_gemm_tc(ctx, act, w, ctx->lin_c, w->rows, nullptr, nullptr, 0, -1, m0[c], rows))) return rc;
            INKQ_CUDA(ctx, cudaEventRecord(ctx->chunk_ev[c], ctx->stream));
            INKQ_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->chunk_ev[c], 0));
            INKQ_CUDA(ctx, cudaMemcpy2DAsync(C_host + static_cast<size_t>(m0[c]) * ldc, static_cast<size_t>(ldc) * sizeof(float),
                                             ctx->lin_c + static_cast<size_t>(m0[c]) * w->rows, static_cast<size_t>(w->rows) * sizeof(float),
                                             static_cast<size_t>(w->rows) * sizeof(float), rows, cudaMemcpyDeviceToHost, ctx->copy_stream));
        }
        INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->copy_stream));
        return inkq_ctx_synchronize(ctx);
    }
    INKQ_CUDA(ctx, cudaMemcpyAsync(ctx->lin_x, x_host, xn * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    if ((rc = inkq_linear(ctx, w, ctx->lin_x, M, ctx->lin_c, w->rows))) return rc;
    INKQ_CUDA(ctx, cudaMemcpy2DAsync(C_host, static_cast<size_t>(ldc) * sizeof(float), ctx->lin_c, static_cast<size_t>(w->rows) * sizeof(float),
                                     static_cast<size_t>(w->rows) * sizeof(float), M, cudaMemcpyDeviceToHost, ctx->stream));
    return inkq_ctx_synchronize(ctx);
}

// ---- weight-only W41 and fp16 lm_head --------------------------------------------------------
int inkq_gemm_w41_f16act(inkq_ctx *ctx, const uint16_t *a16_dev, int M, const inkq_weight *w, float *C_dev, int ldc)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && a16_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, w->scheme == INKQ_W41 || w->scheme == INKQ_A81W41, "weight-only matmul needs Q4_1 weights");
    INKQ_REQUIRE(ctx, M >= 1 && ldc >= w->rows, "bad M or ldc");
    if (M == 1 && (reinterpret_cast<uintptr_t>(a16_dev) & 3) == 0) return launch_gemv_w41(ctx, a16_dev, w, C_dev);   // decode: stream the weights
    return launch_gemm_w41_tc(ctx, a16_dev, M, w, C_dev, ldc);
}

int inkq_gemm_w41_f16act_simt(inkq_ctx *ctx, const uint16_t *a16_dev, int M, const inkq_weight *w, float *C_dev, int ldc)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && a16_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, w->scheme == INKQ_W41 || w->scheme == INKQ_A81W41, "weight-only matmul needs Q4_1 weights");
    INKQ_REQUIRE(ctx, M >= 1 && ldc >= w->rows, "bad M or ldc");
    return launch_gemm_w41_f16(ctx, a16_dev, M, w, C_dev, ldc);
}

int inkq_f16w_create_dev(inkq_ctx *ctx, int N, int K, const uint16_t *w16_dev, int n_begin, int n_end, inkq_f16w **out)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    INKQ_REQUIRE(ctx, w16_dev != nullptr && N > 0 && K > 0 && K % 8 == 0, "bad fp16 weight arguments (K must be a multiple of 8)");
    INKQ_REQUIRE(ctx, 0 <= n_begin && n_begin < n_end && n_end <= N, "row range out of bounds");
    inkq_f16w *w = new (std::nothrow) inkq_f16w();
    if (w == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
    w->ctx = ctx;
    w->rows = n_end - n_begin;
    w->K = K;
    w->bytes = static_cast<size_t>(w->rows) * K * 2;
    if ((rc = dev_alloc(ctx, &w->w, static_cast<size_t>(w->rows) * K))) {
        delete w;
        return rc;
    }
    cudaError_t e = cudaMemcpyAsync(w->w, w16_dev + static_cast<size_t>(n_begin) * K, w->bytes, cudaMemcpyDeviceToDevice, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(w->w);
        delete w;
        return fail(ctx, INKQ_ERR_CUDA, std::string("fp16 weight copy: ") + cudaGetErrorString(e));
    }
    *out = w;
    return INKQ_OK;
}

int inkq_f16w_create(inkq_ctx *ctx, int N, int K, const uint16_t *w16_host, int n_begin, int n_end, inkq_f16w **out)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    INKQ_REQUIRE(ctx, w16_host != nullptr && N > 0 && K > 0 && K % 8 == 0, "bad fp16 weight arguments (K must be a multiple of 8)");
    INKQ_REQUIRE(ctx, 0 <= n_begin && n_begin < n_end && n_end <= N, "row range out of bounds");
    inkq_f16w *w = new (std::nothrow) inkq_f16w();
    if (w == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
    w->ctx = ctx;
    w->rows = n_end - n_begin;
    w->K = K;
    w->bytes = static_cast<size_t>(w->rows) * K * 2;
    if ((rc = dev_alloc(ctx, &w->w, static_cast<size_t>(w->rows) * K))) {
        delete w;
        return rc;
    }
    cudaError_t e = cudaMemcpy(w->w, w16_host + static_cast<size_t>(n_begin) * K, w->bytes, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(w->w);
        delete w;
        return fail(ctx, INKQ_ERR_CUDA, std::string("fp16 weight upload: ") + cudaGetErrorString(e));
    }
    *out = w;
    return INKQ_OK;
}

int inkq_f16w_destroy(inkq_f16w *w)
{
    if (w == nullptr) return INKQ_OK;
    cudaSetDevice(w->ctx->device);
    cudaFree(w->w);
    delete w;
    return INKQ_OK;
}

int inkq_f16w_matmul_prec(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc, int precision)
{
    return inkq::f16w_matmul_impl(ctx, w, x_dev, M, C_dev, ldc, precision, nullptr);
}

}  // extern "C"

int inkq::f16w_matmul_impl(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc, int precision, const ExtraDst *extra)
{
    int rc = use(ctx);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && x_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, M >= 1 && ldc >= w->rows, "bad M or ldc");
    INKQ_REQUIRE(ctx, precision == INKQ_F16W_ACT_FP32 || precision == INKQ_F16W_ACT_FP16, "unknown precision");
    // few rows: the weights are streamed once per 4 rows by the CUDA-core kernel (fp32 activations, exact products)
    const bool aligned = w->rows % 4 == 0 && ldc % 4 == 0 && (reinterpret_cast<uintptr_t>(C_dev) & 15) == 0;
    if (M < 16 || w->K % 64 != 0 || !aligned) return launch_f16w_matmul(ctx, w, x_dev, M, C_dev, ldc, extra);
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0, "x must be 16-byte aligned");
    const int passes = precision == INKQ_F16W_ACT_FP32 ? 2 : 1;
    const size_t need = static_cast<size_t>(M) * w->K * passes;
    if (ctx->f16_x_cap < need) {
        INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));   // earlier launches may still read the old buffer
        cudaFree(ctx->f16_x);
        ctx->f16_x_cap = 0;
        if ((rc = dev_alloc(ctx, &ctx->f16_x, need))) return rc;
        ctx->f16_x_cap = need;
    }
    if (ctx->f16_scale_cap < static_cast<size_t>(M)) {
        INKQ_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        cudaFree(ctx->f16_scale);
        ctx->f16_scale_cap = 0;
        if ((rc = dev_alloc(ctx, &ctx->f16_scale, static_cast<size_t>(M)))) return rc;
        ctx->f16_scale_cap = static_cast<size_t>(M);
    }
    return launch_f16w_gemm_tc(ctx, w, x_dev, M, C_dev, ldc, passes, ctx->f16_x, ctx->f16_scale, extra);
}

extern "C" {

int inkq_f16w_matmul(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, float *C_dev, int ldc)
{
    return inkq_f16w_matmul_prec(ctx, w, x_dev, M, C_dev, ldc, INKQ_F16W_ACT_FP32);
}

}  // extern "C"
