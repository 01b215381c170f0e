// inkq_linear_m1_static: the decode (M == 1) forward of a quantized linear layer for
// callers that must not allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits - a real-time serving
// loop whose latency budget cannot absorb the implicit device synchronisation of an
// allocation, a host that has handed the whole device heap to another allocator, a
// plugin running inside someone else's pre-sized memory pool.  inkq_linear keeps
// its quantized-activation scratch in the context and grows it with cudaMalloc when
// a larger shape shows up; this entry point never does.  Its scratch - one
// quantized activation row: the int8 values plus the per-block scale, scaled sum
// and integer sum planes - lives in the fixed array below, which every device that
// loads this library carries until the process exits (40 KiB: 16 KiB of int8 values and
// three padded planes of 8 KiB).
//
// Limits and rules
//   * K <= INKQ_STATIC_MAX_K (16384); larger K is rejected with INKQ_ERR_UNSUPPORTED.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and caches it; make that first
//     call before starting any stream capture.
//   * All calls on a device share the one array.  It keeps whatever the previous call
//     left; nothing in it has to start at zero, because the quantizer rewrites every
//     byte the QGEMV reads (all K int8 values and all four rows of the padded planes).
//     Two calls whose kernels overlap on the GPU (different streams, no ordering)
//     race on it: order them.
//   * It calls no cudaMalloc, cudaFree or any allocating library routine.
// Same arithmetic and the same result bits as inkq_linear with M == 1 (which fuses the
// quantizer into the QGEMV's prologue; here they are two launches).
#include <cuda_runtime.h>

#include <mutex>

#include "inkq_internal.h"

namespace inkq {

constexpr int STATIC_MAX_K = 16384;
constexpr int STATIC_PLANE = 4 * (STATIC_MAX_K / QK);  // [K/32][M_ld = 4] entries of one plane
constexpr size_t STATIC_BYTES = STATIC_MAX_K + 3 * sizeof(float) * STATIC_PLANE;
static_assert(STATIC_BYTES == 40 * 1024, "the documented size of the static scratch is 40 KiB");

// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer to pass on.
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_BYTES];

constexpr int MAX_DEVICES = 64;
static std::mutex g_static_mu;
static unsigned char *g_static_ptr[MAX_DEVICES];  // device address of the array, per device

static int static_scratch_for(inkq_ctx *ctx, unsigned char **out)
{
    if (ctx->device < 0 || ctx->device >= MAX_DEVICES) return fail(ctx, INKQ_ERR_UNSUPPORTED, "device index beyond the static-scratch table");
    std::lock_guard<std::mutex> lk(g_static_mu);
    if (g_static_ptr[ctx->device] == nullptr) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);  // the context's device is current (set by the caller below)
        if (e != cudaSuccess || p == nullptr)
            return fail(ctx, INKQ_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
        g_static_ptr[ctx->device] = static_cast<unsigned char *>(p);
    }
    *out = g_static_ptr[ctx->device];
    return INKQ_OK;
}

}  // namespace inkq

using namespace inkq;

extern "C" int inkq_linear_m1_static(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, float *C_dev)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    INKQ_REQUIRE(ctx, w != nullptr && x_dev != nullptr && C_dev != nullptr, "null handle, input or output");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(x_dev) & 15) == 0, "x must be 16-byte aligned");
    if (w->K > STATIC_MAX_K)
        return fail(ctx, INKQ_ERR_UNSUPPORTED,
                    "K = " + std::to_string(w->K) + " exceeds the static scratch of inkq_linear_m1_static (K <= " + std::to_string(STATIC_MAX_K) + ")");
    unsigned char *base = nullptr;
    int rc = static_scratch_for(ctx, &base);
    if (rc) return rc;
    // carve the one activation row out of the fixed array
    Act a;
    a.ctx = ctx;
    a.max_rows = 1;
    a.K = w->K;
    a.M = 0;
    a.M_ld = 0;
    a.qmode = -1;
    a.q = reinterpret_cast<int8_t *>(base);
    a.d = reinterpret_cast<float *>(base + STATIC_MAX_K);
    a.s = a.d + STATIC_PLANE;
    a.isum = reinterpret_cast<int32_t *>(a.s + STATIC_PLANE);
    const int qmode = (w->scheme == INKQ_A81W41) ? INKQ_Q8_1_F16 : INKQ_Q8_0_F16;  // as inkq_linear does for M == 1
    if ((rc = launch_quantize(ctx, qmode, x_dev, 1, w->K, &a))) return rc;
    return launch_gemv(ctx, &a, w, C_dev);
}
