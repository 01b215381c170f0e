// Column-sharded (tensor-parallel) linear layer whose exchange step is part of the matmul kernel.
//
// Rank r of P owns the weight rows [r*N/P, (r+1)*N/P) and therefore the output columns of that
// range (every C[:, n] depends on weight row n only: the reference parallelises its CPU kernels
// over the same 8-column groups, qwen3/src/qwen/quantized_gemx_kernels.cc:364-365).  Instead of
// writing its [M][N/P] shard locally and running an all-gather afterwards, the epilogue of the
// QGEMM / QGEMV stores every finished C element into the [M][N] buffer of EVERY rank through
// peer-mapped pointers (plain st.global over NVLink, 128 bytes per warp store), tile by tile while
// the other tiles are still being computed.  What remains of the collective is one small barrier
// kernel: every rank tells every peer "my stores are done" and waits for the same from them.
//
// A peer set is P buffers of equal size, one per rank, each mapped into every process:
//   * separate processes (one per GPU): inkq_peer_export turns a rank's buffer into an 80-byte
//     blob (CUDA IPC handle of its allocation + offset + size), the host exchanges the blobs by
//     any means it has (the Python side uses torch.distributed.all_gather_object) and
//     inkq_peerset_open maps the others;
//   * one process driving several GPUs with peer access enabled, or several buffers on one GPU:
//     inkq_peerset_from_pointers takes the P pointers as they are.
// The first INKQ_PEER_RESERVED_BYTES of every buffer belong to the barrier and must be zero when
// the set is made: words 0..7 count the arrivals of ranks 0..7 at this rank, word 16 is this
// rank's own barrier count.
//
// The barrier's wait is bounded (timeout_ms of the device's nanosecond timer); when it runs out the
// kernel records it in the context's flag word and returns, inkq_ctx_synchronize then reports
// INKQ_ERR_TIMEOUT and the context stays usable.  No TMA, no multicast: only ordinary loads, stores
// and one system-scope reduction per peer touch another GPU's memory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <new>

#include "inkq_internal.h"

namespace inkq {

struct PeerBlob {           // what inkq_peer_export writes: INKQ_PEER_HANDLE_BYTES
    cudaIpcMemHandle_t h;   // 64 bytes
    uint64_t offset;        // of the buffer inside its allocation
    uint64_t bytes;
};
static_assert(sizeof(PeerBlob) == INKQ_PEER_HANDLE_BYTES, "blob size is part of the ABI");

struct PeerPtrs {
    char *p[MAX_PEERS];
};

__device__ __forceinline__ uint64_t global_timer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One CTA of 32 threads; thread p handles peer p.
__global__ void k_peer_barrier(PeerPtrs pp, int world, int rank, uint64_t timeout_ns, int *flag)
{
    uint32_t *mine = reinterpret_cast<uint32_t *>(pp.p[rank]);
    const uint32_t epoch = mine[16] + 1;     // read by every thread before thread 0 rewrites it below
    __syncwarp();
    const int p = threadIdx.x;
    if (p < world && p != rank) {
        // every store this rank issued before this kernel (the matmul's epilogue) precedes the arrival
        __threadfence_system();
        uint32_t *theirs = reinterpret_cast<uint32_t *>(pp.p[p]) + rank;
        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(theirs) : "memory");
        const uint64_t t0 = global_timer_ns();
        // arrivals only grow, and a peer can be at most one barrier ahead: compare as a signed distance
        while (static_cast<int32_t>(ld_acquire_sys(mine + p) - epoch) < 0) {
            if (global_timer_ns() - t0 > timeout_ns) {
                atomicExch(flag, 2);
                break;
            }
            __nanosleep(200);
        }
    }
    __syncwarp();
    if (p == 0) mine[16] = epoch;
}

static int check_set(inkq_ctx *ctx, const inkq_peerset *ps)
{
    INKQ_REQUIRE(ctx, ps != nullptr, "null peer set");
    INKQ_REQUIRE(ctx, ps->ctx == ctx, "the peer set belongs to another context");
    return INKQ_OK;
}

}  // namespace inkq

using namespace inkq;

extern "C" {

int inkq_peer_export(inkq_ctx *ctx, void *dev_ptr, size_t bytes, void *blob_out)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    INKQ_REQUIRE(ctx, dev_ptr != nullptr && blob_out != nullptr && bytes > INKQ_PEER_RESERVED_BYTES, "null pointer or a buffer not larger than its reserved head");
    INKQ_REQUIRE(ctx, (reinterpret_cast<uintptr_t>(dev_ptr) & 255) == 0, "the buffer must be 256-byte aligned");
    // the IPC handle names a whole allocation: find its base
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    cudaDriverEntryPointQueryResult qres;
    void *fn = nullptr;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        return fail(ctx, INKQ_ERR_UNSUPPORTED, "cuMemGetAddressRange entry point not available");
    }
    CUdeviceptr base = 0;
    size_t range = 0;
    CUresult cr = reinterpret_cast<RangeFn>(fn)(&base, &range, reinterpret_cast<CUdeviceptr>(dev_ptr));
    if (cr != CUDA_SUCCESS) return fail(ctx, INKQ_ERR_CUDA, "cuMemGetAddressRange failed with code " + std::to_string(static_cast<int>(cr)));
    PeerBlob b;
    std::memset(&b, 0, sizeof(b));
    b.offset = reinterpret_cast<CUdeviceptr>(dev_ptr) - base;
    b.bytes = bytes;
    INKQ_REQUIRE(ctx, b.offset + bytes <= range, "the buffer runs past the end of its allocation");
    INKQ_CUDA(ctx, cudaIpcGetMemHandle(&b.h, reinterpret_cast<void *>(base)));
    std::memcpy(blob_out, &b, sizeof(b));
    return INKQ_OK;
}

static int new_set(inkq_ctx *ctx, int world, int rank, size_t bytes, inkq_peerset **out)
{
    INKQ_REQUIRE(ctx, out != nullptr, "null output pointer");
    *out = nullptr;
    INKQ_REQUIRE(ctx, world >= 1 && world <= MAX_PEERS && rank >= 0 && rank < world, "world must be 1..8 and rank inside it");
    INKQ_REQUIRE(ctx, bytes > INKQ_PEER_RESERVED_BYTES, "a peer buffer must be larger than its reserved head");
    inkq_peerset *ps = new (std::nothrow) inkq_peerset();
    if (ps == nullptr) return fail(ctx, INKQ_ERR_ALLOC, "host allocation failed");
    ps->ctx = ctx;
    ps->world = world;
    ps->rank = rank;
    ps->bytes = bytes;
    for (int i = 0; i < MAX_PEERS; i++) {
        ps->ptr[i] = nullptr;
        ps->opened[i] = nullptr;
    }
    *out = ps;
    return INKQ_OK;
}

int inkq_peerset_open(inkq_ctx *ctx, int world, int rank, void *local_ptr, const void *blobs, inkq_peerset **out)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    INKQ_REQUIRE(ctx, local_ptr != nullptr && blobs != nullptr, "null pointer");
    INKQ_REQUIRE(ctx, world >= 1 && world <= MAX_PEERS && rank >= 0 && rank < world, "world must be 1..8 and rank inside it");
    const PeerBlob *bl = static_cast<const PeerBlob *>(blobs);
    PeerBlob mine;
    std::memcpy(&mine, bl + rank, sizeof(mine));
    int rc = new_set(ctx, world, rank, static_cast<size_t>(mine.bytes), out);
    if (rc) return rc;
    inkq_peerset *ps = *out;
    ps->ptr[rank] = static_cast<char *>(local_ptr);
    for (int p = 0; p < world; p++) {
        if (p == rank) continue;
        PeerBlob b;
        std::memcpy(&b, bl + p, sizeof(b));
        if (b.bytes != mine.bytes) {
            inkq_peerset_destroy(ps);
            *out = nullptr;
            return fail(ctx, INKQ_ERR_INVALID, "the ranks' buffers differ in size");
        }
        void *base = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&base, b.h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            inkq_peerset_destroy(ps);
            *out = nullptr;
            return fail(ctx, INKQ_ERR_CUDA, std::string("cudaIpcOpenMemHandle of rank ") + std::to_string(p) + ": " + cudaGetErrorString(e));
        }
        ps->opened[p] = base;
        ps->ptr[p] = static_cast<char *>(base) + b.offset;
    }
    return INKQ_OK;
}

int inkq_peerset_from_pointers(inkq_ctx *ctx, int world, int rank, void *const *ptrs, size_t bytes, inkq_peerset **out)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    INKQ_REQUIRE(ctx, ptrs != nullptr, "null pointer array");
    int rc = new_set(ctx, world, rank, bytes, out);
    if (rc) return rc;
    for (int p = 0; p < world; p++) {
        if (ptrs[p] == nullptr || (reinterpret_cast<uintptr_t>(ptrs[p]) & 255) != 0) {
            delete *out;
            *out = nullptr;
            return fail(ctx, INKQ_ERR_INVALID, "every buffer must be non-null and 256-byte aligned");
        }
        (*out)->ptr[p] = static_cast<char *>(ptrs[p]);
    }
    return INKQ_OK;
}

int inkq_peerset_destroy(inkq_peerset *ps)
{
    if (ps == nullptr) return INKQ_OK;
    cudaSetDevice(ps->ctx->device);
    cudaStreamSynchronize(ps->ctx->stream);
    for (int p = 0; p < MAX_PEERS; p++)
        if (ps->opened[p] != nullptr) cudaIpcCloseMemHandle(ps->opened[p]);
    delete ps;
    return INKQ_OK;
}

int inkq_linear_scatter(inkq_ctx *ctx, const inkq_weight *w, const float *x_dev, int M, inkq_peerset *ps, size_t byte_offset, int ldc)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    int rc = check_set(ctx, ps);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && M >= 1, "null weight handle or M < 1");
    INKQ_REQUIRE(ctx, byte_offset >= INKQ_PEER_RESERVED_BYTES && byte_offset % 4 == 0, "the offset must be a multiple of 4 past the reserved head");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    const size_t last = byte_offset + (static_cast<size_t>(M - 1) * ldc + w->rows) * sizeof(float);
    INKQ_REQUIRE(ctx, last <= ps->bytes, "the output does not fit into the peer buffers");
    ExtraDst extra = {};
    for (int p = 0; p < ps->world; p++)
        if (p != ps->rank) extra.p[extra.n++] = reinterpret_cast<float *>(ps->ptr[p] + byte_offset);
    return linear_impl(ctx, w, x_dev, M, reinterpret_cast<float *>(ps->ptr[ps->rank] + byte_offset), ldc, &extra);
}

int inkq_gemm_scatter(inkq_ctx *ctx, const inkq_act *act, const inkq_weight *w, inkq_peerset *ps, size_t byte_offset, int ldc)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    int rc = check_set(ctx, ps);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, act != nullptr && w != nullptr, "null handle");
    INKQ_REQUIRE(ctx, act->M > 1, "the activation handle must hold more than one quantized row (one row: inkq_linear_scatter)");
    INKQ_REQUIRE(ctx, act->K == w->K, "activation and weight K differ");
    INKQ_REQUIRE(ctx, w->scheme != INKQ_W41, "a weight-only layer takes fp16 activations");
    INKQ_REQUIRE(ctx, (w->scheme == INKQ_A81W41) == (act->qmode != INKQ_Q8_0_F16),
                 "activation quantizer mode does not match the weight scheme (Q8_1 for A81W41, Q8_0 otherwise)");
    INKQ_REQUIRE(ctx, byte_offset >= INKQ_PEER_RESERVED_BYTES && byte_offset % 4 == 0, "the offset must be a multiple of 4 past the reserved head");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    const size_t last = byte_offset + (static_cast<size_t>(act->M - 1) * ldc + w->rows) * sizeof(float);
    INKQ_REQUIRE(ctx, last <= ps->bytes, "the output does not fit into the peer buffers");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    ExtraDst extra = {};
    for (int p = 0; p < ps->world; p++)
        if (p != ps->rank) extra.p[extra.n++] = reinterpret_cast<float *>(ps->ptr[p] + byte_offset);
    return launch_gemm_tc(ctx, act, w, reinterpret_cast<float *>(ps->ptr[ps->rank] + byte_offset), ldc, nullptr, &extra);
}

int inkq_f16w_matmul_scatter(inkq_ctx *ctx, const inkq_f16w *w, const float *x_dev, int M, inkq_peerset *ps, size_t byte_offset, int ldc, int precision)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    int rc = check_set(ctx, ps);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, w != nullptr && M >= 1, "null weight handle or M < 1");
    INKQ_REQUIRE(ctx, byte_offset >= INKQ_PEER_RESERVED_BYTES && byte_offset % 4 == 0, "the offset must be a multiple of 4 past the reserved head");
    INKQ_REQUIRE(ctx, ldc >= w->rows, "ldc is smaller than the number of weight rows");
    const size_t last = byte_offset + (static_cast<size_t>(M - 1) * ldc + w->rows) * sizeof(float);
    INKQ_REQUIRE(ctx, last <= ps->bytes, "the output does not fit into the peer buffers");
    ExtraDst extra = {};
    for (int p = 0; p < ps->world; p++)
        if (p != ps->rank) extra.p[extra.n++] = reinterpret_cast<float *>(ps->ptr[p] + byte_offset);
    return f16w_matmul_impl(ctx, w, x_dev, M, reinterpret_cast<float *>(ps->ptr[ps->rank] + byte_offset), ldc, precision, &extra);
}

int inkq_peer_barrier(inkq_ctx *ctx, inkq_peerset *ps, int timeout_ms)
{
    if (ctx == nullptr) return fail(nullptr, INKQ_ERR_INVALID, "null context");
    int rc = check_set(ctx, ps);
    if (rc) return rc;
    INKQ_REQUIRE(ctx, timeout_ms >= 1 && timeout_ms <= 10000, "timeout_ms must be within 1..10000");
    INKQ_CUDA(ctx, cudaSetDevice(ctx->device));
    PeerPtrs pp;
    for (int p = 0; p < MAX_PEERS; p++) pp.p[p] = ps->ptr[p];
    k_peer_barrier<<<1, 32, 0, ctx->stream>>>(pp, ps->world, ps->rank, static_cast<uint64_t>(timeout_ms) * 1000000ull, ctx->dev_flag);
    return after_launch(ctx, "k_peer_barrier");
}

}  // extern "C"
