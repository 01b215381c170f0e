// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk/tensor TMA copies, tcgen05
// (tensor memory allocation, UMMA issue/commit, TMEM loads), proxy fences.
// Every wait is bounded: after INKQ_SPIN_LIMIT_CYCLES the wait gives up and
// returns false so that the kernel can record the failure and leave cleanly.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace inkq {

// ~2 s at 2 GHz.  Legitimate waits in these kernels last microseconds.
#ifndef INKQ_SPIN_LIMIT_CYCLES
#define INKQ_SPIN_LIMIT_CYCLES (4000000000LL)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
// One probe of the barrier (returns at once when the phase is incomplete).
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the limit ran out, or as soon as *abort (a
// shared-memory word another role sets when its own wait ran out) is non-zero.
// After `eager` failed probes the thread sleeps `sleep_ns` between probes (0 = never:
// for waits on the critical path, a sleep costs far more than the probes it saves), so
// a role that is far ahead of its consumer does not take issue slots from the warps
// doing the arithmetic; the clock is read only every 64 probes.
__device__ __forceinline__ bool mbar_wait_abortable(volatile int *abort, uint64_t *bar, uint32_t parity, uint32_t sleep_ns = 256u,
                                                    uint32_t eager = 2u)
{
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
#pragma unroll 1
    for (uint32_t spin = 1;; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (sleep_ns != 0u && spin > eager) __nanosleep(sleep_ns);
        if ((spin & 63u) == 0u && (*abort != 0 || clock64() - t0 > INKQ_SPIN_LIMIT_CYCLES)) return false;
    }
}
// Wait used when a kernel leaves after a failed wait: its own asynchronous copies may still be in flight and must
// land before the CTA's shared memory is given up.  Ignores any abort word; bounded by `limit_cycles` (copies complete
// within microseconds; the default is about a millisecond).
__device__ __forceinline__ bool mbar_wait_drain(uint64_t *bar, uint32_t parity, long long limit_cycles = 2000000LL)
{
    const long long t0 = clock64();
#pragma unroll 1
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(200u);
        if (clock64() - t0 > limit_cycles) return false;
    }
}
// ---- fences -------------------------------------------------------------------
// Make generic-proxy shared-memory writes visible to the async proxy (UMMA / TMA reads).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- TMA ------------------------------------------------------------------------
// Untiled bulk copy global -> shared, completion counted in bytes on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void tma_bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
// Tiled 2-D tensor copy global -> shared (no multicast).  x is the innermost
// coordinate; x * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_tensor2d_g2s(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tensor memory ------------------------------------------------------------------
// Whole-warp calls (.sync.aligned).
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- UMMA ----------------------------------------------------------------------------
// Shared-memory matrix descriptor (K-major operands).  Offsets are in bytes.
//   bits [0,14)  start address >> 4      bits [16,30) leading-dimension byte offset >> 4
//   bits [32,46) stride-dimension byte offset >> 4     bits [46,48) version = 1 (sm_100)
//   bits [61,64) swizzle mode: 0 none, 2 128-byte, 4 64-byte, 6 32-byte
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t swizzle_mode)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr >> 4) & 0x3FFFu);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= static_cast<uint64_t>(1) << 46;
    d |= static_cast<uint64_t>(swizzle_mode & 7u) << 61;
    return d;
}
// Instruction descriptor for kind::i8: D = s32, A and B signed 8-bit, both K-major.
//   bits [4,6) D format (2 = s32); [7,10) A format (1 = s8); [10,13) B format (1 = s8);
//   bit 15 / 16 A / B major (0 = K); [17,23) N >> 3; [24,29) M >> 4.
__device__ __host__ __forceinline__ uint32_t umma_idesc_i8(int umma_m, int umma_n)
{
    return (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(umma_n >> 3) << 17) | (static_cast<uint32_t>(umma_m >> 4) << 24);
}
// Instruction descriptor for kind::f16: D = f32 (1), A and B fp16 (0), K-major.
__device__ __host__ __forceinline__ uint32_t umma_idesc_f16(int umma_m, int umma_n)
{
    return (1u << 4) | (0u << 7) | (0u << 10) | (static_cast<uint32_t>(umma_n >> 3) << 17) | (static_cast<uint32_t>(umma_m >> 4) << 24);
}
// One thread issues.  D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- TMEM -> registers (whole warp; lane i reads TMEM lane base+i, N consecutive columns) ----
__device__ __forceinline__ void tmem_ld_x4(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t *r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_x16(uint32_t taddr, uint32_t *r)
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Per-warpgroup register re-balancing; all four warps of a warpgroup execute the same one.
// inc blocks until the CTA's other warpgroups have released enough registers with dec: the
// caller must make sure the requests never exceed the releases.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc()
{
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec()
{
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---- misc -----------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p)
{
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// 32 contiguous bytes in one request (256-bit load; p must be 32-byte aligned): a whole sector per lane
__device__ __forceinline__ void ldg_stream_v8(const void *p, uint4 &lo, uint4 &hi)
{
    asm("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
        : "l"(p));
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void *p)
{
    uint2 v;
    asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

}  // namespace inkq
