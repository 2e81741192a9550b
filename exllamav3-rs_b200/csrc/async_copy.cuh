// mbarrier + bulk asynchronous copy (TMA unit, untiled) helpers for sm_100a.
// Every wait is bounded: after the limit the caller records a status word and leaves the kernel.
#pragma once
#include <stdint.h>

namespace exl3 {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// try_wait with a suspend-time hint: the thread may sleep up to `ns` nanoseconds inside the instruction instead of
// returning at once, which keeps waiting warps from eating issue slots.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait with sleeping polls (about limit * ns nanoseconds at most).
__device__ __forceinline__ bool mbar_wait_sleep(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 20), uint32_t ns = 2000)
{
    if (mbar_try_wait(bar, parity)) return true;
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait_hint(bar, parity, ns)) return true;
    return false;
}
// Bounded wait: false when the phase did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22))
{
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// Warp-uniform bounded wait: every lane polls, the warp agrees on the outcome (keeps .aligned instructions and
// __syncwarp that follow the wait convergent even if a time-out hits only some lanes).
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22))
{
    const bool ok = mbar_wait(bar, parity, limit);
    return __all_sync(0xffffffffu, ok);
}
// Warp-uniform form of mbar_wait_sleep.
__device__ __forceinline__ bool mbar_wait_sleep_warp(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 20), uint32_t ns = 2000)
{
    const bool ok = mbar_wait_sleep(bar, parity, limit, ns);
    return __all_sync(0xffffffffu, ok);
}
// global -> shared bulk copy; dst/src 16-byte aligned, bytes % 16 == 0; completion counted on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

}  // namespace exl3
