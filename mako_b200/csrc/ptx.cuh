// Thin wrappers over the sm_100a instructions the row pipeline uses: mbarrier (CTA scope), the untiled bulk
// asynchronous copy global -> shared (TMA, no multicast), named barriers. Every wait is bounded.
#pragma once
#include <cstdint>

namespace mk {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_barrier_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

// One potentially blocking probe of the barrier phase: the hardware parks the thread until the phase completes or
// the suspend-time hint (nanoseconds) runs out, so a waiting warp does not compete for issue slots by spinning.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after `limit` probes and reports false, so that a lost copy or a logic error ends the
// kernel with a status instead of hanging the GPU. (2^17 probes of up to 20 us each: a few seconds at most.)
// The same wait by polling (no suspension): for the one lane whose reaction time is on a ring stage's round trip.
// Bounded like the other: about a million probes.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22))
{
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok)
            return true;
    }
    return false;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 17))
{
    for (uint32_t i = 0; i < limit; ++i)
        if (mbar_try_wait(bar, parity))
            return true;
    return false;
}

// Untiled bulk copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16. The data is read once: it is marked evict-first in L2,
// so that a batch of rows larger than L2 does not push out what is used again (code, histories, scratch).
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar)
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// Programmatic dependent launch. wait: blocks until the grids this one was launched behind have completed and their
// writes are visible (returns at once in a launch without that dependency). launch_dependents: the grid launched
// behind this one may start being scheduled once every CTA of this grid has said so or exited.
__device__ __forceinline__ void griddep_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void griddep_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void named_barrier(uint32_t id, uint32_t n_threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n_threads) : "memory");
}

// Order-preserving map float -> uint32 (larger float, larger key); -0 is folded onto +0 first; NaN -> 0.
__device__ __forceinline__ uint32_t order_key(float v)
{
    if (v != v)
        return 0u;
    const uint32_t u = __float_as_uint(v + 0.0f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float key_to_float(uint32_t k)
{
    const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(u);
}

// 2^x on the special-function unit: relative error about 2^-22, results below 2^-126 flushed to zero, 2^-inf = +0.
// For sums whose error margin is reported with them; never for a weight the reference computes with expf.
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two fp32 lanes in one instruction (sm_100: fma/mul on a 64-bit register pair): halves the issue slots of a dot
// product whose operands already sit in adjacent registers (the halves of a float4).
__device__ __forceinline__ float2 mul2(float2 a, float2 b)
{
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c)
{
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

} // namespace mk
