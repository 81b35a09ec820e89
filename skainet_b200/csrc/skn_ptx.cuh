// Thin inline-PTX wrappers used by the sm_100a kernels: mbarrier, 1-D bulk async copy
// (TMA), programmatic dependent launch, packed fp32 arithmetic.  Every wait is bounded.
#pragma once
#include <stdint.h>

__device__ __forceinline__ uint32_t skn_smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void skn_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(skn_smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void skn_fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// orders this thread's earlier generic-proxy shared-memory accesses before later
// async-proxy (bulk copy) accesses
__device__ __forceinline__ void skn_fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void skn_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(skn_smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void skn_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(skn_smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool skn_mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(skn_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t skn_globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: gives up after ~2 s of wall time and returns false.  The caller records
// the failure in the status word and skips the work that depended on the data.
__device__ __forceinline__ bool skn_mbar_wait(uint64_t *bar, uint32_t parity) {
    if (skn_mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = skn_globaltimer_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 1024; ++i)
            if (skn_mbar_try_wait(bar, parity)) return true;
        if (skn_globaltimer_ns() - t0 > 2000000000ull) return false;
    }
}

// global -> shared bulk copy; src, dst 16-byte aligned, bytes a multiple of 16.
// Completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void skn_bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     skn_smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(skn_smem_u32(bar))
                 : "memory");
}

// programmatic dependent launch: block until the grids this one depends on have
// completed and their memory is visible (no-op when launched without the attribute)
__device__ __forceinline__ void skn_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// allow the next grid in the stream to start its prologue
__device__ __forceinline__ void skn_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// packed fp32: two independent fused multiply-adds per instruction
__device__ __forceinline__ uint64_t skn_pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ uint64_t skn_pack2u(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void skn_unpack2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t skn_fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t skn_add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
