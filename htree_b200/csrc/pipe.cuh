// Asynchronous bulk copies global -> shared memory completing on an mbarrier (the TMA engine of sm_90+/sm_100), and the
// bounded waits that go with them.  Used by the pipelined tensor-core forward: a warp keeps the operand blocks of its
// next chunks in flight into its own shared-memory ring while it computes the current one, without holding registers
// for them.  Single-CTA copies only: every source is this GPU's own memory and no copy is shared between CTAs.
#pragma once
#include <stdint.h>

namespace htree {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// makes freshly initialised barriers visible to the asynchronous proxy that completes the copies on them
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
// orders this thread's earlier generic-proxy accesses of shared memory before later asynchronous-proxy writes to it
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// one arrival plus the announcement of `bytes` bytes that the copies issued next will deliver
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// `bytes` (a multiple of 16) from global memory (16-byte aligned) to this CTA's shared memory (16-byte aligned)
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// One attempt to see phase `parity` of the barrier completed; the instruction may suspend the warp for a bounded,
// implementation-defined time.  Callers loop with an iteration limit.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: false if the phase did not complete within `cap` attempts (the caller then flags the error, waits - again
// bounded - for the copies it still has in flight, and returns).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int cap) {
    for (int it = 0; it < cap; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)));
    return v;
}

}  // namespace htree
