// Bulk-async (TMA, untiled) weight streaming primitives: mbarrier set-up, bounded waits, and
// global->shared bulk copies that complete on an mbarrier.  No cluster multicast is used anywhere.
//
// A memory-bound decode kernel keeps HBM busy by having tens of KB of bulk copies in flight per
// SM, issued by one thread; because weights never depend on the previous kernel, the first stages
// are issued before the kernel waits for its predecessor (programmatic dependent launch), so the
// data is already in shared memory when the predecessor's results become visible.
#pragma once
#include "common.cuh"

namespace qw {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Barrier among the first `nthreads` threads of the block (the consumer warps), id 1.
__device__ __forceinline__ void consumer_sync(int nthreads) { asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory"); }

// 16-byte aligned addresses, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Waits for the phase with the given parity.  Bounded: gives up after `limit` polls (each poll may
// itself block for a hardware-defined time), records ERR_WAIT_TIMEOUT and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, unsigned parity, ErrorWord *err, unsigned limit = 1u << 22) {
    const uint32_t a = smem_u32(bar);
    for (unsigned i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(a), "r"(parity)
            : "memory");
        if (ok) return true;
        // another waiter already gave up (e.g. the role that feeds this barrier): do not sit out the whole limit
        if (err && (i & 255u) == 255u && *reinterpret_cast<volatile unsigned int *>(&err->code)) return false;
    }
    report(err, ERR_WAIT_TIMEOUT, __LINE__);
    return false;
}

}  // namespace qw
