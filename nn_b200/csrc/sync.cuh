// Shared-memory barrier and bulk-copy helpers (inline PTX) used by the streaming kernels.
// Every wait is bounded: it gives up after kWaitSpins tries and reports failure to its caller,
// which records it in the context's status word and unwinds.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace nnq {

constexpr unsigned kWaitSpins = 1u << 19;    // bound of every mbarrier wait (about a second in all)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// global -> shared bulk copy (one contiguous tile), completion counted on an mbarrier
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    // the last operand caps the time one try may suspend the thread (nanoseconds)
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
// Bounded wait: returns false when the limit ran out (the caller records it and bails out).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    for (unsigned i = 0; i < kWaitSpins; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}


// Bounded wait written as one PTX loop: try, leave on success, else count down.
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n .reg .u32 n;\n mov.u32 n, %3;\n"
        "W_%=:\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n @p bra D_%=;\n"
        " sub.u32 n, n, 1;\n setp.ne.u32 p, n, 0;\n @p bra W_%=;\n mov.u32 %0, 0;\n bra E_%=;\n"
        "D_%=:\n mov.u32 %0, 1;\nE_%=:\n}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(kWaitSpins) : "memory");
    return ok != 0;
}

}  // namespace nnq
