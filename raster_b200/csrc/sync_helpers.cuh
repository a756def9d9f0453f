// Device helpers shared by the kernels that use mbarriers and bulk async copies:
// barrier init / arrive / time-bounded wait, the global timer, 1-D bulk copies.
#pragma once
#include <stdint.h>

namespace rstq {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");  // no state token: nothing to wait for
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar),
                 "r"(bytes)
                 : "memory");
}
// Raise the phase's expected byte count without arriving: for copies that complete on a barrier whose
// (single) arrival comes later, with the rest of the bytes.
__device__ __forceinline__ void mbar_expect_only(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// non-blocking test of a phase
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long gtime_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Slow path of a time-bounded wait.  Returns false when the limit ran out or
// another warp already gave up (abort flag); the caller then skips its work but
// keeps meeting every CTA barrier so nobody is left waiting.
static __device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    const unsigned long long t0 = gtime_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try(bar, parity)) return true;
        if (*abort_flag) return false;
        if (gtime_ns() - t0 > kWaitLimitNs) {
            *abort_flag = 1;
            return false;
        }
    }
}
// Wait with a short inline spin first (the common case: the other side is a few hundred
// cycles away), then the timed slow path.
__device__ __forceinline__ bool mbar_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
#pragma unroll 1
    for (int i = 0; i < 1024; ++i)
        if (mbar_test(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag);
}
// Wait of a warp that is not on the critical path: mbarrier.try_wait suspends the thread in
// hardware until the phase completes or a system time limit passes, so a waiting warp issues a
// handful of instructions per microsecond instead of a polling loop that competes for issue
// slots with the warps doing the work.
__device__ __forceinline__ bool mbar_block(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_test(bar, parity)) return true;  // one instruction when the phase is already complete
#pragma unroll 1
    for (int i = 0; i < 256; ++i)  // each try may suspend for a while: no timer reads on this path
        if (mbar_try(bar, parity)) return true;
    return mbar_wait(bar, parity, abort_flag);
}
// Warp-wide wait that polls from lane 0 only, sleeping between polls: a producer warp that is
// a long way ahead of its consumer then leaves the barrier unit and the issue slots to the
// warps that are on the critical path.  All 32 lanes must call it; all get the same answer.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    int got = 1;
    if ((threadIdx.x & 31) == 0) {
        got = 0;
#pragma unroll 1
        for (int i = 0; i < 4096 && !got; ++i) {
            got = mbar_test(bar, parity);
            if (!got) __nanosleep(32);
        }
        if (!got) got = mbar_wait(bar, parity, abort_flag);
    }
    return __shfl_sync(0xffffffffu, got, 0) != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                              uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}
// The same copy with an L2 eviction hint: data that is read once (a weight stream) is marked
// evict-first so that it does not push the small, reused buffers (activations, scratch) out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_copy_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                                   uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
}  // namespace rstq
