// Waiting primitives shared by the persistent single-token decode kernels: mbarrier and bulk-copy wrappers,
// relaxed / acquire loads for polling, and a grid-wide barrier over a monotonic counter.  Every wait is bounded: after ~2 s it sets a bit in the
// device status word, every CTA sees the bit at its next wait and returns.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace uocr {

constexpr long long kSpinLimit = 4000000000LL;   // cycles
constexpr uint32_t kStatusRouter = 1u, kStatusBarrier = 2u, kStatusCopy = 4u, kStatusRange = 16u;

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// 1-D bulk copy global -> shared; size and both addresses are multiples of 16 bytes
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Bounded wait on an mbarrier phase.  Returns false after the limit (status bit set).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t *status, int *s_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kSpinLimit) {
            atomicOr(status, kStatusCopy);
            s_flag[1] = 1;
            // one more bounded wait so that the copy does not land after this CTA has gone
            const long long t1 = clock64();
            while (!mbar_try_wait(bar, parity) && clock64() - t1 < kSpinLimit) {}
            return false;
        }
    }
    return true;
}

// Grid-wide barrier over a monotonic counter.  All CTAs are co-resident (cooperative launch).
// Arrival is a release (it orders the whole CTA's earlier writes, which reached thread 0 through the CTA
// barrier); the wait polls with relaxed loads and ends with one fence.
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool grid_barrier(unsigned long long *ctr, unsigned long long target, uint32_t *status,
                                             int *s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        red_release_add_u64(ctr, 1ULL);
        int ok = 1;
        if (ld_relaxed_u64(ctr) < target) {
            const long long t0 = clock64();
            uint32_t polls = 0;
            while (ld_relaxed_u64(ctr) < target) {
                if ((++polls & 63u) == 0u) {
                    if (ld_volatile_u32(status) & (kStatusBarrier | kStatusCopy)) { ok = 0; break; }
                    if (clock64() - t0 > kSpinLimit) { atomicOr(status, kStatusBarrier); ok = 0; break; }
                }
            }
        }
        __threadfence();
        if (s_flag[1] != 0) ok = 0;     // a bulk copy of this CTA timed out: leave; the others time out in turn
        *s_flag = ok;
    }
    __syncthreads();
    return *s_flag != 0;
}

}  // namespace uocr
