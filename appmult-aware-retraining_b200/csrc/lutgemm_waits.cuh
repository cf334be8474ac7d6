// Bounded shared-memory barrier (mbarrier) waits for the sm_100a LUT-GEMM kernels.
//
// Warps of one CTA hand buffers to each other through mbarriers.  No wait in this library spins without a
// limit: after kWaitLimitNs the waiting thread records an id in a device error word (read and cleared by
// the host through lutgemm_device_error) and raises the CTA's abort word, which makes every later wait of
// that CTA return at once - the kernel always terminates, with a result the host knows to be invalid.
#pragma once

#include "lutgemm_common.cuh"

namespace lutgemm {

constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // one second per wait

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One attempt: returns at once when the phase with this parity is complete, otherwise the hardware suspends the
// thread until it completes or a short, implementation-defined time has passed (so a waiting warp does not
// spend issue slots and shared-memory bandwidth on polling).
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long wait_clock_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the phase with the given parity, for at most kWaitLimitNs.  `what` identifies the wait in the error
// word; `error_word` is the device-global word (device_error_word()), `abort_word` a word in the CTA's shared memory.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int what, volatile int *abort_word,
                                          int *error_word) {
    if (mbar_try(bar, parity)) return;
    const unsigned long long t0 = wait_clock_ns();
    do {
        if (mbar_try(bar, parity)) return;
        if (*abort_word) return;
    } while (wait_clock_ns() - t0 < kWaitLimitNs);
    *abort_word = 1;
    atomicExch(error_word, what);
}

// address of the device error word on the current device (nullptr if the lookup failed)
int *device_error_word();

}  // namespace lutgemm
