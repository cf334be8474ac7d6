// Bounded shared-memory barrier (mbarrier) waits for the sm_100a LUT-GEMM kernels.
//
// Warps of one CTA hand buffers to each other through mbarriers.  No wait in this library spins without a
// limit: after kWaitLimit polls the waiting thread records an id in a device error word (read and cleared by
// the host through lutgemm_device_error) and raises the CTA's abort word, which makes every later wait of
// that CTA return at once - the kernel always terminates, with a result the host knows to be invalid.
#pragma once

#include "lutgemm_common.cuh"

namespace lutgemm {

constexpr int kWaitLimit = 1 << 22;  // polls; with the back-off below a fraction of a second

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity.  `what` identifies the wait in the error word; `error_word` is
// the device-global word (device_error_word()), `abort_word` a word in the CTA's shared memory.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int what, volatile int *abort_word,
                                          int *error_word) {
    for (int i = 0; i < kWaitLimit; ++i) {
        if (mbar_test(bar, parity)) return;
        if (i > 64) {
            if (*abort_word) return;
            __nanosleep(32);
        }
    }
    *abort_word = 1;
    atomicExch(error_word, what);
}

// address of the device error word on the current device (nullptr if the lookup failed)
int *device_error_word();

}  // namespace lutgemm
