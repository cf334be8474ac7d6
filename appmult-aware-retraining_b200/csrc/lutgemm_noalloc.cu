// Weight-gradient entry point that allocates nothing.
//
// Some callers cannot hand the library a scratch buffer because they are not allowed to allocate device
// memory at the point where the gradient is needed: a latency-critical path on which cudaMalloc (an
// implicit device synchronisation) is not acceptable, a host runtime that was given a fixed memory budget
// up front, or a binding without access to the caller's allocator.  For them the partial sums of the weight-gradient kernels live in a fixed array that is part
// of the library image: every GPU that loads the library holds these kNoAllocScratchBytes until the
// process exits, and problems whose partial sums do not fit are refused.
#include <cuda_runtime.h>

#include <mutex>

#include "lutgemm.h"
#include "lutgemm_kernels.h"

namespace {

constexpr size_t kNoAllocScratchBytes = size_t(LUTGEMM_NOALLOC_SCRATCH_BYTES);
constexpr int kMaxDevices = 64;

// The scratch itself.  In host code this name is only a handle for the runtime, not a device address;
// the address each device gave it is looked up once per device below and handed to the kernels.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices];  // per device, filled on the first call made with that device current

// Address of the scratch array on the current device, or nullptr after recording the CUDA error.
void *scratch_on_current_device() {
    int dev = 0;
    if (!lutgemm::cuda_ok(cudaGetDevice(&dev)) || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[dev]) return g_scratch_addr[dev];
    void *ptr = nullptr;
    if (!lutgemm::cuda_ok(cudaGetSymbolAddress(&ptr, g_noalloc_scratch)) || ptr == nullptr) return nullptr;
    g_scratch_addr[dev] = ptr;
    return ptr;
}

}  // namespace

extern "C" {

size_t lutgemm_noalloc_scratch_capacity(void) { return kNoAllocScratchBytes; }

int lutgemm_backward_gw_noalloc(const float *gc, const uint8_t *a, const uint8_t *w, float *gw,
                                const int16_t *lut_gw, int bits, int M, int K, int N, void *stream) {
    if (!gc || !a || !w || !gw || !lut_gw || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    void *scratch = scratch_on_current_device();
    if (!scratch) return LUTGEMM_E_CUDA;
    // Same kernels and dispatch as lutgemm_backward with ga == NULL; only the home of the partial sums
    // differs.  Every partial sum the reduction reads is written earlier in the same call, so nothing in
    // the array has to start at zero and nothing is cleared here.
    const int rc = lutgemm_backward(gc, a, w, nullptr, gw, nullptr, lut_gw, bits, M, K, N, scratch,
                                    kNoAllocScratchBytes, stream);
    return rc == LUTGEMM_E_SCRATCH ? LUTGEMM_E_TOOLARGE : rc;
}

}  // extern "C"
