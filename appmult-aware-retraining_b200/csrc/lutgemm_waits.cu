// Device error word of the bounded waits (lutgemm_waits.cuh), its host-side reader, and a self-test kernel
// whose wait can never be satisfied: the time-out path is exercised without hanging a GPU.
#include "lutgemm_kernels.h"
#include "lutgemm_waits.cuh"

namespace lutgemm {

__device__ int g_wait_error = 0;  // 0 = ok, otherwise the id of the wait that gave up

int *device_error_word() {
    int *p = nullptr;
    if (!cuda_ok(cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_wait_error))) return nullptr;
    return p;
}

namespace {

// one warp waits on a barrier that nothing ever arrives on; the wait must run out, record id 99 and return
__global__ void bounded_wait_selftest_kernel(int *error_word) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar), 1);
    }
    __syncthreads();
    mbar_wait(smem_u32(&bar), 0, 99, &abort_word, error_word);
}

}  // namespace

int bounded_wait_selftest(cudaStream_t stream) {
    int *ew = device_error_word();
    if (!ew) return LUTGEMM_E_CUDA;
    bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(ew);
    return launch_status();
}

int read_and_clear_device_error(int *value) {
    int v = 0;
    if (!cuda_ok(cudaMemcpyFromSymbol(&v, g_wait_error, sizeof(int)))) return LUTGEMM_E_CUDA;
    if (v != 0) {
        const int zero = 0;
        if (!cuda_ok(cudaMemcpyToSymbol(g_wait_error, &zero, sizeof(int)))) return LUTGEMM_E_CUDA;
    }
    *value = v;
    return LUTGEMM_OK;
}

}  // namespace lutgemm
