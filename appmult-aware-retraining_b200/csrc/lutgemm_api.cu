// C ABI of liblutgemm_b200.so (declared in include/lutgemm.h): argument validation and dispatch.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "lutgemm.h"
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace {

constexpr int kMaxDevices = 64;
int g_num_sms[kMaxDevices];  // 0 = not queried yet; written with the same value by every thread

int current_num_sms() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1;
    if (dev >= 0 && dev < kMaxDevices && g_num_sms[dev] > 0) return g_num_sms[dev];
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return -1;
    if (dev >= 0 && dev < kMaxDevices) g_num_sms[dev] = sms;
    return sms;
}

thread_local char g_msg[256];

}  // namespace

extern "C" {

int lutgemm_version(void) { return 100; }

const char *lutgemm_status_string(int status) {
    switch (status) {
        case LUTGEMM_OK: return "ok";
        case LUTGEMM_E_BADARG: return "bad argument (null pointer, non-positive size or misaligned buffer)";
        case LUTGEMM_E_BITS: return "unsupported bit-width (supported: 4, 6, 7, 8)";
        case LUTGEMM_E_SCRATCH: return "scratch buffer too small";
        case LUTGEMM_E_TOOLARGE: return "problem size beyond what this entry point supports";
        case LUTGEMM_E_CUDA: {
            cudaError_t e = cudaPeekAtLastError();
            snprintf(g_msg, sizeof(g_msg), "CUDA failure: %s", cudaGetErrorString(e));
            return g_msg;
        }
    }
    return "unknown status";
}

int lutgemm_lut_elem_num(int bits) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    return lutgemm::lut_elem_num(bits);
}

int lutgemm_bits_from_elem_num(long elem_num) {
    const int all[4] = {4, 6, 7, 8};
    for (int b : all)
        if (lutgemm::lut_elem_num(b) == elem_num) return b;
    return LUTGEMM_E_BITS;
}

int lutgemm_forward(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                    int N, void *stream) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (!a || !w || !c || !lut || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(c) & 3) || (reinterpret_cast<uintptr_t>(lut) & 1)) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    // Large-M problems with reasonably filled 512x64 tiles go to the slab kernel; small or skinny ones
    // to the row-broadcast kernel.  LUTGEMM_FORWARD_KERNEL=rowbcast|slab overrides (for A/B timing).
    const long tm = (M + 511) / 512, tn = (N + 63) / 64;
    const double fill = (double)M * N / ((double)tm * 512 * tn * 64);
    bool slab = M >= 512 && N >= 32 && fill >= 0.6;
    if (const char *force = getenv("LUTGEMM_FORWARD_KERNEL")) {
        if (!strcmp(force, "rowbcast")) slab = false;
        if (!strcmp(force, "slab")) slab = true;
    }
    if (slab) return lutgemm::forward_slab(a, w, c, lut, bits, M, K, N, sms, static_cast<cudaStream_t>(stream));
    return lutgemm::forward_rowbcast(a, w, c, lut, bits, M, K, N, sms, static_cast<cudaStream_t>(stream));
}

size_t lutgemm_backward_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || M <= 0 || K <= 0 || N <= 0) return 0;
    const int sms = current_num_sms();
    if (sms <= 0) return 0;
    const int splits = lutgemm::gw_num_splits(bits, M, K, N, sms);
    return splits > 1 ? (size_t)splits * K * N * sizeof(float) : 0;
}

int lutgemm_backward(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                     const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N, void *scratch,
                     size_t scratch_bytes, void *stream) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (!gc || !a || !w || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    if ((ga && !lut_ga) || (gw && !lut_gw)) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(gc) & 3) || (reinterpret_cast<uintptr_t>(ga) & 3) ||
        (reinterpret_cast<uintptr_t>(gw) & 3) || (reinterpret_cast<uintptr_t>(scratch) & 3) ||
        (reinterpret_cast<uintptr_t>(lut_ga) & 1) || (reinterpret_cast<uintptr_t>(lut_gw) & 1))
        return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gw) {
        // the weight gradient goes first: under data parallelism its all-reduce can then overlap gA
        const int splits = lutgemm::gw_num_splits(bits, M, K, N, sms);
        if (splits > 1 && (!scratch || scratch_bytes < (size_t)splits * K * N * sizeof(float)))
            return LUTGEMM_E_SCRATCH;
        int rc = lutgemm::backward_gw(gc, a, w, gw, lut_gw, bits, M, K, N, static_cast<float *>(scratch), splits, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    if (ga) {
        int rc = lutgemm::backward_ga(gc, a, w, ga, lut_ga, bits, M, K, N, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

}  // extern "C"
