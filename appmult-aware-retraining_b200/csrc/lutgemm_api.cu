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

// tile fill of a [rows x cols] problem cut into 512 x 64 slab tiles
double slab_fill(long rows, long cols) {
    const long tr = (rows + 511) / 512, tc = (cols + 63) / 64;
    return (double)rows * (double)cols / ((double)tr * 512.0 * (double)tc * 64.0);
}

bool env_is(const char *name, const char *value) {
    const char *e = getenv(name);
    return e && !strcmp(e, value);
}

struct BackwardPlan {
    bool gw_slab, ga_slab;
    int gw_splits;        // row-broadcast grad_w kernel: slabs of M
    size_t gw_scratch, ga_scratch;
};

// Kernel choice for the two gradients.  Slab kernels amortise one slab build over 512 rows of the
// reduction dimension (M for grad_w, N for grad_a), so they need that dimension long and the tiles
// reasonably full; everything else goes to the row/column-broadcast kernels.
// LUTGEMM_BACKWARD_KERNEL=bcast|slab overrides (for A/B timing).
BackwardPlan plan_backward(int bits, int M, int K, int N, int sms) {
    BackwardPlan pl{};
    // measured on B200 at 4096^3: the gradient slab kernels beat the broadcast kernels only where the
    // latter suffer bank conflicts (7 and 8 bits); at 4 and 6 bits a table row is conflict-free already
    pl.gw_slab = bits >= 7 && M >= 512 && N >= 32 && slab_fill(M, N) >= 0.6;
    pl.ga_slab = bits >= 7 && N >= 384 && M >= 32 && slab_fill(N, M) >= 0.6;
    if (env_is("LUTGEMM_BACKWARD_KERNEL", "bcast")) pl.gw_slab = pl.ga_slab = false;
    if (env_is("LUTGEMM_BACKWARD_KERNEL", "slab")) pl.gw_slab = pl.ga_slab = true;
    pl.gw_splits = pl.gw_slab ? 1 : lutgemm::gw_num_splits(bits, M, K, N, sms);
    if (pl.gw_slab) {
        const int rb = lutgemm::slab_grad_row_blocks(M);
        pl.gw_scratch = rb > 1 ? (size_t)rb * K * N * sizeof(float) : 0;
    } else {
        pl.gw_scratch = pl.gw_splits > 1 ? (size_t)pl.gw_splits * K * N * sizeof(float) : 0;
    }
    if (pl.ga_slab) {
        const int rb = lutgemm::slab_grad_row_blocks(N);
        pl.ga_scratch = rb > 1 ? (size_t)rb * K * M * sizeof(float) : 0;
    }
    return pl;
}

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
    if (slab) {
        // Two implementations of the slab algorithm: barrier-synchronous (default: faster on B200 at 7 and
        // 8 bits, 12.8 vs 17.6 ms at 8-bit 4096^3, where four producer warps cannot build slabs fast
        // enough) and warp-specialised (LUTGEMM_SLAB_IMPL=ws).
        if (env_is("LUTGEMM_SLAB_IMPL", "ws"))
            return lutgemm::forward_slab_ws(a, w, c, lut, bits, M, K, N, sms, static_cast<cudaStream_t>(stream));
        return lutgemm::forward_slab(a, w, c, lut, bits, M, K, N, sms, static_cast<cudaStream_t>(stream));
    }
    return lutgemm::forward_rowbcast(a, w, c, lut, bits, M, K, N, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_device_error(int *value) {
    if (!value) return LUTGEMM_E_BADARG;
    return lutgemm::slab_ws_read_and_clear_error(value);
}

int lutgemm_selftest_bounded_wait(void *stream) {
    return lutgemm::slab_ws_bounded_wait_selftest(static_cast<cudaStream_t>(stream));
}

size_t lutgemm_backward_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || M <= 0 || K <= 0 || N <= 0) return 0;
    const int sms = current_num_sms();
    if (sms <= 0) return 0;
    const BackwardPlan pl = plan_backward(bits, M, K, N, sms);
    return pl.gw_scratch > pl.ga_scratch ? pl.gw_scratch : pl.ga_scratch;
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
    const BackwardPlan pl = plan_backward(bits, M, K, N, sms);
    float *sc = static_cast<float *>(scratch);
    if (gw) {
        // the weight gradient goes first: under data parallelism its all-reduce can then overlap gA
        if (pl.gw_scratch && (!scratch || scratch_bytes < pl.gw_scratch)) return LUTGEMM_E_SCRATCH;
        const bool sync_impl = !env_is("LUTGEMM_SLAB_IMPL", "ws");
        int rc = !pl.gw_slab ? lutgemm::backward_gw(gc, a, w, gw, lut_gw, bits, M, K, N, sc, pl.gw_splits, sms, s)
                 : sync_impl ? lutgemm::backward_gw_slab(gc, a, w, gw, lut_gw, bits, M, K, N, sc, sms, s)
                             : lutgemm::backward_gw_slab_ws(gc, a, w, gw, lut_gw, bits, M, K, N, sc, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    if (ga) {
        if (pl.ga_scratch && (!scratch || scratch_bytes < pl.ga_scratch)) return LUTGEMM_E_SCRATCH;
        const bool sync_impl = !env_is("LUTGEMM_SLAB_IMPL", "ws");
        int rc = !pl.ga_slab ? lutgemm::backward_ga(gc, a, w, ga, lut_ga, bits, M, K, N, sms, s)
                 : sync_impl ? lutgemm::backward_ga_slab(gc, a, w, ga, lut_ga, bits, M, K, N, sc, sms, s)
                             : lutgemm::backward_ga_slab_ws(gc, a, w, ga, lut_ga, bits, M, K, N, sc, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

}  // extern "C"
