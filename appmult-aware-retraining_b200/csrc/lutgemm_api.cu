// C ABI of liblutgemm_b200.so (declared in include/lutgemm.h): argument validation and dispatch.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "lutgemm.h"
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace {

constexpr int kMaxDevices = 64;
int g_num_sms[kMaxDevices];  // 0 = not queried yet; written with the same value by every thread

int current_num_sms() {
    int dev = 0;
    if (!lutgemm::cuda_ok(cudaGetDevice(&dev))) return -1;
    if (dev >= 0 && dev < kMaxDevices && g_num_sms[dev] > 0) return g_num_sms[dev];
    int sms = 0;
    if (!lutgemm::cuda_ok(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) || sms <= 0) return -1;
    if (dev >= 0 && dev < kMaxDevices) g_num_sms[dev] = sms;
    return sms;
}

thread_local char g_msg[256];

// tile fill of a [rows x cols] problem cut into 512 x 64 slab tiles
double slab_fill(long rows, long cols) {
    const long tr = (rows + 511) / 512, tc = (cols + 63) / 64;
    return (double)rows * (double)cols / ((double)tr * 512.0 * (double)tc * 64.0);
}

// tile fill of a [rows x cols] problem cut into 1024 x 32 slab tiles
double tall_fill(long rows, long cols) {
    const long tr = (rows + 1023) / 1024, tc = (cols + 31) / 32;
    return (double)rows * (double)cols / ((double)tr * 1024.0 * (double)tc * 32.0);
}

// kernel-family overrides set through lutgemm_set_kernel_choice (0 = automatic choice by shape)
std::atomic<int> g_force_forward{0}, g_force_backward{0}, g_force_tile{0};

// the CUDA error behind the calling thread's last LUTGEMM_E_CUDA (launchers clear the runtime's own record)
thread_local cudaError_t g_last_cuda_error = cudaSuccess;

// kernels launched by this library in this process (every launch site reports through launch_status)
std::atomic<unsigned long long> g_kernel_launches{0};

struct BackwardPlan {
    bool gw_slab, ga_slab;
    bool gw_tall, ga_tall;  // slab kernel with the 1024 x 32 tile instead of 512 x 64
    int gw_splits;        // row-broadcast grad_w kernel: slabs of M
    size_t gw_scratch, ga_scratch;
    // slab grad_w kernels read the activation codes from a transposed copy at[k][m] kept behind the partial
    // sums in the scratch buffer (their row-code fetch is then coalesced; for a convolution it also
    // replaces one implicit-im2col gather per column tile by a single one)
    size_t gw_at_offset;  // bytes into the scratch buffer, a multiple of 16
    int gw_at_pitch;      // 0 = no transposed copy
};

// Kernel choice for the two gradients.  Slab kernels amortise one slab build over 512 rows of the
// reduction dimension (M for grad_w, N for grad_a), so they need that dimension long and the tiles
// reasonably full; everything else goes to the row/column-broadcast kernels.
// lutgemm_set_kernel_choice overrides the choice (tests, A/B timing).
BackwardPlan plan_backward(int bits, int M, int K, int N, int sms) {
    BackwardPlan pl{};
    // measured on B200 at 4096^3 (ms, grad_w / grad_a): tall fp32-slab 15.9 / 16.4 (8 bit), 14.1 / 14.4 (7 bit)
    // against broadcast about 24 / 24 and 17 / 17: the slab kernels win where the broadcast gathers suffer
    // bank conflicts (7 and 8 bits); at 4 and 6 bits a table row is conflict-free and the broadcast kernels
    // (11.5 / 11.6) beat the slab kernels.  grad_a needs N >= 768 for a slab: on convolution shapes with
    // N <= 512 the column-broadcast kernel is faster at both 7 and 8 bits.
    pl.gw_slab = bits >= 7 && M >= 512 && N >= 32 && slab_fill(M, N) >= 0.6;
    // (a partly filled slab tile only pays against the column-broadcast kernel, which runs at about 37 % of the
    // roofline at 7 bits and 29 % at 8 bits whatever N is, when the better of the two tilings is this full)
    const double ga_fill = slab_fill(N, M) > tall_fill(N, M) ? slab_fill(N, M) : tall_fill(N, M);
    pl.ga_slab = bits >= 7 && N >= 768 && M >= 32 && ga_fill >= (bits == 7 ? 0.85 : 0.7);
    const int force = g_force_backward.load(std::memory_order_relaxed), tile = g_force_tile.load(std::memory_order_relaxed);
    if (force == LUTGEMM_BACKWARD_BCAST) pl.gw_slab = pl.ga_slab = false;
    if (force == LUTGEMM_BACKWARD_SLAB) pl.gw_slab = pl.ga_slab = true;
    // (the tall kernel is the faster one per look-up: at N = 1536, where its tiles are 75 % full and the wide ones
    // full, grad_a of a 12608 x 384 problem takes 1.82 against 1.89 ms, at N = 2560 (83 %) 2.40 against 2.76 ms)
    pl.gw_tall = pl.gw_slab && tall_fill(M, N) >= 0.7 * slab_fill(M, N);
    pl.ga_tall = pl.ga_slab && tall_fill(N, M) >= 0.7 * slab_fill(N, M);
    if (tile == LUTGEMM_TILE_WIDE) pl.gw_tall = pl.ga_tall = false;
    if (tile == LUTGEMM_TILE_TALL) { pl.gw_tall = pl.gw_slab; pl.ga_tall = pl.ga_slab; }
    pl.gw_splits = pl.gw_slab ? 1 : lutgemm::gw_num_splits(bits, M, K, N, sms);
    if (pl.gw_slab) {
        const int rb = pl.gw_tall ? lutgemm::slab_tall_row_blocks(M) : lutgemm::slab_f32_row_blocks(M);
        pl.gw_scratch = rb > 1 ? (size_t)rb * K * N * sizeof(float) : 0;
        pl.gw_at_offset = (pl.gw_scratch + 15) & ~(size_t)15;
        pl.gw_at_pitch = (M + 15) & ~15;
        pl.gw_scratch = pl.gw_at_offset + (size_t)pl.gw_at_pitch * K;
    } else {
        pl.gw_scratch = pl.gw_splits > 1 ? (size_t)pl.gw_splits * K * N * sizeof(float) : 0;
    }
    if (pl.ga_slab) {
        const int rb = pl.ga_tall ? lutgemm::slab_tall_row_blocks(N) : lutgemm::slab_f32_row_blocks(N);
        pl.ga_scratch = rb > 1 ? (size_t)rb * K * M * sizeof(float) : 0;
    }
    return pl;
}

}  // namespace

namespace lutgemm {

void record_cuda_error(cudaError_t e) { g_last_cuda_error = e; }

int launch_status() {
    g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return LUTGEMM_OK;
    g_last_cuda_error = e;
    return LUTGEMM_E_CUDA;
}

}  // namespace lutgemm

extern "C" {

int lutgemm_version(void) { return 200; }

const char *lutgemm_status_string(int status) {
    switch (status) {
        case LUTGEMM_OK: return "ok";
        case LUTGEMM_E_BADARG: return "bad argument (null pointer, non-positive size or misaligned buffer)";
        case LUTGEMM_E_BITS: return "unsupported bit-width (supported: 4, 6, 7, 8)";
        case LUTGEMM_E_SCRATCH: return "scratch buffer too small";
        case LUTGEMM_E_TOOLARGE: return "problem size beyond what this entry point supports";
        case LUTGEMM_E_CUDA: {
            snprintf(g_msg, sizeof(g_msg), "CUDA failure: %s", cudaGetErrorString(g_last_cuda_error));
            return g_msg;
        }
    }
    return "unknown status";
}

int lutgemm_set_tma(int on) {
    lutgemm::slab_fwd_set_tma(on != 0);
    return LUTGEMM_OK;
}

int lutgemm_set_handover(int on) {
    lutgemm::slab_tall_set_handover(on != 0);
    return LUTGEMM_OK;
}

unsigned long long lutgemm_kernel_launches(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

int lutgemm_set_kernel_choice(int forward, int backward, int grad_tile) {
    if (forward < 0 || forward > 2 || backward < 0 || backward > 2 || grad_tile < 0 || grad_tile > 2)
        return LUTGEMM_E_BADARG;
    g_force_forward.store(forward, std::memory_order_relaxed);
    g_force_backward.store(backward, std::memory_order_relaxed);
    g_force_tile.store(grad_tile, std::memory_order_relaxed);
    return LUTGEMM_OK;
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

// ---- shared bodies of the GEMM and the implicit-im2col entry points ------------------------------------
// Large-M problems with reasonably filled 512x64 tiles go to the slab kernel; small or skinny ones to the
// row-broadcast kernel.  lutgemm_set_kernel_choice overrides the choice (tests, A/B timing).
static bool forward_uses_slab(int M, int N) {
    bool slab = M >= 512 && N >= 32 && slab_fill(M, N) >= 0.6;
    const int force = g_force_forward.load(std::memory_order_relaxed);
    if (force == LUTGEMM_FORWARD_ROWBCAST) slab = false;
    if (force == LUTGEMM_FORWARD_SLAB) slab = true;
    return slab;
}

static int codes_pitch(int M) { return (M + 15) & ~15; }

// `scratch` (optional, K * codes_pitch(M) bytes, 16-byte aligned): the slab kernel then reads the activation
// codes from a transposed copy made there first, which stays valid on return.
static int forward_impl(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                        int N, const lutgemm::ConvGeom &conv, void *scratch, size_t scratch_bytes, void *stream,
                        const lutgemm::LayerEpilogue *epi = nullptr) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (!a || !w || (!c && !epi) || !lut || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(c) & 3) || (reinterpret_cast<uintptr_t>(lut) & 1) ||
        (reinterpret_cast<uintptr_t>(scratch) & 15))
        return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (forward_uses_slab(M, N)) {
        const uint8_t *at = nullptr;
        const int pitch = codes_pitch(M);
        if (scratch) {
            if (scratch_bytes < (size_t)pitch * K) return LUTGEMM_E_SCRATCH;
            const int trc = lutgemm::transpose_codes(a, static_cast<uint8_t *>(scratch), M, K, pitch, conv, bits, s);
            if (trc != LUTGEMM_OK) return trc;
            at = static_cast<const uint8_t *>(scratch);
        }
        return lutgemm::forward_slab(a, w, c, lut, bits, M, K, N, conv, at, pitch, epi, sms, s);
    }
    return lutgemm::forward_rowbcast(a, w, c, lut, bits, M, K, N, conv, epi, sms, s);
}

int lutgemm_forward(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                    int N, void *stream) {
    lutgemm::ConvGeom none{};
    return forward_impl(a, w, c, lut, bits, M, K, N, none, nullptr, 0, stream);
}

size_t lutgemm_forward_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || M <= 0 || K <= 0 || N <= 0) return 0;
    if (!forward_uses_slab(M, N)) return 0;
    return (size_t)codes_pitch(M) * K;
}

int lutgemm_forward_ws(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                       int N, void *scratch, size_t scratch_bytes, void *stream) {
    lutgemm::ConvGeom none{};
    return forward_impl(a, w, c, lut, bits, M, K, N, none, scratch, scratch_bytes, stream);
}

int lutgemm_device_error(int *value) {
    if (!value) return LUTGEMM_E_BADARG;
    return lutgemm::read_and_clear_device_error(value);
}

int lutgemm_selftest_bounded_wait(void *stream) {
    return lutgemm::bounded_wait_selftest(static_cast<cudaStream_t>(stream));
}

size_t lutgemm_backward_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || M <= 0 || K <= 0 || N <= 0) return 0;
    const int sms = current_num_sms();
    if (sms <= 0) return 0;
    const BackwardPlan pl = plan_backward(bits, M, K, N, sms);
    return pl.gw_scratch > pl.ga_scratch ? pl.gw_scratch : pl.ga_scratch;
}

static int backward_impl(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                         const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N,
                         const lutgemm::ConvGeom &conv, const uint8_t *codes_t, void *scratch, size_t scratch_bytes,
                         void *stream) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (!gc || !a || !w || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    if ((ga && !lut_ga) || (gw && !lut_gw)) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(gc) & 3) || (reinterpret_cast<uintptr_t>(ga) & 3) ||
        (reinterpret_cast<uintptr_t>(gw) & 3) || (reinterpret_cast<uintptr_t>(scratch) & 15) ||
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
        const uint8_t *at = codes_t;  // left by the forward pass (same layout), or made here
        if (pl.gw_slab && pl.gw_at_pitch && !at) {
            uint8_t *dst = static_cast<uint8_t *>(scratch) + pl.gw_at_offset;
            const int trc = lutgemm::transpose_codes(a, dst, M, K, pl.gw_at_pitch, conv, bits, s);
            if (trc != LUTGEMM_OK) return trc;
            at = dst;
        }
        int rc = !pl.gw_slab ? lutgemm::backward_gw(gc, a, w, gw, lut_gw, bits, M, K, N, conv, sc, pl.gw_splits, sms, s)
                 : pl.gw_tall ? lutgemm::backward_gw_slab_tall(gc, a, w, gw, lut_gw, nullptr, bits, M, K, N, conv, sc, at, pl.gw_at_pitch, sms, s)
                             : lutgemm::backward_gw_slab_f32(gc, a, w, gw, lut_gw, bits, M, K, N, conv, sc, at, pl.gw_at_pitch, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    if (ga) {
        if (pl.ga_scratch && (!scratch || scratch_bytes < pl.ga_scratch)) return LUTGEMM_E_SCRATCH;
        int rc = !pl.ga_slab ? lutgemm::backward_ga(gc, a, w, ga, lut_ga, bits, M, K, N, conv, sms, s)
                 : pl.ga_tall ? lutgemm::backward_ga_slab_tall(gc, a, w, ga, lut_ga, nullptr, bits, M, K, N, conv, sc, sms, s)
                             : lutgemm::backward_ga_slab_f32(gc, a, w, ga, lut_ga, bits, M, K, N, conv, sc, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

int lutgemm_backward(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                     const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N, void *scratch,
                     size_t scratch_bytes, void *stream) {
    lutgemm::ConvGeom none{};
    return backward_impl(gc, a, w, ga, gw, lut_ga, lut_gw, bits, M, K, N, none, nullptr, scratch, scratch_bytes, stream);
}

int lutgemm_backward_ws(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                        const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N,
                        const uint8_t *codes_t, void *scratch, size_t scratch_bytes, void *stream) {
    if (reinterpret_cast<uintptr_t>(codes_t) & 15) return LUTGEMM_E_BADARG;
    lutgemm::ConvGeom none{};
    return backward_impl(gc, a, w, ga, gw, lut_ga, lut_gw, bits, M, K, N, none, codes_t, scratch, scratch_bytes, stream);
}

// ---- gradient tables in fp32 (bits <= 7) -------------------------------------------------------------------------
// Always the tall slab kernels: their fp32 shared-memory table takes either entry type; tiles of small problems
// are mostly empty, which costs time, not correctness.
size_t lutgemm_backward_f32lut_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || bits > 7 || M <= 0 || K <= 0 || N <= 0) return 0;
    const size_t rb_w = lutgemm::slab_tall_row_blocks(M), rb_a = lutgemm::slab_tall_row_blocks(N);
    const size_t gw_need = rb_w > 1 ? rb_w * K * N * sizeof(float) : 0;
    const size_t ga_need = rb_a > 1 ? rb_a * K * M * sizeof(float) : 0;
    return gw_need > ga_need ? gw_need : ga_need;
}

int lutgemm_backward_f32lut(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                            const float *lut_ga, const float *lut_gw, int bits, int M, int K, int N, void *scratch,
                            size_t scratch_bytes, void *stream) {
    if (!lutgemm::bits_supported(bits) || bits > 7) return LUTGEMM_E_BITS;
    if (!gc || !a || !w || M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    if ((ga && !lut_ga) || (gw && !lut_gw)) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(gc) & 3) || (reinterpret_cast<uintptr_t>(ga) & 3) ||
        (reinterpret_cast<uintptr_t>(gw) & 3) || (reinterpret_cast<uintptr_t>(scratch) & 15) ||
        (reinterpret_cast<uintptr_t>(lut_ga) & 3) || (reinterpret_cast<uintptr_t>(lut_gw) & 3))
        return LUTGEMM_E_BADARG;
    if (lutgemm_backward_f32lut_scratch_bytes(bits, M, K, N) > (scratch ? scratch_bytes : 0)) return LUTGEMM_E_SCRATCH;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    lutgemm::ConvGeom none{};
    float *sc = static_cast<float *>(scratch);
    if (gw) {
        const int rc = lutgemm::backward_gw_slab_tall(gc, a, w, gw, nullptr, lut_gw, bits, M, K, N, none, sc, nullptr, 0, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    if (ga) {
        const int rc = lutgemm::backward_ga_slab_tall(gc, a, w, ga, nullptr, lut_ga, bits, M, K, N, none, sc, sms, s);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

// ---- convolution entry points (implicit im2col) ------------------------------------------------------------
static int make_geom(int B, int C, int H, int W, int kh, int kw, int stride, int pad, int dil, lutgemm::ConvGeom *g) {
    if (B <= 0 || C <= 0 || H <= 0 || W <= 0 || kh <= 0 || kw <= 0 || stride <= 0 || pad < 0 || dil <= 0)
        return LUTGEMM_E_BADARG;
    const long Ho = ((long)H + 2L * pad - (long)dil * (kh - 1) - 1) / stride + 1;
    const long Wo = ((long)W + 2L * pad - (long)dil * (kw - 1) - 1) / stride + 1;
    if (Ho <= 0 || Wo <= 0) return LUTGEMM_E_BADARG;
    if ((long)B * Ho * Wo > 0x7fffffffL || (long)C * kh * kw > 0x7fffffffL) return LUTGEMM_E_TOOLARGE;
    g->enabled = 1; g->B = B; g->C = C; g->H = H; g->W = W; g->kh = kh; g->kw = kw;
    g->stride = stride; g->pad = pad; g->dil = dil; g->Ho = (int)Ho; g->Wo = (int)Wo;
    return LUTGEMM_OK;
}

int lutgemm_conv2d_forward(const uint8_t *x, const uint8_t *wmat, uint32_t *y, const uint16_t *lut, int bits, int B,
                           int C, int H, int W, int Cout, int kh, int kw, int stride, int pad, int dil,
                           void *stream) {
    lutgemm::ConvGeom g{};
    const int rc = make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    return forward_impl(x, wmat, y, lut, bits, B * g.Ho * g.Wo, C * kh * kw, Cout, g, nullptr, 0, stream);
}

size_t lutgemm_conv2d_forward_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                            int stride, int pad, int dil) {
    lutgemm::ConvGeom g{};
    if (make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g) != LUTGEMM_OK) return 0;
    return lutgemm_forward_scratch_bytes(bits, B * g.Ho * g.Wo, C * kh * kw, Cout);
}

int lutgemm_conv2d_forward_ws(const uint8_t *x, const uint8_t *wmat, uint32_t *y, const uint16_t *lut, int bits, int B,
                              int C, int H, int W, int Cout, int kh, int kw, int stride, int pad, int dil,
                              void *scratch, size_t scratch_bytes, void *stream) {
    lutgemm::ConvGeom g{};
    const int rc = make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    return forward_impl(x, wmat, y, lut, bits, B * g.Ho * g.Wo, C * kh * kw, Cout, g, scratch, scratch_bytes, stream);
}

// ---- activation gradient of a convolution ------------------------------------------------------------------
// Windows that do not overlap (kernel extent <= stride, e.g. 1x1 convolutions and patch embeddings): every image
// position receives at most one (m,k) term, so the GEMM-shaped grad_a kernels write it in place.  Overlapping
// windows: the pixel-mode slab kernel, one launch per stride class (lutgemm_slab_grad_tall.cu).  Either way no
// unfolded gradient [M,K] exists.
static bool conv_windows_overlap(const lutgemm::ConvGeom &g) {
    return g.dil * (g.kh - 1) + 1 > g.stride || g.dil * (g.kw - 1) + 1 > g.stride;
}

// the stride class (ph, pw) of geometry g; false when the class has no pixels or no taps
static bool make_pixel_class(const lutgemm::ConvGeom &g, int ph, int pw, lutgemm::PixelClass *px) {
    *px = lutgemm::PixelClass{};
    px->H = g.H; px->W = g.W; px->C = g.C; px->ph = ph; px->pw = pw; px->s = g.stride; px->Ho = g.Ho; px->Wo = g.Wo;
    px->T = g.kh * g.kw;
    px->Hc = ph < g.H ? (g.H - ph + g.stride - 1) / g.stride : 0;
    px->Wc = pw < g.W ? (g.W - pw + g.stride - 1) / g.stride : 0;
    int n = 0;
    for (int i = 0; i < g.kh; ++i)
        for (int j = 0; j < g.kw; ++j) {
            const int dh = i * g.dil - g.pad, dw = j * g.dil - g.pad;
            const int rh = (((ph - dh) % g.stride) + g.stride) % g.stride, rw = (((pw - dw) % g.stride) + g.stride) % g.stride;
            if (rh != 0 || rw != 0) continue;
            px->dh[n] = (int8_t)dh; px->dw[n] = (int8_t)dw; px->t[n] = (uint8_t)(i * g.kw + j);
            ++n;
        }
    px->ntaps = n;
    px->P = g.B * px->Hc * px->Wc;
    return n > 0 && px->Hc > 0 && px->Wc > 0;
}

// pixel mode is limited by the tap tables of PixelClass
static bool pixel_mode_supported(const lutgemm::ConvGeom &g) {
    const int max_d = (g.kh > g.kw ? g.kh : g.kw) * g.dil;
    return g.kh * g.kw <= lutgemm::kMaxTaps && g.kh * g.kw <= 256 && max_d <= 127 && g.pad <= 127;
}

// Per stride class: the slab kernel in pixel mode pays where its row dimension taps * Cout is long enough to
// amortise the slab build; otherwise, and always at 4 and 6 bits where a table row is free of bank conflicts, the
// column-broadcast gather kernel in pixel mode.  The slab kernel's time does not depend on the codes; the broadcast
// kernel's bank conflicts do (weight codes clustered around the zero point conflict less than uniform ones).
// Measured on B200, ResNet-18 layers at batch 256, broadcast with uniform / clustered codes against slab, ms:
//   7 bits  3x3 512->512 (4608 rows) 2.92 / 2.13 : 2.42    3x3 256->256 (2304 rows) 2.91 / 2.12 : 3.13
//   8 bits  3x3 512->512             3.94 / 2.73 : 2.68    3x3 256->256             3.92 / 2.69 : 3.63
//           3x3 256->512 stride 2 (classes of 2048, 1024, 1024, 512 rows) 2.63 / 1.82 : 1.53
// Trained layers have clustered codes, so the choice leans that way: from 8192 rows at 7 bits (a wash between the two
// distributions at 4608), from 4096 rows or Cout >= 512 at 8 bits, where the gather is up to four-way conflicted.
static bool gx_class_uses_slab(int bits, const lutgemm::PixelClass &px, int Cout) {
    const int force = g_force_backward.load(std::memory_order_relaxed);
    if (force == LUTGEMM_BACKWARD_BCAST) return false;
    if (force == LUTGEMM_BACKWARD_SLAB) return true;
    const long rows = (long)px.ntaps * Cout;
    return bits == 7 ? rows >= 8192 : bits == 8 && (rows >= 4096 || Cout >= 512);
}

static size_t conv_gx_scratch_bytes(int bits, const lutgemm::ConvGeom &g, int Cout) {
    const int M = g.B * g.Ho * g.Wo, K = g.C * g.kh * g.kw;
    if (!conv_windows_overlap(g)) {
        const int sms = current_num_sms();
        return sms > 0 ? plan_backward(bits, M, K, Cout, sms).ga_scratch : 0;
    }
    size_t need = 0;
    lutgemm::PixelClass px;
    for (int ph = 0; ph < g.stride; ++ph)
        for (int pw = 0; pw < g.stride; ++pw)
            if (make_pixel_class(g, ph, pw, &px) && gx_class_uses_slab(bits, px, Cout)) {
                const size_t n = lutgemm::gx_class_scratch_bytes(bits, Cout, px, g.B);
                need = n > need ? n : need;
            }
    return need;
}

size_t lutgemm_conv2d_backward_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                             int stride, int pad, int dil) {
    lutgemm::ConvGeom g{};
    if (!lutgemm::bits_supported(bits) || Cout <= 0 || make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g) != LUTGEMM_OK)
        return 0;
    const int sms = current_num_sms();
    if (sms <= 0) return 0;
    const int M = B * g.Ho * g.Wo, K = C * kh * kw;
    // the weight-gradient and the activation-gradient kernels run one after the other on the same buffer
    const size_t gw_need = plan_backward(bits, M, K, Cout, sms).gw_scratch;
    const size_t gx_need = conv_gx_scratch_bytes(bits, g, Cout);
    return gw_need > gx_need ? gw_need : gx_need;
}

int lutgemm_conv2d_backward_ws(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, float *gw,
                               const int16_t *lut_ga, const int16_t *lut_gw, int bits, int B, int C, int H, int W,
                               int Cout, int kh, int kw, int stride, int pad, int dil, const uint8_t *codes_t,
                               void *scratch, size_t scratch_bytes, void *stream) {
    lutgemm::ConvGeom g{};
    int rc = make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    if (reinterpret_cast<uintptr_t>(codes_t) & 15) return LUTGEMM_E_BADARG;
    if (gx && !lut_ga) return LUTGEMM_E_BADARG;
    const int M = B * g.Ho * g.Wo, K = C * kh * kw;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (gw) {
        // first, so that under data parallelism its all-reduce can overlap the activation gradient
        rc = backward_impl(gy, x, wmat, nullptr, gw, nullptr, lut_gw, bits, M, K, Cout, g, codes_t, scratch, scratch_bytes,
                           stream);
        if (rc != LUTGEMM_OK) return rc;
    }
    if (!gx) return LUTGEMM_OK;
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (!gy || !x || !wmat || Cout <= 0) return LUTGEMM_E_BADARG;
    if ((reinterpret_cast<uintptr_t>(gx) & 3) || (reinterpret_cast<uintptr_t>(scratch) & 15)) return LUTGEMM_E_BADARG;
    const bool overlap = conv_windows_overlap(g);
    const bool every_pixel_written = overlap ? stride == 1 : (stride == 1 && kh == 1 && kw == 1 && pad == 0);
    if (!every_pixel_written &&
        !lutgemm::cuda_ok(cudaMemsetAsync(gx, 0, (size_t)B * C * H * W * sizeof(float), s)))
        return LUTGEMM_E_CUDA;
    if (!overlap)  // conv.enabled makes the grad_a kernels write (m,k) to the image position it came from
        return backward_impl(gy, x, wmat, gx, nullptr, lut_ga, nullptr, bits, M, K, Cout, g, nullptr, scratch, scratch_bytes,
                             stream);
    if (!pixel_mode_supported(g)) return LUTGEMM_E_TOOLARGE;
    if (conv_gx_scratch_bytes(bits, g, Cout) > (scratch ? scratch_bytes : 0)) return LUTGEMM_E_SCRATCH;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    lutgemm::PixelClass px;
    lutgemm::PixelClass bcast[lutgemm::kMaxClassesPerLaunch];  // classes for the broadcast kernel, launched in groups
    int nb = 0;
    for (int ph = 0; ph < stride; ++ph)
        for (int pw = 0; pw < stride; ++pw) {
            if (!make_pixel_class(g, ph, pw, &px)) continue;
            if (gx_class_uses_slab(bits, px, Cout)) {
                rc = lutgemm::backward_gx_class(gy, x, wmat, gx, lut_ga, bits, Cout, px, B, static_cast<float *>(scratch), sms, s);
                if (rc != LUTGEMM_OK) return rc;
                continue;
            }
            bcast[nb++] = px;
            if (nb == lutgemm::kMaxClassesPerLaunch) {
                rc = lutgemm::backward_gx_bcast(gy, x, wmat, gx, lut_ga, bits, Cout, bcast, nb, sms, s);
                if (rc != LUTGEMM_OK) return rc;
                nb = 0;
            }
        }
    if (nb) return lutgemm::backward_gx_bcast(gy, x, wmat, gx, lut_ga, bits, Cout, bcast, nb, sms, s);
    return LUTGEMM_OK;
}

int lutgemm_conv2d_backward(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, float *gw,
                            const int16_t *lut_ga, const int16_t *lut_gw, int bits, int B, int C, int H, int W,
                            int Cout, int kh, int kw, int stride, int pad, int dil, void *scratch,
                            size_t scratch_bytes, void *stream) {
    return lutgemm_conv2d_backward_ws(gy, x, wmat, gx, gw, lut_ga, lut_gw, bits, B, C, H, W, Cout, kh, kw, stride, pad,
                                      dil, nullptr, scratch, scratch_bytes, stream);
}

// ---- forward with the layer's de-quantisation applied where the kernel stores ------------------------------------
static int make_epilogue(const float *box, const float *sumw_t, const float *taps, const float *s_a, const float *s_w,
                         const float *z_a, const float *z_w, const float *bias, float *out, int L,
                         lutgemm::LayerEpilogue *e) {
    if (!box || !sumw_t || !taps || !s_a || !s_w || !z_a || !z_w || !out || L <= 0) return LUTGEMM_E_BADARG;
    if (reinterpret_cast<uintptr_t>(out) & 3) return LUTGEMM_E_BADARG;
    e->box = box; e->sumw_t = sumw_t; e->taps = taps; e->s_a = s_a; e->s_w = s_w; e->z_a = z_a; e->z_w = z_w;
    e->bias = bias; e->out = out; e->L = L;
    return LUTGEMM_OK;
}

// Shared body: with complete sums per tile the de-quantisation runs where the kernel stores; when cutting K across
// CTAs fills the GPU better (few output tiles), the sums go through a uint32 buffer behind the transposed codes in
// `scratch` and the one-pass epilogue kernel finishes them.
static size_t align16(size_t n) { return (n + 15) & ~(size_t)15; }

static bool layer_forward_needs_sums(int M, int K, int N, int sms) {
    return forward_uses_slab(M, N) && lutgemm::slab_fwd_ksplits(M, K, N, sms) > 1;
}

static size_t layer_forward_scratch_bytes(int bits, int M, int K, int N) {
    if (!lutgemm::bits_supported(bits) || M <= 0 || K <= 0 || N <= 0) return 0;
    const int sms = current_num_sms();
    if (sms <= 0) return 0;
    const size_t codes = align16(lutgemm_forward_scratch_bytes(bits, M, K, N));
    return codes + (layer_forward_needs_sums(M, K, N, sms) ? (size_t)M * N * sizeof(uint32_t) : 0);
}

static int layer_forward_impl(const uint8_t *a, const uint8_t *w, const uint16_t *lut, int bits, int M, int K, int N,
                              const lutgemm::ConvGeom &conv, const lutgemm::LayerEpilogue &e, void *scratch,
                              size_t scratch_bytes, void *stream) {
    if (!lutgemm::bits_supported(bits)) return LUTGEMM_E_BITS;
    if (M <= 0 || K <= 0 || N <= 0) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    const size_t codes = lutgemm_forward_scratch_bytes(bits, M, K, N);
    if (!layer_forward_needs_sums(M, K, N, sms))
        return forward_impl(a, w, nullptr, lut, bits, M, K, N, conv, scratch, scratch ? codes : 0, stream, &e);
    if (!scratch || scratch_bytes < layer_forward_scratch_bytes(bits, M, K, N)) return LUTGEMM_E_SCRATCH;
    uint32_t *sums = reinterpret_cast<uint32_t *>(static_cast<char *>(scratch) + align16(codes));
    const int rc = forward_impl(a, w, sums, lut, bits, M, K, N, conv, scratch, codes, stream);
    if (rc != LUTGEMM_OK) return rc;
    return lutgemm::conv_epilogue(sums, e.box, e.sumw_t, e.taps, e.s_a, e.s_w, e.z_a, e.z_w, e.bias, e.out, M, e.L, N, sms,
                                  static_cast<cudaStream_t>(stream));
}

size_t lutgemm_conv2d_forward_layer_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                                  int stride, int pad, int dil) {
    lutgemm::ConvGeom g{};
    if (make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g) != LUTGEMM_OK) return 0;
    return layer_forward_scratch_bytes(bits, B * g.Ho * g.Wo, C * kh * kw, Cout);
}

size_t lutgemm_forward_layer_scratch_bytes(int bits, int M, int K, int N) {
    return layer_forward_scratch_bytes(bits, M, K, N);
}

int lutgemm_conv2d_forward_layer(const uint8_t *x, const uint8_t *wmat, const uint16_t *lut, int bits, int B, int C, int H,
                                 int W, int Cout, int kh, int kw, int stride, int pad, int dil, const float *box,
                                 const float *sumw_t, const float *taps, const float *s_a, const float *s_w,
                                 const float *z_a, const float *z_w, const float *bias, float *out, void *scratch,
                                 size_t scratch_bytes, void *stream) {
    lutgemm::ConvGeom g{};
    int rc = make_geom(B, C, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    if (!x || !wmat || !lut || Cout <= 0) return LUTGEMM_E_BADARG;
    lutgemm::LayerEpilogue e{};
    rc = make_epilogue(box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, out, g.Ho * g.Wo, &e);
    if (rc != LUTGEMM_OK) return rc;
    return layer_forward_impl(x, wmat, lut, bits, B * g.Ho * g.Wo, C * kh * kw, Cout, g, e, scratch, scratch_bytes, stream);
}

int lutgemm_forward_layer(const uint8_t *a, const uint8_t *w, const uint16_t *lut, int bits, int M, int K, int N,
                          const float *box, const float *sumw_t, const float *taps, const float *s_a, const float *s_w,
                          const float *z_a, const float *z_w, const float *bias, float *out, void *scratch,
                          size_t scratch_bytes, void *stream) {
    if (!a || !w || !lut) return LUTGEMM_E_BADARG;
    lutgemm::ConvGeom none{};
    lutgemm::LayerEpilogue e{};
    const int rc = make_epilogue(box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, out, 1, &e);
    if (rc != LUTGEMM_OK) return rc;
    return layer_forward_impl(a, w, lut, bits, M, K, N, none, e, scratch, scratch_bytes, stream);
}

// ---- layer prologue / epilogue ---------------------------------------------------------------------------
int lutgemm_quantize_activations(const float *x, long stride_b, long stride_c, long stride_h, long stride_w, int B,
                                 int C, int H, int W, const float *scale, const float *zp_neg, float qmax,
                                 uint8_t *codes, float *chansum, void *stream) {
    if (!x || !scale || !zp_neg || !codes || B <= 0 || C <= 0 || H <= 0 || W <= 0 || !(qmax >= 1.f && qmax <= 255.f))
        return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::quantize_codes(x, stride_b, stride_c, stride_h, stride_w, B, C, H, W, scale, zp_neg, qmax, codes,
                                   chansum, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_quantize_activations_backward(const float *x, long stride_b, long stride_c, long stride_h, long stride_w,
                                          int B, int C, int H, int W, const float *scale, const float *zp_neg,
                                          float qmax, const float *gcodes, const float *box_t, const float *s_w,
                                          const float *z_w, float *gx, void *stream) {
    if (!x || !scale || !zp_neg || !gcodes || !s_w || !z_w || !gx || B <= 0 || C <= 0 || H <= 0 || W <= 0)
        return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::quantize_backward(x, stride_b, stride_c, stride_h, stride_w, B, C, H, W, scale, zp_neg, qmax, gcodes,
                                      box_t, s_w, z_w, gx, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_conv2d_epilogue(const uint32_t *y, const float *box, const float *sumw_t, const float *taps,
                            const float *s_a, const float *s_w, const float *z_a, const float *z_w, const float *bias,
                            float *out, long M, int L, int Cout, void *stream) {
    if (!y || !box || !sumw_t || !taps || !s_a || !s_w || !z_a || !z_w || !out || M <= 0 || L <= 0 || Cout <= 0)
        return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::conv_epilogue(y, box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, out, M, L, Cout, sms,
                                  static_cast<cudaStream_t>(stream));
}

// ---- small kernels of the layer wiring -----------------------------------------------------------------------
int lutgemm_layer_update_ranges(const float *act_lo, const float *act_hi, const float *w_lo, const float *w_hi,
                                float *act_min, float *act_max, float *act_seen, float *w_min, float *w_max, float *w_seen,
                                float keep, float momentum, float a_qmax, float w_qmax, float eps, float *quant,
                                void *stream) {
    if (!act_lo || !act_hi || !w_lo || !w_hi || !act_min || !act_max || !act_seen || !w_min || !w_max || !w_seen || !quant)
        return LUTGEMM_E_BADARG;
    return lutgemm::layer_update_ranges(act_lo, act_hi, w_lo, w_hi, act_min, act_max, act_seen, w_min, w_max, w_seen, keep,
                                        momentum, a_qmax, w_qmax, eps, quant, static_cast<cudaStream_t>(stream));
}

int lutgemm_layer_weight_prep(const float *weight, long s_co, long s_c, long s_h, long s_w, int Cout, int Cin, int kh, int kw,
                              const float *quant, float qmax, uint8_t *wmat, float *wsum, void *stream) {
    if (!weight || !quant || !wmat || !wsum || Cout <= 0 || Cin <= 0 || kh <= 0 || kw <= 0 || kh * kw > 4096)
        return LUTGEMM_E_BADARG;
    return lutgemm::layer_weight_prep(weight, s_co, s_c, s_h, s_w, Cout, Cin, kh, kw, quant, qmax, wmat, wsum,
                                      static_cast<cudaStream_t>(stream));
}

int lutgemm_layer_cross_terms(const float *wsum, int Cout, int Cin, int H, int W, int kh, int kw, int stride, int pad,
                              int dil, float *sumw_t, float *taps, void *stream) {
    lutgemm::ConvGeom g{};
    const int rc = make_geom(1, Cin, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    if (!wsum || !sumw_t || !taps || Cout <= 0) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::layer_cross_terms(wsum, Cout, g, sumw_t, taps, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_layer_window_sum(const float *img, int B, int H, int W, int kh, int kw, int stride, int pad, int dil,
                             float *box, void *stream) {
    lutgemm::ConvGeom g{};
    const int rc = make_geom(B, 1, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    if (!img || !box) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::layer_window_sum(img, g, box, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_layer_window_sum_adjoint(const float *gsum, int B, int H, int W, int kh, int kw, int stride, int pad, int dil,
                                     float *out, void *stream) {
    lutgemm::ConvGeom g{};
    const int rc = make_geom(B, 1, H, W, kh, kw, stride, pad, dil, &g);
    if (rc != LUTGEMM_OK) return rc;
    if (!gsum || !out) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::layer_window_sum_adjoint(gsum, g, out, sms, static_cast<cudaStream_t>(stream));
}

int lutgemm_layer_weight_grad(const float *gwmat, const float *tapg, const float *weight, long s_co, long s_c, long s_h,
                              long s_w, int Cout, int Cin, int kh, int kw, const float *quant, float qmax, float *gw,
                              void *stream) {
    if (!gwmat || !tapg || !weight || !quant || !gw || Cout <= 0 || Cin <= 0 || kh <= 0 || kw <= 0) return LUTGEMM_E_BADARG;
    const int sms = current_num_sms();
    if (sms <= 0) return LUTGEMM_E_CUDA;
    return lutgemm::layer_weight_grad_finish(gwmat, tapg, weight, s_co, s_c, s_h, s_w, Cout, Cin, kh, kw, quant, qmax, gw,
                                             sms, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
