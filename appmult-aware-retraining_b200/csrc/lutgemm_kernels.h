// Internal launch interfaces between the C-ABI translation unit and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lutgemm {

// Failure bookkeeping: the CUDA error behind a LUTGEMM_E_CUDA status is kept per host thread so that
// lutgemm_status_string can name it (cudaGetLastError clears the runtime's own record).
void record_cuda_error(cudaError_t e);
inline bool cuda_ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    record_cuda_error(e);
    return false;
}
// status of the launch just made on this thread
int launch_status();

struct ConvGeom;    // lutgemm_common.cuh; geometry.enabled == 0 means `a` is a plain [M,K] matrix
struct PixelClass;  // lutgemm_common.cuh; the input pixels of one stride class of a convolution and their taps
struct LayerEpilogue;  // lutgemm_common.cuh; optional de-quantisation applied where the forward kernels store

// `epi` (optional): the kernel stores the de-quantised fp32 layer output epi->out instead of the uint32 sums c
int forward_rowbcast(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                     int N, const ConvGeom &conv, const LayerEpilogue *epi, int num_sms, cudaStream_t stream);

// `at` (optional): the activation codes transposed, at[k][m] with rows at_pitch bytes apart (transpose_codes)
int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 const ConvGeom &conv, const uint8_t *at, int at_pitch, const LayerEpilogue *epi, int num_sms,
                 cudaStream_t stream);

// operand chunks of forward_slab by bulk-tensor copies (default) or by vector loads through registers
void slab_fwd_set_tma(bool on);
// number of K ranges forward_slab cuts a problem into when it is free to (1 = none; a fused epilogue needs 1)
int slab_fwd_ksplits(int M, int K, int N, int num_sms);

// rows of the reduction dimension per CTA tile of the fp32-slab gradient kernels, and the block count
constexpr int kSlabF32Rows = 512;
int slab_f32_row_blocks(int rdim);
// gradient slab kernels with an fp32 slab (conversion done once per slab entry, in the build)
// `at` (optional): the row codes transposed, at[k][m] with rows at_pitch bytes apart (transpose_codes)
int backward_gw_slab_f32(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                         int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                         int at_pitch, int num_sms, cudaStream_t stream);
int backward_ga_slab_f32(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                         int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms,
                         cudaStream_t stream);
// the same with a tall tile (1024 rows x 32 columns): half the slab-build work per look-up
constexpr int kSlabTallRows = 1024;
int slab_tall_row_blocks(int rdim);
// lut_f32 (optional, bits <= 7): the gradient table as fp32 in the same padded layout; it replaces the int16
// table and the 1/16 scale
int backward_gw_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                          const float *lut_f32, int bits, int M, int K, int N, const ConvGeom &conv, float *scratch,
                          const uint8_t *at, int at_pitch, int num_sms, cudaStream_t stream);
int backward_ga_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                          const float *lut_f32, int bits, int M, int K, int N, const ConvGeom &conv, float *scratch,
                          int num_sms, cudaStream_t stream);
// reads (and clears) the device-side error word of the bounded barrier waits; synchronises the device
int read_and_clear_device_error(int *value);
// launches a one-warp kernel whose barrier wait can never be satisfied (it must time out with error id 99)
int bounded_wait_selftest(cudaStream_t stream);
// out[k][c] (or out[c][k] when transpose) = 1/16 * sum over row blocks of part[b][k][c], b ascending; with
// `scatter` (columns are unfolded rows of that convolution) or `px` (columns are pixels of that class, k a
// channel) the sums go to their positions in the image gradient instead
int slab_reduce_blocks(const float *part, float *out, int K, int C, int nblocks, bool transpose, const ConvGeom *scatter,
                       const PixelClass *px, float scale, int num_sms, cudaStream_t stream);
// activation gradient of a convolution for the input pixels of one stride class, written into gx[B,C,H,W]
// (tall slab kernel in pixel mode: no unfolded gradient, no col2im); scratch: gx_class_scratch_bytes()
size_t gx_class_scratch_bytes(int bits, int Cout, const PixelClass &px, int B);
int backward_gx_class(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut_ga, int bits,
                      int Cout, const PixelClass &px, int B, float *scratch, int num_sms, cudaStream_t stream);
// the same with the column-broadcast gather kernel (whole table in shared memory, no slab) for `nclasses` stride
// classes at once (up to four per launch, so that small images still fill the GPU): better where the row dimension
// taps * Cout is too short to amortise a slab build
int backward_gx_bcast(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut_ga, int bits,
                      int Cout, const PixelClass *classes, int nclasses, int num_sms, cudaStream_t stream);
// hand-over between the warps of the tall gradient kernels: per-buffer mbarriers (default) or one CTA barrier per k
void slab_tall_set_handover(bool on);


// at[k][m] = a[m][k] cut to `bits` bits (or the unfolded code image when conv.enabled); rows `pitch` bytes apart,
// pitch a multiple of 16 and >= M, columns m >= M are written as 0
int transpose_codes(const uint8_t *a, uint8_t *at, int M, int K, int pitch, const ConvGeom &conv, int bits,
                    cudaStream_t stream);

// quantisation prologue / epilogue of an approximate convolution layer (lutgemm_quant.cu); strides in elements
int quantize_codes(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                   const float *zp_neg, float qmax, uint8_t *codes, float *chansum, int num_sms, cudaStream_t stream);
int quantize_backward(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                      const float *zp_neg, float qmax, const float *gcodes, const float *boxT, const float *s_w,
                      const float *z_w, float *gx, int num_sms, cudaStream_t stream);
int conv_epilogue(const uint32_t *y, const float *box, const float *sumw_t, const float *taps, const float *s_a,
                  const float *s_w, const float *z_a, const float *z_w, const float *bias, float *out, long M, int L,
                  int Cout, int num_sms, cudaStream_t stream);

// small one-pass kernels of the layer wiring (lutgemm_layer_aux.cu); strides in elements, quant = {s_a, z_a, s_w, z_w}
int layer_update_ranges(const float *act_lo, const float *act_hi, const float *w_lo, const float *w_hi, float *act_min,
                        float *act_max, float *act_seen, float *w_min, float *w_max, float *w_seen, float keep,
                        float momentum, float a_qmax, float w_qmax, float eps, float *quant, cudaStream_t stream);
int layer_weight_prep(const float *weight, long s_co, long s_c, long s_h, long s_w, int Cout, int Cin, int kh, int kw,
                      const float *quant, float qmax, uint8_t *wmat, float *wsum, cudaStream_t stream);
int layer_cross_terms(const float *wsum, int Cout, const ConvGeom &g, float *sumw_t, float *taps, int num_sms,
                      cudaStream_t stream);
int layer_window_sum(const float *img, const ConvGeom &g, float *box, int num_sms, cudaStream_t stream);
int layer_window_sum_adjoint(const float *gsum, const ConvGeom &g, float *out, int num_sms, cudaStream_t stream);
int layer_weight_grad_finish(const float *gwmat, const float *tapg, const float *weight, long s_co, long s_c, long s_h,
                             long s_w, int Cout, int Cin, int kh, int kw, const float *quant, float qmax, float *gw,
                             int num_sms, cudaStream_t stream);

// number of slabs the weight-gradient kernel splits M into (1 = no scratch needed)
int gw_num_splits(int bits, int M, int K, int N, int num_sms);

// with conv.enabled (a convolution whose windows do not overlap) ga is the image gradient gx[B,C,H,W] and every
// (m,k) is written to the position its activation came from; the caller zero-fills gx where nothing lands
int backward_ga(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                int M, int K, int N, const ConvGeom &conv, int num_sms, cudaStream_t stream);

int backward_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                int M, int K, int N, const ConvGeom &conv, float *scratch, int num_splits, int num_sms,
                cudaStream_t stream);

}  // namespace lutgemm
