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

struct ConvGeom;  // lutgemm_common.cuh; geometry.enabled == 0 means `a` is a plain [M,K] matrix

int forward_rowbcast(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                     int N, const ConvGeom &conv, int num_sms, cudaStream_t stream);

// `at` (optional): the activation codes transposed, at[k][m] with rows at_pitch bytes apart (transpose_codes)
int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 const ConvGeom &conv, const uint8_t *at, int at_pitch, int num_sms, cudaStream_t stream);

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
int backward_gw_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                          int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                          int at_pitch, int num_sms, cudaStream_t stream);
int backward_ga_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                          int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms,
                          cudaStream_t stream);
// reads (and clears) the device-side error word of the bounded barrier waits; synchronises the device
int read_and_clear_device_error(int *value);
// launches a one-warp kernel whose barrier wait can never be satisfied (it must time out with error id 99)
int bounded_wait_selftest(cudaStream_t stream);
// out[k][c] (or out[c][k] when transpose) = 1/16 * sum over row blocks of part[b][k][c], b ascending
int slab_reduce_blocks(const float *part, float *out, int K, int C, int nblocks, bool transpose, int bkl_L,
                       int num_sms, cudaStream_t stream);


// at[k][m] = a[m][k] (or the unfolded code image when conv.enabled); rows `pitch` bytes apart, pitch a multiple
// of 16 and >= M, columns m >= M are written as 0
int transpose_codes(const uint8_t *a, uint8_t *at, int M, int K, int pitch, const ConvGeom &conv, cudaStream_t stream);

// gx[B,C,H,W] from the unfolded activation gradient gcol[B][C*kh*kw][Ho*Wo] (deterministic gather)
int col2im_gather(const float *gcol, float *gx, const ConvGeom &g, int num_sms, cudaStream_t stream);

// quantisation prologue / epilogue of an approximate convolution layer (lutgemm_quant.cu); strides in elements
int quantize_codes(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                   const float *zp_neg, float qmax, uint8_t *codes, float *chansum, int num_sms, cudaStream_t stream);
int quantize_backward(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                      const float *zp_neg, float qmax, const float *gcodes, const float *boxT, const float *s_w,
                      const float *z_w, float *gx, int num_sms, cudaStream_t stream);
int conv_epilogue(const uint32_t *y, const float *box, const float *sumw_t, const float *taps, const float *s_a,
                  const float *s_w, const float *z_a, const float *z_w, const float *bias, float *out, long M, int L,
                  int Cout, int num_sms, cudaStream_t stream);

// number of slabs the weight-gradient kernel splits M into (1 = no scratch needed)
int gw_num_splits(int bits, int M, int K, int N, int num_sms);

int backward_ga(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                int M, int K, int N, const ConvGeom &conv, int num_sms, cudaStream_t stream);

int backward_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                int M, int K, int N, const ConvGeom &conv, float *scratch, int num_splits, int num_sms,
                cudaStream_t stream);

}  // namespace lutgemm
