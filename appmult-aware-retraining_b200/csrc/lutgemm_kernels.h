// Internal launch interfaces between the C-ABI translation unit and the kernel translation units.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace lutgemm {

int forward_rowbcast(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                     int N, int num_sms, cudaStream_t stream);

int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 int num_sms, cudaStream_t stream);

int backward_gw_slab(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                     int M, int K, int N, float *scratch, int num_sms, cudaStream_t stream);
int backward_ga_slab(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                     int M, int K, int N, float *scratch, int num_sms, cudaStream_t stream);
// number of 512-row blocks the slab gradient kernels cut their reduction dimension into
int slab_grad_row_blocks(int rdim);

// number of slabs the weight-gradient kernel splits M into (1 = no scratch needed)
int gw_num_splits(int bits, int M, int K, int N, int num_sms);

int backward_ga(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                int M, int K, int N, int num_sms, cudaStream_t stream);

int backward_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                int M, int K, int N, float *scratch, int num_splits, int num_sms, cudaStream_t stream);

}  // namespace lutgemm
