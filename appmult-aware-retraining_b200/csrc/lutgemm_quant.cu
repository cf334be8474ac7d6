// Quantisation prologue / de-quantisation epilogue of an approximate convolution layer, one pass each
// (the reference runs them as a dozen PyTorch elementwise kernels around its operator,
// micronet+/app_layers.py:147-181):
//
//   quantize:           codes[b,c,h,w] = clamp(rint(x / s_a - z_a), 0, qmax) as uint8, NCHW-contiguous, from
//                       an activation tensor of any dense layout (NCHW or channels-last), plus the channel
//                       sums chansum[b,h,w] = sum_c codes the zero-point cross term needs
//   epilogue:           out[m,co] = s_a s_w (y[m,co] + z_w box[m] + z_a sumw[l,co] + z_a z_w taps[l]) (+ bias[co])
//   quantize_backward:  gx = [0 <= rint(x / s_a - z_a) <= qmax] * s_w * (gcodes[b,c,h,w] + z_w boxT[b,h,w])
//                       written in the layout of x (straight-through rounding, clamp mask)
//
// Scales and zero points are read from device memory (they are module buffers refreshed every step), so
// no call synchronises with the host.
#include "lutgemm.h"
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

namespace {

__device__ __forceinline__ float code_of(float x, const Divisor &scale, float zp_neg) {
    return rintf(__fsub_rn(quotient(x, scale), zp_neg));  // two roundings, as x / scale - zp in PyTorch
}

// Tile of 32 channels x 32 columns of one image row (b, h).  Reads follow the input's fastest dimension,
// writes follow w: for a channels-last input that is a transposition through shared memory.
template <bool BACKWARD>
__global__ void __launch_bounds__(256) quant_tile_kernel(const float *__restrict__ x, long sb, long sc, long sh, long sw,
                                                         int B, int C, int H, int W, const float *__restrict__ scale_p,
                                                         const float *__restrict__ zp_p, float qmax,
                                                         uint8_t *__restrict__ codes, float *__restrict__ chansum,
                                                         const float *__restrict__ gcodes, const float *__restrict__ boxT,
                                                         const float *__restrict__ sw_p, const float *__restrict__ zw_p,
                                                         float *__restrict__ gx) {
    __shared__ float tile[32][33];
    const Divisor scale = make_divisor(*scale_p);
    const float zp = *zp_p;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const int ct = (C + 31) / 32;
    const bool chan_fast = sc == 1 && sw != 1;
    // one tile per CTA: blockIdx.x = (column tile, channel tile), blockIdx.y = image row, blockIdx.z = image (no
    // 64-bit divisions to decode a linear tile index: they cost more than the tile's arithmetic)
    {
        const int c0 = (int)(blockIdx.x % ct) * 32;
        const int w0 = (int)(blockIdx.x / ct) * 32;
        const int h = blockIdx.y, b = blockIdx.z;
        const float *xrow = x + b * sb + h * sh;
        // tile[c][w] = q (forward) or the clamp mask (backward)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = ty + 8 * r;
            const int c = chan_fast ? c0 + tx : c0 + i, w = chan_fast ? w0 + i : w0 + tx;
            float v = 0.f;
            if (c < C && w < W) {
                const float q = code_of(xrow[c * sc + w * sw], scale, zp);
                v = BACKWARD ? ((q >= 0.f && q <= qmax) ? 1.f : 0.f) : fminf(fmaxf(q, 0.f), qmax);
            }
            if (chan_fast) tile[tx][i] = v; else tile[i][tx] = v;
        }
        __syncthreads();
        if (!BACKWARD) {
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int c = c0 + ty + 8 * r, w = w0 + tx;
                if (c < C && w < W) codes[(((size_t)b * C + c) * H + h) * W + w] = (uint8_t)tile[ty + 8 * r][tx];
            }
            if (chansum && ty == 0 && w0 + tx < W) {
                float s = 0.f;
#pragma unroll 8
                for (int c = 0; c < 32; ++c) s += tile[c][tx];  // codes of channels >= C are 0
                atomicAdd(chansum + ((size_t)b * H + h) * W + w0 + tx, s);  // integer-valued sums < 2^24: exact in any order
            }
        } else {
            const float swt = *sw_p, zw = *zw_p;
            // g[c][w] = mask * s_w * (gcodes + z_w boxT), gathered along w, then written along x's fast dimension
            float gv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int c = c0 + ty + 8 * r, w = w0 + tx;
                gv[r] = 0.f;
                if (c < C && w < W) {
                    float g = gcodes[(((size_t)b * C + c) * H + h) * W + w];
                    if (boxT) g = __fadd_rn(g, __fmul_rn(zw, boxT[((size_t)b * H + h) * W + w]));
                    gv[r] = tile[ty + 8 * r][tx] * __fmul_rn(swt, g);
                }
            }
            __syncthreads();
#pragma unroll
            for (int r = 0; r < 4; ++r) tile[ty + 8 * r][tx] = gv[r];
            __syncthreads();
            float *grow = gx + b * sb + h * sh;
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int i = ty + 8 * r;
                const int c = chan_fast ? c0 + tx : c0 + i, w = chan_fast ? w0 + i : w0 + tx;
                if (c < C && w < W) grow[c * sc + w * sw] = chan_fast ? tile[tx][i] : tile[i][tx];
            }
        }
    }
}

__global__ void __launch_bounds__(256) conv_epilogue_kernel(const uint32_t *__restrict__ y, const float *__restrict__ box,
                                                            const float *__restrict__ sumw_t, const float *__restrict__ taps,
                                                            const float *__restrict__ sa_p, const float *__restrict__ sw_p,
                                                            const float *__restrict__ za_p, const float *__restrict__ zw_p,
                                                            const float *__restrict__ bias, float *__restrict__ out, long M,
                                                            int L, int Cout) {
    const float s = *sa_p * *sw_p, za = *za_p, zw = *zw_p, zz = za * zw;
    // a warp per output row m (32 rows per CTA per step), lanes over the output channels: the row terms and the
    // position l = m mod L are computed once per row, and nothing divides by Cout per element
    const int lane = threadIdx.x & 31, wrow = threadIdx.x >> 5;
    for (long m = (long)blockIdx.x * 8 + wrow; m < M; m += (long)gridDim.x * 8) {
        const int l = (int)(m % L);
        // separately rounded products and sums, in the order the PyTorch expression evaluates them
        const float zw_box = __fmul_rn(zw, box[m]), zz_taps = __fmul_rn(zz, taps[l]);
        const uint32_t *yrow = y + m * Cout;
        const float *srow = sumw_t + (size_t)l * Cout;
        float *orow = out + m * Cout;
        for (int co = lane; co < Cout; co += 32) {
            float acc = (float)yrow[co];
            acc = __fadd_rn(acc, zw_box);
            acc = __fadd_rn(acc, __fmul_rn(za, srow[co]));
            acc = __fadd_rn(acc, zz_taps);
            float o = __fmul_rn(s, acc);
            if (bias) o = __fadd_rn(o, bias[co]);
            orow[co] = o;
        }
    }
}

}  // namespace

int quantize_codes(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                   const float *zp_neg, float qmax, uint8_t *codes, float *chansum, int num_sms, cudaStream_t stream) {
    (void)num_sms;
    if (H > 65535 || B > 65535) return LUTGEMM_E_TOOLARGE;
    const dim3 grid((unsigned)(((W + 31) / 32) * ((C + 31) / 32)), (unsigned)H, (unsigned)B);
    quant_tile_kernel<false><<<grid, 256, 0, stream>>>(x, sb, sc, sh, sw, B, C, H, W, scale, zp_neg, qmax, codes, chansum,
                                                       nullptr, nullptr, nullptr, nullptr, nullptr);
    return launch_status();
}

int quantize_backward(const float *x, long sb, long sc, long sh, long sw, int B, int C, int H, int W, const float *scale,
                      const float *zp_neg, float qmax, const float *gcodes, const float *boxT, const float *s_w,
                      const float *z_w, float *gx, int num_sms, cudaStream_t stream) {
    (void)num_sms;
    if (H > 65535 || B > 65535) return LUTGEMM_E_TOOLARGE;
    const dim3 grid((unsigned)(((W + 31) / 32) * ((C + 31) / 32)), (unsigned)H, (unsigned)B);
    quant_tile_kernel<true><<<grid, 256, 0, stream>>>(x, sb, sc, sh, sw, B, C, H, W, scale, zp_neg, qmax, nullptr, nullptr,
                                                      gcodes, boxT, s_w, z_w, gx);
    return launch_status();
}

int conv_epilogue(const uint32_t *y, const float *box, const float *sumw_t, const float *taps, const float *s_a,
                  const float *s_w, const float *z_a, const float *z_w, const float *bias, float *out, long M, int L,
                  int Cout, int num_sms, cudaStream_t stream) {
    const long blocks = (M + 7) / 8;
    const int grid = (int)(blocks < 32L * num_sms ? blocks : 32L * num_sms);
    conv_epilogue_kernel<<<grid, 256, 0, stream>>>(y, box, sumw_t, taps, s_a, s_w, z_a, z_w, bias, out, M, L, Cout);
    return launch_status();
}

}  // namespace lutgemm
