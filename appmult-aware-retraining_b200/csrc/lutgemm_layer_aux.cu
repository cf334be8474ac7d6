// Small one-pass kernels around the LUT kernels of an approximate layer.  Each replaces a chain of PyTorch
// elementwise / slicing kernels (ten to twenty launches each) of the layer wiring in lutgemm_layers.py; the
// reference runs the same arithmetic as PyTorch expressions in ApproxConv2d.forward and its observers,
// micronet+/app_layers.py:21-53, 147-184.
//
//   update_ranges      observers + quantisation parameters: running min/max of the weights, exponential moving
//                      average of the activation min/max, scales and zero points (:21-53, :155-160)
//   weight_prep        weight codes of one layer, transposed to the [Cin*kh*kw, Cout] matrix the LUT kernels take,
//                      and their sums over the input channels per (output channel, tap)
//   cross_terms        sumw_t[l,co] = sum of the weight codes over the taps valid at output position l, and
//                      taps[l] = Cin * number of valid taps: the z_a-terms of the layer expression (:178-180)
//   window_sum         box[m] = sum over the kernel window of the channel-summed activation codes: the z_w-term
//   window_sum_adjoint its adjoint (backward of the z_w-term)
//   weight_grad_finish gradient w.r.t. the fp32 weight from the gradient w.r.t. the weight codes: cross term,
//                      clamp mask, activation scale (backward of :147-150 for the weight)
// All scalars live in device memory: no call synchronises with the host.
#include "lutgemm.h"
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

namespace {

__device__ __forceinline__ float code_of(float x, const Divisor &scale, float zp_neg) {
    return rintf(__fsub_rn(quotient(x, scale), zp_neg));  // two roundings, as x / scale - zp in PyTorch
}

// one thread: the layer's observers and quantisation parameters
__global__ void update_ranges_kernel(const float *act_lo, const float *act_hi, const float *w_lo, const float *w_hi,
                                     float *act_min, float *act_max, float *act_seen, float *w_min, float *w_max,
                                     float *w_seen, float keep, float momentum, float a_qmax, float w_qmax, float eps,
                                     float *quant) {
    // activations: exponential moving average of the batch range, keep = 1 - momentum (the first batch sets it)
    float amin = *act_lo, amax = *act_hi;
    if (*act_seen != 0.f) {
        amin = __fadd_rn(__fmul_rn(keep, *act_min), __fmul_rn(momentum, *act_lo));
        amax = __fadd_rn(__fmul_rn(keep, *act_max), __fmul_rn(momentum, *act_hi));
    }
    *act_min = amin; *act_max = amax; *act_seen = 1.f;
    // weights: running range
    float wmin = *w_lo, wmax = *w_hi;
    if (*w_seen != 0.f) { wmin = fminf(wmin, *w_min); wmax = fmaxf(wmax, *w_max); }
    *w_min = wmin; *w_max = wmax; *w_seen = 1.f;
    const float s_a = fmaxf(__fdiv_rn(__fsub_rn(amax, amin), a_qmax), eps);
    const float s_w = fmaxf(__fdiv_rn(__fsub_rn(wmax, wmin), w_qmax), eps);
    quant[0] = s_a;
    quant[1] = rintf(__fdiv_rn(amin, s_a));
    quant[2] = s_w;
    quant[3] = rintf(__fdiv_rn(wmin, s_w));
}

// One block per output channel: codes of weight[co, :, :, :] (any strides) written as column co of wmat[K, Cout],
// K ordered (cin, kh, kw); wsum[co, t] = sum over cin of the codes of tap t (integers: exact in any order).
__global__ void __launch_bounds__(256) weight_prep_kernel(const float *__restrict__ weight, long s_co, long s_c, long s_h,
                                                          long s_w, int Cout, int Cin, int kh, int kw,
                                                          const float *__restrict__ quant, float qmax,
                                                          uint8_t *__restrict__ wmat, float *__restrict__ wsum) {
    extern __shared__ float tap_sum[];  // [kh*kw]
    const int T = kh * kw, K = Cin * T, co = blockIdx.x;
    const Divisor scale = make_divisor(quant[2]);
    const float zp = quant[3];
    for (int t = threadIdx.x; t < T; t += blockDim.x) tap_sum[t] = 0.f;
    __syncthreads();
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const int c = k / T, t = k - c * T, i = t / kw, j = t - i * kw;
        const float q = fminf(fmaxf(code_of(weight[co * s_co + c * s_c + i * s_h + j * s_w], scale, zp), 0.f), qmax);
        wmat[(size_t)k * Cout + co] = (uint8_t)q;
        atomicAdd(&tap_sum[t], q);
    }
    __syncthreads();
    for (int t = threadIdx.x; t < T; t += blockDim.x) wsum[(size_t)co * T + t] = tap_sum[t];
}

__device__ __forceinline__ bool tap_inside(const ConvGeom &g, int oh, int ow, int i, int j) {
    const int ih = oh * g.stride - g.pad + i * g.dil, iw = ow * g.stride - g.pad + j * g.dil;
    return (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W;
}

// sumw_t[l, co] = sum over the taps inside the image at output position l of wsum[co, t] (ascending t);
// taps[l] = Cin * number of those taps
__global__ void __launch_bounds__(256) cross_terms_kernel(const float *__restrict__ wsum, int Cout, const ConvGeom g,
                                                          float *__restrict__ sumw_t, float *__restrict__ taps) {
    const int L = g.Ho * g.Wo, T = g.kh * g.kw;
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < (long)L * Cout; idx += (long)gridDim.x * blockDim.x) {
        const int l = (int)(idx / Cout), co = (int)(idx - (long)l * Cout), oh = l / g.Wo, ow = l - oh * g.Wo;
        float s = 0.f;
        int n = 0;
        for (int t = 0; t < T; ++t)
            if (tap_inside(g, oh, ow, t / g.kw, t % g.kw)) { s += wsum[(size_t)co * T + t]; ++n; }
        sumw_t[idx] = s;
        if (co == 0) taps[l] = (float)n * (float)g.C;
    }
}

// box[(b*Ho + oh)*Wo + ow] = sum over the taps inside the image of img[b, ih, iw]   (ascending tap order)
__global__ void __launch_bounds__(256) window_sum_kernel(const float *__restrict__ img, const ConvGeom g,
                                                         float *__restrict__ box) {
    const long M = (long)g.B * g.Ho * g.Wo;
    for (long m = blockIdx.x * (long)blockDim.x + threadIdx.x; m < M; m += (long)gridDim.x * blockDim.x) {
        const int ow = (int)(m % g.Wo), oh = (int)((m / g.Wo) % g.Ho);
        const long b = m / ((long)g.Wo * g.Ho);
        const float *src = img + b * g.H * g.W;
        float s = 0.f;
        for (int i = 0; i < g.kh; ++i) {
            const int ih = oh * g.stride - g.pad + i * g.dil;
            if ((unsigned)ih >= (unsigned)g.H) continue;
            for (int j = 0; j < g.kw; ++j) {
                const int iw = ow * g.stride - g.pad + j * g.dil;
                if ((unsigned)iw < (unsigned)g.W) s += src[ih * g.W + iw];
            }
        }
        box[m] = s;
    }
}

// out[b, h, w] = sum over the taps (i, j) that connect (h, w) to an output position of gsum[b, oh, ow]
__global__ void __launch_bounds__(256) window_sum_adjoint_kernel(const float *__restrict__ gsum, const ConvGeom g,
                                                                 float *__restrict__ out) {
    const long P = (long)g.B * g.H * g.W;
    for (long p = blockIdx.x * (long)blockDim.x + threadIdx.x; p < P; p += (long)gridDim.x * blockDim.x) {
        const int w = (int)(p % g.W), h = (int)((p / g.W) % g.H);
        const long b = p / ((long)g.W * g.H);
        const float *src = gsum + b * g.Ho * g.Wo;
        float s = 0.f;
        for (int i = 0; i < g.kh; ++i) {
            const int th = h + g.pad - i * g.dil;
            if (th < 0 || th % g.stride) continue;
            const int oh = th / g.stride;
            if (oh >= g.Ho) continue;
            for (int j = 0; j < g.kw; ++j) {
                const int tw = w + g.pad - j * g.dil;
                if (tw < 0 || tw % g.stride) continue;
                const int ow = tw / g.stride;
                if (ow < g.Wo) s += src[oh * g.Wo + ow];
            }
        }
        out[p] = s;
    }
}

// gw[co, c, i, j] = [0 <= code(weight) <= qmax] * s_a * (gwmat[(c*kh+i)*kw+j, co] + z_a * tapg[co, (i*kw+j)])
// weight given by its strides, gw contiguous [Cout, Cin, kh, kw]
__global__ void __launch_bounds__(256) weight_grad_finish_kernel(const float *__restrict__ gwmat, const float *__restrict__ tapg,
                                                                 const float *__restrict__ weight, long s_co, long s_c,
                                                                 long s_h, long s_w, int Cout, int Cin, int kh, int kw,
                                                                 const float *__restrict__ quant, float qmax,
                                                                 float *__restrict__ gw) {
    const int T = kh * kw, K = Cin * T;
    const float s_a = quant[0], z_a = quant[1], zp = quant[3];
    const Divisor scale = make_divisor(quant[2]);
    for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < (long)K * Cout; idx += (long)gridDim.x * blockDim.x) {
        const int k = (int)(idx / Cout), co = (int)(idx - (long)k * Cout);  // gwmat is read in its own order
        const int c = k / T, t = k - c * T, i = t / kw, j = t - i * kw;
        const float q = code_of(weight[co * s_co + c * s_c + i * s_h + j * s_w], scale, zp);
        const float gq = __fadd_rn(gwmat[idx], __fmul_rn(z_a, tapg[(size_t)co * T + t]));
        gw[(size_t)co * K + k] = (q >= 0.f && q <= qmax) ? __fmul_rn(s_a, gq) : 0.f;
    }
}

int grid_for(long items, int num_sms) {
    const long blocks = (items + 255) / 256;
    return (int)(blocks < 16L * num_sms ? (blocks > 0 ? blocks : 1) : 16L * num_sms);
}

}  // namespace

int layer_update_ranges(const float *act_lo, const float *act_hi, const float *w_lo, const float *w_hi, float *act_min,
                        float *act_max, float *act_seen, float *w_min, float *w_max, float *w_seen, float keep,
                        float momentum, float a_qmax, float w_qmax, float eps, float *quant, cudaStream_t stream) {
    update_ranges_kernel<<<1, 1, 0, stream>>>(act_lo, act_hi, w_lo, w_hi, act_min, act_max, act_seen, w_min, w_max, w_seen,
                                              keep, momentum, a_qmax, w_qmax, eps, quant);
    return launch_status();
}

int layer_weight_prep(const float *weight, long s_co, long s_c, long s_h, long s_w, int Cout, int Cin, int kh, int kw,
                      const float *quant, float qmax, uint8_t *wmat, float *wsum, cudaStream_t stream) {
    weight_prep_kernel<<<Cout, 256, kh * kw * sizeof(float), stream>>>(weight, s_co, s_c, s_h, s_w, Cout, Cin, kh, kw, quant,
                                                                      qmax, wmat, wsum);
    return launch_status();
}

int layer_cross_terms(const float *wsum, int Cout, const ConvGeom &g, float *sumw_t, float *taps, int num_sms,
                      cudaStream_t stream) {
    cross_terms_kernel<<<grid_for((long)g.Ho * g.Wo * Cout, num_sms), 256, 0, stream>>>(wsum, Cout, g, sumw_t, taps);
    return launch_status();
}

int layer_window_sum(const float *img, const ConvGeom &g, float *box, int num_sms, cudaStream_t stream) {
    window_sum_kernel<<<grid_for((long)g.B * g.Ho * g.Wo, num_sms), 256, 0, stream>>>(img, g, box);
    return launch_status();
}

int layer_window_sum_adjoint(const float *gsum, const ConvGeom &g, float *out, int num_sms, cudaStream_t stream) {
    window_sum_adjoint_kernel<<<grid_for((long)g.B * g.H * g.W, num_sms), 256, 0, stream>>>(gsum, g, out);
    return launch_status();
}

int layer_weight_grad_finish(const float *gwmat, const float *tapg, const float *weight, long s_co, long s_c, long s_h,
                             long s_w, int Cout, int Cin, int kh, int kw, const float *quant, float qmax, float *gw,
                             int num_sms, cudaStream_t stream) {
    weight_grad_finish_kernel<<<grid_for((long)Cin * kh * kw * Cout, num_sms), 256, 0, stream>>>(
        gwmat, tapg, weight, s_co, s_c, s_h, s_w, Cout, Cin, kh, kw, quant, qmax, gw);
    return launch_status();
}

}  // namespace lutgemm
