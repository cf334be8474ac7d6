/*
 * CPU oracle for the approximate-multiplier LUT-GEMM (TEST INFRASTRUCTURE, not product code).
 *
 * This file restates, in plain C, the arithmetic of the reference CUDA operator so that the
 * sm_100a kernels can be checked against it.  Only the test-suite, the smoke check and the
 * cpu_baseline / reference legs of the benchmark may call into it; the product path never does.
 *
 * What each function follows in the reference (paths relative to the reference project):
 *   geometry            self_ops/src/approx_mult.h:12-41      (ROW = 2^b+1, COL = 2^b+2, tail padding,
 *                                                              null code 2^b, FACTOR = 1/16)
 *   oracle_forward      self_ops/src/approx_gemm_forward.cu:183-208  (idx = a*COL + b; uint32 += uint16)
 *                       self_ops/src/approx_gemm_forward.cu:142-176  (out-of-range lanes use the null
 *                                                              code whose row/column is all zero)
 *   oracle_backward     self_ops/src/approx_gemm_backward.cu:213-241 (gA: ascending n, fp32 FMA of
 *                                                              gC * float(int16), one final *FACTOR)
 *                       self_ops/src/approx_gemm_backward.cu:447-475 (gB: ascending m, same arithmetic)
 *   oracle_im2col_*     self_ops/ops_py/approx_ops.py:556-571 (pad with code 0, unfold with K ordered
 *                                                              (cin, kh, kw), rows ordered (b, oh, ow))
 *
 * Parity pin: the reference ships no tests or golden vectors for this path.  The oracle is pinned
 * instead (a) against the reference's own gather expression evaluated by importing its Python LUT
 * loader in the development container (fixtures under tests/golden/, generator committed beside
 * them) and (b) against the reference's checked-in LUT files' self-consistency headers.
 *
 * Build: gcc -O3 -fopenmp -shared -fPIC (see oracle/build_oracle.py).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_FACTOR (1.0f / 16.0f)

static int geom(int bits, int *row, int *col, int *elems) {
    int pad;
    switch (bits) {
        case 4: pad = 718; break;
        case 6: pad = 830; break;
        case 7: pad = 638; break;
        case 8: pad = 0; break;
        default: return -1;
    }
    *row = (1 << bits) + 1;
    *col = (1 << bits) + 2;
    *elems = (*row) * (*col) + pad;
    return 0;
}

int oracle_lut_elem_num(int bits) {
    int r, c, e;
    if (geom(bits, &r, &c, &e)) return -1;
    return e;
}

int oracle_lut_col_num(int bits) {
    int r, c, e;
    if (geom(bits, &r, &c, &e)) return -1;
    return c;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* C[m,n] = sum_k lut[a[m,k]*COL + w[k,n]]  (uint32 wrap-around accumulate, as the reference) */
int oracle_forward(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits,
                   long M, long K, long N) {
    int row, col, elems;
    if (geom(bits, &row, &col, &elems)) return -1;
#pragma omp parallel for schedule(static)
    for (long m = 0; m < M; ++m) {
        uint32_t *cm = c + m * N;
        for (long n = 0; n < N; ++n) cm[n] = 0u;
        for (long k = 0; k < K; ++k) {
            const uint16_t *lrow = lut + (long)a[m * K + k] * col;
            const uint8_t *wk = w + k * N;
            for (long n = 0; n < N; ++n) cm[n] += lrow[wk[n]];
        }
    }
    return 0;
}

/*
 * gA[m,k] = FACTOR * sum_{n ascending} gC[m,n] * float(lut_ga[a[m,k]*COL + w[k,n]])
 * gW[k,n] = FACTOR * sum_{m ascending} float(lut_gw[a[m,k]*COL + w[k,n]]) * gC[m,n]
 * Each term is one fused multiply-add in fp32, which is what the reference kernels compile to.
 */
int oracle_backward(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                    const int16_t *lut_ga, const int16_t *lut_gw, int bits, long M, long K, long N) {
    int row, col, elems;
    if (geom(bits, &row, &col, &elems)) return -1;
    if (ga) {
#pragma omp parallel for schedule(static)
        for (long m = 0; m < M; ++m) {
            const float *gcm = gc + m * N;
            for (long k = 0; k < K; ++k) {
                const int16_t *lrow = lut_ga + (long)a[m * K + k] * col;
                const uint8_t *wk = w + k * N;
                float acc = 0.0f;
                for (long n = 0; n < N; ++n) acc = fmaf(gcm[n], (float)lrow[wk[n]], acc);
                ga[m * K + k] = acc * ORACLE_FACTOR;
            }
        }
    }
    if (gw) {
#pragma omp parallel for schedule(static)
        for (long k = 0; k < K; ++k) {
            float *gwk = gw + k * N;
            const uint8_t *wk = w + k * N;
            for (long n = 0; n < N; ++n) gwk[n] = 0.0f;
            for (long m = 0; m < M; ++m) {
                const int16_t *lrow = lut_gw + (long)a[m * K + k] * col;
                const float *gcm = gc + m * N;
                for (long n = 0; n < N; ++n) gwk[n] = fmaf((float)lrow[wk[n]], gcm[n], gwk[n]);
            }
            for (long n = 0; n < N; ++n) gwk[n] *= ORACLE_FACTOR;
        }
    }
    return 0;
}

/* float64 evaluation of the same sums, used to bound the fp32 rounding of any summation order */
int oracle_backward_f64(const float *gc, const uint8_t *a, const uint8_t *w, double *ga, double *gw,
                        double *ga_abs, double *gw_abs, const int16_t *lut_ga, const int16_t *lut_gw,
                        int bits, long M, long K, long N) {
    int row, col, elems;
    if (geom(bits, &row, &col, &elems)) return -1;
#pragma omp parallel for schedule(static)
    for (long m = 0; m < M; ++m) {
        const float *gcm = gc + m * N;
        for (long k = 0; k < K; ++k) {
            const int16_t *lrow = lut_ga + (long)a[m * K + k] * col;
            const uint8_t *wk = w + k * N;
            double acc = 0.0, aabs = 0.0;
            for (long n = 0; n < N; ++n) {
                double t = (double)gcm[n] * (double)lrow[wk[n]];
                acc += t;
                aabs += fabs(t);
            }
            ga[m * K + k] = acc / 16.0;
            if (ga_abs) ga_abs[m * K + k] = aabs / 16.0;
        }
    }
#pragma omp parallel for schedule(static)
    for (long k = 0; k < K; ++k) {
        const uint8_t *wk = w + k * N;
        for (long n = 0; n < N; ++n) {
            gw[k * N + n] = 0.0;
            if (gw_abs) gw_abs[k * N + n] = 0.0;
        }
        for (long m = 0; m < M; ++m) {
            const int16_t *lrow = lut_gw + (long)a[m * K + k] * col;
            const float *gcm = gc + m * N;
            for (long n = 0; n < N; ++n) {
                double t = (double)lrow[wk[n]] * (double)gcm[n];
                gw[k * N + n] += t;
                if (gw_abs) gw_abs[k * N + n] += fabs(t);
            }
        }
        for (long n = 0; n < N; ++n) {
            gw[k * N + n] /= 16.0;
            if (gw_abs) gw_abs[k * N + n] /= 16.0;
        }
    }
    return 0;
}

/*
 * im2col of a code tensor x[B,C,H,W] (uint8) -> col[B*Ho*Wo, C*kh*kw]; spatial padding is code 0
 * (it contributes LUT[0][w], not zero), K index = (c*kh + i)*kw + j, row index = (b*Ho + oh)*Wo + ow.
 */
int oracle_im2col_u8(const uint8_t *x, uint8_t *col, long B, long C, long H, long W, long kh, long kw,
                     long stride, long pad, long dil) {
    long Ho = (H + 2 * pad - dil * (kh - 1) - 1) / stride + 1;
    long Wo = (W + 2 * pad - dil * (kw - 1) - 1) / stride + 1;
    long Kc = C * kh * kw;
#pragma omp parallel for schedule(static)
    for (long r = 0; r < B * Ho * Wo; ++r) {
        long b = r / (Ho * Wo), oh = (r / Wo) % Ho, ow = r % Wo;
        for (long c = 0; c < C; ++c)
            for (long i = 0; i < kh; ++i)
                for (long j = 0; j < kw; ++j) {
                    long ih = oh * stride - pad + i * dil, iw = ow * stride - pad + j * dil;
                    uint8_t v = 0;
                    if (ih >= 0 && ih < H && iw >= 0 && iw < W) v = x[((b * C + c) * H + ih) * W + iw];
                    col[r * Kc + (c * kh + i) * kw + j] = v;
                }
    }
    return 0;
}

/* adjoint of the above for fp32 gradients: gx[B,C,H,W] += gcol (padding positions are dropped) */
int oracle_col2im_f32(const float *gcol, float *gx, long B, long C, long H, long W, long kh, long kw,
                      long stride, long pad, long dil) {
    long Ho = (H + 2 * pad - dil * (kh - 1) - 1) / stride + 1;
    long Wo = (W + 2 * pad - dil * (kw - 1) - 1) / stride + 1;
    long Kc = C * kh * kw;
    memset(gx, 0, sizeof(float) * (size_t)(B * C * H * W));
    /* serial over rows inside one image so the fp32 add order is deterministic (ascending row, k) */
#pragma omp parallel for schedule(static)
    for (long b = 0; b < B; ++b)
        for (long oh = 0; oh < Ho; ++oh)
            for (long ow = 0; ow < Wo; ++ow) {
                long r = (b * Ho + oh) * Wo + ow;
                for (long c = 0; c < C; ++c)
                    for (long i = 0; i < kh; ++i)
                        for (long j = 0; j < kw; ++j) {
                            long ih = oh * stride - pad + i * dil, iw = ow * stride - pad + j * dil;
                            if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                                gx[((b * C + c) * H + ih) * W + iw] += gcol[r * Kc + (c * kh + i) * kw + j];
                        }
            }
    return 0;
}
