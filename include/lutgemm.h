/*
 * lutgemm.h - C ABI of the sm_100a approximate-multiplier LUT-GEMM library (liblutgemm_b200.so).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle (cudaStream_t passed
 * as void*; NULL = the legacy default stream).  All functions return 0 on success and a negative
 * LUTGEMM_E_* status otherwise; nothing here prints, exits or throws.  The library keeps no mutable
 * host state apart from idempotent per-device attribute caches, so calls are re-entrant across
 * host threads.  Each entry point names the reference interface it replaces (paths are relative to
 * the reference project changmg/AppMult-Aware-Retraining).
 *
 * Table wire format (self_ops/src/approx_mult.h:12-41, self_ops/ops_py/approx_ops.py:18-79):
 * a flat array of LUT_ELEM_NUM entries, entry (a, w) at a*(2^bits+2) + w, everything outside
 * [0,2^bits)^2 zero.  LUT_ELEM_NUM is 1024 / 5120 / 17408 / 66306 for bits = 4 / 6 / 7 / 8.
 * Operand codes must lie in [0, 2^bits); the kernels mask codes to `bits` bits so a stray code can
 * never read outside the staged table.
 */
#ifndef LUTGEMM_H
#define LUTGEMM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LUTGEMM_OK 0
#define LUTGEMM_E_BADARG (-1)      /* null pointer, non-positive size, misaligned buffer */
#define LUTGEMM_E_BITS (-2)        /* bits not in {4,6,7,8} */
#define LUTGEMM_E_CUDA (-3)        /* a CUDA runtime call or the kernel launch failed */
#define LUTGEMM_E_SCRATCH (-4)     /* scratch buffer too small */
#define LUTGEMM_E_TOOLARGE (-5)    /* size beyond what the entry point supports */

/* Library version (major*10000 + minor*100 + patch). */
int lutgemm_version(void);

/* Number of kernels this library has launched in this process so far (all entry points, all threads):
 * the difference of two readings counts the launches in between.  No counterpart in the reference. */
unsigned long long lutgemm_kernel_launches(void);

/*
 * Kernel-family override, process-wide; 0 (LUTGEMM_KERNEL_AUTO) in every position restores the automatic
 * choice by problem shape, which is the default.  Meant for tests that must reach every kernel family on one
 * shape and for A/B timing; results do not depend on it (forward bit-identical, gradients within fp32
 * summation order).  forward: row-broadcast or slab kernel; backward: broadcast or slab gradient kernels;
 * grad_tile: 512 x 64 or 1024 x 32 slab tile.  Call the *_scratch_bytes functions after changing it.
 * No counterpart in the reference (one kernel per operator there).
 */
#define LUTGEMM_KERNEL_AUTO 0
#define LUTGEMM_FORWARD_ROWBCAST 1
#define LUTGEMM_FORWARD_SLAB 2
#define LUTGEMM_BACKWARD_BCAST 1
#define LUTGEMM_BACKWARD_SLAB 2
#define LUTGEMM_TILE_WIDE 1
#define LUTGEMM_TILE_TALL 2
int lutgemm_set_kernel_choice(int forward, int backward, int grad_tile);

/*
 * How the 16 warps of a CTA of the tall gradient slab kernels pass slab buffers to each other, process-wide:
 * 1 (default) = through per-buffer shared-memory barriers with one arrival per warp, so warps may drift by half a
 * read phase; 0 = one CTA-wide barrier per k.  Same results either way; exists for A/B timing and tests.
 * No counterpart in the reference.
 */
int lutgemm_set_handover(int on);

/*
 * How the forward slab kernel fetches its operand-code chunks when it has the transposed copy of the activation
 * codes, process-wide: 1 (default) = tiled bulk-tensor copies (TMA) issued by one thread straight into shared
 * memory, 0 = 16-byte vector loads through registers.  Same results either way; exists for A/B timing and tests.
 * No counterpart in the reference (its kernels load byte-wise or with 4-byte loads, approx_gemm_forward.cu:142-176).
 */
int lutgemm_set_tma(int on);

/* Human-readable text for a status code; for LUTGEMM_E_CUDA the CUDA error behind the calling thread's
 * last such status is appended.  The returned pointer is valid until the thread's next call. */
const char *lutgemm_status_string(int status);

/* Padded flat table length for a bit-width, or LUTGEMM_E_BITS.
 * Replaces the compile-time LUT_ELEM_NUM of self_ops/src/approx_mult.h:12-38. */
int lutgemm_lut_elem_num(int bits);

/* Inverse of the above: bit-width whose padded table has `elem_num` entries, or LUTGEMM_E_BITS.
 * The reference fixes the bit-width at compile time (approx_mult.h:12); here it is inferred from
 * the table the caller passes, so one binary serves every width. */
int lutgemm_bits_from_elem_num(long elem_num);

/*
 * Forward:  c[m,n] = sum_{k<K} lut[a[m,k]*(2^bits+2) + w[k,n]]      (uint32 accumulate, exact)
 *   a   [M,K] uint8 row-major      w [K,N] uint8 row-major      c [M,N] uint32 row-major (overwritten)
 *   lut flat uint16 [lutgemm_lut_elem_num(bits)]
 * Replaces approx_gemm_forward_gpu, self_ops/src/approx_gemm_forward.cu:241-314 (kernel :37-229),
 * bound to Python at self_ops/src/op_register.cpp:16.
 */
int lutgemm_forward(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits,
                    int M, int K, int N, void *stream);

/*
 * Forward with a workspace.  With `scratch` (lutgemm_forward_scratch_bytes() bytes, 16-byte aligned; 0 bytes
 * means the kernel chosen for this shape has no use for it and NULL may be passed) the activation codes are
 * first transposed into it ([K][M rounded up to 16] uint8) and the main kernel reads them from there with
 * coalesced loads; results are identical to lutgemm_forward.  No counterpart in the reference.
 */
size_t lutgemm_forward_scratch_bytes(int bits, int M, int K, int N);
int lutgemm_forward_ws(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                       int N, void *scratch, size_t scratch_bytes, void *stream);

/*
 * Scratch bytes lutgemm_backward needs for a problem (0 when none is needed).  The weight-gradient
 * kernel splits its long reduction over M into slabs whose partial sums live in this buffer, followed
 * by a transposed copy of the activation codes.
 * No counterpart in the reference (its GB kernel never splits M, approx_gemm_backward.cu:587-608).
 */
size_t lutgemm_backward_scratch_bytes(int bits, int M, int K, int N);

/*
 * Backward:  ga[m,k] = (1/16) * sum_{n<N} gc[m,n] * float(lut_ga[a[m,k]*(2^bits+2) + w[k,n]])
 *            gw[k,n] = (1/16) * sum_{m<M} float(lut_gw[a[m,k]*(2^bits+2) + w[k,n]]) * gc[m,n]
 *   gc [M,N] float32    ga [M,K] float32 (overwritten)    gw [K,N] float32 (overwritten)
 *   lut_ga, lut_gw flat int16 tables holding round(16 * dAM/da) and round(16 * dAM/dw)
 *   ga or gw may be NULL to skip that gradient.
 *   scratch: device buffer of at least lutgemm_backward_scratch_bytes() bytes, 16-byte aligned (may be
 *   NULL when that is 0); its contents on return are unspecified.
 * Replaces approx_gemm_backward_gpu, self_ops/src/approx_gemm_backward.cu:506-624 (kernels :13-258
 * and :261-492), bound to Python at self_ops/src/op_register.cpp:18.
 */
int lutgemm_backward(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                     const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N,
                     void *scratch, size_t scratch_bytes, void *stream);

/*
 * lutgemm_backward with the transposed activation codes that lutgemm_forward_ws left in its workspace for the
 * same `a` (codes_t, [K][M rounded up to 16] uint8; may be NULL): the weight-gradient kernel then skips its own
 * transposition.  Same results.  No counterpart in the reference.
 */
int lutgemm_backward_ws(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                        const int16_t *lut_ga, const int16_t *lut_gw, int bits, int M, int K, int N,
                        const uint8_t *codes_t, void *scratch, size_t scratch_bytes, void *stream);

/*
 * Backward with the gradient tables in fp32 (bit-widths up to 7): the same sums as lutgemm_backward with
 * float(lut) replaced by the fp32 entry and without the 1/16 factor,
 *   ga[m,k] = sum_n gc[m,n] * lut_ga[a[m,k]*(2^bits+2) + w[k,n]],   gw[k,n] = sum_m lut_gw[...] * gc[m,n].
 * The tables use the padded flat layout of the wire format with float entries.  For callers whose gradient
 * tables are not multiples of 1/16 (the reference rounds them to that grid when it writes its LUT files,
 * scripts/gen_bp_lut.py:171-183, and its kernels only take the int16 form, approx_gemm_backward.cu:506-529).
 * At 8 bits an fp32 table (256 KB) does not fit next to the slabs in shared memory: LUTGEMM_E_BITS.
 * scratch: lutgemm_backward_f32lut_scratch_bytes() bytes, 16-byte aligned.  No counterpart in the reference.
 */
size_t lutgemm_backward_f32lut_scratch_bytes(int bits, int M, int K, int N);
int lutgemm_backward_f32lut(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, float *gw,
                            const float *lut_ga, const float *lut_gw, int bits, int M, int K, int N, void *scratch,
                            size_t scratch_bytes, void *stream);

/*
 * Convolution forward with the im2col fused into the operand loader (this entry point writes no unfolded
 * tensor; lutgemm_conv2d_forward_ws below trades one uint8 copy of the unfolded codes for faster loads):
 *   y[(b*Ho+oh)*Wo+ow, n] = sum_{c,i,j} lut[ x[b,c,oh*stride-pad+i*dil,ow*stride-pad+j*dil] * (2^bits+2) + wmat[(c*kh+i)*kw+j, n] ]
 * with code 0 outside the image (spatial padding looks up lut[0][w], as in the reference).
 *   x    [B,C,H,W] uint8 codes (NCHW)       wmat [C*kh*kw, Cout] uint8 (the weight viewed [Cout,-1], transposed)
 *   y    [B*Ho*Wo, Cout] uint32, i.e. NHWC;  Ho = (H + 2*pad - dil*(kh-1) - 1)/stride + 1, Wo likewise
 * Replaces approx_conv2d_op's F.pad + F.unfold + transpose/reshape + approx_gemm_forward chain,
 * self_ops/ops_py/approx_ops.py:556-571 (square stride/padding/dilation, groups = 1, no bias, :545-547).
 */
int lutgemm_conv2d_forward(const uint8_t *x, const uint8_t *wmat, uint32_t *y, const uint16_t *lut, int bits,
                           int B, int C, int H, int W, int Cout, int kh, int kw, int stride, int pad, int dil,
                           void *stream);

/* Scratch bytes lutgemm_conv2d_backward needs: per-row-block partial sums of the gradient kernels and, for the
 * weight gradient, a transposed uint8 copy of the unfolded activation CODES (M*K bytes) when the caller passes
 * none.  No fp32 unfolded gradient is ever materialised.  No counterpart in the reference. */
size_t lutgemm_conv2d_backward_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                             int stride, int pad, int dil);

/*
 * Convolution backward through the gradient tables, activations gathered on the fly as in the forward:
 *   gw[(c*kh+i)*kw+j, n] = 1/16 * sum_m lut_gw[a[m,k]][wmat[k,n]] * gy[m,n]                 ([C*kh*kw, Cout] fp32)
 *   gx[b,c,h,w] = 1/16 * sum over the taps (i,j) that reach (h,w) and over n of
 *                 gy[m(b,h,w,i,j), n] * lut_ga[x[b,c,h,w]][wmat[(c*kh+i)*kw+j, n]]          ([B,C,H,W] fp32)
 *   gy [B*Ho*Wo, Cout] fp32 (NHWC).  gx or gw may be NULL.
 * gx is computed per input pixel (every tap that touches a pixel sees the same activation code, so the sum over
 * taps joins the sum over n); the unfolded activation gradient [B*Ho*Wo, C*kh*kw] the reference forms and folds
 * back (autograd of F.unfold) never exists.  Overlapping windows with more than 128 taps are refused
 * (LUTGEMM_E_TOOLARGE).  Sums are deterministic.
 * Replaces the autograd chain of approx_conv2d_op (unfold backward + approx_gemm_backward),
 * self_ops/ops_py/approx_ops.py:181-205,556-571.
 */
int lutgemm_conv2d_backward(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, float *gw,
                            const int16_t *lut_ga, const int16_t *lut_gw, int bits, int B, int C, int H, int W,
                            int Cout, int kh, int kw, int stride, int pad, int dil, void *scratch,
                            size_t scratch_bytes, void *stream);

/*
 * Convolution forward / backward sharing one transposed copy of the unfolded activation codes.
 * lutgemm_conv2d_forward_ws: as lutgemm_conv2d_forward; with `scratch`
 * (lutgemm_conv2d_forward_scratch_bytes() bytes, 16-byte aligned; 0 = not used for this shape) the uint8
 * im2col is written there once, transposed ([C*kh*kw][B*Ho*Wo rounded up to 16]), instead of being gathered
 * by every tile of the main kernel, and stays valid on return.
 * lutgemm_conv2d_backward_ws: as lutgemm_conv2d_backward; `codes_t` (may be NULL) is that buffer as the
 * forward pass of the same layer left it, which saves the weight-gradient kernel its own transposition.
 * No counterpart in the reference (it materialises the unfolded activations in fp32, twice).
 */
size_t lutgemm_conv2d_forward_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                            int stride, int pad, int dil);
int lutgemm_conv2d_forward_ws(const uint8_t *x, const uint8_t *wmat, uint32_t *y, const uint16_t *lut, int bits, int B,
                              int C, int H, int W, int Cout, int kh, int kw, int stride, int pad, int dil,
                              void *scratch, size_t scratch_bytes, void *stream);
int lutgemm_conv2d_backward_ws(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, float *gw,
                               const int16_t *lut_ga, const int16_t *lut_gw, int bits, int B, int C, int H, int W,
                               int Cout, int kh, int kw, int stride, int pad, int dil, const uint8_t *codes_t,
                               void *scratch, size_t scratch_bytes, void *stream);

/*
 * Quantisation prologue of an approximate convolution layer, one pass:
 *   codes[b,c,h,w] = uint8(clamp(rint(x[b,c,h,w] / *scale - *zp_neg), 0, qmax))     NCHW-contiguous
 *   chansum[b,h,w] += sum_c codes[b,c,h,w]      (optional; the caller zeroes it; exact, the sums are integers)
 * x is any dense 4-D fp32 tensor given by its element strides (NCHW or channels-last); scale and zp_neg are
 * device pointers to one float each (module buffers), so nothing synchronises with the host.
 * Replaces the elementwise chain of ApproxConv2d.forward, micronet+/app_layers.py:147-150,163-166
 * (x / scale - zero_point, round with straight-through gradient, clamp) and the uint8 cast of
 * self_ops/ops_py/approx_ops.py:563.
 */
int lutgemm_quantize_activations(const float *x, long stride_b, long stride_c, long stride_h, long stride_w, int B,
                                 int C, int H, int W, const float *scale, const float *zp_neg, float qmax,
                                 uint8_t *codes, float *chansum, void *stream);

/*
 * Backward of the prologue (straight-through rounding, clamp mask), fused with the zero-point cross term
 * and the weight scale:
 *   gx[b,c,h,w] = [0 <= rint(x / *scale - *zp_neg) <= qmax] * *s_w * (gcodes[b,c,h,w] + *z_w * box_t[b,h,w])
 * gcodes is NCHW-contiguous (what lutgemm_conv2d_backward returns for an un-scaled grad_out), box_t may be
 * NULL, gx has the strides of x.  Replaces the autograd chain of the same lines.
 */
int lutgemm_quantize_activations_backward(const float *x, long stride_b, long stride_c, long stride_h, long stride_w,
                                          int B, int C, int H, int W, const float *scale, const float *zp_neg,
                                          float qmax, const float *gcodes, const float *box_t, const float *s_w,
                                          const float *z_w, float *gx, void *stream);

/*
 * De-quantisation epilogue of an approximate convolution layer, one pass over the accumulators:
 *   out[m,co] = *s_a * *s_w * (y[m,co] + *z_w * box[m] + *z_a * sumw_t[l,co] + *z_a * *z_w * taps[l]) (+ bias[co])
 * with m = b*L + l, y the uint32 result of lutgemm_conv2d_forward ([M, Cout]), box [M] the window sums of the
 * activation codes, sumw_t [L, Cout] the window sums of the weight codes, taps [L] the valid-tap counts times
 * Cin; each product and sum is rounded separately, in this order.  bias may be NULL.
 * Replaces micronet+/app_layers.py:175-184 (three cross-term convolutions, adds, scale).
 */
int lutgemm_conv2d_epilogue(const uint32_t *y, const float *box, const float *sumw_t, const float *taps,
                            const float *s_a, const float *s_w, const float *z_a, const float *z_w, const float *bias,
                            float *out, long M, int L, int Cout, void *stream);

/*
 * Forward of a whole approximate layer in one kernel: lutgemm_conv2d_forward_ws (or lutgemm_forward_ws for a
 * linear layer, L = 1) with lutgemm_conv2d_epilogue applied to the sums while they are still in registers, so the
 * uint32 accumulators [M, Cout] are neither written nor read back:
 *   out[m,co] = *s_a * *s_w * (sum[m,co] + *z_w * box[m] + *z_a * sumw_t[l,co] + *z_a * *z_w * taps[l]) (+ bias[co])
 * with m = b*L + l; arguments as for the two functions it combines.  scratch: lutgemm_*_forward_layer_scratch_bytes()
 * bytes, 16-byte aligned: first the transposed-codes workspace of lutgemm_conv2d_forward_scratch_bytes /
 * lutgemm_forward_scratch_bytes (valid on return, reusable by the backward of the same layer), then - only for
 * shapes with so few output tiles that the kernel cuts K across CTAs, whose partial sums have to meet in memory -
 * room for the uint32 sums, which the one-pass epilogue kernel then finishes.  scratch may be NULL when the
 * function returns 0 bytes.
 * Replaces self_ops.approx_conv2d_op's forward plus micronet+/app_layers.py:175-184.
 */
size_t lutgemm_conv2d_forward_layer_scratch_bytes(int bits, int B, int C, int H, int W, int Cout, int kh, int kw,
                                                  int stride, int pad, int dil);
size_t lutgemm_forward_layer_scratch_bytes(int bits, int M, int K, int N);
int lutgemm_conv2d_forward_layer(const uint8_t *x, const uint8_t *wmat, const uint16_t *lut, int bits, int B, int C, int H,
                                 int W, int Cout, int kh, int kw, int stride, int pad, int dil, const float *box,
                                 const float *sumw_t, const float *taps, const float *s_a, const float *s_w,
                                 const float *z_a, const float *z_w, const float *bias, float *out, void *scratch,
                                 size_t scratch_bytes, void *stream);
int lutgemm_forward_layer(const uint8_t *a, const uint8_t *w, const uint16_t *lut, int bits, int M, int K, int N,
                          const float *box, const float *sumw_t, const float *taps, const float *s_a, const float *s_w,
                          const float *z_a, const float *z_w, const float *bias, float *out, void *scratch,
                          size_t scratch_bytes, void *stream);

/*
 * Small one-pass kernels of the layer wiring; each stands for a chain of PyTorch elementwise / slicing kernels of
 * ApproxConv2d.forward, its observers and their autograd backward (micronet+/app_layers.py:21-53, 147-184).
 * quant is a device array {s_a, z_a, s_w, z_w} (activation scale, activation zero point, weight scale, weight zero
 * point, the zero points being round(min / scale)); strides are in elements; nothing synchronises with the host.
 *
 * lutgemm_layer_update_ranges: the layer's observers and quantisation parameters in one launch.  act_lo/act_hi,
 *   w_lo/w_hi: min and max of this batch's activations and of the weights (device scalars); the act_ and w_ state: the
 *   exponential moving average (keep = 1 - momentum) of the activation range, the running range of the weights and
 *   their "seen" flags (0 before the first batch), updated in place; quant = {max((amax-amin)/a_qmax, eps),
 *   round(amin/s_a), max((wmax-wmin)/w_qmax, eps), round(wmin/s_w)}.   (:21-53, :155-160)
 * lutgemm_layer_weight_prep: wmat[(c*kh+i)*kw+j, co] = uint8(clamp(round(weight[co,c,i,j]/s_w - z_w), 0, qmax)) and
 *   wsum[co, i*kw+j] = sum_c of those codes.   (:147-150, :173 and the uint8 cast / transposition of
 *   self_ops/ops_py/approx_ops.py:563-564)
 * lutgemm_layer_cross_terms: sumw_t[l, co] = sum of wsum[co, t] over the taps t inside the image at output
 *   position l; taps[l] = Cin * their number (the convolutions with a constant image of :179-180).
 * lutgemm_layer_window_sum: box[b, oh, ow] = sum of img[b, ., .] over the kernel window (zero padding), img the
 *   channel sums of the activation codes (the convolution with a constant weight of :178).
 * lutgemm_layer_window_sum_adjoint: out[b, h, w] = sum of gsum[b, oh, ow] over the windows that contain (h, w).
 * lutgemm_layer_weight_grad: gw[co,c,i,j] = [0 <= round(weight/s_w - z_w) <= qmax] * s_a *
 *   (gwmat[(c*kh+i)*kw+j, co] + z_a * tapg[co, i*kw+j]), gw contiguous.
 */
int lutgemm_layer_update_ranges(const float *act_lo, const float *act_hi, const float *w_lo, const float *w_hi,
                                float *act_min, float *act_max, float *act_seen, float *w_min, float *w_max, float *w_seen,
                                float keep, float momentum, float a_qmax, float w_qmax, float eps, float *quant,
                                void *stream);
int lutgemm_layer_weight_prep(const float *weight, long s_co, long s_c, long s_h, long s_w, int Cout, int Cin, int kh, int kw,
                              const float *quant, float qmax, uint8_t *wmat, float *wsum, void *stream);
int lutgemm_layer_cross_terms(const float *wsum, int Cout, int Cin, int H, int W, int kh, int kw, int stride, int pad,
                              int dil, float *sumw_t, float *taps, void *stream);
int lutgemm_layer_window_sum(const float *img, int B, int H, int W, int kh, int kw, int stride, int pad, int dil,
                             float *box, void *stream);
int lutgemm_layer_window_sum_adjoint(const float *gsum, int B, int H, int W, int kh, int kw, int stride, int pad, int dil,
                                     float *out, void *stream);
int lutgemm_layer_weight_grad(const float *gwmat, const float *tapg, const float *weight, long s_co, long s_c, long s_h,
                              long s_w, int Cout, int Cin, int kh, int kw, const float *quant, float qmax, float *gw,
                              void *stream);

/*
 * Weight gradient only, with no device memory taken from anyone: same result as lutgemm_backward with
 * ga == NULL, but the kernels' partial sums go to a fixed array inside the library image instead of a
 * caller-supplied scratch buffer.  Meant for callers that may not allocate when the gradient is due -
 * a runtime with a memory budget fixed at start-up, a binding that cannot reach the framework's
 * allocator, code on a path where cudaMalloc's implicit synchronisation is not acceptable.
 *   - The array is LUTGEMM_NOALLOC_SCRATCH_BYTES (32 MiB) per GPU that loads the library, held until
 *     the process exits; lutgemm_noalloc_scratch_capacity() returns the figure.  A problem whose partial
 *     sums need more is refused with LUTGEMM_E_TOOLARGE (lutgemm_backward_scratch_bytes tells the need: on
 *     the slab path one K*N*4-byte block per 1024 or 512 rows of M plus a transposed copy of the codes,
 *     K*M bytes; splits*K*N*4 on the split-M path; nothing for small M).
 *   - The first call made with a given device current looks up the array's address on that device
 *     (cudaGetSymbolAddress); make that first call before any stream capture begins.
 *   - All calls share the one array per device and it keeps whatever the last call left there.  Nothing
 *     in it has to be zero on entry (every partial sum is written before it is read).  Two calls that
 *     overlap on the same GPU - different streams, or different host threads - race on it: serialise them.
 *   - The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
 * No counterpart in the reference.
 */
#define LUTGEMM_NOALLOC_SCRATCH_BYTES (32u << 20)
size_t lutgemm_noalloc_scratch_capacity(void);
int lutgemm_backward_gw_noalloc(const float *gc, const uint8_t *a, const uint8_t *w, float *gw,
                                const int16_t *lut_gw, int bits, int M, int K, int N, void *stream);

/*
 * Reads and clears the device-side error word of the pipelined kernels into *value (0 = no error).
 * Their warps hand slabs to each other through shared-memory barriers; every wait on such a barrier is
 * bounded, and a wait that runs out records which one it was instead of hanging the GPU.  A non-zero
 * value means the results of launches since the last call are invalid.  Synchronises the device.
 * No counterpart in the reference (its kernels have no inter-warp waits).
 */
int lutgemm_device_error(int *value);

/*
 * Launches a one-warp kernel that waits on a shared-memory barrier nothing ever arrives on.  The wait
 * is bounded like every wait in the library: it gives up after one second, records error
 * id 99 (readable through lutgemm_device_error) and the kernel returns; the context stays usable.
 * Exists so that the time-out path can be exercised without hanging a GPU.  No counterpart in the
 * reference.
 */
int lutgemm_selftest_bounded_wait(void *stream);

#ifdef __cplusplus
}
#endif
#endif /* LUTGEMM_H */
