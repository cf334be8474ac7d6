// Shared device/host helpers of the sm_100a LUT-GEMM kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "lutgemm.h"

namespace lutgemm {

// ---- table geometry of the wire format (reference: self_ops/src/approx_mult.h:12-41) -------------
__host__ __device__ constexpr int lut_col_num(int bits) { return (1 << bits) + 2; }
__host__ __device__ constexpr int lut_row_num(int bits) { return (1 << bits) + 1; }
__host__ __device__ constexpr int lut_tail_pad(int bits) {
    return bits == 4 ? 718 : bits == 6 ? 830 : bits == 7 ? 638 : 0;
}
__host__ __device__ constexpr int lut_elem_num(int bits) {
    return lut_row_num(bits) * lut_col_num(bits) + lut_tail_pad(bits);
}
constexpr float kGradFactor = 1.0f / 16.0f;  // approx_mult.h:41

inline bool bits_supported(int bits) { return bits == 4 || bits == 6 || bits == 7 || bits == 8; }

// ---- implicit im2col ---------------------------------------------------------------------------
// Geometry of a convolution whose unfolded activation matrix a[m,k] is never materialised:
//   m = (b*Ho + oh)*Wo + ow,  k = (c*kh + i)*kw + j,  a[m,k] = x[b,c,oh*stride-pad+i*dil,ow*stride-pad+j*dil]
// or code 0 outside the image (the reference pads the code tensor with 0 before unfolding,
// self_ops/ops_py/approx_ops.py:556-563, so padding looks up LUT[0][w]).
struct ConvGeom {
    int enabled;
    int B, C, H, W, kh, kw, stride, pad, dil, Ho, Wo;
};

__device__ __forceinline__ uint32_t conv_code(const uint8_t *__restrict__ x, const ConvGeom &g, int m, int k) {
    const int L = g.Ho * g.Wo, kk = g.kh * g.kw;
    const int b = m / L, l = m - b * L, oh = l / g.Wo, ow = l - oh * g.Wo;
    const int c = k / kk, r = k - c * kk, i = r / g.kw, j = r - i * g.kw;
    const int ih = oh * g.stride - g.pad + i * g.dil, iw = ow * g.stride - g.pad + j * g.dil;
    if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
        return x[((size_t)(b * g.C + c) * g.H + ih) * g.W + iw];
    return 0u;
}

// 16 consecutive k of one unfolded row, packed little-endian into four words (k >= K gives 0)
__device__ __forceinline__ uint4 conv_code16(const uint8_t *__restrict__ x, const ConvGeom &g, int m, int kbase, int K) {
    const int L = g.Ho * g.Wo, kk = g.kh * g.kw;
    const int b = m / L, l = m - b * L, oh = l / g.Wo, ow = l - oh * g.Wo;
    int c = kbase / kk, r = kbase - c * kk, i = r / g.kw, j = r - i * g.kw;
    const int ih0 = oh * g.stride - g.pad, iw0 = ow * g.stride - g.pad;
    const uint8_t *xb = x + (size_t)b * g.C * g.H * g.W;
    uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        const int ih = ih0 + i * g.dil, iw = iw0 + j * g.dil;
        if (kbase + q < K && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
            t[q >> 2] |= (uint32_t)xb[((size_t)c * g.H + ih) * g.W + iw] << (8 * (q & 3));
        if (++j == g.kw) { j = 0; if (++i == g.kh) { i = 0; ++c; } }
    }
    return make_uint4(t[0], t[1], t[2], t[3]);
}

// Where grad_a[m,k] of a convolution lands in the image gradient gx[B,C,H,W] when the kernel windows do not
// overlap (every image position is touched by at most one (m,k)): the position a[m,k] was read from, or -1
// for padding.  Used by the gradient kernels to write such convolutions' activation gradient in place.
__device__ __forceinline__ long conv_scatter_index(const ConvGeom &g, int m, int k) {
    const int L = g.Ho * g.Wo, kk = g.kh * g.kw;
    const int b = m / L, l = m - b * L, oh = l / g.Wo, ow = l - oh * g.Wo;
    const int c = k / kk, r = k - c * kk, i = r / g.kw, j = r - i * g.kw;
    const int ih = oh * g.stride - g.pad + i * g.dil, iw = ow * g.stride - g.pad + j * g.dil;
    if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
        return (((long)b * g.C + c) * g.H + ih) * g.W + iw;
    return -1;
}

// Input pixels of one stride class of a convolution - h = ph + s*hh, w = pw + s*ww - and the kernel taps that
// reach them.  The activation gradient of an input pixel sums, over those taps (i,j) and the output channels n,
// gy[(b, (h - dh)/s, (w - dw)/s), n] * T(x[b,c,h,w], wmat[(c*T + t), n])  with dh = i*dil - pad, t = i*kw + j.
constexpr int kMaxTaps = 128;
struct PixelClass {
    int H, W, C;            // image
    int Hc, Wc;             // pixels of the class per image
    int ph, pw, s;
    int Ho, Wo;             // output positions of the convolution
    int ntaps, T;           // taps of the class; kh*kw
    int P;                  // pixels of the class over all images: B * Hc * Wc
    int8_t dh[kMaxTaps], dw[kMaxTaps];
    uint8_t t[kMaxTaps];
};
// up to four classes handled by one launch (all classes of a stride-2 convolution): class i owns the pixel tiles
// [tile_begin[i], tile_begin[i+1])
constexpr int kMaxClassesPerLaunch = 4;
struct PixelClassSet {
    int n;
    int tile_begin[kMaxClassesPerLaunch + 1];
    PixelClass c[kMaxClassesPerLaunch];
};
// pixel p of the class (counted over all images) -> offset of (b, channel 0, h, w) in the NCHW image
__host__ __device__ __forceinline__ size_t pixel_class_offset(const PixelClass &px, int p) {
    const int per = px.Hc * px.Wc, b = p / per, r = p - b * per, hh = r / px.Wc, ww = r - hh * px.Wc;
    return (size_t)b * px.C * px.H * px.W + (size_t)(px.ph + px.s * hh) * px.W + (px.pw + px.s * ww);
}

// De-quantisation of an approximate layer applied where a forward kernel stores its sums (out != nullptr):
//   out[m,n] = s_a s_w (sum[m,n] + z_w box[m] + z_a sumw_t[l,n] + z_a z_w taps[l]) (+ bias[n]),   l = m mod L
// every product and sum rounded separately in this order (the order the layer expression of
// micronet+/app_layers.py:175-184 evaluates them).  All scalars are device pointers: nothing syncs with the host.
struct LayerEpilogue {
    const float *box, *sumw_t, *taps, *s_a, *s_w, *z_a, *z_w, *bias;
    float *out;
    int L;
};
struct LayerEpilogueScalars {
    float s, za, zw, zz;
};
__device__ __forceinline__ LayerEpilogueScalars load_epilogue_scalars(const LayerEpilogue &e) {
    LayerEpilogueScalars v;
    v.za = *e.z_a;
    v.zw = *e.z_w;
    v.s = __fmul_rn(*e.s_a, *e.s_w);
    v.zz = __fmul_rn(v.za, v.zw);
    return v;
}
// row terms: z_w box[m] and z_a z_w taps[l], shared by every column of the row
__device__ __forceinline__ float epilogue_value(const LayerEpilogue &e, const LayerEpilogueScalars &v, uint32_t sum,
                                                float zw_box, float zz_taps, int l, int n, int N) {
    float acc = (float)sum;
    acc = __fadd_rn(acc, zw_box);
    acc = __fadd_rn(acc, __fmul_rn(v.za, e.sumw_t[(size_t)l * N + n]));
    acc = __fadd_rn(acc, zz_taps);
    float o = __fmul_rn(v.s, acc);
    if (e.bias) o = __fadd_rn(o, e.bias[n]);
    return o;
}

// ---- quotient by a divisor that is the same for many elements -----------------------------------
// x / s with the IEEE round-to-nearest result, from r = __frcp_rn(s) computed once: q0 = x r, then one fused
// correction with the exact remainder (Markstein's sequence; compared bit for bit with the IEEE division on
// 1.2e11 random operand pairs, divisor mantissas near all ones and near a power of two included).  The IEEE
// division itself costs about 47 instructions per element here.  Operands whose quotient or remainder could leave
// the normal range, infinities and divisors outside 2^-60 .. 2^60 take the IEEE division.
struct Divisor {
    float s, r;
    bool fast;
};
__device__ __forceinline__ Divisor make_divisor(float s) {
    Divisor d;
    d.s = s;
    d.r = __frcp_rn(s);
    const float as = fabsf(s);
    d.fast = as > 0x1p-60f && as < 0x1p60f;
    return d;
}
__device__ __forceinline__ float quotient(float x, const Divisor &d) {
    const float ax = fabsf(x);
    if (!d.fast || ax > 0x1p60f || (ax < 0x1p-60f && ax != 0.f)) return __fdiv_rn(x, d.s);
    const float q0 = x * d.r;
    return fmaf(fmaf(-q0, d.s, x), d.r, q0);
}

// ---- small device helpers ----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// 16-bit shared-memory gathers that land zero-/sign-extended in a 32-bit register (no cvt needed)
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int32_t lds_s16(uint32_t addr) {
    int32_t v;
    asm("ld.shared.s16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// byte i of v (one PRMT whatever i is; shift + mask costs two instructions for the middle bytes)
__device__ __forceinline__ uint32_t byte_of(uint32_t v, int i) { return __byte_perm(v, 0u, 0x4440u + i); }
// base + STRIDE * (byte i of v) in one integer dot-product instruction (STRIDE must fit a byte)
template <int STRIDE>
__device__ __forceinline__ uint32_t byte_scaled_add(uint32_t v, int i, uint32_t base) {
    static_assert(STRIDE > 0 && STRIDE < 256, "stride must fit one byte of the dot-product operand");
    return __dp4a(v, (uint32_t)STRIDE << (8 * i), base);
}

// Stage the padded wire-format table into shared memory as a dense [2^BITS][2^BITS] array of 16-bit
// entries.  TRANSPOSE=false: dst[a][w]; TRANSPOSE=true: dst[w][a].  The reference copies the padded
// table verbatim once per output tile (approx_gemm_forward.cu:81-92); here a persistent CTA stages
// it once per launch into the layout its gather pattern wants.
template <int BITS, bool TRANSPOSE, typename T>
__device__ __forceinline__ void stage_table(T *dst, const T *__restrict__ src, int tid, int nthreads) {
    constexpr int Q = 1 << BITS;
    constexpr int COL = lut_col_num(BITS);
    if (!TRANSPOSE) {
        if ((reinterpret_cast<uintptr_t>(src) & 3u) == 0) {
            // rows start at a*COL (COL even) so pairs of entries are 4-byte aligned
            const uint32_t *s32 = reinterpret_cast<const uint32_t *>(src);
            uint32_t *d32 = reinterpret_cast<uint32_t *>(dst);
#pragma unroll 8
            for (int i = tid; i < Q * Q / 2; i += nthreads) {
                int a = i / (Q / 2), wp = i % (Q / 2);
                d32[i] = __ldg(s32 + a * (COL / 2) + wp);
            }
        } else {
#pragma unroll 8
            for (int i = tid; i < Q * Q; i += nthreads) dst[i] = src[(i >> BITS) * COL + (i & (Q - 1))];
        }
    } else {
        // consecutive threads take consecutive a (contiguous shared-memory writes, strided L2 reads)
#pragma unroll 8
        for (int i = tid; i < Q * Q; i += nthreads) {
            int w = i >> BITS, a = i & (Q - 1);
            dst[i] = src[a * COL + w];
        }
    }
}

}  // namespace lutgemm
