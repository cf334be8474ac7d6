// Gradient LUT-GEMM kernels for sm_100a, fp32 column-gathered slab with a TALL tile (16*RW rows x 32 columns).
//
//   grad_w:  gw[k,n] = 1/16 * sum_m T(a[m,k], w[k,n]) * gc[m,n]     rows r = m, columns c = n
//   grad_a:  ga[m,k] = 1/16 * sum_n gc[m,n] * T(a[m,k], w[k,n])     rows r = n, columns c = m
//   grad_x:  gx[b,c,h,w] = 1/16 * sum_{taps (i,j)} sum_n gy[m(b,h,w,i,j), n] * T(x[b,c,h,w], wmat[(c,i,j), n])
//            rows r = (tap, n), columns = input pixels, the k loop runs over the input channels c
//
// Per k a slab U_k[x][c] = T(x, cc[k,c]) is gathered once, then every row reads slab row rc[r,k] contiguously
// (conflict-free: with RW = 64 half a warp per row and two fp32 columns per lane in one 64-bit load, otherwise a
// warp per row and one column per lane) and multiplies it with its grad_out entries held in registers (RW per
// thread).  The 2^b-row build is paid once per 16*RW rows; two slab buffers, so slab k+1 is built
// while slab k is read.
//
// grad_x is the activation gradient of a convolution WITHOUT the unfolded intermediate: every tap that
// touches an input pixel sees the same activation code, so the sum over taps joins the sum over n in one
// long row dimension (kh*kw*Cout rows: 576 for a 3x3 convolution with 64 output channels, which is why the
// kernel exists with RW = 36 as well), the column codes are the code image itself, the row codes are kh*kw
// rows of the weight matrix, and the result is written straight into the image gradient - no col2im, no
// atomics.  A strided convolution is cut into stride^2 classes of input pixels (h mod stride, w mod stride)
// that each see a fixed subset of the taps; one launch per class.
//
// Hand-over between the warps of a CTA: per slab buffer a "full" barrier (all 16 warps have built their part)
// and an "empty" barrier (all 16 warps have finished reading it), both mbarriers with one arrival per warp.
// A warp reads the first half of its rows of slab k, then - once slab k-1 has been released - adds up the
// partial sums of k-1 if it is its turn, builds its part of slab k+1, and reads the second half of its rows:
// each wait has half a read phase of slack, so warps drift instead of lining up behind a CTA barrier per k.
// Every wait is bounded (lutgemm_waits.cuh).
// Partial sums: one per lane, warp and k; the 16 warps are added in ascending order by one warp (rotating
// with k), row blocks by slab_reduce_blocks in ascending order: results are deterministic.
// grad_w takes its row codes from a transposed copy at[k][m] of the activation codes when the caller has one.
// Replaces ApproxGemmBackwardKernelForGA / ForGB, self_ops/src/approx_gemm_backward.cu:13-258, 261-492, and for
// grad_x the unfold backward of self_ops/ops_py/approx_ops.py:556-571.
#include <type_traits>

#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"
#include "lutgemm_waits.cuh"

#ifndef LUTGEMM_TALL_HALFWARP_ROWS
#define LUTGEMM_TALL_HALFWARP_ROWS 1
#endif

namespace lutgemm {
namespace sgt {

enum { kGw = 1, kGa = 2, kGx = 3 };

template <int BITS, int RW_>
struct Cfg {
    static constexpr int Q = 1 << BITS;
    static constexpr bool F32_TABLE = BITS <= 7;
    static constexpr int HALF = Q / 2;
    static constexpr int TT_STRIDE = F32_TABLE ? Q + 1 : HALF + 1;  // words per table row
    static constexpr int WARPS = 16, THREADS = 512, RW = RW_, RT = WARPS * RW, CT = 32;
    static constexpr int KC = 16;                       // k per global fetch (16 codes per row in registers)
    static constexpr int SC = BITS == 8 ? 8 : 16;       // k per shared-memory stage
    static constexpr int U_STRIDE = 34;  // words per slab row: 32 floats + 2 (8-byte aligned rows, conflict-free stores)
    static constexpr int P_STRIDE = 33;
    static constexpr int NSEG = RT / 16;                // 16-row code segments per k
    static constexpr int RC_LOADS = (KC * NSEG + THREADS - 1) / THREADS;  // row-code vectors per thread and group
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = SC * RT, CC_STAGE = SC * CT;
    static constexpr int P_BYTES = WARPS * P_STRIDE * 4;
    static constexpr int OFF_U = TT_BYTES;
    static constexpr int OFF_RC = OFF_U + 2 * U_BYTES;
    static constexpr int OFF_CC = OFF_RC + 2 * RC_STAGE;
    static constexpr int OFF_PART = OFF_CC + 2 * CC_STAGE;
    static constexpr int OFF_BAR = (OFF_PART + 2 * P_BYTES + 15) & ~15;
    static constexpr int SMEM = OFF_BAR + 4 * 8 + 16;   // four mbarriers and the abort word
    static_assert(RW % 4 == 0 && RW <= 64, "rows per warp");
};

struct Args {
    const uint8_t *a;
    const uint8_t *w;
    const int16_t *lut;
    const float *lut_f32;      // optional (bits <= 7): the table as fp32 in the same padded layout, used instead of lut
    float factor;              // result scale: 1/16 for the 16x fixed-point int16 tables, 1 for fp32 tables
    const float *gc;
    float *out;
    int M, K, N;               // kGx: M = pixels of the class (all images), K = channels, N = Cout
    int RDIM, CDIM;
    int tiles_r, tiles_c;
    int ksplits, k_per_split;  // a tile's k range is cut into independent work items (outputs are per k)
    int direct;
    int vec_a, vec_w, vec_g;
    ConvGeom conv;
    int ga_scatter;     // grad_a of a convolution whose windows do not overlap: results go straight to the image
    const uint8_t *at;  // grad_w only, optional: transposed row codes at[k][m], rows at_pitch bytes apart
    int at_pitch;       // a multiple of 16; columns m >= M hold 0
    int *error_word;    // device error word of the bounded waits
    PixelClass px;      // kGx only
};

// USE_AT (grad_w only): the row codes come from the transposed copy p.at; the other instantiation keeps the
// direct / implicit-im2col fetch, so neither carries the other's registers.
// HANDOVER: per-buffer mbarriers (see the file comment) instead of one CTA barrier per k.
template <int BITS, int MODE, int RW, bool USE_AT, bool HANDOVER>
__global__ void __launch_bounds__(512, 1) slab_grad_tall_kernel(const Args p) {
    using C = Cfg<BITS, RW>;
    constexpr int WARPS = C::WARPS;
    constexpr int Q = C::Q, HALF = C::HALF, TTS = C::TT_STRIDE, RT = C::RT, CT = C::CT, KC = C::KC, SC = C::SC;
    constexpr int US = C::U_STRIDE, PS = C::P_STRIDE, THREADS = C::THREADS, NSEG = C::NSEG, RCL = C::RC_LOADS;
    constexpr int HALVES = KC / SC;  // shared-memory stages per fetched group of 16 k
    // slab reads in flight ahead of their use (per row, or per pair of columns with HW): 4 at 8 bits (2 and 3 are 1 - 2 %
    // slower, 8 is 3 % slower), 2 at 7 bits and below (4 is 1 % slower)
    constexpr int PF = BITS == 8 ? 4 : 2;
    // HW: half a warp per slab row and two columns per lane (64-bit slab reads) instead of a warp per row and one
    // column per lane: lanes 0-15 take the first RW/2 rows of the warp, lanes 16-31 the others
    constexpr bool HW = LUTGEMM_TALL_HALFWARP_ROWS && MODE != kGx && RW == 64 && HANDOVER;
    constexpr uint32_t MASK4 = (Q - 1) * 0x01010101u;
    constexpr int COL = lut_col_num(BITS);
    static_assert(MODE != kGw || USE_AT || RT % THREADS == 0, "grad_w without a transposed copy: whole rows per thread");

    const int M = p.M, K = p.K, N = p.N;
    const int RDIM = p.RDIM, CDIM = p.CDIM;

    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *rc_s = smem + C::OFF_RC;
    uint8_t *cc_s = smem + C::OFF_CC;
    float *part_s = reinterpret_cast<float *>(smem + C::OFF_PART);
    const uint32_t tt_addr = smem_u32(smem);
    const uint32_t u_addr = smem_u32(smem + C::OFF_U);
    const uint32_t bar_full = smem_u32(smem + C::OFF_BAR), bar_empty = bar_full + 16;
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem + C::OFF_BAR + 32);
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;

    // ---- stage the gradient table; x = row code, y = column code, T(x,y) = lut[a*COL + w] ----------------
    // (grad_w: rows are activation codes; grad_a / grad_x: rows are weight codes)
#pragma unroll 8
    for (int idx = tid; idx < Q * Q; idx += THREADS) {
        const int hi_idx = idx >> BITS, lo_idx = idx & (Q - 1);  // global read contiguous in lo_idx
        const int x = MODE == kGw ? hi_idx : lo_idx, y = MODE == kGw ? lo_idx : hi_idx;
        if (C::F32_TABLE) {
            reinterpret_cast<float *>(smem)[y * TTS + x] =
                p.lut_f32 ? p.lut_f32[hi_idx * COL + lo_idx] : (float)p.lut[hi_idx * COL + lo_idx];
        } else {
            const int16_t v = p.lut[hi_idx * COL + lo_idx];
            // int16 pairs {T(i,y), T(i+HALF,y)} in offset-binary (v + 32768) for the magic-number conversion
            reinterpret_cast<uint16_t *>(smem)[(y * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] =
                (uint16_t)v ^ (uint16_t)0x8000u;
        }
    }
    if (tid == 0) *abort_word = 0;

    // ---- operand staging.  A group of 16 k is fetched into registers (row-code vectors and one column-
    //      code vector per thread) and written to shared memory SC k at a time:
    //      rc_s[stage][kk][r] (RT row codes per k), cc_s[stage][kk][c] (32 column codes per k) --------------
    uint4 prc[RCL], pcc = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int j = 0; j < RCL; ++j) prc[j] = make_uint4(0, 0, 0, 0);
    auto load16 = [&](const uint8_t *src, int valid) -> uint4 {  // up to 16 bytes, the rest 0
        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 16; ++q)
            if (q < valid) t[q >> 2] |= (uint32_t)src[q] << (8 * (q & 3));
        return make_uint4(t[0], t[1], t[2], t[3]);
    };
    auto a_codes16 = [&](int m, int kbase) -> uint4 {  // a[m][kbase..kbase+15]
        m = min(m, M - 1);
        if (kbase >= K) return make_uint4(0, 0, 0, 0);
        if (p.conv.enabled) return conv_code16(p.a, p.conv, m, kbase, K);
        const uint8_t *src = p.a + (size_t)m * K + kbase;
        if (p.vec_a) return *reinterpret_cast<const uint4 *>(src);
        return load16(src, min(16, K - kbase));
    };
    auto w_codes16 = [&](int k, int n) -> uint4 {  // w[k][n..n+15]
        if (k >= K || n >= N) return make_uint4(0, 0, 0, 0);
        const uint8_t *src = p.w + (size_t)k * N + n;
        if (p.vec_w) return *reinterpret_cast<const uint4 *>(src);
        return load16(src, min(16, N - n));
    };
    // grad_x: row codes of channel k, rows r..r+15 with r = tap*N + n -> weight rows (k*T + t[tap])
    auto gx_row_codes16 = [&](int k, int r) -> uint4 {
        if (k >= K || r >= RDIM) return make_uint4(0, 0, 0, 0);
        int q = r / N, n = r - q * N;
        if (p.vec_w)  // N % 16 == 0: the 16 rows lie inside one tap
            return *reinterpret_cast<const uint4 *>(p.w + ((size_t)k * p.px.T + p.px.t[q]) * N + n);
        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (r + i < RDIM) t[i >> 2] |= (uint32_t)p.w[((size_t)k * p.px.T + p.px.t[q]) * N + n] << (8 * (i & 3));
            if (++n == N) { n = 0; ++q; }
        }
        return make_uint4(t[0], t[1], t[2], t[3]);
    };
    // grad_x: the code of pixel column `col` in channels kbase..kbase+15
    auto gx_col_codes16 = [&](int col, int kbase) -> uint4 {
        if (col >= CDIM || kbase >= K) return make_uint4(0, 0, 0, 0);
        const size_t plane = (size_t)p.px.H * p.px.W;
        const uint8_t *src = p.a + pixel_class_offset(p.px, col) + (size_t)kbase * plane;
        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 16; ++q)
            if (kbase + q < K) t[q >> 2] |= (uint32_t)src[q * plane] << (8 * (q & 3));
        return make_uint4(t[0], t[1], t[2], t[3]);
    };
    auto fetch_group = [&](int r0, int c0, int group) {
        const int kbase = group * KC;
        if (MODE == kGw && USE_AT) {
            // row codes from the transposed copy at[k][m]: 16 rows per load, coalesced like the w operand
#pragma unroll
            for (int j = 0; j < RCL; ++j) {
                const int idx = tid + THREADS * j;  // (k, 16-row segment)
                const int gk = kbase + idx / NSEG, gm = r0 + (idx % NSEG) * 16;
                prc[j] = (idx < KC * NSEG && gk < K && gm < p.at_pitch)
                             ? *reinterpret_cast<const uint4 *>(p.at + (size_t)gk * p.at_pitch + gm)
                             : make_uint4(0, 0, 0, 0);
            }
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else if (MODE == kGw) {
#pragma unroll
            for (int j = 0; j < RCL; ++j) prc[j] = a_codes16(r0 + tid + THREADS * j, kbase);
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else {
#pragma unroll
            for (int j = 0; j < RCL; ++j) {
                const int idx = tid + THREADS * j;  // (k, 16-row segment)
                const int gk = kbase + idx / NSEG, gr = r0 + (idx % NSEG) * 16;
                if (idx >= KC * NSEG) prc[j] = make_uint4(0, 0, 0, 0);
                else prc[j] = MODE == kGx ? gx_row_codes16(gk, gr) : w_codes16(gk, gr);
            }
            if (tid < CT) pcc = MODE == kGx ? gx_col_codes16(c0 + tid, kbase) : a_codes16(c0 + tid, kbase);
        }
    };
    // writes the k range [half*SC, half*SC + SC) of the fetched group to `stage`
    auto store_stage = [&](int stage, int half) {
        uint8_t *rs = rc_s + stage * C::RC_STAGE;
        uint8_t *cs = cc_s + stage * C::CC_STAGE;
        const uint32_t tc[4] = {pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4};
        if (MODE == kGw && !USE_AT) {
#pragma unroll
            for (int j = 0; j < RCL; ++j) {
                const uint32_t tr[4] = {prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4};
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (q / SC == half || HALVES == 1)
                        rs[(q % SC) * RT + tid + THREADS * j] = (uint8_t)(tr[q >> 2] >> (8 * (q & 3)));
            }
        } else {
#pragma unroll
            for (int j = 0; j < RCL; ++j) {
                const int idx = tid + THREADS * j, kq = idx / NSEG;
                if (idx < KC * NSEG && (kq / SC == half || HALVES == 1))
                    *reinterpret_cast<uint4 *>(rs + (kq % SC) * RT + (idx % NSEG) * 16) =
                        make_uint4(prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4);
            }
        }
        if (MODE == kGw) {
            if (tid < KC * CT / 16) {
                const int kq = tid / (CT / 16);
                if (kq / SC == half || HALVES == 1)
                    *reinterpret_cast<uint4 *>(cs + (kq % SC) * CT + (tid % (CT / 16)) * 16) =
                        make_uint4(tc[0], tc[1], tc[2], tc[3]);
            }
        } else if (tid < CT) {
#pragma unroll
            for (int q = 0; q < 16; ++q)
                if (q / SC == half || HALVES == 1) cs[(q % SC) * CT + tid] = (uint8_t)(tc[q >> 2] >> (8 * (q & 3)));
        }
    };
    // build slab `buf` for the k at (stage, kk): warp wp fills the 64-bit column pair (2wp, 2wp+1).
    // Lanes run over x, so the table reads are contiguous and the 64-bit slab stores (row stride 34 words)
    // fall on distinct bank pairs within each half-warp.
    auto build = [&](int buf, int stage, int kk) {
        const uint32_t cw = *reinterpret_cast<const uint16_t *>(cc_s + stage * C::CC_STAGE + kk * CT + wp * 2);
        const uint32_t y0 = cw & 0xffu, y1 = cw >> 8;
        const uint32_t ub = u_addr + buf * C::U_BYTES + wp * 8;
        // The table reads of the warp's share are issued before its first store where that measured faster (the
        // stores order later reads behind them): always with the fp32 table (7 bits: grad_w 13.70 -> 13.28 ms,
        // grad_a 13.87 -> 13.48 ms at 4096^3), at 8 bits for grad_w only (14.00 -> 13.77 ms; grad_a 14.06 -> 14.50 ms).
        constexpr bool READS_FIRST = C::F32_TABLE || MODE == kGw;
        constexpr int NJ = C::F32_TABLE ? (Q + 31) / 32 : HALF / 32;
        uint32_t r0[NJ], r1[NJ];
        auto read = [&](int j) {
            const int x = lane + 32 * j;  // fp32 table: code x; int16 table: the pair of codes (x, x + HALF)
            if (Q >= 32 || x < Q) {
                r0[j] = lds_u32(tt_addr + (y0 * TTS + x) * 4);
                r1[j] = lds_u32(tt_addr + (y1 * TTS + x) * 4);
            }
        };
        auto store = [&](int j) {
            const int x = lane + 32 * j;
            if constexpr (C::F32_TABLE) {
                if (Q >= 32 || x < Q)
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ub + x * (US * 4)), "r"(r0[j]), "r"(r1[j]) : "memory");
            } else {
                // 0x4B000000 | u is the float 2^23 + u; minus (2^23 + 32768) leaves the signed entry exactly
                const float f00 = __uint_as_float((r0[j] & 0xffffu) | 0x4B000000u) - 8421376.0f;
                const float f01 = __uint_as_float((r1[j] & 0xffffu) | 0x4B000000u) - 8421376.0f;
                const float f10 = __uint_as_float(__byte_perm(r0[j], 0x4B000000u, 0x7632)) - 8421376.0f;
                const float f11 = __uint_as_float(__byte_perm(r1[j], 0x4B000000u, 0x7632)) - 8421376.0f;
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + x * (US * 4)), "f"(f00), "f"(f01) : "memory");
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + (x + HALF) * (US * 4)), "f"(f10), "f"(f11)
                             : "memory");
            }
        };
        if constexpr (READS_FIRST) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) read(j);
#pragma unroll
            for (int j = 0; j < NJ; ++j) store(j);
        } else {
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                read(j);
                store(j);
            }
        }
    };
    // add the 16 warps' partial sums of one k in ascending warp order and store the tile's 32 columns
    auto reduce_store = [&](int k, float *obase, int c0) {
        const float *ps = part_s + (k & 1) * (WARPS * PS) + lane;
        float v = ps[0];
#pragma unroll
        for (int wv = 1; wv < WARPS; ++wv) v += ps[wv * PS];
        const int col = c0 + lane;
        if (col < CDIM) {
            if (p.direct && MODE == kGx) {
                obase[pixel_class_offset(p.px, col) + (size_t)k * p.px.H * p.px.W] = v * p.factor;
            } else if (p.direct && MODE == kGa) {
                if (p.ga_scatter) {
                    const long o = conv_scatter_index(p.conv, col, k);
                    if (o >= 0) obase[o] = v * p.factor;
                } else {
                    obase[(size_t)col * K + k] = v * p.factor;
                }
            } else {
                obase[(size_t)k * CDIM + col] = p.direct ? v * p.factor : v;
            }
        }
    };

    const int items = p.tiles_r * p.tiles_c * p.ksplits;
    bool first_item = true;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int tile = item / p.ksplits;
        const int kbeg = (item % p.ksplits) * p.k_per_split, kend = min(K, kbeg + p.k_per_split);
        const int tr = tile / p.tiles_c, tc = tile % p.tiles_c;
        const int r0 = tr * RT, c0 = tc * CT;

        // the grad_out block of this tile: g[r] for the warp's RW rows and the lane's column
        float g[RW];
        if constexpr (HW) {
            // g[2i + j] = grad_out at (row h * RW/2 + i of the warp, column 2 * cp + j of the tile)
            const int h = lane >> 4, cp = lane & 15;
            if (MODE == kGw) {
                const int n = c0 + 2 * cp;
#pragma unroll
                for (int i = 0; i < RW / 2; ++i) {
                    const int m = r0 + wp * RW + h * (RW / 2) + i;
                    if (m < M && n + 1 < N && p.vec_g) {
                        const float2 t = *reinterpret_cast<const float2 *>(p.gc + (size_t)m * N + n);
                        g[2 * i] = t.x; g[2 * i + 1] = t.y;
                    } else {
                        g[2 * i] = (m < M && n < N) ? p.gc[(size_t)m * N + n] : 0.f;
                        g[2 * i + 1] = (m < M && n + 1 < N) ? p.gc[(size_t)m * N + n + 1] : 0.f;
                    }
                }
            } else {
                const int nb = r0 + wp * RW + h * (RW / 2);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int m = c0 + 2 * cp + j;
                    const float *src = p.gc + (size_t)min(m, M - 1) * N + min(nb, N - 1);
                    if (m < M && p.vec_g && nb + RW / 2 <= N) {
#pragma unroll
                        for (int i = 0; i < RW / 2; i += 4) {
                            const float4 t = *reinterpret_cast<const float4 *>(src + i);
                            g[2 * i + j] = t.x; g[2 * (i + 1) + j] = t.y; g[2 * (i + 2) + j] = t.z; g[2 * (i + 3) + j] = t.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < RW / 2; ++i)
                            g[2 * i + j] = (m < M && nb + i < N) ? p.gc[(size_t)m * N + nb + i] : 0.f;
                    }
                }
            }
        } else if (MODE == kGw) {
            const int n = c0 + lane;
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int m = r0 + wp * RW + r;
                g[r] = (m < M && n < N) ? p.gc[(size_t)m * N + n] : 0.f;
            }
        } else if (MODE == kGa) {
            // g[r] = gc[m = c0 + lane][n = r0 + RW*wp + r]
            const int m = c0 + lane;
            const int nb = r0 + wp * RW;
            const float *src = p.gc + (size_t)min(m, M - 1) * N + nb;
            if (m < M && p.vec_g && nb + RW <= N) {
#pragma unroll
                for (int r = 0; r < RW; r += 4) {
                    const float4 t = *reinterpret_cast<const float4 *>(src + r);
                    g[r] = t.x; g[r + 1] = t.y; g[r + 2] = t.z; g[r + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < RW; ++r) g[r] = (m < M && nb + r < N) ? src[r] : 0.f;
            }
        } else {
            // g[r] = gy[m(pixel, tap), n] for row (tap, n) = r0 + RW*wp + r; 0 where the tap leaves the output
            const int col = c0 + lane;
            int h = 0, w = 0, b = 0;
            if (col < CDIM) {
                const int per = p.px.Hc * p.px.Wc;
                b = col / per;
                const int rr = col - b * per, hh = rr / p.px.Wc;
                h = p.px.ph + p.px.s * hh;
                w = p.px.pw + p.px.s * (rr - hh * p.px.Wc);
            }
            const int rb = r0 + wp * RW;
            auto row_src = [&](int r) -> const float * {  // &gy[m][n] of row r, or nullptr
                if (col >= CDIM || r >= RDIM) return nullptr;
                const int q = r / N, n = r - q * N;
                const int th = h - p.px.dh[q], tw = w - p.px.dw[q];
                if (th < 0 || tw < 0) return nullptr;
                const int oh = th / p.px.s, ow = tw / p.px.s;
                if (oh * p.px.s != th || ow * p.px.s != tw || oh >= p.px.Ho || ow >= p.px.Wo) return nullptr;
                return p.gc + ((size_t)(b * p.px.Ho + oh) * p.px.Wo + ow) * N + n;
            };
            if (p.vec_g) {  // N % 4 == 0: four consecutive rows share their tap
#pragma unroll
                for (int r = 0; r < RW; r += 4) {
                    const float *src = row_src(rb + r);
                    const float4 t = src ? *reinterpret_cast<const float4 *>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
                    g[r] = t.x; g[r + 1] = t.y; g[r + 2] = t.z; g[r + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const float *src = row_src(rb + r);
                    g[r] = src ? *src : 0.f;
                }
            }
        }

        // kbeg is a multiple of 16, so the first stage is half 0 of its group
        fetch_group(r0, c0, kbeg / KC);
        __syncthreads();  // previous item (or the table staging) is done with every buffer
        store_stage((kbeg / SC) & 1, 0);
        if (HANDOVER && tid == 0) {
            // fresh barriers for this item: phases restart at 0 (nobody is waiting or arriving here)
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                if (!first_item) asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar_full + 8 * b) : "memory");
                mbar_init(bar_full + 8 * b, WARPS);
            }
        }
        first_item = false;
        __syncthreads();
        build(kbeg & 1, (kbeg / SC) & 1, 0);
        if (HANDOVER) {
            __syncwarp();
            // slab kbeg is complete once every warp has arrived; the other buffer starts out released
            if (lane == 0) {
                mbar_arrive(bar_full + 8 * (kbeg & 1));
                mbar_arrive(bar_empty + 8 * ((kbeg & 1) ^ 1));
            }
        } else {
            __syncthreads();
        }

        float *obase = p.out + (p.direct ? (size_t)0 : (size_t)tr * K * CDIM);

        // use slab k: slab row rc[r,k], one fp32 column per lane, for rows [RB, RE) of this warp
        auto use_rows = [&](int k, int stage, int kk, float (&s)[4], auto rb_tag, auto re_tag) {
            constexpr int RB = decltype(rb_tag)::value, RE = decltype(re_tag)::value;
            const uint8_t *rbase = rc_s + stage * C::RC_STAGE + kk * RT + wp * RW;
            const uint32_t ub = u_addr + (k & 1) * C::U_BYTES + lane * 4;
            // slab row address = base + 136 * code in one integer dot-product instruction
            auto row_addr = [&](uint32_t v, int i) { return byte_scaled_add<US * 4>(v, i, ub); };
            constexpr int W0 = RB / 4, W1 = (RE + 3) / 4;  // code words (four rows each) this range touches
            uint32_t rv[W1 - W0];
            if constexpr (RW % 16 == 0 && RB % 16 == 0 && RE % 16 == 0) {
                const uint4 *rp = reinterpret_cast<const uint4 *>(rbase);
#pragma unroll
                for (int q = RB / 16; q < RE / 16; ++q) {
                    const uint4 t = rp[q];
                    rv[4 * q - W0] = t.x; rv[4 * q + 1 - W0] = t.y; rv[4 * q + 2 - W0] = t.z; rv[4 * q + 3 - W0] = t.w;
                }
            } else {
                const uint32_t *rp32 = reinterpret_cast<const uint32_t *>(rbase);
#pragma unroll
                for (int q = W0; q < W1; ++q) rv[q - W0] = rp32[q];
            }
            float pf[PF];
#pragma unroll
            for (int r = RB; r < RB + PF; ++r)
                asm volatile("ld.shared.f32 %0, [%1];" : "=f"(pf[(r - RB) % PF]) : "r"(row_addr(rv[(r >> 2) - W0], r & 3)));
#pragma unroll
            for (int r = RB; r < RE; ++r) {
                const float f = pf[(r - RB) % PF];
                if (r + PF < RE)
                    asm volatile("ld.shared.f32 %0, [%1];"
                                 : "=f"(pf[(r - RB) % PF]) : "r"(row_addr(rv[((r + PF) >> 2) - W0], (r + PF) & 3)));
                s[r & 3] = fmaf(f, g[r], s[r & 3]);
            }
        };
        // HW: rows [IB, IE) of this half-warp's RW/2 rows; s[0], s[2] belong to the lane's first column, s[1], s[3] to
        // its second
        auto use_rows_hw = [&](int k, int stage, int kk, float (&s)[4], auto ib_tag, auto ie_tag) {
            constexpr int IB = decltype(ib_tag)::value, IEND = decltype(ie_tag)::value;
            static_assert(IB % 16 == 0 && IEND % 16 == 0, "whole 16-row code vectors");
            const uint8_t *rbase = rc_s + stage * C::RC_STAGE + kk * RT + wp * RW + (lane >> 4) * (RW / 2);
            const uint32_t ub = u_addr + (k & 1) * C::U_BYTES + (lane & 15) * 8;
            uint32_t rv[(IEND - IB) / 4];
#pragma unroll
            for (int q = IB / 16; q < IEND / 16; ++q) {
                const uint4 t = reinterpret_cast<const uint4 *>(rbase)[q];
                rv[4 * q - IB / 4] = t.x; rv[4 * q + 1 - IB / 4] = t.y; rv[4 * q + 2 - IB / 4] = t.z; rv[4 * q + 3 - IB / 4] = t.w;
            }
            float pa[PF], pb[PF];
            auto fetch = [&](int i) {
                asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                             : "=f"(pa[(i - IB) % PF]), "=f"(pb[(i - IB) % PF])
                             : "r"(byte_scaled_add<US * 4>(rv[(i - IB) >> 2], i & 3, ub)));
            };
#pragma unroll
            for (int i = IB; i < IB + PF; ++i) fetch(i);
#pragma unroll
            for (int i = IB; i < IEND; ++i) {
                const float fa = pa[(i - IB) % PF], fb = pb[(i - IB) % PF];
                if (i + PF < IEND) fetch(i + PF);
                s[2 * (i & 1)] = fmaf(fa, g[2 * i], s[2 * (i & 1)]);
                s[2 * (i & 1) + 1] = fmaf(fb, g[2 * i + 1], s[2 * (i & 1) + 1]);
            }
        };
        using I0 = std::integral_constant<int, 0>;
        using IH = std::integral_constant<int, (RW / 2) & ~3>;
        using IE = std::integral_constant<int, RW>;
        using IQ = std::integral_constant<int, ((RW / 4) + 15) & ~15>;  // HW: half of a half-warp's rows

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / SC, kk = k % SC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * SC < kend;
            // the registers are free for the next group once the last stage of the current one is written
            if (kk == 0 && have_next_chunk && (chunk + 1) % HALVES == 0) fetch_group(r0, c0, (chunk + 1) / HALVES);
            float s[4] = {0.f, 0.f, 0.f, 0.f};
            if (HANDOVER) {
                // phase of either barrier that belongs to this step: its (kl / 2)-th since the item began
                const int b = k & 1;
                const uint32_t par = ((k - kbeg) >> 1) & 1;
                mbar_wait(bar_full + 8 * b, par, 1 + b, abort_word, p.error_word);         // slab k is complete
                if constexpr (HW) use_rows_hw(k, stage, kk, s, I0{}, IQ{});
                else use_rows(k, stage, kk, s, I0{}, IH{});
                mbar_wait(bar_empty + 8 * (b ^ 1), par, 3 + b, abort_word, p.error_word);  // slab k-1 is released
                if (k > kbeg && wp == ((k - 1) & (WARPS - 1))) reduce_store(k - 1, obase, c0);
                if (k + 1 < kend) {
                    build((k + 1) & 1, ((k + 1) / SC) & 1, (k + 1) % SC);
                    if (kk == SC - 2 && have_next_chunk) store_stage(stage ^ 1, (chunk + 1) % HALVES);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * (b ^ 1));
                }
                if constexpr (HW) {
                    use_rows_hw(k, stage, kk, s, IQ{}, IH{});
                    // the two halves of the warp hold the same two columns for different rows
                    float ca = s[0] + s[2], cb = s[1] + s[3];
                    ca += __shfl_xor_sync(0xffffffffu, ca, 16);
                    cb += __shfl_xor_sync(0xffffffffu, cb, 16);
                    if (lane < 16) {
                        float *pp = part_s + (k & 1) * (WARPS * PS) + wp * PS + 2 * lane;
                        pp[0] = ca;
                        pp[1] = cb;
                    }
                } else {
                    use_rows(k, stage, kk, s, IH{}, IE{});
                    part_s[(k & 1) * (WARPS * PS) + wp * PS + lane] = (s[0] + s[1]) + (s[2] + s[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_empty + 8 * b);
            } else {
                // Half of the warps (alternating groups of four, so that every scheduler has both kinds) run the
                // side work - building slab k+1 and adding up the partial sums of k-1 - before their gathers,
                // the other half after them, so that its dependent shared-memory chains overlap gather streams.
                const bool side_first = (wp >> 2) & 1;
                auto side_work = [&]() {
                    if (k + 1 < kend) build((k + 1) & 1, ((k + 1) / SC) & 1, (k + 1) % SC);
                    if (k > kbeg && wp == ((k - 1) & (WARPS - 1))) reduce_store(k - 1, obase, c0);
                };
                if (side_first) { side_work(); use_rows(k, stage, kk, s, I0{}, IE{}); }
                else { use_rows(k, stage, kk, s, I0{}, IE{}); side_work(); }
                part_s[(k & 1) * (WARPS * PS) + wp * PS + lane] = (s[0] + s[1]) + (s[2] + s[3]);
                if (kk == SC - 2 && have_next_chunk) store_stage(stage ^ 1, (chunk + 1) % HALVES);
                __syncthreads();
            }
        }
        if (HANDOVER) __syncthreads();  // every warp has stored its partial sums of the last k
        if (wp == ((kend - 1) & (WARPS - 1))) reduce_store(kend - 1, obase, c0);
    }
}

}  // namespace sgt

int slab_tall_row_blocks(int rdim) { return (rdim + kSlabTallRows - 1) / kSlabTallRows; }

namespace {

bool g_tall_handover = true;  // per-buffer mbarrier hand-over (false: one CTA barrier per k)


template <int BITS, int MODE, int RW>
int launch_slab_grad_tall(sgt::Args p, float *out, float *scratch, int num_sms, cudaStream_t stream) {
    using C = sgt::Cfg<BITS, RW>;
    static_assert(C::SMEM <= 232448, "shared memory budget");
    const bool use_at = MODE == sgt::kGw && p.at != nullptr;
    const bool ho = g_tall_handover;
    auto kern = use_at ? (ho ? sgt::slab_grad_tall_kernel<BITS, MODE, RW, MODE == sgt::kGw, true>
                             : sgt::slab_grad_tall_kernel<BITS, MODE, RW, MODE == sgt::kGw, false>)
                       : (ho ? sgt::slab_grad_tall_kernel<BITS, MODE, RW, false, true>
                             : sgt::slab_grad_tall_kernel<BITS, MODE, RW, false, false>);
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM)))
        return LUTGEMM_E_CUDA;
    p.error_word = device_error_word();
    if (!p.error_word) return LUTGEMM_E_CUDA;
    p.tiles_r = (p.RDIM + C::RT - 1) / C::RT;
    p.tiles_c = (p.CDIM + C::CT - 1) / C::CT;
    p.direct = p.tiles_r == 1;
    p.out = p.direct ? out : scratch;
    // cut K so that the persistent grid's last wave is as full as possible (k ranges are multiples of 16)
    const long tiles = (long)p.tiles_r * p.tiles_c;
    const int kchunks = (p.K + C::KC - 1) / C::KC;
    int ksplits = 1;
    double best = -1.0;
    for (int sp = 1; sp <= 16 && sp <= kchunks; ++sp) {
        const int per = ((kchunks + sp - 1) / sp) * C::KC;
        if ((p.K + per - 1) / per != sp) continue;
        const long it = tiles * sp;
        const long waves = (it + num_sms - 1) / num_sms;
        const double eff = (double)it / (double)(waves * num_sms) * (double)per / (double)(per + 8);
        if (eff > best + 1e-9) { best = eff; ksplits = sp; }
    }
    p.ksplits = ksplits;
    p.k_per_split = ((kchunks + ksplits - 1) / ksplits) * C::KC;
    const long items = tiles * ksplits;
    const int grid = (int)(items < num_sms ? items : num_sms);
    kern<<<grid, C::THREADS, C::SMEM, stream>>>(p);
    return launch_status();
}

template <int BITS, int MODE>
int launch_gemm_grad_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                          const float *lut_f32, int M, int K, int N, const ConvGeom &conv, float *scratch,
                          const uint8_t *at, int at_pitch, int num_sms, cudaStream_t stream) {
    static_assert(sgt::Cfg<BITS, 64>::RT == kSlabTallRows, "tile height");
    if (lut_f32 && !sgt::Cfg<BITS, 64>::F32_TABLE) return LUTGEMM_E_BITS;
    sgt::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = gc; p.M = M; p.K = K; p.N = N;
    p.lut_f32 = lut_f32;
    p.factor = lut_f32 ? 1.0f : kGradFactor;
    p.RDIM = MODE == sgt::kGa ? N : M;
    p.CDIM = MODE == sgt::kGa ? M : N;
    p.conv = conv;
    p.at = MODE == sgt::kGw ? at : nullptr;
    p.at_pitch = at_pitch;
    p.ga_scatter = (MODE == sgt::kGa && conv.enabled) ? 1 : 0;
    p.vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    const int rc = launch_slab_grad_tall<BITS, MODE, 64>(p, out, scratch, num_sms, stream);
    if (rc != LUTGEMM_OK) return rc;
    const int tiles_r = (p.RDIM + kSlabTallRows - 1) / kSlabTallRows;
    if (tiles_r > 1)
        return slab_reduce_blocks(scratch, out, K, p.CDIM, tiles_r, MODE == sgt::kGa, p.ga_scatter ? &conv : nullptr,
                                  nullptr, p.factor, num_sms, stream);
    return LUTGEMM_OK;
}

// cost of one (k, column tile) step in shared-memory wavefronts: rows read plus the slab build
long gx_step_cost(int bits, long rdim, int rw) {
    const long rt = 16L * rw, q = 1L << bits;
    return ((rdim + rt - 1) / rt) * (rt + (bits == 8 ? 3 * q / 2 : 2 * q));
}

template <int BITS>
int launch_gx_class(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut, int Cout,
                    const PixelClass &px, int B, float *scratch, int num_sms, cudaStream_t stream) {
    sgt::Args p{};
    p.a = x; p.w = wmat; p.lut = lut; p.gc = gy;
    p.factor = kGradFactor;
    p.M = B * px.Hc * px.Wc; p.K = px.C; p.N = Cout;
    p.RDIM = px.ntaps * Cout;
    p.CDIM = p.M;
    p.px = px;
    p.vec_w = (Cout % 16 == 0) && ((reinterpret_cast<uintptr_t>(wmat) & 15) == 0);
    p.vec_g = (Cout % 4 == 0) && ((reinterpret_cast<uintptr_t>(gy) & 15) == 0);
    int rw = 64;
    for (int cand : {36, 32})
        if (gx_step_cost(BITS, p.RDIM, cand) < gx_step_cost(BITS, p.RDIM, rw)) rw = cand;
    int rc;
    if (rw == 36) rc = launch_slab_grad_tall<BITS, sgt::kGx, 36>(p, gx, scratch, num_sms, stream);
    else if (rw == 32) rc = launch_slab_grad_tall<BITS, sgt::kGx, 32>(p, gx, scratch, num_sms, stream);
    else rc = launch_slab_grad_tall<BITS, sgt::kGx, 64>(p, gx, scratch, num_sms, stream);
    if (rc != LUTGEMM_OK) return rc;
    const int tiles_r = (p.RDIM + 16 * rw - 1) / (16 * rw);
    if (tiles_r > 1)
        return slab_reduce_blocks(scratch, gx, p.K, p.CDIM, tiles_r, false, nullptr, &px, kGradFactor, num_sms, stream);
    return LUTGEMM_OK;
}

}  // namespace

void slab_tall_set_handover(bool on) { g_tall_handover = on; }

int backward_gw_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                          const float *lut_f32, int bits, int M, int K, int N, const ConvGeom &conv, float *scratch,
                          const uint8_t *at, int at_pitch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_gemm_grad_tall<4, sgt::kGw>(gc, a, w, gw, lut_gw, lut_f32, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 6: return launch_gemm_grad_tall<6, sgt::kGw>(gc, a, w, gw, lut_gw, lut_f32, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 7: return launch_gemm_grad_tall<7, sgt::kGw>(gc, a, w, gw, lut_gw, lut_f32, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 8: return launch_gemm_grad_tall<8, sgt::kGw>(gc, a, w, gw, lut_gw, lut_f32, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int backward_ga_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                          const float *lut_f32, int bits, int M, int K, int N, const ConvGeom &conv, float *scratch,
                          int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_gemm_grad_tall<4, sgt::kGa>(gc, a, w, ga, lut_ga, lut_f32, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 6: return launch_gemm_grad_tall<6, sgt::kGa>(gc, a, w, ga, lut_ga, lut_f32, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 7: return launch_gemm_grad_tall<7, sgt::kGa>(gc, a, w, ga, lut_ga, lut_f32, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 8: return launch_gemm_grad_tall<8, sgt::kGa>(gc, a, w, ga, lut_ga, lut_f32, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

size_t gx_class_scratch_bytes(int bits, int Cout, const PixelClass &px, int B) {
    const long rdim = (long)px.ntaps * Cout;
    int rw = 64;
    for (int cand : {36, 32})
        if (gx_step_cost(bits, rdim, cand) < gx_step_cost(bits, rdim, rw)) rw = cand;
    const long tiles_r = (rdim + 16L * rw - 1) / (16L * rw);
    return tiles_r > 1 ? (size_t)tiles_r * px.C * ((size_t)B * px.Hc * px.Wc) * sizeof(float) : 0;
}

int backward_gx_class(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut_ga, int bits,
                      int Cout, const PixelClass &px, int B, float *scratch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_gx_class<4>(gy, x, wmat, gx, lut_ga, Cout, px, B, scratch, num_sms, stream);
        case 6: return launch_gx_class<6>(gy, x, wmat, gx, lut_ga, Cout, px, B, scratch, num_sms, stream);
        case 7: return launch_gx_class<7>(gy, x, wmat, gx, lut_ga, Cout, px, B, scratch, num_sms, stream);
        case 8: return launch_gx_class<8>(gy, x, wmat, gx, lut_ga, Cout, px, B, scratch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
