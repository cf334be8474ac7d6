// Backward LUT-GEMM for sm_100a (gradient-table gathers fused with the grad_out multiply, fp32).
//
//   gA[m,k] = 1/16 * sum_n gC[m,n] * float(LUTa[a[m,k]][w[k,n]])      (ga_colbcast_kernel)
//   gW[k,n] = 1/16 * sum_m float(LUTw[a[m,k]][w[k,n]]) * gC[m,n]      (gw_rowbcast_kernel)
//
// Both kernels keep the whole int16 gradient table in shared memory and make ONE of the two table
// indices warp-uniform so a gather stays inside a single table row:
//   gA: a thread owns gA[m, k..k+R) for C rows m; a[m,k] is fixed per thread, the weight code
//       w[k,n] is the same for all lanes (they share the k set), and the table is staged TRANSPOSED
//       ([w][a]) so the uniform index selects the row.  n ascends exactly as in the reference, so
//       the fp32 sum order per element is the reference's.
//   gW: a thread owns gW[k..k+R, n..n+C); w[k,n] is fixed per thread, the activation code a[m,k] is
//       warp-uniform, table staged as [a][w].  The reduction over M (262144 rows for the CIFAR
//       convolutions, against a 576x64 output) is split into slabs across CTAs; partial sums go to a
//       scratch buffer and a second kernel adds the slabs in ascending order (deterministic).
// grad_x (PIX instantiation of the gA kernel): the activation gradient of a convolution per INPUT PIXEL.  A thread
// owns C pixels of one stride class and R input channels; the "n" loop runs over (tap, n): for tap (i,j) the
// grad_out rows are those of the output positions the tap connects the pixels to (zero rows where it leaves the
// output), the weight rows are (channel, tap).  The activation code of a pixel is the same for every tap, so
// the accumulators collect the whole sum over taps and output channels and are stored straight into
// gx[B,C,H,W]: no unfolded gradient, no col2im.
// Replaces ApproxGemmBackwardKernelForGA / ForGB, self_ops/src/approx_gemm_backward.cu:13-258,261-492, and for
// grad_x the unfold backward of self_ops/ops_py/approx_ops.py:556-571.
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

// ------------------------------------------------------------------------------------------------
// gA
// ------------------------------------------------------------------------------------------------
template <int BITS, int R, int C, int WM, int WK>
struct GaCfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int THREADS = 32 * WM * WK;
    static constexpr int MT = WM * 32 * C;
    static constexpr int KT = WK * R;
    static constexpr int NT = 16;
    static constexpr int GSTRIDE = NT * 4 + 16;  // bytes; odd multiple of 16 -> conflict-free 128-bit row reads
    static constexpr int LUT_BYTES = Q * Q * 2;
    static constexpr int G_STAGE = MT * GSTRIDE;
    static constexpr int W_STAGE = KT * NT;
    static constexpr int OFF_ROWINFO = LUT_BYTES + 2 * (G_STAGE + W_STAGE);
    static constexpr int SMEM = OFF_ROWINFO;
    static constexpr int SMEM_PIX = OFF_ROWINFO + MT * 16;  // grad_x: {first output row, hh, ww} per pixel of the tile
};

// PIX: grad_x per input pixel of the stride classes in `set` (tiles_m counts the pixel tiles of all of them, K =
// channels, a = the code image, w = the weight matrix [C*T, N], gc = grad_out [B*Ho*Wo, N], ga = gx[B,C,H,W]).
template <int BITS, int R, int C, int WM, int WK, bool PIX>
__global__ void __launch_bounds__(32 * WM * WK, WM * WK <= 8 ? (C <= 2 ? 4 : 2) : 1)
ga_colbcast_kernel(const float *__restrict__ gc, const uint8_t *__restrict__ a, const uint8_t *__restrict__ w,
                   float *__restrict__ ga, const int16_t *__restrict__ lut, int M, int K, int N, int tiles_m,
                   int tiles_k, int vec_g, int vec_w, int vec_o, const ConvGeom conv,
                   const __grid_constant__ PixelClassSet set) {
    using Cfg = GaCfg<BITS, R, C, WM, WK>;
    constexpr int MT = Cfg::MT, KT = Cfg::KT, NT = Cfg::NT, GS = Cfg::GSTRIDE, THREADS = Cfg::THREADS;
    constexpr uint32_t MASK = Cfg::Q - 1, MASK4 = MASK * 0x01010101u;
    static_assert(R % 4 == 0 && R <= 16, "R k-columns per thread");

    extern __shared__ __align__(16) uint8_t smem[];
    int16_t *lut_s = reinterpret_cast<int16_t *>(smem);
    uint8_t *g_s = smem + Cfg::LUT_BYTES;
    uint8_t *w_s = g_s + 2 * Cfg::G_STAGE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WK, wk = warp % WK;

    stage_table<BITS, true>(lut_s, lut, tid, THREADS);
    const uint32_t lut_addr = smem_u32(lut_s);
    const int nnt = (N + NT - 1) / NT;
    int4 *rowinfo = reinterpret_cast<int4 *>(smem + Cfg::OFF_ROWINFO);  // PIX only
    const PixelClass *pxp = &set.c[0];                                     // PIX only: the class of the current tile

    // PIX: step = (tap q, n tile): grad_out rows of the output positions tap q connects the tile's pixels to
    auto load_tile_pix = [&](int m0, int k0, int step, int buf) {
        const PixelClass &px = *pxp;
        uint8_t *gs = g_s + buf * Cfg::G_STAGE;
        uint8_t *ws = w_s + buf * Cfg::W_STAGE;
        const int q = step / nnt, nbase = (step - q * nnt) * NT;
        // pixel (hh, ww) of the class sits at h = ph + s*hh; tap q reaches output row (h - dh)/s = hh + eh
        const int eh = (px.ph - px.dh[q]) / px.s, ew = (px.pw - px.dw[q]) / px.s;
        const int moff = eh * px.Wo + ew;
        for (int id = tid; id < MT * (NT / 4); id += THREADS) {
            const int r = id / (NT / 4), nc = (id % (NT / 4)) * 4;
            const int4 info = rowinfo[r];  // {m of tap offset 0, hh, ww, valid}
            const int oh = info.y + eh, ow = info.z + ew, gn = nbase + nc;
            float *dst = reinterpret_cast<float *>(gs + r * GS + nc * 4);
            const bool ok = info.w && (unsigned)oh < (unsigned)px.Ho && (unsigned)ow < (unsigned)px.Wo && gn < N;
            const float *src = gc + (size_t)(info.x + moff) * N + gn;
            if (ok && vec_g) cp_async16(dst, src);
            else if (ok) {
#pragma unroll
                for (int e = 0; e < 4; ++e) dst[e] = gn + e < N ? src[e] : 0.f;
            } else *reinterpret_cast<float4 *>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const int t = px.t[q];
        if (vec_w) {
            for (int id = tid; id < KT; id += THREADS) {
                const int gk = k0 + id;
                if (gk < K && nbase < N) cp_async16(ws + id * NT, w + ((size_t)gk * px.T + t) * N + nbase);
                else *reinterpret_cast<uint4 *>(ws + id * NT) = make_uint4(0, 0, 0, 0);
            }
        } else {
            for (int id = tid; id < KT * NT; id += THREADS) {
                const int kk = id / NT, nn = id % NT;
                const int gk = k0 + kk, gn = nbase + nn;
                ws[id] = (gk < K && gn < N) ? w[((size_t)gk * px.T + t) * N + gn] : (uint8_t)0;
            }
        }
        cp_async_commit();
    };

    auto load_tile = [&](int m0, int k0, int nt, int buf) {
        if (PIX) { load_tile_pix(m0, k0, nt, buf); return; }
        uint8_t *gs = g_s + buf * Cfg::G_STAGE;
        uint8_t *ws = w_s + buf * Cfg::W_STAGE;
        const int nbase = nt * NT;
        if (vec_g) {
            for (int id = tid; id < MT * (NT / 4); id += THREADS) {
                int r = id / (NT / 4), nc = (id % (NT / 4)) * 4;
                int gm = m0 + r, gn = nbase + nc;
                if (gm < M && gn < N) cp_async16(gs + r * GS + nc * 4, gc + (size_t)gm * N + gn);
                else *reinterpret_cast<float4 *>(gs + r * GS + nc * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            for (int id = tid; id < MT * NT; id += THREADS) {
                int r = id / NT, nn = id % NT;
                int gm = m0 + r, gn = nbase + nn;
                *reinterpret_cast<float *>(gs + r * GS + nn * 4) = (gm < M && gn < N) ? gc[(size_t)gm * N + gn] : 0.f;
            }
        }
        if (vec_w) {
            for (int id = tid; id < KT; id += THREADS) {
                int gk = k0 + id;
                if (gk < K && nbase < N) cp_async16(ws + id * NT, w + (size_t)gk * N + nbase);
                else *reinterpret_cast<uint4 *>(ws + id * NT) = make_uint4(0, 0, 0, 0);
            }
        } else {
            for (int id = tid; id < KT * NT; id += THREADS) {
                int kk = id / NT, nn = id % NT;
                int gk = k0 + kk, gn = nbase + nn;
                ws[id] = (gk < K && gn < N) ? w[(size_t)gk * N + gn] : (uint8_t)0;
            }
        }
        cp_async_commit();
    };

    for (int tile = blockIdx.x; tile < tiles_m * tiles_k; tile += gridDim.x) {
        int m0 = (tile / tiles_k) * MT;
        const int k0 = (tile % tiles_k) * KT;
        if (PIX) {
            const int tm = tile / tiles_k;
            int ci = 0;
            while (ci + 1 < set.n && tm >= set.tile_begin[ci + 1]) ++ci;
            pxp = &set.c[ci];
            m0 = (tm - set.tile_begin[ci]) * MT;
            M = pxp->P;
        }
        const PixelClass &px = *pxp;
        const int kth = k0 + wk * R;           // first k of this thread
        const int mth = m0 + wm * 32 * C + lane;  // first m of this thread; rows mth + 32*j

        // activation codes of the thread's outputs, four k per register: the gather address is then
        // row base + 2 * code in one integer dot-product instruction
        uint32_t acode[R / 4][C];
        float acc[R][C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int m = mth + 32 * j;
#pragma unroll
            for (int q = 0; q < R / 4; ++q) acode[q][j] = 0u;
            if (m < M && PIX) {
                // the pixel's code in channels kth .. kth+R-1 (planes H*W apart)
                const uint8_t *src = a + pixel_class_offset(px, m);
                const size_t plane = (size_t)px.H * px.W;
#pragma unroll
                for (int i = 0; i < R; ++i)
                    if (kth + i < K) acode[i >> 2][j] |= ((uint32_t)src[(kth + i) * plane] & MASK) << (8 * (i & 3));
            } else if (m < M) {
                if (conv.enabled) {
                    const uint4 t = conv_code16(a, conv, m, kth, K);
                    const uint32_t tw[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
                    for (int q = 0; q < R / 4; ++q) acode[q][j] = tw[q] & MASK4;
                } else {
#pragma unroll
                    for (int i = 0; i < R; ++i)
                        if (kth + i < K) acode[i >> 2][j] |= ((uint32_t)a[(size_t)m * K + kth + i] & MASK) << (8 * (i & 3));
                }
            }
#pragma unroll
            for (int i = 0; i < R; ++i) acc[i][j] = 0.f;
        }

        if (PIX) {
            // where the tile's pixels sit: output row index for tap offset 0 and the class coordinates
            for (int r = tid; r < MT; r += THREADS) {
                const int pm = m0 + r;
                int4 info = make_int4(0, 0, 0, 0);
                if (pm < M) {
                    const int per = px.Hc * px.Wc, b = pm / per, rr = pm - b * per, hh = rr / px.Wc, ww = rr - hh * px.Wc;
                    info = make_int4((b * px.Ho + hh) * px.Wo + ww, hh, ww, 1);
                }
                rowinfo[r] = info;
            }
            __syncthreads();
        }
        const int nsteps = PIX ? px.ntaps * nnt : nnt;
        load_tile(m0, k0, 0, 0);
        for (int nt = 0; nt < nsteps; ++nt) {
            cp_async_wait<0>();
            __syncthreads();
            if (nt + 1 < nsteps) load_tile(m0, k0, nt + 1, (nt + 1) & 1);
            const uint8_t *gs = g_s + (nt & 1) * Cfg::G_STAGE + (wm * 32 * C + lane) * GS;
            const uint8_t *ws = w_s + (nt & 1) * Cfg::W_STAGE + (wk * R) * NT;
#pragma unroll 1
            for (int n4 = 0; n4 < NT; n4 += 4) {
                uint32_t w4[R];
                float4 g4[C];
#pragma unroll
                for (int i = 0; i < R; ++i) w4[i] = *reinterpret_cast<const uint32_t *>(ws + i * NT + n4) & MASK4;
#pragma unroll
                for (int j = 0; j < C; ++j) g4[j] = *reinterpret_cast<const float4 *>(gs + (32 * j) * GS + n4 * 4);
#pragma unroll
                for (int nn = 0; nn < 4; ++nn) {
#pragma unroll
                    for (int i = 0; i < R; ++i) {
                        // table row of the weight code (already cut to BITS bits): at 7 bits a row is 256 bytes, so one
                        // byte permutation puts the code where the row offset needs it
                        const uint32_t wrow = BITS == 7 ? lut_addr + __byte_perm(w4[i], 0u, 0x4404u | (nn << 4))
                                                        : lut_addr + (byte_of(w4[i], nn) << (BITS + 1));
#pragma unroll
                        for (int j = 0; j < C; ++j) {
                            const float g = nn == 0 ? g4[j].x : nn == 1 ? g4[j].y : nn == 2 ? g4[j].z : g4[j].w;
                            acc[i][j] = fmaf(g, (float)lds_s16(byte_scaled_add<2>(acode[i >> 2][j], i & 3, wrow)), acc[i][j]);
                        }
                    }
                }
            }
        }

#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int m = mth + 32 * j;
            if (m >= M) continue;
            if (PIX) {
                float *obase = ga + pixel_class_offset(px, m);
                const size_t plane = (size_t)px.H * px.W;
#pragma unroll
                for (int i = 0; i < R; ++i)
                    if (kth + i < K) obase[(kth + i) * plane] = acc[i][j] * kGradFactor;
                continue;
            }
            if (conv.enabled) {
                // a convolution whose windows do not overlap: (m,k) goes straight to the image position it was
                // read from (consecutive lanes are consecutive output positions)
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    if (kth + i >= K) continue;
                    const long o = conv_scatter_index(conv, m, kth + i);
                    if (o >= 0) ga[o] = acc[i][j] * kGradFactor;
                }
                continue;
            }
            float *orow = ga + (size_t)m * K + kth;
            if (vec_o) {
#pragma unroll
                for (int i = 0; i < R; i += 4)
                    if (kth + i < K)
                        *reinterpret_cast<float4 *>(orow + i) =
                            make_float4(acc[i][j] * kGradFactor, acc[i + 1][j] * kGradFactor,
                                        acc[i + 2][j] * kGradFactor, acc[i + 3][j] * kGradFactor);
            } else {
#pragma unroll
                for (int i = 0; i < R; ++i)
                    if (kth + i < K) orow[i] = acc[i][j] * kGradFactor;
            }
        }
        __syncthreads();
    }
}

template <int BITS, int R, int C, int WM, int WK, bool PIX = false>
static int launch_ga(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut, int M,
                     int K, int N, const ConvGeom &conv, int num_sms, cudaStream_t stream,
                     const PixelClassSet *set = nullptr) {
    using Cfg = GaCfg<BITS, R, C, WM, WK>;
    auto kern = ga_colbcast_kernel<BITS, R, C, WM, WK, PIX>;
    constexpr int SMEM = PIX ? Cfg::SMEM_PIX : Cfg::SMEM;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM)))
        return LUTGEMM_E_CUDA;
    const int tiles_m = PIX ? set->tile_begin[set->n] : (M + Cfg::MT - 1) / Cfg::MT, tiles_k = (K + Cfg::KT - 1) / Cfg::KT;
    const long tiles = (long)tiles_m * tiles_k;
    int ctas_per_sm = 1;  // persistent grid: as many CTAs as the SMs hold at once
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, Cfg::THREADS, SMEM) != cudaSuccess ||
        ctas_per_sm < 1)
        ctas_per_sm = 1;
    const int grid = (int)(tiles < (long)num_sms * ctas_per_sm ? tiles : (long)num_sms * ctas_per_sm);
    const int vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    const int vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    const int vec_o = (K % 4 == 0) && ((reinterpret_cast<uintptr_t>(ga) & 15) == 0);
    kern<<<grid, Cfg::THREADS, SMEM, stream>>>(gc, a, w, ga, lut, M, K, N, tiles_m, tiles_k, vec_g, vec_w, vec_o, conv,
                                               set ? *set : PixelClassSet{});
    return launch_status();
}

int backward_ga(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                int M, int K, int N, const ConvGeom &conv, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_ga<4, 8, 4, 2, 4>(gc, a, w, ga, lut_ga, M, K, N, conv, num_sms, stream);
        case 6: return launch_ga<6, 8, 4, 2, 4>(gc, a, w, ga, lut_ga, M, K, N, conv, num_sms, stream);
        // (two columns per thread and four CTAs per SM instead of four and two measured 1-3 % slower: the kernel
        // is bound by the bank conflicts of its gather, not by latency)
        case 7: return launch_ga<7, 8, 4, 2, 4>(gc, a, w, ga, lut_ga, M, K, N, conv, num_sms, stream);
        // the 128 KB table leaves room for one CTA per SM only: make it 16 warps
        case 8: return launch_ga<8, 8, 4, 4, 4>(gc, a, w, ga, lut_ga, M, K, N, conv, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

template <int BITS, int R, int C, int WM, int WK>
static int launch_gx_bcast(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut_ga,
                           int Cout, const PixelClass *classes, int nclasses, int num_sms, cudaStream_t stream) {
    constexpr int MT = GaCfg<BITS, R, C, WM, WK>::MT;
    ConvGeom none{};
    for (int first = 0; first < nclasses; first += kMaxClassesPerLaunch) {
        PixelClassSet set{};
        set.n = nclasses - first < kMaxClassesPerLaunch ? nclasses - first : kMaxClassesPerLaunch;
        for (int i = 0; i < set.n; ++i) {
            set.c[i] = classes[first + i];
            set.tile_begin[i + 1] = set.tile_begin[i] + (set.c[i].P + MT - 1) / MT;
        }
        const int rc = launch_ga<BITS, R, C, WM, WK, true>(gy, x, wmat, gx, lut_ga, 0, classes[first].C, Cout, none, num_sms,
                                                           stream, &set);
        if (rc != LUTGEMM_OK) return rc;
    }
    return LUTGEMM_OK;
}

int backward_gx_bcast(const float *gy, const uint8_t *x, const uint8_t *wmat, float *gx, const int16_t *lut_ga, int bits,
                      int Cout, const PixelClass *classes, int nclasses, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_gx_bcast<4, 8, 4, 2, 4>(gy, x, wmat, gx, lut_ga, Cout, classes, nclasses, num_sms, stream);
        case 6: return launch_gx_bcast<6, 8, 4, 2, 4>(gy, x, wmat, gx, lut_ga, Cout, classes, nclasses, num_sms, stream);
        case 7: return launch_gx_bcast<7, 8, 4, 2, 4>(gy, x, wmat, gx, lut_ga, Cout, classes, nclasses, num_sms, stream);
        case 8: return launch_gx_bcast<8, 8, 4, 4, 4>(gy, x, wmat, gx, lut_ga, Cout, classes, nclasses, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

// ------------------------------------------------------------------------------------------------
// gW
// ------------------------------------------------------------------------------------------------
template <int BITS, int R, int C, int WK, int WN>
struct GwCfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int THREADS = 32 * WK * WN;
    static constexpr int KT = WK * R;
    static constexpr int NT = WN * 32 * C;
    static constexpr int MT = 16;
    static constexpr int LUT_BYTES = Q * Q * 2;
    static constexpr int A_STAGE = MT * KT;
    static constexpr int G_STAGE = MT * NT * 4;
    static constexpr int SMEM = LUT_BYTES + 2 * (A_STAGE + G_STAGE);
};

constexpr int kGwWideR = 4, kGwWideC = 8, kGwNarrowR = 16, kGwNarrowC = 2, kGwWarps = 8;
constexpr int kGwMinRowsPerSplit = 512;

template <int BITS, int R, int C, int WK, int WN>
__global__ void __launch_bounds__(32 * WK * WN, 1)
gw_rowbcast_kernel(const float *__restrict__ gc, const uint8_t *__restrict__ a, const uint8_t *__restrict__ w,
                   float *__restrict__ out, const int16_t *__restrict__ lut, int M, int K, int N, int tiles_k,
                   int tiles_n, int num_splits, int rows_per_split, float out_scale, int vec_a, int vec_g,
                   const ConvGeom conv) {
    using Cfg = GwCfg<BITS, R, C, WK, WN>;
    constexpr int MT = Cfg::MT, KT = Cfg::KT, NT = Cfg::NT, THREADS = Cfg::THREADS;
    constexpr uint32_t MASK = Cfg::Q - 1;
    static_assert(R == 4 || R == 16, "R k-rows per thread");
    static_assert(C == 2 || C == 8, "C columns per lane");

    extern __shared__ __align__(16) uint8_t smem[];
    int16_t *lut_s = reinterpret_cast<int16_t *>(smem);
    uint8_t *a_s = smem + Cfg::LUT_BYTES;
    uint8_t *g_s = a_s + 2 * Cfg::A_STAGE;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wk = warp / WN, wn = warp % WN;

    stage_table<BITS, false>(lut_s, lut, tid, THREADS);
    const uint32_t lut_addr = smem_u32(lut_s);

    auto load_tile = [&](int k0, int n0, int mbase, int mend, int buf) {
        uint8_t *as = a_s + buf * Cfg::A_STAGE;
        float *gs = reinterpret_cast<float *>(g_s + buf * Cfg::G_STAGE);
        if (vec_a) {
            for (int id = tid; id < MT * (KT / 16); id += THREADS) {
                int r = id / (KT / 16), kc = (id % (KT / 16)) * 16;
                int gm = mbase + r, gk = k0 + kc;
                if (gm < mend && gk < K) cp_async16(as + r * KT + kc, a + (size_t)gm * K + gk);
                else *reinterpret_cast<uint4 *>(as + r * KT + kc) = make_uint4(0, 0, 0, 0);
            }
        } else {
            for (int id = tid; id < MT * KT; id += THREADS) {
                int r = id / KT, kk = id % KT;
                int gm = mbase + r, gk = k0 + kk;
                as[id] = !(gm < mend && gk < K) ? (uint8_t)0
                         : conv.enabled          ? (uint8_t)conv_code(a, conv, gm, gk)
                                                 : a[(size_t)gm * K + gk];
            }
        }
        if (vec_g) {
            for (int id = tid; id < MT * (NT / 4); id += THREADS) {
                int r = id / (NT / 4), nc = (id % (NT / 4)) * 4;
                int gm = mbase + r, gn = n0 + nc;
                if (gm < mend && gn < N) cp_async16(gs + r * NT + nc, gc + (size_t)gm * N + gn);
                else *reinterpret_cast<float4 *>(gs + r * NT + nc) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        } else {
            for (int id = tid; id < MT * NT; id += THREADS) {
                int r = id / NT, nn = id % NT;
                int gm = mbase + r, gn = n0 + nn;
                gs[id] = (gm < mend && gn < N) ? gc[(size_t)gm * N + gn] : 0.f;
            }
        }
        cp_async_commit();
    };

    const long items = (long)tiles_k * tiles_n * num_splits;
    for (long item = blockIdx.x; item < items; item += gridDim.x) {
        const int split = (int)(item % num_splits);
        const int tile = (int)(item / num_splits);
        const int k0 = (tile / tiles_n) * KT, n0 = (tile % tiles_n) * NT;
        const int mbeg = split * rows_per_split;
        const int mend = min(M, mbeg + rows_per_split);
        // column of accumulator j: lanes interleave in groups of 4 columns so that every 128-bit read
        // of the grad_out tile is contiguous across the warp (C == 8), or plain pairs (C == 2)
        auto col_of = [&](int j) { return C == 8 ? (j >> 2) * 128 + lane * 4 + (j & 3) : lane * C + j; };
        const int kth = k0 + wk * R, nth = n0 + wn * 32 * C;

        // weight codes of the thread's outputs, four k per register (gather address = row base + 2 * code)
        uint32_t wcode[R / 4][C];
        float acc[R][C];
#pragma unroll
        for (int j = 0; j < C; ++j) {
#pragma unroll
            for (int q = 0; q < R / 4; ++q) wcode[q][j] = 0u;
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const int k = kth + i, n = nth + col_of(j);
                if (k < K && n < N) wcode[i >> 2][j] |= ((uint32_t)w[(size_t)k * N + n] & MASK) << (8 * (i & 3));
                acc[i][j] = 0.f;
            }
        }

        const int nmt = (mend - mbeg + MT - 1) / MT;
        if (nmt > 0) load_tile(k0, n0, mbeg, mend, 0);
        for (int mt = 0; mt < nmt; ++mt) {
            cp_async_wait<0>();
            __syncthreads();
            if (mt + 1 < nmt) load_tile(k0, n0, mbeg + (mt + 1) * MT, mend, (mt + 1) & 1);
            const uint8_t *as = a_s + (mt & 1) * Cfg::A_STAGE + wk * R;
            const float *gs = reinterpret_cast<const float *>(g_s + (mt & 1) * Cfg::G_STAGE) + wn * 32 * C +
                              (C == 8 ? lane * 4 : lane * C);
#pragma unroll 2
            for (int mm = 0; mm < MT; ++mm) {
                uint32_t av[R / 4];
                if constexpr (R == 4) {
                    av[0] = *reinterpret_cast<const uint32_t *>(as + mm * KT);
                } else {
                    uint4 t = *reinterpret_cast<const uint4 *>(as + mm * KT);
                    av[0] = t.x; av[1] = t.y; av[2] = t.z; av[3] = t.w;
                }
                float g[C];
                if constexpr (C == 8) {
                    float4 t0 = *reinterpret_cast<const float4 *>(gs + mm * NT);
                    float4 t1 = *reinterpret_cast<const float4 *>(gs + mm * NT + 128);
                    g[0] = t0.x; g[1] = t0.y; g[2] = t0.z; g[3] = t0.w;
                    g[4] = t1.x; g[5] = t1.y; g[6] = t1.z; g[7] = t1.w;
                } else {
                    float2 t0 = *reinterpret_cast<const float2 *>(gs + mm * NT);
                    g[0] = t0.x; g[1] = t0.y;
                }
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const uint32_t arow = lut_addr + ((byte_of(av[i / 4], i % 4) & MASK) << (BITS + 1));
#pragma unroll
                    for (int j = 0; j < C; ++j)
                        acc[i][j] = fmaf((float)lds_s16(byte_scaled_add<2>(wcode[i >> 2][j], i & 3, arow)), g[j], acc[i][j]);
                }
            }
        }

        float *obase = out + (num_splits > 1 ? (size_t)split * K * N : (size_t)0);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int k = kth + i;
            if (k >= K) continue;
#pragma unroll
            for (int j = 0; j < C; ++j)
                if (nth + col_of(j) < N) obase[(size_t)k * N + nth + col_of(j)] = acc[i][j] * out_scale;
        }
        __syncthreads();
    }
}

__global__ void gw_reduce_splits_kernel(const float *__restrict__ partial, float *__restrict__ gw, long KN,
                                        int num_splits, float scale) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < KN; i += (long)gridDim.x * blockDim.x) {
        float s = 0.f;
        for (int p = 0; p < num_splits; ++p) s += partial[(size_t)p * KN + i];
        gw[i] = s * scale;
    }
}

static bool gw_use_narrow(int N) { return N <= 128; }

int gw_num_splits(int bits, int M, int K, int N, int num_sms) {
    (void)bits;
    const int kt = gw_use_narrow(N) ? kGwWarps * kGwNarrowR : kGwWarps * kGwWideR;
    const int nt = gw_use_narrow(N) ? 32 * kGwNarrowC : 32 * kGwWideC;
    const long tiles = (long)((K + kt - 1) / kt) * ((N + nt - 1) / nt);
    long want = (2L * num_sms + tiles - 1) / tiles;
    long cap = M / kGwMinRowsPerSplit;
    if (want > cap) want = cap;
    if (want < 1) want = 1;
    if (want > 4096) want = 4096;
    return (int)want;
}

template <int BITS, int R, int C, int WK, int WN>
static int launch_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut, int M,
                     int K, int N, const ConvGeom &conv, float *scratch, int num_splits, int num_sms,
                     cudaStream_t stream) {
    using Cfg = GwCfg<BITS, R, C, WK, WN>;
    auto kern = gw_rowbcast_kernel<BITS, R, C, WK, WN>;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM)))
        return LUTGEMM_E_CUDA;
    const int tiles_k = (K + Cfg::KT - 1) / Cfg::KT, tiles_n = (N + Cfg::NT - 1) / Cfg::NT;
    const long items = (long)tiles_k * tiles_n * num_splits;
    const int ctas_per_sm = Cfg::SMEM <= 100 * 1024 ? 2 : 1;
    const int grid = (int)(items < (long)num_sms * ctas_per_sm ? items : (long)num_sms * ctas_per_sm);
    int rows_per_split = (M + num_splits - 1) / num_splits;
    rows_per_split = (rows_per_split + Cfg::MT - 1) / Cfg::MT * Cfg::MT;
    const int vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    const int vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    float *out = num_splits > 1 ? scratch : gw;
    const float scale = num_splits > 1 ? 1.0f : kGradFactor;
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(gc, a, w, out, lut, M, K, N, tiles_k, tiles_n, num_splits,
                                                    rows_per_split, scale, vec_a, vec_g, conv);
    if (launch_status() != LUTGEMM_OK) return LUTGEMM_E_CUDA;
    if (num_splits > 1) {
        const long KN = (long)K * N;
        const int rgrid = (int)((KN + 255) / 256 < 4L * num_sms ? (KN + 255) / 256 : 4L * num_sms);
        gw_reduce_splits_kernel<<<rgrid, 256, 0, stream>>>(scratch, gw, KN, num_splits, kGradFactor);
        if (launch_status() != LUTGEMM_OK) return LUTGEMM_E_CUDA;
    }
    return LUTGEMM_OK;
}

template <int BITS>
static int dispatch_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut, int M,
                       int K, int N, const ConvGeom &conv, float *scratch, int num_splits, int num_sms,
                       cudaStream_t stream) {
    if (gw_use_narrow(N))
        return launch_gw<BITS, kGwNarrowR, kGwNarrowC, kGwWarps, 1>(gc, a, w, gw, lut, M, K, N, conv, scratch,
                                                                     num_splits, num_sms, stream);
    return launch_gw<BITS, kGwWideR, kGwWideC, kGwWarps, 1>(gc, a, w, gw, lut, M, K, N, conv, scratch, num_splits,
                                                             num_sms, stream);
}

int backward_gw(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                int M, int K, int N, const ConvGeom &conv, float *scratch, int num_splits, int num_sms,
                cudaStream_t stream) {
    switch (bits) {
        case 4: return dispatch_gw<4>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_splits, num_sms, stream);
        case 6: return dispatch_gw<6>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_splits, num_sms, stream);
        case 7: return dispatch_gw<7>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_splits, num_sms, stream);
        case 8: return dispatch_gw<8>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_splits, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

// at[k][m..m+15] per thread: lanes run over m, so the 16-byte stores are coalesced.  For the unfolded code
// image the (channel, tap) of k and the (image, row, column) of the first m are decoded once per thread and m
// advances incrementally; for a plain [M,K] matrix the byte loads of the 32 k of a block share sectors.
__global__ void __launch_bounds__(1024) transpose_codes_kernel(const uint8_t *__restrict__ a, uint8_t *__restrict__ at,
                                                               int M, int K, int pitch, const ConvGeom g, uint32_t mask4) {
    const int k = blockIdx.y * 32 + threadIdx.y;
    const int m0 = (blockIdx.x * 32 + threadIdx.x) * 16;
    if (k >= K || m0 >= pitch) return;
    uint32_t v[4] = {0u, 0u, 0u, 0u};
    if (g.enabled) {
        const int L = g.Ho * g.Wo, kk = g.kh * g.kw;
        const int c = k / kk, r = k - c * kk, i = r / g.kw, j = r - i * g.kw;
        int b = m0 / L, l = m0 - b * L, oh = l / g.Wo, ow = l - oh * g.Wo;
        const int dh = i * g.dil - g.pad, dw = j * g.dil - g.pad;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const int ih = oh * g.stride + dh, iw = ow * g.stride + dw;
            if (m0 + e < M && (unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
                v[e >> 2] |= (uint32_t)a[((size_t)(b * g.C + c) * g.H + ih) * g.W + iw] << (8 * (e & 3));
            if (++ow == g.Wo) { ow = 0; if (++oh == g.Ho) { oh = 0; ++b; } }
        }
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e)
            if (m0 + e < M) v[e >> 2] |= (uint32_t)a[(size_t)(m0 + e) * K + k] << (8 * (e & 3));
    }
    *reinterpret_cast<uint4 *>(at + (size_t)k * pitch + m0) = make_uint4(v[0] & mask4, v[1] & mask4, v[2] & mask4, v[3] & mask4);
}

// The same for a convolution whose output plane is a multiple of 16 positions and whose input plane fits
// shared memory: one CTA stages the plane x[b,c,:,:] once (coalesced) and writes the kh*kw shifted copies of
// it, 16 output positions per thread and store.
__global__ void __launch_bounds__(256) transpose_codes_plane_kernel(const uint8_t *__restrict__ x, uint8_t *__restrict__ at,
                                                                    int pitch, const ConvGeom g, uint32_t mask4) {
    extern __shared__ __align__(16) uint8_t plane[];
    const int bc = blockIdx.x, b = bc / g.C, c = bc - b * g.C;
    const int HW = g.H * g.W, L = g.Ho * g.Wo, kk = g.kh * g.kw;
    const uint8_t *src = x + (size_t)bc * HW;
    if ((HW & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        for (int i = threadIdx.x; i < HW / 16; i += blockDim.x)
            reinterpret_cast<uint4 *>(plane)[i] = reinterpret_cast<const uint4 *>(src)[i];
    } else {
        for (int i = threadIdx.x; i < HW; i += blockDim.x) plane[i] = src[i];
    }
    __syncthreads();
    const int chunks = L / 16;
    for (int q = threadIdx.x; q < kk * chunks; q += blockDim.x) {
        const int tap = q / chunks, l0 = (q - tap * chunks) * 16;
        const int i = tap / g.kw, j = tap - i * g.kw;
        const int dh = i * g.dil - g.pad, dw = j * g.dil - g.pad;
        int oh = l0 / g.Wo, ow = l0 - oh * g.Wo;
        uint32_t v[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const int ih = oh * g.stride + dh, iw = ow * g.stride + dw;
            if ((unsigned)ih < (unsigned)g.H && (unsigned)iw < (unsigned)g.W)
                v[e >> 2] |= (uint32_t)plane[ih * g.W + iw] << (8 * (e & 3));
            if (++ow == g.Wo) { ow = 0; ++oh; }
        }
        *reinterpret_cast<uint4 *>(at + (size_t)(c * kk + tap) * pitch + (size_t)b * L + l0) =
            make_uint4(v[0] & mask4, v[1] & mask4, v[2] & mask4, v[3] & mask4);
    }
}

// Plain [M,K] matrix with 16-byte aligned rows (K a multiple of 16): a CTA moves a tile of 128 rows x 64 k through
// shared memory - 16-byte loads along k, 16-byte stores along m - instead of gathering single bytes from global memory.
__global__ void __launch_bounds__(512) transpose_codes_tiled_kernel(const uint8_t *__restrict__ a, uint8_t *__restrict__ at,
                                                                    int M, int K, int pitch, uint32_t mask4) {
    constexpr int TM = 128, TK = 64, TP = TK + 4;  // tile pitch in bytes: rows 17 words apart, the transposed byte reads
                                                   // of 32 rows fall on 32 different banks
    __shared__ __align__(16) uint8_t tile[TM * TP];
    const int m0 = blockIdx.x * TM, k0 = blockIdx.y * TK;
    const int tid = threadIdx.x;
    {   // load: thread = (row, 16-k chunk); 4 chunks per row
        const int r = tid >> 2, q = tid & 3;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (m0 + r < M && k0 + q * 16 < K) v = *reinterpret_cast<const uint4 *>(a + (size_t)(m0 + r) * K + k0 + q * 16);
        uint32_t *dst = reinterpret_cast<uint32_t *>(tile + r * TP + q * 16);
        dst[0] = v.x & mask4; dst[1] = v.y & mask4; dst[2] = v.z & mask4; dst[3] = v.w & mask4;
    }
    __syncthreads();
    {   // store: thread = (k, 16-row chunk); 8 chunks per k
        const int k = tid >> 3, c = tid & 7;
        if (k0 + k < K && m0 + c * 16 < pitch) {
            uint32_t v[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e >> 2] |= (uint32_t)tile[(c * 16 + e) * TP + k] << (8 * (e & 3));
            *reinterpret_cast<uint4 *>(at + (size_t)(k0 + k) * pitch + m0 + c * 16) = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
}

int transpose_codes(const uint8_t *a, uint8_t *at, int M, int K, int pitch, const ConvGeom &conv, int bits,
                    cudaStream_t stream) {
    const uint32_t mask4 = ((1u << bits) - 1u) * 0x01010101u;  // codes are cut to `bits` bits on their way through
    // (small planes leave a CTA too little to do: they take the generic kernel)
    if (conv.enabled && (conv.Ho * conv.Wo) % 16 == 0 && conv.Ho * conv.Wo >= 256 && conv.H * conv.W <= 96 * 1024 &&
        (long)conv.B * conv.C <= 0x7fffffffL) {
        // every column m < M is written (M = B * Ho * Wo is a multiple of 16, so pitch == M)
        const int smem = (conv.H * conv.W + 15) & ~15;
        if (smem > 48 * 1024 &&
            !cuda_ok(cudaFuncSetAttribute(transpose_codes_plane_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)))
            return LUTGEMM_E_CUDA;
        transpose_codes_plane_kernel<<<conv.B * conv.C, 256, smem, stream>>>(a, at, pitch, conv, mask4);
        return launch_status();
    }
    if (!conv.enabled && K % 16 == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (K + 63) / 64 <= 65535) {
        const dim3 tgrid((pitch + 127) / 128, (K + 63) / 64);
        transpose_codes_tiled_kernel<<<tgrid, 512, 0, stream>>>(a, at, M, K, pitch, mask4);
        return launch_status();
    }
    const dim3 block(32, 32), grid((pitch / 16 + 31) / 32, (K + 31) / 32);
    if (grid.y > 65535u) return LUTGEMM_E_TOOLARGE;
    transpose_codes_kernel<<<grid, block, 0, stream>>>(a, at, M, K, pitch, conv, mask4);
    return launch_status();
}

}  // namespace lutgemm
