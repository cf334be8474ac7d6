// Forward LUT-GEMM for sm_100a:  c[m,n] = sum_k LUT[a[m,k]][w[k,n]]  (exact uint32 accumulate).
//
// "Row-broadcast" kernel.  The whole 2^b x 2^b table sits in shared memory as dense uint16 rows
// (128 KB at 8 bits).  All 32 lanes of a warp work on the SAME rows m, so the activation code
// a[m,k] - and with it the table row - is warp-uniform; lane l owns C adjacent output columns and
// supplies the column index w[k,n].  A gather therefore touches one table row only:
//   b <= 6 : a row is <= 32 words, so every gather is bank-conflict free (equal words broadcast),
//   b  = 7 : 64 words, at most 2-way,      b = 8 : 128 words, at most 4-way,
// instead of the up-to-32-way random pattern of a thread tile that mixes rows.  CTAs are persistent
// (grid = #SMs) and stage the table once per launch; operand tiles stream through a two-stage
// cp.async pipeline.  Replaces ApproxGemmForwardKernel, self_ops/src/approx_gemm_forward.cu:37-229.
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

template <int BITS, int R, int C, int WM, int WN>
struct FwdCfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int THREADS = 32 * WM * WN;
    static constexpr int MT = WM * R;
    static constexpr int NT = WN * 32 * C;
    static constexpr int KT = 32;
    static constexpr int LUT_BYTES = Q * Q * 2;
    static constexpr int A_STAGE = MT * KT;
    static constexpr int W_STAGE = KT * NT;
    static constexpr int SMEM = LUT_BYTES + 2 * (A_STAGE + W_STAGE);
};

template <int BITS, int R, int C, int WM, int WN>
__global__ void __launch_bounds__(32 * WM * WN, 1)
fwd_rowbcast_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ w, uint32_t *__restrict__ c,
                    const uint16_t *__restrict__ lut, int M, int K, int N, int tiles_m, int tiles_n,
                    int vec_a, int vec_w, int vec_c, const ConvGeom conv, const LayerEpilogue epi) {
    using Cfg = FwdCfg<BITS, R, C, WM, WN>;
    constexpr int KT = Cfg::KT, MT = Cfg::MT, NT = Cfg::NT, THREADS = Cfg::THREADS;
    constexpr uint32_t MASK = Cfg::Q - 1;
    static_assert(C == 2 || C == 4 || C == 8, "C columns per lane");

    extern __shared__ __align__(16) uint8_t smem[];
    uint16_t *lut_s = reinterpret_cast<uint16_t *>(smem);
    uint8_t *a_s = smem + Cfg::LUT_BYTES;
    uint8_t *w_s = a_s + 2 * Cfg::A_STAGE;

    const int tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const int wm = warp / WN, wn = warp % WN;

    stage_table<BITS, false>(lut_s, lut, tid, THREADS);
    const uint32_t lut_addr = smem_u32(lut_s);

    const int nkt = (K + KT - 1) / KT;

    auto load_tile = [&](int m0, int n0, int kt, int buf) {
        uint8_t *as = a_s + buf * Cfg::A_STAGE;
        uint8_t *ws = w_s + buf * Cfg::W_STAGE;
        const int kbase = kt * KT;
        if (vec_a) {
            for (int id = tid; id < MT * (KT / 16); id += THREADS) {
                int r = id / (KT / 16), kc = (id % (KT / 16)) * 16;
                int gm = min(m0 + r, M - 1), gk = kbase + kc;
                if (gk < K) cp_async16(as + r * KT + kc, a + (size_t)gm * K + gk);
                else *reinterpret_cast<uint4 *>(as + r * KT + kc) = make_uint4(0, 0, 0, 0);
            }
        } else {
            for (int id = tid; id < MT * KT; id += THREADS) {
                int r = id / KT, kk = id % KT;
                int gm = min(m0 + r, M - 1), gk = kbase + kk;
                as[id] = gk >= K ? (uint8_t)0 : conv.enabled ? (uint8_t)conv_code(a, conv, gm, gk) : a[(size_t)gm * K + gk];
            }
        }
        if (vec_w) {
            for (int id = tid; id < KT * (NT / 16); id += THREADS) {
                int kk = id / (NT / 16), nc = (id % (NT / 16)) * 16;
                int gk = kbase + kk, gn = n0 + nc;
                if (gk < K && gn < N) cp_async16(ws + kk * NT + nc, w + (size_t)gk * N + gn);
                else *reinterpret_cast<uint4 *>(ws + kk * NT + nc) = make_uint4(0, 0, 0, 0);
            }
        } else {
            for (int id = tid; id < KT * NT; id += THREADS) {
                int kk = id / NT, nn = id % NT;
                int gk = kbase + kk, gn = n0 + nn;
                ws[id] = (gk < K && gn < N) ? w[(size_t)gk * N + gn] : (uint8_t)0;
            }
        }
        cp_async_commit();
    };

    for (int tile = blockIdx.x; tile < tiles_m * tiles_n; tile += gridDim.x) {
        const int m0 = (tile / tiles_n) * MT, n0 = (tile % tiles_n) * NT;
        uint32_t acc[R][C];
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int j = 0; j < C; ++j) acc[i][j] = 0u;

        load_tile(m0, n0, 0, 0);
        for (int kt = 0; kt < nkt; ++kt) {
            cp_async_wait<0>();
            __syncthreads();
            if (kt + 1 < nkt) load_tile(m0, n0, kt + 1, (kt + 1) & 1);
            const uint8_t *as = a_s + (kt & 1) * Cfg::A_STAGE + (wm * R) * KT;
            const uint8_t *ws = w_s + (kt & 1) * Cfg::W_STAGE + wn * 32 * C + lane * C;
            const int kcount = min(KT, K - kt * KT);

            auto step = [&](uint32_t (&woff)[C], const uint32_t (&arow)[R]) {
#pragma unroll
                for (int i = 0; i < R; ++i) {
#pragma unroll
                    for (int j = 0; j < C; ++j) acc[i][j] += lds_u16(arow[i] + woff[j]);
                }
            };
            auto load_w = [&](int k, uint32_t (&woff)[C]) {
                const uint8_t *p = ws + k * NT;
                if constexpr (C == 8) {
                    uint2 v = *reinterpret_cast<const uint2 *>(p);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        woff[j] = (byte_of(v.x, j) & MASK) * 2u;
                        woff[4 + j] = (byte_of(v.y, j) & MASK) * 2u;
                    }
                } else if constexpr (C == 4) {
                    uint32_t v = *reinterpret_cast<const uint32_t *>(p);
#pragma unroll
                    for (int j = 0; j < 4; ++j) woff[j] = (byte_of(v, j) & MASK) * 2u;
                } else {
                    uint32_t v = *reinterpret_cast<const uint16_t *>(p);
#pragma unroll
                    for (int j = 0; j < 2; ++j) woff[j] = (byte_of(v, j) & MASK) * 2u;
                }
            };

            if (kcount == KT) {
#pragma unroll 1
                for (int k4 = 0; k4 < KT; k4 += 4) {
                    uint32_t a4[R];
#pragma unroll
                    for (int i = 0; i < R; ++i) a4[i] = *reinterpret_cast<const uint32_t *>(as + i * KT + k4);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) {
                        uint32_t woff[C], arow[R];
                        load_w(k4 + kk, woff);
#pragma unroll
                        for (int i = 0; i < R; ++i) arow[i] = lut_addr + ((byte_of(a4[i], kk) & MASK) << (BITS + 1));
                        step(woff, arow);
                    }
                }
            } else {
#pragma unroll 1
                for (int k = 0; k < kcount; ++k) {
                    uint32_t woff[C], arow[R];
                    load_w(k, woff);
#pragma unroll
                    for (int i = 0; i < R; ++i) arow[i] = lut_addr + (((uint32_t)as[i * KT + k] & MASK) << (BITS + 1));
                    step(woff, arow);
                }
            }
        }

        // epilogue: each lane owns C adjacent columns of R rows
        const int nbase = n0 + wn * 32 * C + lane * C;
        LayerEpilogueScalars ev{};
        if (epi.out) ev = load_epilogue_scalars(epi);
#pragma unroll
        for (int i = 0; i < R; ++i) {
            const int m = m0 + wm * R + i;
            if (m >= M) continue;
            if (epi.out) {
                // the layer's de-quantisation applied to the sums in registers
                const int l = m % epi.L;
                const float zw_box = __fmul_rn(ev.zw, epi.box[m]), zz_taps = __fmul_rn(ev.zz, epi.taps[l]);
                float *orow = epi.out + (size_t)m * N;
#pragma unroll
                for (int j = 0; j < C; ++j)
                    if (nbase + j < N) orow[nbase + j] = epilogue_value(epi, ev, acc[i][j], zw_box, zz_taps, l, nbase + j, N);
                continue;
            }
            uint32_t *crow = c + (size_t)m * N;
            if (vec_c) {
                if constexpr (C >= 4) {
#pragma unroll
                    for (int j = 0; j < C; j += 4)
                        if (nbase + j < N)
                            *reinterpret_cast<uint4 *>(crow + nbase + j) =
                                make_uint4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]);
                } else {
                    if (nbase < N) *reinterpret_cast<uint2 *>(crow + nbase) = make_uint2(acc[i][0], acc[i][1]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < C; ++j)
                    if (nbase + j < N) crow[nbase + j] = acc[i][j];
            }
        }
        __syncthreads();  // every warp is done with both operand buffers before the next tile's loads
    }
}

template <int BITS, int R, int C, int WM, int WN>
static int launch_fwd(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                      const ConvGeom &conv, const LayerEpilogue *epi, int num_sms, cudaStream_t stream) {
    using Cfg = FwdCfg<BITS, R, C, WM, WN>;
    auto kern = fwd_rowbcast_kernel<BITS, R, C, WM, WN>;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM)))
        return LUTGEMM_E_CUDA;
    const int tiles_m = (M + Cfg::MT - 1) / Cfg::MT, tiles_n = (N + Cfg::NT - 1) / Cfg::NT;
    const long tiles = (long)tiles_m * tiles_n;
    const int ctas_per_sm = Cfg::SMEM <= 100 * 1024 ? 2 : 1;
    const int grid = (int)(tiles < (long)num_sms * ctas_per_sm ? tiles : (long)num_sms * ctas_per_sm);
    const int vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    const int vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    const int vec_c = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(a, w, c, lut, M, K, N, tiles_m, tiles_n, vec_a, vec_w, vec_c, conv,
                                                    epi ? *epi : LayerEpilogue{});
    return launch_status();
}

template <int BITS>
static int dispatch_fwd(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                        const ConvGeom &conv, const LayerEpilogue *epi, int num_sms, cudaStream_t stream) {
    if (N <= 128) return launch_fwd<BITS, 16, 2, 8, 1>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
    return launch_fwd<BITS, 8, 8, 8, 1>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
}

int forward_rowbcast(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                     int N, const ConvGeom &conv, const LayerEpilogue *epi, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return dispatch_fwd<4>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
        case 6: return dispatch_fwd<6>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
        case 7: return dispatch_fwd<7>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
        case 8: return dispatch_fwd<8>(a, w, c, lut, M, K, N, conv, epi, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
