// Warp-specialised "column-gathered slab" LUT-GEMM kernels for sm_100a (forward, grad_w, grad_a).
//
// Same arithmetic and shared-memory layouts as the barrier-synchronous slab kernel (lutgemm_slab.cu):
// for each k a slab U_k[x][c] = TABLE(x, cc[k,c]) is gathered once and every row r of the 512-row tile
// then reads slab row rc[r,k] contiguously (64 look-ups per conflict-free shared-memory wavefront).
// Here the two phases run on different warps, coupled by mbarriers instead of a CTA-wide barrier per k:
//
//   warps 0-3  (producers): stream operand chunks from global memory (row codes transposed into
//                           [k][r] byte rows, column codes as they are), build slab k+1, and in the
//                           gradient modes combine the 16 consumer partial sums of k-1 in fixed order;
//   warps 4-19 (consumers): for every k read 32 slab rows each and accumulate (integer accumulators
//                           for the forward, fp32 FMAs against the register-resident grad_out block
//                           for the gradients).
//
// Pipeline state: two slab buffers (slab_full / slab_empty), two row-code stages (rc_full / rc_empty)
// and, for the gradients, two partial-sum buffers (part_full / part_empty).  Consumers never wait for
// each other, only for a producer that is normally a slab ahead, so their shared-memory latencies
// overlap instead of lining up behind a barrier.  Every mbarrier wait is bounded: after kWaitLimit
// polls the thread records an error code in g_slab_ws_error and raises an abort word that makes every
// later wait of the CTA return at once, so the kernel always terminates.
// Replaces ApproxGemmForwardKernel (self_ops/src/approx_gemm_forward.cu:37-229) and
// ApproxGemmBackwardKernelForGA / ForGB (self_ops/src/approx_gemm_backward.cu:13-258, 261-492).
#include <stdlib.h>

#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

__device__ int g_slab_ws_error = 0;  // 0 = ok, otherwise the id of the wait that gave up

namespace ws {

enum { kFwd = 0, kGw = 1, kGa = 2 };
constexpr int kProducerWarps = 4, kConsumerWarps = 16;
constexpr int kProducers = kProducerWarps * 32, kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kProducers + kConsumers;
constexpr int kWaitLimit = 1 << 22;

template <int BITS>
struct Cfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int HALF = Q / 2;
    static constexpr int TT_STRIDE = HALF + 1;
    static constexpr int RT = 512, CT = 64, KC = 16;
    static constexpr int U_STRIDE = 33, P_STRIDE = 66;
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = KC * RT, CC_STAGE = KC * CT;
    static constexpr int P_BYTES = 16 * P_STRIDE * 4;
    static constexpr int OFF_U = TT_BYTES;
    static constexpr int OFF_RC = OFF_U + 2 * U_BYTES;
    static constexpr int OFF_CC = OFF_RC + 2 * RC_STAGE;
    static constexpr int OFF_PART = OFF_CC + 2 * CC_STAGE;
    static constexpr int OFF_BAR_FWD = OFF_PART;
    static constexpr int OFF_BAR_BWD = OFF_PART + 2 * P_BYTES;
    static constexpr int SMEM_FWD = OFF_BAR_FWD + 16 * 8;
    static constexpr int SMEM_BWD = OFF_BAR_BWD + 16 * 8;
    static constexpr int NSETS = HALF > 32 ? HALF / 32 : 1;
};

struct Args {
    const uint8_t *a;
    const uint8_t *w;
    const void *lut;
    const float *gc;
    void *out;
    int M, K, N;
    int tiles_r, tiles_c;
    int ksplits, k_per_split;
    int direct;
    int vec_a, vec_w, vec_o, vec_g;
};

// barrier slots
enum { B_SLAB_FULL = 0, B_SLAB_EMPTY = 2, B_RC_FULL = 4, B_RC_EMPTY = 6, B_PART_FULL = 8, B_PART_EMPTY = 10 };

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait for the phase with the given parity.  A wait that runs out records its id in
// g_slab_ws_error and raises the CTA's abort word; from then on every wait of the CTA returns at once,
// so the kernel still terminates (with a wrong result, which the host learns from the error word).
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, int what, volatile int *abort_word) {
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return;
        if (i > 64) {
            if (*abort_word) return;
            __nanosleep(32);
        }
    }
    *abort_word = 1;
    atomicExch(&g_slab_ws_error, what);
}

template <int BITS, int MODE>
__global__ void __launch_bounds__(kThreads, 1) slab_ws_kernel(const Args p) {
    using C = Cfg<BITS>;
    constexpr int Q = C::Q, HALF = C::HALF, TTS = C::TT_STRIDE, RT = C::RT, CT = C::CT, KC = C::KC;
    constexpr int US = C::U_STRIDE, PS = C::P_STRIDE, NSETS = C::NSETS;
    constexpr uint32_t MASK4 = (Q - 1) * 0x01010101u;
    constexpr int COL = lut_col_num(BITS);
    constexpr int OFF_BAR = MODE == kFwd ? C::OFF_BAR_FWD : C::OFF_BAR_BWD;

    const int M = p.M, K = p.K, N = p.N;
    const int CDIM = MODE == kGa ? M : N;

    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tt_s = reinterpret_cast<uint32_t *>(smem);
    uint8_t *rc_s = smem + C::OFF_RC;
    uint8_t *cc_s = smem + C::OFF_CC;
    float *part_s = reinterpret_cast<float *>(smem + C::OFF_PART);
    const uint32_t bar0 = smem_u32(smem + OFF_BAR);
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem + OFF_BAR + 12 * 8);
    const uint32_t tt_addr = smem_u32(tt_s);
    const uint32_t u_addr = smem_u32(smem + C::OFF_U);

    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;

    // ---- table staging (all threads): tt[y][i] = { T(i, y), T(i + HALF, y) } -------------------------
    {
        const uint16_t *lut = reinterpret_cast<const uint16_t *>(p.lut);
        uint16_t *tt16 = reinterpret_cast<uint16_t *>(tt_s);
        for (int idx = tid; idx < Q * Q; idx += kThreads) {
            const int hi_idx = idx >> BITS, lo_idx = idx & (Q - 1);
            const uint16_t v = lut[hi_idx * COL + lo_idx];
            const int x = MODE == kGa ? lo_idx : hi_idx, y = MODE == kGa ? hi_idx : lo_idx;
            tt16[(y * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] = v;
        }
    }
    if (tid == 0) {
        *abort_word = 0;
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar0 + (B_SLAB_FULL + b) * 8, kProducers);
            mbar_init(bar0 + (B_SLAB_EMPTY + b) * 8, kConsumers);
            mbar_init(bar0 + (B_RC_FULL + b) * 8, kProducers);
            mbar_init(bar0 + (B_RC_EMPTY + b) * 8, kConsumers);
            mbar_init(bar0 + (B_PART_FULL + b) * 8, kConsumers);
            mbar_init(bar0 + (B_PART_EMPTY + b) * 8, kProducers);
        }
    }
    __syncthreads();

    const int items = MODE == kFwd ? p.tiles_r * p.tiles_c * p.ksplits : p.tiles_r * p.tiles_c;
    uint32_t it = 0;  // k iterations done by this CTA (slab / partial buffer = it & 1)
    uint32_t ch = 0;  // operand chunks done by this CTA (row-code stage = ch & 1)

    if (wp < kProducerWarps) {
        // =============================== producers ======================================================
        const int ptid = tid;  // 0..127
        uint4 prc[4], pcc = make_uint4(0, 0, 0, 0);

        auto fetch_chunk = [&](int r0, int c0, int chunk) {
            const int kbase = chunk * KC;
            if (MODE != kGa) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint8_t *src = p.a + (size_t)min(r0 + ptid + 128 * j, M - 1) * K + kbase;
                    if (p.vec_a) {
                        prc[j] = kbase < K ? *reinterpret_cast<const uint4 *>(src) : make_uint4(0, 0, 0, 0);
                    } else {
                        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            if (kbase + q < K) t[q >> 2] |= (uint32_t)src[q] << (8 * (q & 3));
                        prc[j] = make_uint4(t[0], t[1], t[2], t[3]);
                    }
                }
                if (ptid < KC * CT / 16) {
                    const int kk = ptid / (CT / 16), cc = (ptid % (CT / 16)) * 16;
                    const int gk = kbase + kk, gn = c0 + cc;
                    if (p.vec_w) {
                        pcc = (gk < K && gn < N) ? *reinterpret_cast<const uint4 *>(p.w + (size_t)gk * N + gn)
                                                  : make_uint4(0, 0, 0, 0);
                    } else {
                        uint32_t t[4] = {0, 0, 0, 0};
                        if (gk < K) {
#pragma unroll
                            for (int q = 0; q < 16; ++q)
                                if (gn + q < N) t[q >> 2] |= (uint32_t)p.w[(size_t)gk * N + gn + q] << (8 * (q & 3));
                        }
                        pcc = make_uint4(t[0], t[1], t[2], t[3]);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int idx = ptid + 128 * j;
                    const int kk = idx / (RT / 16), rr = (idx % (RT / 16)) * 16;
                    const int gk = kbase + kk, gn = r0 + rr;
                    if (p.vec_w) {
                        prc[j] = (gk < K && gn < N) ? *reinterpret_cast<const uint4 *>(p.w + (size_t)gk * N + gn)
                                                     : make_uint4(0, 0, 0, 0);
                    } else {
                        uint32_t t[4] = {0, 0, 0, 0};
                        if (gk < K) {
#pragma unroll
                            for (int q = 0; q < 16; ++q)
                                if (gn + q < N) t[q >> 2] |= (uint32_t)p.w[(size_t)gk * N + gn + q] << (8 * (q & 3));
                        }
                        prc[j] = make_uint4(t[0], t[1], t[2], t[3]);
                    }
                }
                if (ptid < CT) {
                    const uint8_t *src = p.a + (size_t)min(c0 + ptid, M - 1) * K + kbase;
                    if (p.vec_a) {
                        pcc = kbase < K ? *reinterpret_cast<const uint4 *>(src) : make_uint4(0, 0, 0, 0);
                    } else {
                        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
                        for (int q = 0; q < 16; ++q)
                            if (kbase + q < K) t[q >> 2] |= (uint32_t)src[q] << (8 * (q & 3));
                        pcc = make_uint4(t[0], t[1], t[2], t[3]);
                    }
                }
            }
        };
        auto store_chunk = [&](int stage) {
            uint8_t *rs = rc_s + stage * C::RC_STAGE;
            uint8_t *cs = cc_s + stage * C::CC_STAGE;
            const uint32_t tc[4] = {pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4};
            if (MODE != kGa) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t tr[4] = {prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4};
#pragma unroll
                    for (int q = 0; q < 16; ++q)
                        rs[q * RT + ptid + 128 * j] = (uint8_t)(tr[q >> 2] >> (8 * (q & 3)));
                }
                if (ptid < KC * CT / 16) {
                    const int kk = ptid / (CT / 16), cc = (ptid % (CT / 16)) * 16;
                    *reinterpret_cast<uint4 *>(cs + kk * CT + cc) = make_uint4(tc[0], tc[1], tc[2], tc[3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int idx = ptid + 128 * j;
                    const int kk = idx / (RT / 16), rr = (idx % (RT / 16)) * 16;
                    *reinterpret_cast<uint4 *>(rs + kk * RT + rr) =
                        make_uint4(prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4);
                }
                if (ptid < CT) {
#pragma unroll
                    for (int q = 0; q < 16; ++q) cs[q * CT + ptid] = (uint8_t)(tc[q >> 2] >> (8 * (q & 3)));
                }
            }
        };
        // producer warp wp fills column pairs 8wp .. 8wp+7 of the slab
        auto build = [&](int buf, int stage, int kk) {
            const uint4 cw4 = *reinterpret_cast<const uint4 *>(cc_s + stage * C::CC_STAGE + kk * CT + wp * 16);
            const uint32_t cw[4] = {cw4.x, cw4.y, cw4.z, cw4.w};
            const uint32_t ub = u_addr + buf * C::U_BYTES;
#pragma unroll
            for (int pp = 0; pp < 8; ++pp) {
                const uint32_t y0 = byte_of(cw[pp >> 1], 2 * (pp & 1)), y1 = byte_of(cw[pp >> 1], 2 * (pp & 1) + 1);
                const int pc = 8 * wp + pp;
#pragma unroll
                for (int j = 0; j < NSETS; ++j) {
                    const int i = lane + 32 * j;
                    if (HALF >= 32 || i < HALF) {
                        const uint32_t r0 = lds_u32(tt_addr + (y0 * TTS + i) * 4);
                        const uint32_t r1 = lds_u32(tt_addr + (y1 * TTS + i) * 4);
                        const uint32_t lo = __byte_perm(r0, r1, 0x5410);
                        const uint32_t hi = __byte_perm(r0, r1, 0x7632);
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + (i * US + pc) * 4), "r"(lo) : "memory");
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + ((i + HALF) * US + pc) * 4), "r"(hi) : "memory");
                    }
                }
            }
        };
        // gradients: add the 16 consumer partial sums of one k in fixed order and store the 64 columns.
        // warp wp owns columns 16wp..16wp+15; lane = 16*half + col; half h adds consumers 8h..8h+7.
        auto reduce_store = [&](uint32_t jt, int k, float *obase, int c0) {
            const float *ps = part_s + (jt & 1) * (16 * PS);
            const int col = 16 * wp + (lane & 15), half = lane >> 4;
            float v = 0.f;
#pragma unroll
            for (int q = 0; q < 8; ++q) v += ps[(8 * half + q) * PS + col];
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (lane < 16 && c0 + col < CDIM) {
                if (p.direct && MODE == kGa) obase[(size_t)(c0 + col) * K + k] = v * kGradFactor;
                else obase[(size_t)k * CDIM + c0 + col] = p.direct ? v * kGradFactor : v;
            }
        };

        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            int tile, kbeg, kend;
            if (MODE == kFwd) {
                tile = item / p.ksplits;
                kbeg = (item % p.ksplits) * p.k_per_split;
                kend = min(K, kbeg + p.k_per_split);
            } else {
                tile = item; kbeg = 0; kend = K;
            }
            const int tr = tile / p.tiles_c, tc_ = tile % p.tiles_c;
            const int r0 = tr * RT, c0 = tc_ * CT;
            float *obase = nullptr;
            if (MODE != kFwd)
                obase = reinterpret_cast<float *>(p.out) + (p.direct ? (size_t)0 : (size_t)tr * K * CDIM);

            fetch_chunk(r0, c0, kbeg / KC);
            for (int kc = kbeg; kc < kend; kc += KC) {
                const int stage = ch & 1;
                // row-code stage free (consumers finished the chunk two back), then publish this chunk
                mbar_wait(bar0 + (B_RC_EMPTY + stage) * 8, ((ch >> 1) & 1) ^ 1, 1, abort_word);
                store_chunk(stage);
                mbar_arrive(bar0 + (B_RC_FULL + stage) * 8);
                asm volatile("bar.sync 1, %0;" ::"n"(kProducers) : "memory");  // column codes visible to all producer warps
                if (kc + KC < kend) fetch_chunk(r0, c0, kc / KC + 1);
                const int kcnt = min(KC, kend - kc);
                for (int kk = 0; kk < kcnt; ++kk) {
                    const int b = it & 1;
                    mbar_wait(bar0 + (B_SLAB_EMPTY + b) * 8, ((it >> 1) & 1) ^ 1, 2, abort_word);
                    build(b, stage, kk);
                    mbar_arrive(bar0 + (B_SLAB_FULL + b) * 8);
                    if (MODE != kFwd && kc + kk > kbeg) {
                        const uint32_t jt = it - 1;
                        mbar_wait(bar0 + (B_PART_FULL + (jt & 1)) * 8, (jt >> 1) & 1, 3, abort_word);
                        reduce_store(jt, kc + kk - 1, obase, c0);
                        mbar_arrive(bar0 + (B_PART_EMPTY + (jt & 1)) * 8);
                    }
                    ++it;
                }
                ++ch;
                // No second barrier is needed: the column-code stage written next is the OTHER one, and a
                // warp can only reach the store after that by passing the next chunk's bar.sync, which
                // every producer warp reaches after finishing this chunk's builds.
            }
            if (MODE != kFwd) {
                const uint32_t jt = it - 1;
                mbar_wait(bar0 + (B_PART_FULL + (jt & 1)) * 8, (jt >> 1) & 1, 4, abort_word);
                reduce_store(jt, kend - 1, obase, c0);
                mbar_arrive(bar0 + (B_PART_EMPTY + (jt & 1)) * 8);
            }
        }
    } else {
        // =============================== consumers ======================================================
        const int cw = wp - kProducerWarps;  // 0..15: rows 32cw .. 32cw+31 of the tile
        for (int item = blockIdx.x; item < items; item += gridDim.x) {
            int tile, kbeg, kend;
            if (MODE == kFwd) {
                tile = item / p.ksplits;
                kbeg = (item % p.ksplits) * p.k_per_split;
                kend = min(K, kbeg + p.k_per_split);
            } else {
                tile = item; kbeg = 0; kend = K;
            }
            const int tr = tile / p.tiles_c, tc_ = tile % p.tiles_c;
            const int r0 = tr * RT, c0 = tc_ * CT;

            uint32_t acc[32][2];
            float g[32][2];
            if (MODE == kFwd) {
#pragma unroll
                for (int r = 0; r < 32; ++r) acc[r][0] = acc[r][1] = 0u;
            } else if (MODE == kGw) {
                const int n = c0 + 2 * lane;
#pragma unroll
                for (int r = 0; r < 32; ++r) {
                    const int m = r0 + cw * 32 + r;
                    g[r][0] = g[r][1] = 0.f;
                    if (m < M) {
                        const float *src = p.gc + (size_t)m * N + n;
                        if (p.vec_g) {
                            if (n < N) { const float2 t = *reinterpret_cast<const float2 *>(src); g[r][0] = t.x; g[r][1] = t.y; }
                        } else {
                            if (n < N) g[r][0] = src[0];
                            if (n + 1 < N) g[r][1] = src[1];
                        }
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int m = c0 + 2 * lane + j;
                    const int nb = r0 + cw * 32;
                    const float *src = p.gc + (size_t)min(m, M - 1) * N + nb;
                    if (m < M && p.vec_g && nb + 32 <= N) {
#pragma unroll
                        for (int r = 0; r < 32; r += 4) {
                            const float4 t = *reinterpret_cast<const float4 *>(src + r);
                            g[r][j] = t.x; g[r + 1][j] = t.y; g[r + 2][j] = t.z; g[r + 3][j] = t.w;
                        }
                    } else {
#pragma unroll
                        for (int r = 0; r < 32; ++r) g[r][j] = (m < M && nb + r < N) ? src[r] : 0.f;
                    }
                }
            }

            for (int kc = kbeg; kc < kend; kc += KC) {
                const int stage = ch & 1;
                mbar_wait(bar0 + (B_RC_FULL + stage) * 8, (ch >> 1) & 1, 5, abort_word);
                const int kcnt = min(KC, kend - kc);
                for (int kk = 0; kk < kcnt; ++kk) {
                    const int b = it & 1;
                    const uint4 *rp = reinterpret_cast<const uint4 *>(rc_s + stage * C::RC_STAGE + kk * RT + cw * 32);
                    const uint4 q0 = rp[0], q1 = rp[1];
                    const uint32_t rv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    const uint32_t ub = u_addr + b * C::U_BYTES + lane * 4;
                    mbar_wait(bar0 + (B_SLAB_FULL + b) * 8, (it >> 1) & 1, 6, abort_word);
                    float s0a = 0.f, s0b = 0.f, s1a = 0.f, s1b = 0.f;
#pragma unroll
                    for (int r = 0; r < 32; ++r) {
                        const uint32_t x = byte_of(rv[r >> 2], r & 3);
                        uint32_t word;
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(word) : "r"(ub + x * (US * 4)));
                        if (MODE == kFwd) {
                            acc[r][0] += word;        // sum(lo) + 65536 * sum(hi)  (mod 2^32)
                            acc[r][1] += word >> 16;  // sum(hi)
                        } else {
                            const float f0 = (float)(int16_t)(word & 0xffffu);
                            const float f1 = (float)((int32_t)word >> 16);
                            if (r & 1) { s0b = fmaf(f0, g[r][0], s0b); s1b = fmaf(f1, g[r][1], s1b); }
                            else       { s0a = fmaf(f0, g[r][0], s0a); s1a = fmaf(f1, g[r][1], s1a); }
                        }
                    }
                    mbar_arrive(bar0 + (B_SLAB_EMPTY + b) * 8);
                    if (MODE != kFwd) {
                        mbar_wait(bar0 + (B_PART_EMPTY + b) * 8, ((it >> 1) & 1) ^ 1, 7, abort_word);
                        *reinterpret_cast<float2 *>(part_s + b * (16 * PS) + cw * PS + 2 * lane) =
                            make_float2(s0a + s0b, s1a + s1b);
                        mbar_arrive(bar0 + (B_PART_FULL + b) * 8);
                    }
                    ++it;
                }
                mbar_arrive(bar0 + (B_RC_EMPTY + stage) * 8);
                ++ch;
            }

            if (MODE == kFwd) {
                const int n = c0 + 2 * lane;
#pragma unroll
                for (int r = 0; r < 32; ++r) {
                    acc[r][0] -= acc[r][1] << 16;
                    const int m = r0 + cw * 32 + r;
                    if (m < M) {
                        uint32_t *crow = reinterpret_cast<uint32_t *>(p.out) + (size_t)m * N;
                        if (p.ksplits > 1) {
                            if (n < N) atomicAdd(crow + n, acc[r][0]);
                            if (n + 1 < N) atomicAdd(crow + n + 1, acc[r][1]);
                        } else if (p.vec_o) {
                            if (n < N) *reinterpret_cast<uint2 *>(crow + n) = make_uint2(acc[r][0], acc[r][1]);
                        } else {
                            if (n < N) crow[n] = acc[r][0];
                            if (n + 1 < N) crow[n + 1] = acc[r][1];
                        }
                    }
                }
            }
        }
    }
}

// Self-test of the bounded wait: one warp waits on a barrier that nothing ever arrives on; the wait
// must run out, record id 99 and return.
__global__ void bounded_wait_selftest_kernel() {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        abort_word = 0;
        mbar_init(smem_u32(&bar), 1);
    }
    __syncthreads();
    mbar_wait(smem_u32(&bar), 0, 99, &abort_word);
}

}  // namespace ws

int slab_ws_bounded_wait_selftest(cudaStream_t stream) {
    ws::bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>();
    return cudaGetLastError() == cudaSuccess ? LUTGEMM_OK : LUTGEMM_E_CUDA;
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
template <int BITS>
static int launch_fwd_ws(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                         int num_sms, cudaStream_t stream) {
    using C = ws::Cfg<BITS>;
    auto kern = ws::slab_ws_kernel<BITS, ws::kFwd>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_FWD) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    ws::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.out = c; p.M = M; p.K = K; p.N = N;
    p.tiles_r = (M + C::RT - 1) / C::RT;
    p.tiles_c = (N + C::CT - 1) / C::CT;
    const long tiles = (long)p.tiles_r * p.tiles_c;
    int ksplits = 1;
    double best = -1.0;
    const int kchunks = (K + C::KC - 1) / C::KC;
    for (int s = 1; s <= 16 && s <= kchunks; ++s) {
        const int per = ((kchunks + s - 1) / s) * C::KC;
        if ((K + per - 1) / per != s) continue;
        const long items = tiles * s;
        const long waves = (items + num_sms - 1) / num_sms;
        const double eff = (double)items / (double)(waves * num_sms) * (double)per / (double)(per + 4);
        if (eff > best + 1e-9) { best = eff; ksplits = s; }
    }
    p.ksplits = ksplits;
    p.k_per_split = ((kchunks + ksplits - 1) / ksplits) * C::KC;
    const long items = tiles * ksplits;
    const int grid = (int)(items < num_sms ? items : num_sms);
    if (ksplits > 1 && cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(uint32_t), stream) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    p.vec_a = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_o = (N % 2 == 0) && ((reinterpret_cast<uintptr_t>(c) & 7) == 0);
    kern<<<grid, ws::kThreads, C::SMEM_FWD, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? LUTGEMM_OK : LUTGEMM_E_CUDA;
}

int forward_slab_ws(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K,
                    int N, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_fwd_ws<4>(a, w, c, lut, M, K, N, num_sms, stream);
        case 6: return launch_fwd_ws<6>(a, w, c, lut, M, K, N, num_sms, stream);
        case 7: return launch_fwd_ws<7>(a, w, c, lut, M, K, N, num_sms, stream);
        case 8: return launch_fwd_ws<8>(a, w, c, lut, M, K, N, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

template <int BITS, int MODE>
static int launch_grad_ws(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                          int M, int K, int N, float *scratch, int num_sms, cudaStream_t stream) {
    using C = ws::Cfg<BITS>;
    auto kern = ws::slab_ws_kernel<BITS, MODE>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BWD) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    const int RDIM = MODE == ws::kGa ? N : M, CDIM = MODE == ws::kGa ? M : N;
    ws::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = gc; p.M = M; p.K = K; p.N = N;
    p.tiles_r = (RDIM + C::RT - 1) / C::RT;
    p.tiles_c = (CDIM + C::CT - 1) / C::CT;
    p.direct = p.tiles_r == 1;
    p.out = p.direct ? out : scratch;
    p.ksplits = 1; p.k_per_split = K;
    p.vec_a = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    const long items = (long)p.tiles_r * p.tiles_c;
    const int grid = (int)(items < num_sms ? items : num_sms);
    kern<<<grid, ws::kThreads, C::SMEM_BWD, stream>>>(p);
    if (cudaGetLastError() != cudaSuccess) return LUTGEMM_E_CUDA;
    if (!p.direct) return slab_reduce_blocks(scratch, out, K, CDIM, p.tiles_r, MODE == ws::kGa, 0, num_sms, stream);
    return LUTGEMM_OK;
}

int backward_gw_slab_ws(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                        int bits, int M, int K, int N, float *scratch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_grad_ws<4, ws::kGw>(gc, a, w, gw, lut_gw, M, K, N, scratch, num_sms, stream);
        case 6: return launch_grad_ws<6, ws::kGw>(gc, a, w, gw, lut_gw, M, K, N, scratch, num_sms, stream);
        case 7: return launch_grad_ws<7, ws::kGw>(gc, a, w, gw, lut_gw, M, K, N, scratch, num_sms, stream);
        case 8: return launch_grad_ws<8, ws::kGw>(gc, a, w, gw, lut_gw, M, K, N, scratch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int backward_ga_slab_ws(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                        int bits, int M, int K, int N, float *scratch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_grad_ws<4, ws::kGa>(gc, a, w, ga, lut_ga, M, K, N, scratch, num_sms, stream);
        case 6: return launch_grad_ws<6, ws::kGa>(gc, a, w, ga, lut_ga, M, K, N, scratch, num_sms, stream);
        case 7: return launch_grad_ws<7, ws::kGa>(gc, a, w, ga, lut_ga, M, K, N, scratch, num_sms, stream);
        case 8: return launch_grad_ws<8, ws::kGa>(gc, a, w, ga, lut_ga, M, K, N, scratch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int slab_ws_read_and_clear_error(int *value) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_slab_ws_error, sizeof(int)) != cudaSuccess) return LUTGEMM_E_CUDA;
    if (v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_slab_ws_error, &zero, sizeof(int)) != cudaSuccess) return LUTGEMM_E_CUDA;
    }
    *value = v;
    return LUTGEMM_OK;
}

}  // namespace lutgemm
