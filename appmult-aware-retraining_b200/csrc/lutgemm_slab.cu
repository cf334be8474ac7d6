// "Column-gathered slab" LUT-GEMM kernels for sm_100a: forward, weight gradient and activation gradient.
//
// A warp-wide table gather whose 32 column indices are random costs ~2.8 shared-memory wavefronts at
// 8 bits even when the table row is warp-uniform (a 256-entry uint16 row spans 4 words per bank).
// These kernels take the data-dependent column index out of the hot gather.  With a CTA tile of
// 512 "rows" r and 64 "columns" c, and for each k one row code rc[r,k] and one column code cc[k,c]:
//
//   build (once per k):   U_k[x][c] = TABLE(x, cc[k,c])   for every code x       (a gather by cc)
//   use   (per row r):    row rc[r,k] of U_k, read contiguously over c
//
// The use-phase read is warp-uniform in x and contiguous in c: one 32-bit shared load per lane
// returns two adjacent 16-bit entries (two columns), conflict-free by construction - 64 table
// look-ups per shared-memory wavefront instead of ~11.  The build reads the table transposed and
// paired ([cc][x], codes x and x + 2^b/2 in one word) with conflict-free 32-bit loads and writes slab
// rows (stride 33 words) with conflict-free 32-bit stores: 2^b * 2 wavefronts per k against 512 for
// the use phase.
//
//   mode      rows r   cols c   rc[r,k]   cc[k,c]   per-thread state                      result
//   forward   m        n        a[m,k]    w[k,n]    32x2 int32 accumulators over k        c[m,n]
//   grad_w    m        n        a[m,k]    w[k,n]    32x2 grad_out values gc[m,n]          gw[k,n] = sum_m
//   grad_a    n        m        w[k,n]    a[m,k]    32x2 grad_out values gc[m,n]          ga[m,k] = sum_n
//
// In the two gradient modes every k yields one partial sum per column and warp; the 16 warps are
// combined in a fixed tree through shared memory, and 512-row blocks are combined by a second kernel
// in ascending block order, so results are deterministic run to run.
// Replaces ApproxGemmForwardKernel (self_ops/src/approx_gemm_forward.cu:37-229) and
// ApproxGemmBackwardKernelForGA / ForGB (self_ops/src/approx_gemm_backward.cu:13-258, 261-492).
#include <stdlib.h>

#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

enum { kFwd = 0, kGw = 1, kGa = 2 };

template <int BITS>
struct SlabCfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int HALF = Q / 2;          // words per transposed-table row (two codes per word)
    static constexpr int TT_STRIDE = HALF + 1;  // words; +1 keeps the transposing stage conflict-free
    static constexpr int THREADS = 512;
    static constexpr int RT = 512;              // rows per CTA tile: 32 per warp
    static constexpr int CT = 64;               // columns per CTA tile: 2 per lane
    static constexpr int KC = 16;               // k per operand stage
    static constexpr int U_STRIDE = 33;         // words per slab row (32 + 1 pad)
    static constexpr int P_STRIDE = 66;         // floats per warp row of the partial-sum buffer
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = KC * RT;
    static constexpr int CC_STAGE = KC * CT;
    static constexpr int P_BYTES = 16 * P_STRIDE * 4;
    static constexpr int SMEM_FWD = TT_BYTES + 2 * U_BYTES + 2 * RC_STAGE + 2 * CC_STAGE;
    static constexpr int SMEM_BWD = SMEM_FWD + 2 * P_BYTES;
    static constexpr int NSETS = HALF > 32 ? HALF / 32 : 1;
};

struct SlabArgs {
    const uint8_t *a;     // [M,K]
    const uint8_t *w;     // [K,N]
    const void *lut;      // padded wire-format table (uint16 or int16)
    const float *gc;      // [M,N] (gradient modes)
    void *out;            // forward: c [M,N] u32; gradients: gw/ga or the partial buffer [rblocks][K][C]
    int M, K, N;
    int tiles_r, tiles_c;
    int ksplits, k_per_split;  // forward only
    int direct;                // gradients: 1 = single row block, write the scaled result in place
    int vec_a, vec_w, vec_o, vec_g;
    // constants handed over as run-time values so that the compiler keeps the multiply-add forms that run
    // on the FMA pipe (the integer ALU pipe is the scarcer one in the use phase)
    uint32_t c_row_bytes;  // U_STRIDE * 4
    uint32_t c_64k;        // 65536
    ConvGeom conv;         // enabled: `a` is the image-code tensor x[B,C,H,W] and a[m,k] is gathered on the fly
    int ga_bkl;            // grad_a output layout: 0 = [M][K], 1 = [B][K][Ho*Wo] (what col2im consumes)
};

// ACC (forward): 0 = two dp2a per word; 1 = full-word add plus shifted add, fixed up at the end;
// 2 = as 1 but the slab-row address and the high-half add are integer multiply-adds (FMA pipe).
template <int BITS, int MODE, int ACC>
__global__ void __launch_bounds__(512, 1) slab_kernel(const SlabArgs p) {
    using Cfg = SlabCfg<BITS>;
    constexpr int Q = Cfg::Q, HALF = Cfg::HALF, TTS = Cfg::TT_STRIDE, RT = Cfg::RT, CT = Cfg::CT, KC = Cfg::KC;
    constexpr int US = Cfg::U_STRIDE, PS = Cfg::P_STRIDE, THREADS = Cfg::THREADS, NSETS = Cfg::NSETS;
    constexpr uint32_t MASK4 = (Q - 1) * 0x01010101u;
    constexpr int COL = lut_col_num(BITS);

    const int M = p.M, K = p.K, N = p.N;
    const int RDIM = MODE == kGa ? N : M;  // extent of the row index r
    const int CDIM = MODE == kGa ? M : N;  // extent of the column index c

    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tt_s = reinterpret_cast<uint32_t *>(smem);
    uint32_t *u_s = reinterpret_cast<uint32_t *>(smem + Cfg::TT_BYTES);
    uint8_t *rc_s = smem + Cfg::TT_BYTES + 2 * Cfg::U_BYTES;
    uint8_t *cc_s = rc_s + 2 * Cfg::RC_STAGE;
    float *part_s = reinterpret_cast<float *>(cc_s + 2 * Cfg::CC_STAGE);

    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;

    // ---- stage the table transposed and paired: tt[y][i] = { T(i, y), T(i + HALF, y) } where x is the
    //      row code and y the column code; T(x, y) = lut[a*COL + w] with (a, w) = (x, y) or (y, x) -------
    {
        const uint16_t *lut = reinterpret_cast<const uint16_t *>(p.lut);
        uint16_t *tt16 = reinterpret_cast<uint16_t *>(tt_s);
        for (int idx = tid; idx < Q * Q; idx += THREADS) {
            const int hi_idx = idx >> BITS, lo_idx = idx & (Q - 1);  // global read is contiguous in lo_idx
            uint16_t v = lut[hi_idx * COL + lo_idx];
            if (MODE != kFwd && ACC == 1) v ^= 0x8000u;  // offset-binary: u = v + 32768 for the magic-number conversion
            const int x = MODE == kGa ? lo_idx : hi_idx, y = MODE == kGa ? hi_idx : lo_idx;
            tt16[(y * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] = v;
        }
    }
    const uint32_t tt_addr = smem_u32(tt_s);
    const uint32_t u_addr = smem_u32(u_s);

    // position of grad_a element (m, k) in the output: [M][K], or [B][K][L] with m = b*L + l
    auto ga_index = [&](int m, int k) -> size_t {
        if (!p.ga_bkl) return (size_t)m * K + k;
        const int L = p.conv.Ho * p.conv.Wo, b = m / L;
        return ((size_t)b * K + k) * L + (m - b * L);
    };

    // ---- operand chunk staging: rc_s[stage][kk][r] (512 row codes per k), cc_s[stage][kk][c] (64) ----
    uint4 prc = make_uint4(0, 0, 0, 0), pcc = make_uint4(0, 0, 0, 0);

    auto fetch_chunk = [&](int r0, int c0, int chunk) {
        const int kbase = chunk * KC;
        if (MODE != kGa) {
            // row codes a[r][kbase..+15]: one row per thread, transposed when stored
            const uint8_t *src = p.a + (size_t)min(r0 + tid, M - 1) * K + kbase;
            if (p.conv.enabled) {
                prc = conv_code16(p.a, p.conv, min(r0 + tid, M - 1), kbase, K);
            } else if (p.vec_a) {
                prc = kbase < K ? *reinterpret_cast<const uint4 *>(src) : make_uint4(0, 0, 0, 0);
            } else {
                uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (kbase + j < K) t[j >> 2] |= (uint32_t)src[j] << (8 * (j & 3));
                prc = make_uint4(t[0], t[1], t[2], t[3]);
            }
            // column codes w[kbase+kk][c0..c0+63]
            if (tid < KC * CT / 16) {
                const int kk = tid / (CT / 16), cc = (tid % (CT / 16)) * 16;
                const int gk = kbase + kk, gn = c0 + cc;
                if (p.vec_w) {
                    pcc = (gk < K && gn < N) ? *reinterpret_cast<const uint4 *>(p.w + (size_t)gk * N + gn)
                                              : make_uint4(0, 0, 0, 0);
                } else {
                    uint32_t t[4] = {0, 0, 0, 0};
                    if (gk < K) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (gn + j < N) t[j >> 2] |= (uint32_t)p.w[(size_t)gk * N + gn + j] << (8 * (j & 3));
                    }
                    pcc = make_uint4(t[0], t[1], t[2], t[3]);
                }
            }
        } else {
            // row codes w[kbase+kk][r0..r0+511]: thread t takes k-row t/32 and 16 consecutive r
            {
                const int kk = tid / (RT / 16), rr = (tid % (RT / 16)) * 16;
                const int gk = kbase + kk, gn = r0 + rr;
                if (p.vec_w) {
                    prc = (gk < K && gn < N) ? *reinterpret_cast<const uint4 *>(p.w + (size_t)gk * N + gn)
                                              : make_uint4(0, 0, 0, 0);
                } else {
                    uint32_t t[4] = {0, 0, 0, 0};
                    if (gk < K) {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (gn + j < N) t[j >> 2] |= (uint32_t)p.w[(size_t)gk * N + gn + j] << (8 * (j & 3));
                    }
                    prc = make_uint4(t[0], t[1], t[2], t[3]);
                }
            }
            // column codes a[c0+c][kbase..+15]: one m-row per thread (64 threads), transposed when stored
            if (tid < CT) {
                const uint8_t *src = p.a + (size_t)min(c0 + tid, M - 1) * K + kbase;
                if (p.conv.enabled) {
                    pcc = conv_code16(p.a, p.conv, min(c0 + tid, M - 1), kbase, K);
                } else if (p.vec_a) {
                    pcc = kbase < K ? *reinterpret_cast<const uint4 *>(src) : make_uint4(0, 0, 0, 0);
                } else {
                    uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (kbase + j < K) t[j >> 2] |= (uint32_t)src[j] << (8 * (j & 3));
                    pcc = make_uint4(t[0], t[1], t[2], t[3]);
                }
            }
        }
    };
    auto store_chunk = [&](int stage) {
        uint8_t *rs = rc_s + stage * Cfg::RC_STAGE;
        uint8_t *cs = cc_s + stage * Cfg::CC_STAGE;
        // codes are masked to BITS bits here, once, so no stray code can index outside a slab or table
        const uint32_t tr[4] = {prc.x & MASK4, prc.y & MASK4, prc.z & MASK4, prc.w & MASK4};
        const uint32_t tc[4] = {pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4};
        if (MODE != kGa) {
#pragma unroll
            for (int j = 0; j < 16; ++j) rs[j * RT + tid] = (uint8_t)(tr[j >> 2] >> (8 * (j & 3)));
            if (tid < KC * CT / 16) {
                const int kk = tid / (CT / 16), cc = (tid % (CT / 16)) * 16;
                *reinterpret_cast<uint4 *>(cs + kk * CT + cc) = make_uint4(tc[0], tc[1], tc[2], tc[3]);
            }
        } else {
            const int kk = tid / (RT / 16), rr = (tid % (RT / 16)) * 16;
            *reinterpret_cast<uint4 *>(rs + kk * RT + rr) = make_uint4(tr[0], tr[1], tr[2], tr[3]);
            if (tid < CT) {
#pragma unroll
                for (int j = 0; j < 16; ++j) cs[j * CT + tid] = (uint8_t)(tc[j >> 2] >> (8 * (j & 3)));
            }
        }
    };
    // build slab `buf` for the k that sits at (stage, kk): warp wp fills column pairs 2wp and 2wp+1
    auto build = [&](int buf, int stage, int kk) {
        const uint32_t cw = *reinterpret_cast<const uint32_t *>(cc_s + stage * Cfg::CC_STAGE + kk * CT + wp * 4);
        const uint32_t ub = u_addr + buf * Cfg::U_BYTES;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
            const uint32_t y0 = byte_of(cw, 2 * pp), y1 = byte_of(cw, 2 * pp + 1);
            const int pc = 2 * wp + pp;
#pragma unroll
            for (int j = 0; j < NSETS; ++j) {
                const int i = lane + 32 * j;
                if (HALF >= 32 || i < HALF) {
                    const uint32_t r0 = lds_u32(tt_addr + (y0 * TTS + i) * 4);
                    const uint32_t r1 = lds_u32(tt_addr + (y1 * TTS + i) * 4);
                    const uint32_t lo = __byte_perm(r0, r1, 0x5410);  // { T(i, y0), T(i, y1) }
                    const uint32_t hi = __byte_perm(r0, r1, 0x7632);  // { T(i+HALF, y0), T(i+HALF, y1) }
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + (i * US + pc) * 4), "r"(lo) : "memory");
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + ((i + HALF) * US + pc) * 4), "r"(hi) : "memory");
                }
            }
        }
    };

    const int items = MODE == kFwd ? p.tiles_r * p.tiles_c * p.ksplits : p.tiles_r * p.tiles_c;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        int tile, kbeg, kend;
        if (MODE == kFwd) {
            // work item = (output tile, K split); splits of one tile are combined with integer atomics,
            // which are exact in any order, so the result stays bit-identical
            tile = item / p.ksplits;
            kbeg = (item % p.ksplits) * p.k_per_split;
            kend = min(K, kbeg + p.k_per_split);
        } else {
            tile = item; kbeg = 0; kend = K;
        }
        const int tr = tile / p.tiles_c, tc = tile % p.tiles_c;
        const int r0 = tr * RT, c0 = tc * CT;

        // per-thread state: integer accumulators (forward) or the grad_out block (gradients)
        uint32_t acc[32][2];
        float g[32][2];
        if (MODE == kFwd) {
#pragma unroll
            for (int r = 0; r < 32; ++r) acc[r][0] = acc[r][1] = 0u;
        } else if (MODE == kGw) {
            const int n = c0 + 2 * lane;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const int m = r0 + wp * 32 + r;
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
            // g[r][j] = gc[m = c0 + 2*lane + j][n = r0 + 32*wp + r]
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int m = c0 + 2 * lane + j;
                const int nb = r0 + wp * 32;
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

        fetch_chunk(r0, c0, kbeg / KC);
        __syncthreads();  // previous item (or the table staging) is done with every buffer
        store_chunk((kbeg / KC) & 1);
        __syncthreads();
        build(kbeg & 1, (kbeg / KC) & 1, 0);
        __syncthreads();

        float *obase = nullptr;  // gradients: where row k of this item's 64 columns goes
        if (MODE != kFwd)
            obase = reinterpret_cast<float *>(p.out) + (p.direct ? (size_t)0 : (size_t)tr * K * CDIM);

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / KC, kk = k % KC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * KC < kend;
            if (kk == 0 && have_next_chunk) fetch_chunk(r0, c0, chunk + 1);
            if (k + 1 < kend) build((k + 1) & 1, ((k + 1) / KC) & 1, (k + 1) % KC);

            if (MODE != kFwd && k > kbeg) {
                // combine the 16 warps' partial sums of k-1 (fixed tree): warp wp owns columns 4wp..4wp+3,
                // lane = 4*grp + col; grp adds warps 2grp and 2grp+1, the 8 groups meet by shuffles
                const float *ps = part_s + ((k - 1) & 1) * (16 * PS);
                const int col = 4 * wp + (lane & 3), grp = lane >> 2;
                float v = ps[(2 * grp) * PS + col] + ps[(2 * grp + 1) * PS + col];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (lane < 4 && c0 + col < CDIM) {
                    if (p.direct && MODE == kGa) obase[ga_index(c0 + col, k - 1)] = v * kGradFactor;
                    else obase[(size_t)(k - 1) * CDIM + c0 + col] = p.direct ? v * kGradFactor : v;
                }
            }

            // use slab k: slab row rc[r,k], two columns per lane, for this warp's 32 rows
            const uint4 *rp = reinterpret_cast<const uint4 *>(rc_s + stage * Cfg::RC_STAGE + kk * RT + wp * 32);
            const uint4 q0 = rp[0], q1 = rp[1];
            const uint32_t rv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
            const uint32_t ub = u_addr + (k & 1) * Cfg::U_BYTES + lane * 4;
            float s0a = 0.f, s0b = 0.f, s1a = 0.f, s1b = 0.f;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                uint32_t x, addr, word;
                if constexpr (ACC == 2) {
                    x = __byte_perm(rv[r >> 2], 0u, 0x4440u + (r & 3));
                    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(addr) : "r"(x), "r"(p.c_row_bytes), "r"(ub));
                } else {
                    x = byte_of(rv[r >> 2], r & 3);
                    addr = ub + x * (US * 4);
                }
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(word) : "r"(addr));
                if (MODE == kFwd) {
                    if constexpr (ACC == 0) {
                        acc[r][0] = __dp2a_lo(word, 0x00000001u, acc[r][0]);
                        acc[r][1] = __dp2a_lo(word, 0x00000100u, acc[r][1]);
                    } else if constexpr (ACC == 1) {
                        acc[r][0] += word;
                        acc[r][1] += word >> 16;
                    } else if constexpr (ACC == 3) {
                        acc[r][0] += word;
                        acc[r][1] = __dp2a_lo(word, 0x00000100u, acc[r][1]);
                    } else {
                        acc[r][0] += word;
                        asm("mad.hi.u32 %0, %1, %2, %0;" : "+r"(acc[r][1]) : "r"(word), "r"(p.c_64k));
                    }
                } else {
                    float f0, f1;
                    if constexpr (ACC == 1) {
                        // 0x4B000000 | u is the float 2^23 + u; subtracting 2^23 + 32768 leaves the signed
                        // entry exactly.  One logic op + one FADD per value instead of a conversion on
                        // the (16 lanes/clk) XU pipe.
                        f0 = __uint_as_float((word & 0xffffu) | 0x4B000000u) - 8421376.0f;
                        f1 = __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7632)) - 8421376.0f;
                    } else {
                        f0 = (float)(int16_t)(word & 0xffffu);
                        f1 = (float)((int32_t)word >> 16);
                    }
                    if (r & 1) { s0b = fmaf(f0, g[r][0], s0b); s1b = fmaf(f1, g[r][1], s1b); }
                    else       { s0a = fmaf(f0, g[r][0], s0a); s1a = fmaf(f1, g[r][1], s1a); }
                }
            }
            if (MODE != kFwd)
                *reinterpret_cast<float2 *>(part_s + (k & 1) * (16 * PS) + wp * PS + 2 * lane) =
                    make_float2(s0a + s0b, s1a + s1b);
            if (kk == KC - 2 && have_next_chunk) store_chunk(stage ^ 1);
            __syncthreads();
        }

        if (MODE == kFwd) {
            const int n = c0 + 2 * lane;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                if constexpr (ACC != 0) acc[r][0] -= acc[r][1] << 16;  // low sum = full-word sum - 65536 * high sum
                const int m = r0 + wp * 32 + r;
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
        } else {
            // flush the last k
            const int k = kend - 1;
            const float *ps = part_s + (k & 1) * (16 * PS);
            const int col = 4 * wp + (lane & 3), grp = lane >> 2;
            float v = ps[(2 * grp) * PS + col] + ps[(2 * grp + 1) * PS + col];
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            if (lane < 4 && c0 + col < CDIM) {
                if (p.direct && MODE == kGa) obase[ga_index(c0 + col, k)] = v * kGradFactor;
                else obase[(size_t)k * CDIM + c0 + col] = p.direct ? v * kGradFactor : v;
            }
        }
    }
}

// out[k][c] (TRANSPOSE=false) or out[c][k] (TRANSPOSE=true) = scale * sum_b part[b][k][c], b ascending.
// With bkl_L > 0 (and TRANSPOSE=false) column c = b*L + l goes to out[(b*K + k)*L + l] instead.
template <bool TRANSPOSE>
__global__ void slab_reduce_blocks_kernel(const float *__restrict__ part, float *__restrict__ out, int K, int C,
                                          int nblocks, float scale, int bkl_L) {
    __shared__ float tile[32][33];
    const int tiles_c = (C + 31) / 32, tiles_k = (K + 31) / 32;
    const size_t KC_ = (size_t)K * C;
    for (int t = blockIdx.x; t < tiles_c * tiles_k; t += gridDim.x) {
        const int k0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + ty + 8 * j, c = c0 + tx;
            float s = 0.f;
            if (k < K && c < C)
                for (int b = 0; b < nblocks; ++b) s += part[(size_t)b * KC_ + (size_t)k * C + c];
            if (TRANSPOSE) tile[ty + 8 * j][tx] = s * scale;
            else if (k < K && c < C) {
                if (bkl_L > 0) out[((size_t)(c / bkl_L) * K + k) * bkl_L + c % bkl_L] = s * scale;
                else out[(size_t)k * C + c] = s * scale;
            }
        }
        if (TRANSPOSE) {
            __syncthreads();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = c0 + ty + 8 * j, k = k0 + tx;
                if (k < K && c < C) out[(size_t)c * K + k] = tile[tx][ty + 8 * j];
            }
            __syncthreads();
        }
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static int env_int(const char *name, int dflt) {
    const char *e = getenv(name);
    return e ? atoi(e) : dflt;
}

template <int BITS, int ACC>
static int launch_fwd_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                           const ConvGeom &conv, int num_sms, cudaStream_t stream) {
    using Cfg = SlabCfg<BITS>;
    auto kern = slab_kernel<BITS, kFwd, ACC>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_FWD) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    SlabArgs p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = nullptr; p.out = c; p.M = M; p.K = K; p.N = N;
    p.conv = conv;
    p.tiles_r = (M + Cfg::RT - 1) / Cfg::RT;
    p.tiles_c = (N + Cfg::CT - 1) / Cfg::CT;
    const long tiles = (long)p.tiles_r * p.tiles_c;
    // pick the K split that best fills the last wave of the persistent grid
    int ksplits = 1;
    double best = -1.0;
    const int kchunks = (K + Cfg::KC - 1) / Cfg::KC;
    for (int s = 1; s <= 16 && s <= kchunks; ++s) {
        const int per = ((kchunks + s - 1) / s) * Cfg::KC;
        if ((K + per - 1) / per != s) continue;  // some split would get no work
        const long items = tiles * s;
        const long waves = (items + num_sms - 1) / num_sms;
        const double eff = (double)items / (double)(waves * num_sms) * (double)per / (double)(per + 6);
        if (eff > best + 1e-9) { best = eff; ksplits = s; }
    }
    p.ksplits = ksplits;
    p.k_per_split = ((kchunks + ksplits - 1) / ksplits) * Cfg::KC;
    const long items = tiles * ksplits;
    const int grid = (int)(items < num_sms ? items : num_sms);
    if (ksplits > 1 && cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(uint32_t), stream) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    p.vec_a = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_o = (N % 2 == 0) && ((reinterpret_cast<uintptr_t>(c) & 7) == 0);
    p.c_row_bytes = Cfg::U_STRIDE * 4;
    p.c_64k = 65536u;
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_FWD, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? LUTGEMM_OK : LUTGEMM_E_CUDA;
}

int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 const ConvGeom &conv, int num_sms, cudaStream_t stream) {
    const int acc = env_int("LUTGEMM_SLAB_ACC", 1);  // 1 measured fastest on B200 (0: +6 %, 2: +45 % time)
#define LUTGEMM_CASE(B)                                                                         \
    case B:                                                                                     \
        if (acc == 0) return launch_fwd_slab<B, 0>(a, w, c, lut, M, K, N, conv, num_sms, stream);     \
        if (acc == 2) return launch_fwd_slab<B, 2>(a, w, c, lut, M, K, N, conv, num_sms, stream);     \
        if (acc == 3) return launch_fwd_slab<B, 3>(a, w, c, lut, M, K, N, conv, num_sms, stream);     \
        return launch_fwd_slab<B, 1>(a, w, c, lut, M, K, N, conv, num_sms, stream);
    switch (bits) {
        LUTGEMM_CASE(4)
        LUTGEMM_CASE(6)
        LUTGEMM_CASE(7)
        LUTGEMM_CASE(8)
    }
#undef LUTGEMM_CASE
    return LUTGEMM_E_BITS;
}

int slab_reduce_blocks(const float *part, float *out, int K, int C, int nblocks, bool transpose, int bkl_L,
                       int num_sms, cudaStream_t stream) {
    const long tiles = (long)((K + 31) / 32) * ((C + 31) / 32);
    const int rgrid = (int)(tiles < 8L * num_sms ? tiles : 8L * num_sms);
    if (transpose && bkl_L == 0)
        slab_reduce_blocks_kernel<true><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, kGradFactor, 0);
    else
        slab_reduce_blocks_kernel<false><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, kGradFactor, bkl_L);
    return cudaGetLastError() == cudaSuccess ? LUTGEMM_OK : LUTGEMM_E_CUDA;
}

// number of 512-row blocks of the reduction dimension (M for grad_w, N for grad_a)
int slab_grad_row_blocks(int rdim) { return (rdim + 511) / 512; }

template <int BITS, int MODE>
static int launch_grad_slab(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                            int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms,
                            cudaStream_t stream) {
    using Cfg = SlabCfg<BITS>;
    auto kern = env_int("LUTGEMM_SLAB_CVT", 1) == 0 ? slab_kernel<BITS, MODE, 0> : slab_kernel<BITS, MODE, 1>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BWD) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    const int RDIM = MODE == kGa ? N : M, CDIM = MODE == kGa ? M : N;
    SlabArgs p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = gc; p.M = M; p.K = K; p.N = N;
    p.conv = conv;
    p.ga_bkl = (MODE == kGa && conv.enabled) ? 1 : 0;
    p.tiles_r = (RDIM + Cfg::RT - 1) / Cfg::RT;
    p.tiles_c = (CDIM + Cfg::CT - 1) / Cfg::CT;
    p.direct = p.tiles_r == 1;
    p.out = p.direct ? out : scratch;
    p.ksplits = 1; p.k_per_split = K;
    p.vec_a = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    p.c_row_bytes = Cfg::U_STRIDE * 4;
    p.c_64k = 65536u;
    const long items = (long)p.tiles_r * p.tiles_c;
    const int grid = (int)(items < num_sms ? items : num_sms);
    kern<<<grid, Cfg::THREADS, Cfg::SMEM_BWD, stream>>>(p);
    if (cudaGetLastError() != cudaSuccess) return LUTGEMM_E_CUDA;
    if (!p.direct)
        return slab_reduce_blocks(scratch, out, K, CDIM, p.tiles_r, MODE == kGa, p.ga_bkl ? conv.Ho * conv.Wo : 0,
                                  num_sms, stream);
    return LUTGEMM_OK;
}

int backward_gw_slab(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw, int bits,
                     int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_grad_slab<4, kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_sms, stream);
        case 6: return launch_grad_slab<6, kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_sms, stream);
        case 7: return launch_grad_slab<7, kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_sms, stream);
        case 8: return launch_grad_slab<8, kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int backward_ga_slab(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga, int bits,
                     int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_grad_slab<4, kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, num_sms, stream);
        case 6: return launch_grad_slab<6, kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, num_sms, stream);
        case 7: return launch_grad_slab<7, kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, num_sms, stream);
        case 8: return launch_grad_slab<8, kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
