// Gradient LUT-GEMM kernels for sm_100a with an fp32 "column-gathered slab" (grad_w and grad_a).
//
//   grad_w:  gw[k,n] = 1/16 * sum_m T(a[m,k], w[k,n]) * gc[m,n]     rows r = m, columns c = n
//   grad_a:  ga[m,k] = 1/16 * sum_n gc[m,n] * T(a[m,k], w[k,n])     rows r = n, columns c = m
//
// As in the forward slab kernel, for every k the CTA first gathers a slab U_k[x][c] = T(x, cc[k,c]) for
// all 2^b row codes x and its 64 columns c, and each of its 512 rows then reads slab row rc[r,k]
// contiguously.  Here the slab holds fp32 values, converted ONCE per slab entry while it is built:
// the use phase is then  "extract code, form address, one 64-bit shared load, two FMAs"  per row and
// lane pair of columns - 5 instructions per 64 table look-ups, with no int16->fp32 conversion (the XU
// pipe converts only 16 lanes/clk) and no unpacking in the hot loop.  The grad_out block of the tile
// (32 rows x 2 columns per thread) stays in registers for the whole k loop.
//
// Shared memory: the gradient table (fp32 [cc][x] for b <= 7, 66 KB at 7 bits; int16 pairs at 8 bits,
// 129 KB, converted with the magic-number trick during the build), the slab(s) (2^b rows x 264 B; two
// buffers for b <= 7, one at 8 bits where two do not fit), operand code stages and the per-warp partial
// sums.  Every k yields one partial sum per column and warp; the 16 warps are combined in a fixed
// tree, 512-row blocks by slab_reduce_blocks in ascending order: results are deterministic.
// Replaces ApproxGemmBackwardKernelForGA / ForGB, self_ops/src/approx_gemm_backward.cu:13-258, 261-492.
#include <stdlib.h>

#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {
namespace sg {

enum { kGw = 1, kGa = 2 };

template <int BITS, int WARPS, int RW_>
struct Cfg {
    static constexpr int Q = 1 << BITS;
    static constexpr bool F32_TABLE = BITS <= 7;
    static constexpr int HALF = Q / 2;
    static constexpr int TT_STRIDE = F32_TABLE ? Q + 1 : HALF + 1;  // words per table row
    static constexpr int THREADS = 32 * WARPS, RT = WARPS * RW_, CT = 64, KC = 16;
    static constexpr int RW = RW_;               // rows per warp (a multiple of 8)
    static constexpr int PPW = 32 / WARPS;       // slab column pairs built per warp
    static constexpr int CPW = CT / WARPS;       // columns whose partial sums a warp combines
    static constexpr int U_STRIDE = 66;  // words per slab row: 64 floats + 2 (conflict-free 64-bit stores)
    static constexpr int P_STRIDE = 66;
    static constexpr int NBUF = BITS == 8 ? 1 : 2;   // slab buffers (and partial-sum buffers)
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = KC * RT, CC_STAGE = KC * CT;
    static constexpr int P_BYTES = WARPS * P_STRIDE * 4;
    static constexpr int OFF_U = TT_BYTES;
    static constexpr int OFF_RC = OFF_U + NBUF * U_BYTES;
    static constexpr int OFF_CC = OFF_RC + 2 * RC_STAGE;
    static constexpr int OFF_PART = OFF_CC + 2 * CC_STAGE;
    static constexpr int SMEM = OFF_PART + NBUF * P_BYTES;
};

struct Args {
    const uint8_t *a;
    const uint8_t *w;
    const int16_t *lut;
    const float *gc;
    float *out;
    int M, K, N;
    int tiles_r, tiles_c;
    int ksplits, k_per_split;  // a tile's k range is cut into independent work items (outputs are per k)
    int direct;
    int vec_a, vec_w, vec_g;
    ConvGeom conv;
    int ga_scatter;  // grad_a of a convolution: results go straight to the image gradient
    const uint8_t *at;  // grad_w only, optional: transposed row codes at[k][m], rows at_pitch bytes apart
    int at_pitch;       // a multiple of 16; columns m >= M hold 0
};

// PF = how many slab-row loads are kept in flight ahead of the FMAs that consume them.  Without explicit
// prefetch the compiler, short of registers, emits load -> use -> load -> use, and a warp's k iteration
// costs RW shared-memory latencies back to back.
template <int BITS, int MODE, int WARPS, int RW_, int PF>
__global__ void __launch_bounds__(32 * WARPS, 1) slab_grad_kernel(const Args p) {
    using C = Cfg<BITS, WARPS, RW_>;
    constexpr int RW = C::RW, PPW = C::PPW, CPW = C::CPW;
    constexpr int Q = C::Q, HALF = C::HALF, TTS = C::TT_STRIDE, RT = C::RT, CT = C::CT, KC = C::KC;
    constexpr int US = C::U_STRIDE, PS = C::P_STRIDE, THREADS = C::THREADS, NBUF = C::NBUF;
    constexpr uint32_t MASK4 = (Q - 1) * 0x01010101u;
    constexpr int COL = lut_col_num(BITS);

    const int M = p.M, K = p.K, N = p.N;
    const int CDIM = MODE == kGa ? M : N;

    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t *rc_s = smem + C::OFF_RC;
    uint8_t *cc_s = smem + C::OFF_CC;
    float *part_s = reinterpret_cast<float *>(smem + C::OFF_PART);
    const uint32_t tt_addr = smem_u32(smem);
    const uint32_t u_addr = smem_u32(smem + C::OFF_U);
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;

    // ---- stage the gradient table; x = row code, y = column code, T(x,y) = lut[a*COL + w] ----------------
#pragma unroll 8
    for (int idx = tid; idx < Q * Q; idx += THREADS) {
        const int hi_idx = idx >> BITS, lo_idx = idx & (Q - 1);  // global read contiguous in lo_idx
        const int16_t v = p.lut[hi_idx * COL + lo_idx];
        const int x = MODE == kGa ? lo_idx : hi_idx, y = MODE == kGa ? hi_idx : lo_idx;
        if (C::F32_TABLE) {
            reinterpret_cast<float *>(smem)[y * TTS + x] = (float)v;
        } else {
            // int16 pairs {T(i,y), T(i+HALF,y)} in offset-binary (v + 32768) for the magic-number conversion
            reinterpret_cast<uint16_t *>(smem)[(y * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] =
                (uint16_t)v ^ (uint16_t)0x8000u;
        }
    }

    // grad_a of a convolution (non-overlapping windows) goes straight to its place in the image gradient
    auto ga_index = [&](int m, int k) -> long {
        if (!p.ga_scatter) return (long)m * K + k;
        return conv_scatter_index(p.conv, m, k);
    };

    // ---- operand chunk staging: rc_s[stage][kk][r] (512 row codes per k), cc_s[stage][kk][c] (64) ------
    uint4 prc = make_uint4(0, 0, 0, 0), pcc = make_uint4(0, 0, 0, 0);
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
    auto fetch_chunk = [&](int r0, int c0, int chunk) {
        const int kbase = chunk * KC;
        if (tid >= RT) return;
        if (MODE == kGw && p.at) {
            // row codes from the transposed copy at[k][m]: 16 rows per load, coalesced like the w operand
            const int gk = kbase + tid / (RT / 16), gm = r0 + (tid % (RT / 16)) * 16;
            prc = (gk < K && gm < p.at_pitch) ? *reinterpret_cast<const uint4 *>(p.at + (size_t)gk * p.at_pitch + gm)
                                              : make_uint4(0, 0, 0, 0);
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else if (MODE == kGw) {
            prc = a_codes16(r0 + tid, kbase);
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else {
            prc = w_codes16(kbase + tid / (RT / 16), r0 + (tid % (RT / 16)) * 16);
            if (tid < CT) pcc = a_codes16(c0 + tid, kbase);
        }
    };
    auto store_chunk = [&](int stage) {
        if (tid >= RT) return;
        uint8_t *rs = rc_s + stage * C::RC_STAGE;
        uint8_t *cs = cc_s + stage * C::CC_STAGE;
        const uint32_t tr[4] = {prc.x & MASK4, prc.y & MASK4, prc.z & MASK4, prc.w & MASK4};
        const uint32_t tc[4] = {pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4};
        if (MODE == kGw && p.at) {
            *reinterpret_cast<uint4 *>(rs + (tid / (RT / 16)) * RT + (tid % (RT / 16)) * 16) =
                make_uint4(tr[0], tr[1], tr[2], tr[3]);
            if (tid < KC * CT / 16)
                *reinterpret_cast<uint4 *>(cs + (tid / (CT / 16)) * CT + (tid % (CT / 16)) * 16) =
                    make_uint4(tc[0], tc[1], tc[2], tc[3]);
        } else if (MODE == kGw) {
#pragma unroll
            for (int q = 0; q < 16; ++q) rs[q * RT + tid] = (uint8_t)(tr[q >> 2] >> (8 * (q & 3)));
            if (tid < KC * CT / 16)
                *reinterpret_cast<uint4 *>(cs + (tid / (CT / 16)) * CT + (tid % (CT / 16)) * 16) =
                    make_uint4(tc[0], tc[1], tc[2], tc[3]);
        } else {
            *reinterpret_cast<uint4 *>(rs + (tid / (RT / 16)) * RT + (tid % (RT / 16)) * 16) =
                make_uint4(tr[0], tr[1], tr[2], tr[3]);
            if (tid < CT) {
#pragma unroll
                for (int q = 0; q < 16; ++q) cs[q * CT + tid] = (uint8_t)(tc[q >> 2] >> (8 * (q & 3)));
            }
        }
    };
    // build slab `buf` for the k at (stage, kk): warp wp fills PPW 64-bit column pairs (columns 2*PPW*wp ...).
    // Lanes run over x, so the table reads are contiguous and the 64-bit slab stores (row stride 66 words)
    // fall on distinct bank pairs within each half-warp.
    auto build = [&](int buf, int stage, int kk) {
        const uint8_t *cp = cc_s + stage * C::CC_STAGE + kk * CT + wp * (2 * PPW);
        const uint32_t cw = PPW == 2 ? *reinterpret_cast<const uint32_t *>(cp) : *reinterpret_cast<const uint16_t *>(cp);
        const uint32_t ub = u_addr + buf * C::U_BYTES;
#pragma unroll
        for (int pp = 0; pp < PPW; ++pp) {
            const uint32_t y0 = byte_of(cw, 2 * pp), y1 = byte_of(cw, 2 * pp + 1);
            const uint32_t col_off = (2 * PPW * wp + 2 * pp) * 4;
            if constexpr (C::F32_TABLE) {
#pragma unroll
                for (int j = 0; j < (Q + 31) / 32; ++j) {
                    const int x = lane + 32 * j;
                    if (Q >= 32 || x < Q) {
                        const uint32_t r0 = lds_u32(tt_addr + (y0 * TTS + x) * 4);
                        const uint32_t r1 = lds_u32(tt_addr + (y1 * TTS + x) * 4);
                        asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ub + x * (US * 4) + col_off), "r"(r0), "r"(r1)
                                     : "memory");
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < HALF / 32; ++j) {
                    const int i = lane + 32 * j;
                    const uint32_t r0 = lds_u32(tt_addr + (y0 * TTS + i) * 4);
                    const uint32_t r1 = lds_u32(tt_addr + (y1 * TTS + i) * 4);
                    // 0x4B000000 | u is the float 2^23 + u; minus (2^23 + 32768) leaves the signed entry exactly
                    const float f00 = __uint_as_float((r0 & 0xffffu) | 0x4B000000u) - 8421376.0f;
                    const float f01 = __uint_as_float((r1 & 0xffffu) | 0x4B000000u) - 8421376.0f;
                    const float f10 = __uint_as_float(__byte_perm(r0, 0x4B000000u, 0x7632)) - 8421376.0f;
                    const float f11 = __uint_as_float(__byte_perm(r1, 0x4B000000u, 0x7632)) - 8421376.0f;
                    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + i * (US * 4) + col_off), "f"(f00), "f"(f01)
                                 : "memory");
                    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + (i + HALF) * (US * 4) + col_off), "f"(f10),
                                 "f"(f11)
                                 : "memory");
                }
            }
        }
    };
    // combine the warps' partial sums of one k (fixed tree): warp wp owns CPW columns, lane = CPW*grp + col;
    // grp adds warps 2grp and 2grp+1, the groups meet by shuffles; then store the columns
    auto reduce_store = [&](int k, float *obase, int c0) {
        const float *ps = part_s + (NBUF == 2 ? (k & 1) : 0) * (WARPS * PS);
        const int col = CPW * wp + (lane & (CPW - 1)), grp = lane / CPW;
        float v = ps[(2 * grp) * PS + col] + ps[(2 * grp + 1) * PS + col];
#pragma unroll
        for (int d = CPW; d < 32; d *= 2) v += __shfl_xor_sync(0xffffffffu, v, d);
        if (lane < CPW && c0 + col < CDIM) {
            if (p.direct && MODE == kGa) {
                const long o = ga_index(c0 + col, k);
                if (o >= 0) obase[o] = v * kGradFactor;
            } else {
                obase[(size_t)k * CDIM + c0 + col] = p.direct ? v * kGradFactor : v;
            }
        }
    };

    const int items = p.tiles_r * p.tiles_c * p.ksplits;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int tile = item / p.ksplits;
        const int kbeg = (item % p.ksplits) * p.k_per_split, kend = min(K, kbeg + p.k_per_split);
        const int tr = tile / p.tiles_c, tc = tile % p.tiles_c;
        const int r0 = tr * RT, c0 = tc * CT;

        // the grad_out block of this tile: g[r][j] for the warp's RW rows and the lane's 2 columns
        float g[RW][2];
        if (MODE == kGw) {
            const int n = c0 + 2 * lane;
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int m = r0 + wp * RW + r;
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
            // g[r][j] = gc[m = c0 + 2*lane + j][n = r0 + RW*wp + r]
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int m = c0 + 2 * lane + j;
                const int nb = r0 + wp * RW;
                const float *src = p.gc + (size_t)min(m, M - 1) * N + nb;
                if (m < M && p.vec_g && nb + RW <= N) {
#pragma unroll
                    for (int r = 0; r < RW; r += 4) {
                        const float4 t = *reinterpret_cast<const float4 *>(src + r);
                        g[r][j] = t.x; g[r + 1][j] = t.y; g[r + 2][j] = t.z; g[r + 3][j] = t.w;
                    }
                } else {
#pragma unroll
                    for (int r = 0; r < RW; ++r) g[r][j] = (m < M && nb + r < N) ? src[r] : 0.f;
                }
            }
        }

        fetch_chunk(r0, c0, kbeg / KC);
        __syncthreads();  // previous item (or the table staging) is done with every buffer
        store_chunk((kbeg / KC) & 1);
        __syncthreads();
        build(NBUF == 2 ? (kbeg & 1) : 0, (kbeg / KC) & 1, 0);
        __syncthreads();

        float *obase = p.out + (p.direct ? (size_t)0 : (size_t)tr * K * CDIM);

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / KC, kk = k % KC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * KC < kend;
            if (kk == 0 && have_next_chunk) fetch_chunk(r0, c0, chunk + 1);
            // Half of the warps (alternating groups of four, so that every scheduler has both kinds) run
            // the side work - building slab k+1 and combining the partial sums of k-1 - before their gathers,
            // the other half after them: the dependent shared-memory chains of the side work then overlap
            // the other group's gather stream instead of all lining up behind the barrier.
            const bool side_first = (wp >> 2) & 1;
            auto side_work = [&]() {
                if (NBUF == 2 && k + 1 < kend) build((k + 1) & 1, ((k + 1) / KC) & 1, (k + 1) % KC);
                if (NBUF == 2 && k > kbeg) reduce_store(k - 1, obase, c0);
            };
            auto use_phase = [&]() {
            // use slab k: slab row rc[r,k], two fp32 columns per lane, for this warp's RW rows
                const uint2 *rp = reinterpret_cast<const uint2 *>(rc_s + stage * C::RC_STAGE + kk * RT + wp * RW);
                uint32_t rv[RW / 4];
#pragma unroll
                for (int q = 0; q < RW / 8; ++q) {
                    const uint2 t = rp[q];
                    rv[2 * q] = t.x; rv[2 * q + 1] = t.y;
                }
                const uint32_t ub = u_addr + (NBUF == 2 ? (k & 1) : 0) * C::U_BYTES + lane * 8;
                float s0a = 0.f, s0b = 0.f, s1a = 0.f, s1b = 0.f;
                float pf0[PF], pf1[PF];
                auto row_addr = [&](uint32_t v, int i) { return ub + byte_of(v, i) * (US * 4); };
#pragma unroll
                for (int r = 0; r < PF; ++r) {
                    asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                                 : "=f"(pf0[r]), "=f"(pf1[r]) : "r"(row_addr(rv[r >> 2], r & 3)));
                }
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const float f0 = pf0[r % PF], f1 = pf1[r % PF];
                    if (r + PF < RW) {
                        asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];"
                                     : "=f"(pf0[r % PF]), "=f"(pf1[r % PF])
                                     : "r"(row_addr(rv[(r + PF) >> 2], (r + PF) & 3)));
                    }
                    if (r & 1) { s0b = fmaf(f0, g[r][0], s0b); s1b = fmaf(f1, g[r][1], s1b); }
                    else       { s0a = fmaf(f0, g[r][0], s0a); s1a = fmaf(f1, g[r][1], s1a); }
                }
                *reinterpret_cast<float2 *>(part_s + (NBUF == 2 ? (k & 1) : 0) * (WARPS * PS) + wp * PS + 2 * lane) =
                    make_float2(s0a + s0b, s1a + s1b);
            };
            if (side_first) { side_work(); use_phase(); } else { use_phase(); side_work(); }
            if (kk == KC - 2 && have_next_chunk) store_chunk(stage ^ 1);
            __syncthreads();
            if (NBUF == 1) {
                // one slab and one partial-sum buffer: everybody has left slab k, so rebuild it for k+1 and
                // combine the partial sums of k, then meet again before slab k+1 is read
                if (k + 1 < kend) build(0, ((k + 1) / KC) & 1, (k + 1) % KC);
                reduce_store(k, obase, c0);
                __syncthreads();
            }
        }
        if (NBUF == 2) reduce_store(kend - 1, obase, c0);
    }
}

}  // namespace sg

int slab_f32_row_blocks(int rdim) { return (rdim + kSlabF32Rows - 1) / kSlabF32Rows; }

// out[k][c] (TRANSPOSE=false) or out[c][k] (TRANSPOSE=true) = scale * sum_b part[b][k][c], b ascending.
// PLACE = 1: column c is an unfolded row m of a convolution with non-overlapping windows and (m,k) goes to its
// position in the image gradient (conv_scatter_index); PLACE = 2: column c is pixel c of a stride class and k a
// channel (pixel_class_offset).  Both with TRANSPOSE=false.
struct ReducePlace {
    ConvGeom conv;
    PixelClass px;
};
template <bool TRANSPOSE, int PLACE>
__global__ void slab_reduce_blocks_kernel(const float *__restrict__ part, float *__restrict__ out, int K, int C,
                                          int nblocks, float scale, const ReducePlace pl) {
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
                if (PLACE == 1) {
                    const long o = conv_scatter_index(pl.conv, c, k);
                    if (o >= 0) out[o] = s * scale;
                } else if (PLACE == 2) {
                    out[pixel_class_offset(pl.px, c) + (size_t)k * pl.px.H * pl.px.W] = s * scale;
                } else {
                    out[(size_t)k * C + c] = s * scale;
                }
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

// The same for plain outputs whose rows of partial sums are 16-byte aligned (C a multiple of 4): 16-byte loads, a
// 32 (k) x 128 (c) tile per step; the transposing form turns the tile in shared memory so that both sides stay
// coalesced.
template <bool TRANSPOSE>
__global__ void __launch_bounds__(256) slab_reduce_blocks_vec_kernel(const float *__restrict__ part, float *__restrict__ out,
                                                                     int K, int C, int nblocks, float scale) {
    __shared__ float tile[TRANSPOSE ? 32 * 129 : 1];
    const int tiles_c = (C + 127) / 128, tiles_k = (K + 31) / 32;
    const size_t KC_ = (size_t)K * C;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8 threads
    for (int t = blockIdx.x; t < tiles_c * tiles_k; t += gridDim.x) {
        const int k0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 128;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + ty + 8 * j, c = c0 + 4 * tx;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < K && c < C) {
                for (int b = 0; b < nblocks; ++b) {
                    const float4 v = *reinterpret_cast<const float4 *>(part + (size_t)b * KC_ + (size_t)k * C + c);
                    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
                }
                s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
                if (!TRANSPOSE) *reinterpret_cast<float4 *>(out + (size_t)k * C + c) = s;
            }
            if (TRANSPOSE) {
                float *d = tile + (ty + 8 * j) * 129 + 4 * tx;
                d[0] = s.x; d[1] = s.y; d[2] = s.z; d[3] = s.w;
            }
        }
        if (TRANSPOSE) {
            __syncthreads();
            for (int cc = ty; cc < 128; cc += 8) {
                const int c = c0 + cc, k = k0 + tx;
                if (k < K && c < C) out[(size_t)c * K + k] = tile[tx * 129 + cc];
            }
            __syncthreads();
        }
    }
}

int slab_reduce_blocks(const float *part, float *out, int K, int C, int nblocks, bool transpose, const ConvGeom *scatter,
                       const PixelClass *px, float scale, int num_sms, cudaStream_t stream) {
    if (!scatter && !px && C % 4 == 0 && (reinterpret_cast<uintptr_t>(part) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        const long vtiles = (long)((K + 31) / 32) * ((C + 127) / 128);
        const int vgrid = (int)(vtiles < 8L * num_sms ? vtiles : 8L * num_sms);
        if (transpose) slab_reduce_blocks_vec_kernel<true><<<vgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale);
        else slab_reduce_blocks_vec_kernel<false><<<vgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale);
        return launch_status();
    }
    const long tiles = (long)((K + 31) / 32) * ((C + 31) / 32);
    const int rgrid = (int)(tiles < 8L * num_sms ? tiles : 8L * num_sms);
    ReducePlace pl{};
    if (scatter) {
        pl.conv = *scatter;
        slab_reduce_blocks_kernel<false, 1><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale, pl);
    } else if (px) {
        pl.px = *px;
        slab_reduce_blocks_kernel<false, 2><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale, pl);
    } else if (transpose) {
        slab_reduce_blocks_kernel<true, 0><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale, pl);
    } else {
        slab_reduce_blocks_kernel<false, 0><<<rgrid, 256, 0, stream>>>(part, out, K, C, nblocks, scale, pl);
    }
    return launch_status();
}

template <int BITS, int MODE, int WARPS, int RW, int PF>
static int launch_slab_grad_w(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                            int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                            int at_pitch, int num_sms, cudaStream_t stream) {
    using C = sg::Cfg<BITS, WARPS, RW>;
    auto kern = sg::slab_grad_kernel<BITS, MODE, WARPS, RW, PF>;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM)))
        return LUTGEMM_E_CUDA;
    const int RDIM = MODE == sg::kGa ? N : M, CDIM = MODE == sg::kGa ? M : N;
    sg::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = gc; p.M = M; p.K = K; p.N = N;
    p.conv = conv;
    p.at = MODE == sg::kGw ? at : nullptr;
    p.at_pitch = at_pitch;
    p.ga_scatter = (MODE == sg::kGa && conv.enabled) ? 1 : 0;
    p.tiles_r = (RDIM + C::RT - 1) / C::RT;
    p.tiles_c = (CDIM + C::CT - 1) / C::CT;
    p.direct = p.tiles_r == 1;
    p.out = p.direct ? out : scratch;
    p.vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    // cut K so that the persistent grid's last wave is as full as possible (k ranges are multiples of KC)
    const long tiles = (long)p.tiles_r * p.tiles_c;
    const int kchunks = (K + C::KC - 1) / C::KC;
    int ksplits = 1;
    double best = -1.0;
    for (int sp = 1; sp <= 16 && sp <= kchunks; ++sp) {
        const int per = ((kchunks + sp - 1) / sp) * C::KC;
        if ((K + per - 1) / per != sp) continue;
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
    if (launch_status() != LUTGEMM_OK) return LUTGEMM_E_CUDA;
    if (!p.direct)
        return slab_reduce_blocks(scratch, out, K, CDIM, p.tiles_r, MODE == sg::kGa, p.ga_scatter ? &conv : nullptr, nullptr,
                                  kGradFactor, num_sms, stream);
    return LUTGEMM_OK;
}

template <int BITS, int MODE>
static int launch_slab_grad(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                            int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                            int at_pitch, int num_sms, cudaStream_t stream) {
    return launch_slab_grad_w<BITS, MODE, 16, 32, 4>(gc, a, w, out, lut, M, K, N, conv, scratch, at, at_pitch, num_sms,
                                                     stream);
}

int backward_gw_slab_f32(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                         int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                         int at_pitch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_slab_grad<4, sg::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 6: return launch_slab_grad<6, sg::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 7: return launch_slab_grad<7, sg::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 8: return launch_slab_grad<8, sg::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int backward_ga_slab_f32(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                         int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms,
                         cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_slab_grad<4, sg::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 6: return launch_slab_grad<6, sg::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 7: return launch_slab_grad<7, sg::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 8: return launch_slab_grad<8, sg::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
