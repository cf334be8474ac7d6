// Forward LUT-GEMM for sm_100a, "column-gathered slab" kernel (large M).
//
// A warp-wide table gather whose 32 column indices are random costs ~2.8 shared-memory wavefronts at
// 8 bits even when the table row is warp-uniform, because a 256-entry row spans 4 words per bank.
// This kernel removes the data-dependent column index from the hot gather:
//
//   for every k, the CTA first builds a slab  U_k[x][n] = LUT[x][w[k,n]]  for all 2^b codes x and its
//   64 output columns n  (a gather by w, done ONCE per k for all 512 rows of the CTA tile), then
//   every output row m only needs row a[m,k] of the slab:  c[m, n..n+63] += U_k[a[m,k]][0..63].
//
// The slab read is warp-uniform in x and contiguous in n: one 32-bit shared load per lane returns
// two adjacent uint16 entries (two columns), conflict-free by construction, i.e. 64 table look-ups
// per shared-memory wavefront.  The two halves are accumulated with dp2a (no unpacking).
// The build reads the table transposed ([w][x], x paired as (i, i + 2^b/2) inside one word) with
// conflict-free 32-bit loads and writes slab rows with conflict-free 32-bit stores (row stride 33
// words), so it costs 2 * 2^b * 64 * 2 B / 128 B = 2^b * 2 wavefronts per k against 512 for the use.
// Accumulators: 512 x 64 int32 per CTA (64 per thread, 512 threads), exact.
// Replaces ApproxGemmForwardKernel, self_ops/src/approx_gemm_forward.cu:37-229.
#include <stdlib.h>

#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"

namespace lutgemm {

template <int BITS>
struct SlabCfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int HALF = Q / 2;         // words per transposed-table row (two codes per word)
    static constexpr int TT_STRIDE = HALF + 1; // words; +1 makes the transposing stage conflict-free
    static constexpr int THREADS = 512;
    static constexpr int WARPS = 16;
    static constexpr int MT = 512;             // 32 rows per warp
    static constexpr int NT = 64;              // 2 columns per lane
    static constexpr int KC = 16;              // k per operand stage
    static constexpr int U_STRIDE = 33;        // words per slab row (32 + 1 pad)
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int A_STAGE = KC * MT;
    static constexpr int W_STAGE = KC * NT;
    static constexpr int SMEM = TT_BYTES + 2 * U_BYTES + 2 * A_STAGE + 2 * W_STAGE;
    static constexpr int NSETS = HALF > 32 ? HALF / 32 : 1;
};

// ACC selects how the two uint16 halves of a slab word reach their accumulators:
//   0: two dp2a;  1: full-word add + shifted add;  2: full-word add + mad.hi.
// Modes 1/2 keep S = sum(lo) + 65536*sum(hi) (mod 2^32) and H = sum(hi); sum(lo) = S - (H << 16).
template <int BITS, int ACC>
__global__ void __launch_bounds__(512, 1)
fwd_slab_kernel(const uint8_t *__restrict__ a, const uint8_t *__restrict__ w, uint32_t *__restrict__ c,
                const uint16_t *__restrict__ lut, int M, int K, int N, int tiles_m, int tiles_n, int ksplits,
                int k_per_split, int vec_a, int vec_w, int vec_c) {
    using Cfg = SlabCfg<BITS>;
    constexpr int Q = Cfg::Q, HALF = Cfg::HALF, TTS = Cfg::TT_STRIDE, MT = Cfg::MT, NT = Cfg::NT, KC = Cfg::KC;
    constexpr int US = Cfg::U_STRIDE, THREADS = Cfg::THREADS, NSETS = Cfg::NSETS;
    constexpr uint32_t MASK = Q - 1;
    constexpr int COL = lut_col_num(BITS);

    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *tt_s = reinterpret_cast<uint32_t *>(smem);
    uint32_t *u_s = reinterpret_cast<uint32_t *>(smem + Cfg::TT_BYTES);
    uint8_t *a_s = smem + Cfg::TT_BYTES + 2 * Cfg::U_BYTES;
    uint8_t *w_s = a_s + 2 * Cfg::A_STAGE;

    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;

    // ---- stage the table transposed and paired: tt[w][i] = { LUT[i][w], LUT[i + HALF][w] } ----------
    {
        uint16_t *tt16 = reinterpret_cast<uint16_t *>(tt_s);
        for (int idx = tid; idx < Q * Q; idx += THREADS) {
            const int x = idx >> BITS, wc = idx & (Q - 1);
            const uint16_t v = lut[x * COL + wc];
            tt16[(wc * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] = v;
        }
    }
    const uint32_t tt_addr = smem_u32(tt_s);
    const uint32_t u_addr = smem_u32(u_s);

    // operand chunk prefetch registers
    uint4 pa = make_uint4(0, 0, 0, 0), pw = make_uint4(0, 0, 0, 0);

    auto fetch_chunk = [&](int m0, int n0, int chunk) {
        const int kbase = chunk * KC;
        const int gm = min(m0 + tid, M - 1);
        const uint8_t *arow = a + (size_t)gm * K + kbase;
        if (vec_a) {
            pa = kbase < K ? *reinterpret_cast<const uint4 *>(arow) : make_uint4(0, 0, 0, 0);
        } else {
            uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (kbase + j < K) t[j >> 2] |= (uint32_t)arow[j] << (8 * (j & 3));
            pa = make_uint4(t[0], t[1], t[2], t[3]);
        }
        if (tid < KC * NT / 16) {
            const int kk = tid / (NT / 16), nc = (tid % (NT / 16)) * 16;
            const int gk = kbase + kk, gn = n0 + nc;
            if (vec_w) {
                pw = (gk < K && gn < N) ? *reinterpret_cast<const uint4 *>(w + (size_t)gk * N + gn) : make_uint4(0, 0, 0, 0);
            } else {
                uint32_t t[4] = {0, 0, 0, 0};
                if (gk < K) {
#pragma unroll
                    for (int j = 0; j < 16; ++j)
                        if (gn + j < N) t[j >> 2] |= (uint32_t)w[(size_t)gk * N + gn + j] << (8 * (j & 3));
                }
                pw = make_uint4(t[0], t[1], t[2], t[3]);
            }
        }
    };
    auto store_chunk = [&](int stage) {
        uint8_t *as = a_s + stage * Cfg::A_STAGE;
        const uint32_t t[4] = {pa.x, pa.y, pa.z, pa.w};
#pragma unroll
        for (int j = 0; j < 16; ++j) as[j * MT + tid] = (uint8_t)(t[j >> 2] >> (8 * (j & 3)));
        if (tid < KC * NT / 16) {
            const int kk = tid / (NT / 16), nc = (tid % (NT / 16)) * 16;
            *reinterpret_cast<uint4 *>(w_s + stage * Cfg::W_STAGE + kk * NT + nc) = pw;
        }
    };
    // build slab `buf` for the k that sits at (stage, kk)
    auto build = [&](int buf, int stage, int kk) {
        const uint32_t wc = *reinterpret_cast<const uint32_t *>(w_s + stage * Cfg::W_STAGE + kk * NT + wp * 4);
        const uint32_t ub = u_addr + buf * Cfg::U_BYTES;
#pragma unroll
        for (int pp = 0; pp < 2; ++pp) {
            const uint32_t w0 = byte_of(wc, 2 * pp) & MASK, w1 = byte_of(wc, 2 * pp + 1) & MASK;
            const int p = 2 * wp + pp;
#pragma unroll
            for (int j = 0; j < NSETS; ++j) {
                const int i = lane + 32 * j;
                if (HALF >= 32 || i < HALF) {
                    const uint32_t r0 = lds_u32(tt_addr + (w0 * TTS + i) * 4);
                    const uint32_t r1 = lds_u32(tt_addr + (w1 * TTS + i) * 4);
                    const uint32_t lo = __byte_perm(r0, r1, 0x5410);
                    const uint32_t hi = __byte_perm(r0, r1, 0x7632);
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + (i * US + p) * 4), "r"(lo) : "memory");
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(ub + ((i + HALF) * US + p) * 4), "r"(hi) : "memory");
                }
            }
        }
    };

    // work item = (output tile, K split); splits of one tile are combined with integer atomics, which
    // are exact in any order, so the result stays bit-identical
    for (int item = blockIdx.x; item < tiles_m * tiles_n * ksplits; item += gridDim.x) {
        const int tile = item / ksplits, ks = item % ksplits;
        const int kbeg = ks * k_per_split, kend = min(K, kbeg + k_per_split);
        const int m0 = (tile / tiles_n) * MT, n0 = (tile % tiles_n) * NT;
        uint32_t acc[32][2];
#pragma unroll
        for (int r = 0; r < 32; ++r) acc[r][0] = acc[r][1] = 0u;

        fetch_chunk(m0, n0, kbeg / KC);
        __syncthreads();  // previous item (or the table staging) is done with every buffer
        store_chunk((kbeg / KC) & 1);
        __syncthreads();
        build(kbeg & 1, (kbeg / KC) & 1, 0);
        __syncthreads();

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / KC, kk = k % KC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * KC < kend;
            if (kk == 0 && have_next_chunk) fetch_chunk(m0, n0, chunk + 1);
            if (k + 1 < kend) build((k + 1) & 1, ((k + 1) / KC) & 1, (k + 1) % KC);

            // use slab k: every lane adds two columns of slab row a[m,k] for its warp's 32 rows
            const uint4 *ap = reinterpret_cast<const uint4 *>(a_s + stage * Cfg::A_STAGE + kk * MT + wp * 32);
            const uint4 a0 = ap[0], a1 = ap[1];
            const uint32_t av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t ub = u_addr + (k & 1) * Cfg::U_BYTES + lane * 4;
#pragma unroll
            for (int r = 0; r < 32; ++r) {
                const uint32_t x = byte_of(av[r >> 2], r & 3) & MASK;
                uint32_t word;
                asm volatile("ld.shared.u32 %0, [%1];" : "=r"(word) : "r"(ub + x * (US * 4)));
                if constexpr (ACC == 0) {
                    acc[r][0] = __dp2a_lo(word, 0x00000001u, acc[r][0]);
                    acc[r][1] = __dp2a_lo(word, 0x00000100u, acc[r][1]);
                } else if constexpr (ACC == 1) {
                    acc[r][0] += word;
                    acc[r][1] += word >> 16;
                } else {
                    acc[r][0] += word;
                    acc[r][1] = __umulhi(word, 65536u) + acc[r][1];
                }
            }
            if (kk == KC - 2 && have_next_chunk) store_chunk(stage ^ 1);
            __syncthreads();
        }

        const int n = n0 + 2 * lane;
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            if constexpr (ACC != 0) acc[r][0] -= acc[r][1] << 16;
            const int m = m0 + wp * 32 + r;
            if (m < M) {
                uint32_t *crow = c + (size_t)m * N;
                if (ksplits > 1) {
                    if (n < N) atomicAdd(crow + n, acc[r][0]);
                    if (n + 1 < N) atomicAdd(crow + n + 1, acc[r][1]);
                } else if (vec_c) {
                    if (n < N) *reinterpret_cast<uint2 *>(crow + n) = make_uint2(acc[r][0], acc[r][1]);
                } else {
                    if (n < N) crow[n] = acc[r][0];
                    if (n + 1 < N) crow[n + 1] = acc[r][1];
                }
            }
        }
    }
}

template <int BITS, int ACC>
static int launch_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                       int num_sms, cudaStream_t stream) {
    using Cfg = SlabCfg<BITS>;
    auto kern = fwd_slab_kernel<BITS, ACC>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    const int tiles_m = (M + Cfg::MT - 1) / Cfg::MT, tiles_n = (N + Cfg::NT - 1) / Cfg::NT;
    const long tiles = (long)tiles_m * tiles_n;
    // pick the K split that best fills the last wave of the persistent grid
    int ksplits = 1;
    double best = -1.0;
    const int kchunks = (K + Cfg::KC - 1) / Cfg::KC;
    for (int s = 1; s <= 16 && s <= kchunks; ++s) {
        const int per = ((kchunks + s - 1) / s) * Cfg::KC;
        const int used = (K + per - 1) / per;  // splits that actually get work
        if (used != s) continue;
        const long items = tiles * s;
        const long waves = (items + num_sms - 1) / num_sms;
        const double eff = (double)items / (double)(waves * num_sms) * (double)per / (double)(per + 6);
        if (eff > best + 1e-9) { best = eff; ksplits = s; }
    }
    const int k_per_split = ((kchunks + ksplits - 1) / ksplits) * Cfg::KC;
    const long items = tiles * ksplits;
    const int grid = (int)(items < num_sms ? items : num_sms);
    if (ksplits > 1 && cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(uint32_t), stream) != cudaSuccess)
        return LUTGEMM_E_CUDA;
    const int vec_a = (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    const int vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    const int vec_c = (N % 2 == 0) && ((reinterpret_cast<uintptr_t>(c) & 7) == 0);
    kern<<<grid, Cfg::THREADS, Cfg::SMEM, stream>>>(a, w, c, lut, M, K, N, tiles_m, tiles_n, ksplits, k_per_split,
                                                    vec_a, vec_w, vec_c);
    return cudaGetLastError() == cudaSuccess ? LUTGEMM_OK : LUTGEMM_E_CUDA;
}

int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 int num_sms, cudaStream_t stream) {
    int acc = 0;
    if (const char *e = getenv("LUTGEMM_SLAB_ACC")) acc = atoi(e);
#define LUTGEMM_SLAB_CASE(B)                                                                   \
    case B:                                                                                    \
        if (acc == 1) return launch_slab<B, 1>(a, w, c, lut, M, K, N, num_sms, stream);        \
        if (acc == 2) return launch_slab<B, 2>(a, w, c, lut, M, K, N, num_sms, stream);        \
        return launch_slab<B, 0>(a, w, c, lut, M, K, N, num_sms, stream);
    switch (bits) {
        LUTGEMM_SLAB_CASE(4)
        LUTGEMM_SLAB_CASE(6)
        LUTGEMM_SLAB_CASE(7)
        LUTGEMM_SLAB_CASE(8)
    }
#undef LUTGEMM_SLAB_CASE
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
