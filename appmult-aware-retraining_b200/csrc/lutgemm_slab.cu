// Forward LUT-GEMM for sm_100a, "column-gathered slab" kernel (large M):
//     c[m,n] = sum_k LUT[a[m,k]][w[k,n]]        exact uint32 accumulate
//
// A warp-wide table gather whose 32 column indices are random costs ~2.8 shared-memory wavefronts at
// 8 bits even when the table row is warp-uniform (a 256-entry uint16 row spans 4 words per bank).
// This kernel takes the data-dependent column index out of the hot gather.  A CTA owns a tile of 512
// rows m and 64 columns n, and for every k
//
//   build (once per k):  U_k[x][n] = LUT[x][w[k,n]]   for every code x and the 64 columns  (gather by w)
//   use   (per row m):   row a[m,k] of U_k, read contiguously over n and added to the accumulators.
//
// The use-phase read is uniform in x and contiguous in n: half a warp reads one slab row, one 64-bit shared load
// per lane returns four adjacent uint16 entries (four columns), conflict-free by construction - 64 table
// look-ups per shared-memory wavefront instead of ~11, and two rows per load instruction.  The build reads the table transposed and paired ([w][x],
// codes x and x + 2^b/2 in one word) with conflict-free 32-bit loads and writes slab rows (stride 34
// words) with conflict-free 64-bit stores: 2^b * 2 wavefronts per k against 512 for the use phase.
// Two slab buffers: slab k+1 is built while slab k is read, one CTA barrier per k.  (Handing the buffers over
// through per-buffer mbarriers, as the gradient kernels do, does not pay here: with polling waits it was slower -
// 11.5 against 10.7 ms at 8 bits for 4096^3 - and with suspending waits 10.38 against 10.42 ms at 8 bits, 8.63
// against 8.68 ms at 7 bits, 8.35 against 7.69 ms at 6 bits: the forward's read phase per k is half as long as
// the gradients'.)
// The two halves of a slab word go to the accumulators as  S += word,  H += word >> 16 ; at the end
// sum(lo) = S - (H << 16) (mod 2^32) and sum(hi) = H.
// Work items are (tile, k range): whole tiles where they fill the persistent grid's waves, otherwise every CTA
// takes an equal contiguous share of all (tile, 16-k chunk) pairs; the parts of a tile that is cut are combined
// with integer atomics, which are exact in any order, so the result stays bit-identical.  The activation codes come either from a
// transposed copy at[k][m] in a workspace (16 rows of one k per 16-byte load, coalesced; for a convolution
// that copy is the uint8 im2col, made once) or, without a workspace, straight from a[m][k] - with
// conv.enabled gathered from the NCHW code image on the fly (implicit im2col) - and transposed byte-wise
// on their way into shared memory.
// Operand delivery with a workspace: the k chunks of at[k][m] (two boxes of 16 k x 256 rows) and of w[k][n] (one box
// of 16 k x 64 columns) are fetched by one elected thread with tiled bulk-tensor copies (TMA) straight into the
// stage the kernel reads, completion counted on an mbarrier that every thread waits on (bounded) before the first
// use of the chunk; the transposition kernel has already cut the activation codes to b bits, the weight codes are
// cut when the build extracts them.  Without a workspace, or when w breaks a TMA alignment rule, the chunks go
// through registers (16-byte vector loads) as before.
// The gradient kernels built on the same idea are in lutgemm_slab_grad_tall.cu and lutgemm_slab_grad.cu.
// Replaces ApproxGemmForwardKernel, self_ops/src/approx_gemm_forward.cu:37-229.
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"
#include "lutgemm_tma.cuh"
#include "lutgemm_waits.cuh"

#ifndef LUTGEMM_FWD_HALFWARP_ROWS
#define LUTGEMM_FWD_HALFWARP_ROWS 1
#endif

namespace lutgemm {
namespace sf {

template <int BITS>
struct Cfg {
    static constexpr int Q = 1 << BITS;
    static constexpr int HALF = Q / 2;          // words per transposed-table row (two codes per word)
    static constexpr int TT_STRIDE = HALF + 1;  // words; +1 keeps the transposing stage conflict-free
    static constexpr int THREADS = 512;
    static constexpr int RT = 512;              // rows per CTA tile: 32 per warp
    static constexpr int CT = 64;               // columns per CTA tile: 2 per lane
    static constexpr int KC = 16;               // k per operand stage
    static constexpr int U_STRIDE = 34;         // words per slab row (32 + 2 pad: 8-byte aligned rows)
    static constexpr int TT_BYTES = (Q * TT_STRIDE * 4 + 127) & ~127;  // the stages behind it are TMA destinations
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = KC * RT;   // [half][kk][256]: two boxes of 16 k x 256 rows
    static constexpr int CC_STAGE = KC * CT;   // [kk][64]
    static constexpr int OFF_BAR = TT_BYTES + 2 * U_BYTES + 2 * RC_STAGE + 2 * CC_STAGE;
    static constexpr int SMEM = OFF_BAR + 2 * 8 + 16;  // one mbarrier per stage and the abort word
    static_assert(U_BYTES % 128 == 0 && RC_STAGE % 128 == 0 && CC_STAGE % 128 == 0, "TMA destinations are 128-byte aligned");
    static constexpr int NSETS = HALF > 32 ? HALF / 32 : 1;
};

struct Args {
    const uint8_t *a;  // [M,K] codes, or the code image x[B,C,H,W] when conv.enabled
    const uint8_t *w;  // [K,N]
    const uint16_t *lut;
    uint32_t *c;       // [M,N]
    int M, K, N;
    int tiles_r, tiles_c;
    int share;  // 1: equal shares of (tile, k chunk) pairs per CTA, cut tiles combined with atomics; 0: whole tiles
    int vec_a, vec_w, vec_c, vec_c4;
    ConvGeom conv;
    const uint8_t *at;  // optional: the activation codes transposed, at[k][m], rows at_pitch bytes apart
    int at_pitch;       // a multiple of 16; columns m >= M hold 0
    LayerEpilogue epi;  // epi.out != nullptr: the de-quantised fp32 layer output is stored instead of c
    int *error_word;    // device error word of the bounded waits (TMA instantiation)
};

// byte offset of activation code (kk, row) inside a row-code stage
__device__ __forceinline__ int rc_off(int kk, int row) { return (row >> 8) * (16 * 256) + kk * 256 + (row & 255); }

// USE_AT: the activation codes come from the transposed workspace copy (p.at); the other instantiation keeps
// the direct / implicit-im2col fetch, so neither carries the other's registers.
// TMA (with USE_AT): operand chunks by bulk-tensor copies (map_at over at[K][pitch], map_w over w[K][N]).
template <int BITS, bool USE_AT, bool TMA>
__global__ void __launch_bounds__(512, 1) slab_fwd_kernel(const Args p, const __grid_constant__ CUtensorMap map_at,
                                                          const __grid_constant__ CUtensorMap map_w) {
    static_assert(!TMA || USE_AT, "bulk-tensor operand loads read the transposed copy");
    using C = Cfg<BITS>;
    constexpr int Q = C::Q, HALF = C::HALF, TTS = C::TT_STRIDE, RT = C::RT, CT = C::CT, KC = C::KC;
    constexpr int US = C::U_STRIDE, THREADS = C::THREADS, NSETS = C::NSETS;
    constexpr uint32_t MASK4 = (Q - 1) * 0x01010101u;
    constexpr int COL = lut_col_num(BITS);
    constexpr bool HW = LUTGEMM_FWD_HALFWARP_ROWS != 0;  // half a warp per slab row in the use phase (64-bit reads)
    const int M = p.M, K = p.K, N = p.N;

    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t *rc_s = smem + C::TT_BYTES + 2 * C::U_BYTES;
    uint8_t *cc_s = rc_s + 2 * C::RC_STAGE;
    const uint32_t tt_addr = smem_u32(smem);
    const uint32_t u_addr = smem_u32(smem + C::TT_BYTES);
    const int tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
    const uint32_t bar_stage = smem_u32(smem + C::OFF_BAR);  // TMA: one barrier per operand stage
    volatile int *abort_word = reinterpret_cast<volatile int *>(smem + C::OFF_BAR + 16);
    uint32_t stage_phase = 0;                                 // TMA: bit s = parity of the next completion of stage s
    if (TMA && tid == 0) {
        *abort_word = 0;
        mbar_init(bar_stage, 1);
        mbar_init(bar_stage + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");  // visible to the copy engine
    }

    // ---- stage the table transposed and paired: tt[w][i] = { LUT[i][w], LUT[i + HALF][w] } ---------------
    {
        uint16_t *tt16 = reinterpret_cast<uint16_t *>(smem);
#pragma unroll 8
        for (int idx = tid; idx < Q * Q; idx += THREADS) {
            const int x = idx >> BITS, y = idx & (Q - 1);  // global read contiguous in y
            tt16[(y * TTS + (x & (HALF - 1))) * 2 + (x >> (BITS - 1))] = p.lut[x * COL + y];
        }
    }

    // ---- operand chunk staging: rc_s[stage][kk][m] (512 activation codes per k), cc_s[stage][kk][n] -----
    uint4 prc = make_uint4(0, 0, 0, 0), pcc = make_uint4(0, 0, 0, 0);
    auto load16 = [&](const uint8_t *src, int valid) -> uint4 {  // up to 16 bytes, the rest 0
        uint32_t t[4] = {0, 0, 0, 0};
#pragma unroll
        for (int q = 0; q < 16; ++q)
            if (q < valid) t[q >> 2] |= (uint32_t)src[q] << (8 * (q & 3));
        return make_uint4(t[0], t[1], t[2], t[3]);
    };
    auto fetch_chunk = [&](int m0, int n0, int chunk) {
        const int kbase = chunk * KC;
        const int m = min(m0 + tid, M - 1);
        if (USE_AT) {
            // 16 rows of one k per thread, coalesced (instead of 16 k of one row, gathered for a convolution)
            const int gk = kbase + tid / (RT / 16), gm = m0 + (tid % (RT / 16)) * 16;
            prc = (gk < K && gm < p.at_pitch) ? *reinterpret_cast<const uint4 *>(p.at + (size_t)gk * p.at_pitch + gm)
                                              : make_uint4(0, 0, 0, 0);
        } else if (kbase >= K) prc = make_uint4(0, 0, 0, 0);
        else if (p.conv.enabled) prc = conv_code16(p.a, p.conv, m, kbase, K);
        else if (p.vec_a) prc = *reinterpret_cast<const uint4 *>(p.a + (size_t)m * K + kbase);
        else prc = load16(p.a + (size_t)m * K + kbase, min(16, K - kbase));
        if (tid < KC * CT / 16) {
            const int gk = kbase + tid / (CT / 16), gn = n0 + (tid % (CT / 16)) * 16;
            if (gk >= K || gn >= N) pcc = make_uint4(0, 0, 0, 0);
            else if (p.vec_w) pcc = *reinterpret_cast<const uint4 *>(p.w + (size_t)gk * N + gn);
            else pcc = load16(p.w + (size_t)gk * N + gn, min(16, N - gn));
        }
    };
    auto store_chunk = [&](int stage) {
        // codes are masked to BITS bits here, once, so no stray code can index outside a slab or the table
        const uint32_t tr[4] = {prc.x & MASK4, prc.y & MASK4, prc.z & MASK4, prc.w & MASK4};
        uint8_t *rs = rc_s + stage * C::RC_STAGE;
        if (USE_AT) {
            *reinterpret_cast<uint4 *>(rs + rc_off(tid / (RT / 16), (tid % (RT / 16)) * 16)) =
                make_uint4(tr[0], tr[1], tr[2], tr[3]);
        } else {
#pragma unroll
            for (int q = 0; q < 16; ++q) rs[rc_off(q, tid)] = (uint8_t)(tr[q >> 2] >> (8 * (q & 3)));
        }
        if (tid < KC * CT / 16)
            *reinterpret_cast<uint4 *>(cc_s + stage * C::CC_STAGE + (tid / (CT / 16)) * CT + (tid % (CT / 16)) * 16) =
                make_uint4(pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4);
    };
    // build slab `buf` for the k that sits at (stage, kk): warp wp fills column pairs 2wp and 2wp+1
    auto build = [&](int buf, int stage, int kk) {
        const uint32_t cw = *reinterpret_cast<const uint32_t *>(cc_s + stage * C::CC_STAGE + kk * CT + wp * 4);
        const uint32_t ub = u_addr + buf * C::U_BYTES + wp * 8;  // this warp's four columns: words 2wp and 2wp+1
        // (chunks that arrive by bulk copy have not been through the masking store: cut the codes to BITS bits here)
        const uint32_t cwm = TMA ? (cw & MASK4) : cw;
        const uint32_t y0 = byte_of(cwm, 0), y1 = byte_of(cwm, 1), y2 = byte_of(cwm, 2), y3 = byte_of(cwm, 3);
        // all table reads of the warp's share are issued before its first store (the stores order later reads behind
        // them)
        uint32_t r0[NSETS], r1[NSETS], r2[NSETS], r3[NSETS];
#pragma unroll
        for (int j = 0; j < NSETS; ++j) {
            const int i = lane + 32 * j;
            if (HALF >= 32 || i < HALF) {
                r0[j] = lds_u32(tt_addr + (y0 * TTS + i) * 4);
                r1[j] = lds_u32(tt_addr + (y1 * TTS + i) * 4);
                r2[j] = lds_u32(tt_addr + (y2 * TTS + i) * 4);
                r3[j] = lds_u32(tt_addr + (y3 * TTS + i) * 4);
            }
        }
#pragma unroll
        for (int j = 0; j < NSETS; ++j) {
            const int i = lane + 32 * j;
            if (HALF >= 32 || i < HALF) {
                // { LUT[i][y0], LUT[i][y1] }, { LUT[i][y2], LUT[i][y3] } and the same for code i + HALF
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ub + i * (US * 4)), "r"(__byte_perm(r0[j], r1[j], 0x5410)),
                             "r"(__byte_perm(r2[j], r3[j], 0x5410)) : "memory");
                asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ub + (i + HALF) * (US * 4)),
                             "r"(__byte_perm(r0[j], r1[j], 0x7632)), "r"(__byte_perm(r2[j], r3[j], 0x7632)) : "memory");
            }
        }
    };

    // TMA: thread 0 starts the three copies of a chunk into `stage` (every thread is past a CTA barrier after its last
    // read of that stage); all threads wait for them before the chunk's first use
    auto tma_issue = [&](int m0, int n0, int chunk, int stage) {
        if (tid != 0) return;
        tma_fence_before_load();
        const uint32_t bar = bar_stage + 8 * stage;
        tma_expect_bytes(bar, C::RC_STAGE + C::CC_STAGE);
        const uint32_t rs = smem_u32(rc_s + stage * C::RC_STAGE), cs = smem_u32(cc_s + stage * C::CC_STAGE);
        tma_load_2d(rs, &map_at, m0, chunk * KC, bar);
        tma_load_2d(rs + KC * 256, &map_at, m0 + 256, chunk * KC, bar);
        tma_load_2d(cs, &map_w, n0, chunk * KC, bar);
    };
    auto tma_wait = [&](int stage) {
        mbar_wait(bar_stage + 8 * stage, (stage_phase >> stage) & 1u, 21 + stage, abort_word, p.error_word);
        stage_phase ^= 1u << stage;
    };

    // Work items are (tile, k range).  Without a K split: whole tiles, round-robin.  With one (p.share): the
    // (tile, 16-k chunk) pairs of the whole problem, tile-major, are cut into gridDim.x equal contiguous shares, so all
    // CTAs finish together; a share covers the tail of one tile's k range, whole tiles and the head of another, and
    // the sums of a tile that is cut are combined with integer atomics (exact in any order).
    const long kchunks = (K + KC - 1) / KC;
    const long total_chunks = (long)p.tiles_r * p.tiles_c * kchunks;
    long cur = p.share ? total_chunks * blockIdx.x / gridDim.x : (long)blockIdx.x;
    const long cur_end = p.share ? total_chunks * (blockIdx.x + 1) / gridDim.x : (long)p.tiles_r * p.tiles_c;
    while (cur < cur_end) {
        int tile, kbeg, kend;
        if (p.share) {
            tile = (int)(cur / kchunks);
            const int kc0 = (int)(cur - (long)tile * kchunks);
            const int kc1 = (int)min(kchunks, (long)kc0 + (cur_end - cur));
            kbeg = kc0 * KC;
            kend = min(K, kc1 * KC);
            cur += kc1 - kc0;
        } else {
            tile = (int)cur;
            kbeg = 0;
            kend = K;
            cur += gridDim.x;
        }
        const bool partial = kbeg != 0 || kend != K;
        const int m0 = (tile / p.tiles_c) * RT, n0 = (tile % p.tiles_c) * CT;

        // HW: half a warp per slab row, two words (four columns) per lane: acc[2 * i + w] belongs to row i of the lane's
        // half and word w.  Otherwise a warp per row, one word (two columns) per lane: acc[r] belongs to row r.
        uint32_t acc[32][2];  // [..][0] = sum of whole words, [..][1] = sum of high halves
#pragma unroll
        for (int r = 0; r < 32; ++r) acc[r][0] = acc[r][1] = 0u;

        if (TMA) {
            __syncthreads();  // previous item (or the table staging and barrier set-up) is done with every buffer
            tma_issue(m0, n0, kbeg / KC, (kbeg / KC) & 1);
            tma_wait((kbeg / KC) & 1);
        } else {
            fetch_chunk(m0, n0, kbeg / KC);
            __syncthreads();  // previous item (or the table staging) is done with every buffer
            store_chunk((kbeg / KC) & 1);
            __syncthreads();
        }
        build(kbeg & 1, (kbeg / KC) & 1, 0);
        __syncthreads();

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / KC, kk = k % KC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * KC < kend;
            if (TMA) {
                // the other stage was last read before the barrier that ended the previous k: refill it now, and
                // make sure it has landed before the last k of this chunk builds the next chunk's first slab
                if (kk == 0 && have_next_chunk) tma_issue(m0, n0, chunk + 1, stage ^ 1);
                if (kk == KC - 1 && have_next_chunk) tma_wait(stage ^ 1);
            } else if (kk == 0 && have_next_chunk) fetch_chunk(m0, n0, chunk + 1);
            // half of the warps (alternating groups of four, so that every scheduler has both kinds) build their share
            // of slab k+1 before their reads of slab k, the other half after them: the build's dependent
            // shared-memory chains then overlap read streams
            const bool build_first = (wp >> 2) & 1;
            if (build_first && k + 1 < kend) build((k + 1) & 1, ((k + 1) / KC) & 1, (k + 1) % KC);

            if constexpr (HW) {
                // use slab k: lanes 0-15 read the slab rows of the warp's rows 0-15, lanes 16-31 those of rows 16-31,
                // 64 bits (four columns) per lane
                const uint4 q0 = *reinterpret_cast<const uint4 *>(rc_s + stage * C::RC_STAGE +
                                                                  rc_off(kk, wp * 32 + (lane >> 4) * 16));
                const uint32_t rv[4] = {q0.x, q0.y, q0.z, q0.w};
                const uint32_t ub = u_addr + (k & 1) * C::U_BYTES + (lane & 15) * 8;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    // slab row address = base + 136 * code in one integer dot-product instruction
                    const uint32_t addr = byte_scaled_add<US * 4>(rv[i >> 2], i & 3, ub);
                    uint32_t w0, w1;
                    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(addr));
                    acc[2 * i][0] += w0;
                    acc[2 * i][1] += w0 >> 16;
                    acc[2 * i + 1][0] += w1;
                    acc[2 * i + 1][1] += w1 >> 16;
                }
            } else {
                // use slab k: slab row a[m,k], two columns per lane, for this warp's 32 rows
                const uint4 *rp = reinterpret_cast<const uint4 *>(rc_s + stage * C::RC_STAGE + rc_off(kk, wp * 32));
                const uint4 q0 = rp[0], q1 = rp[1];
                const uint32_t rv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                const uint32_t ub = u_addr + (k & 1) * C::U_BYTES + lane * 4;
#pragma unroll
                for (int r = 0; r < 32; ++r) {
                    // slab row address = base + 136 * code in one integer dot-product instruction
                    const uint32_t addr = byte_scaled_add<US * 4>(rv[r >> 2], r & 3, ub);
                    uint32_t word;
                    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(word) : "r"(addr));
                    acc[r][0] += word;
                    acc[r][1] += word >> 16;
                }
            }
            if (!build_first && k + 1 < kend) build((k + 1) & 1, ((k + 1) / KC) & 1, (k + 1) % KC);
            if (!TMA && kk == KC - 2 && have_next_chunk) store_chunk(stage ^ 1);
            __syncthreads();
        }

        LayerEpilogueScalars ev{};
        if (p.epi.out) ev = load_epilogue_scalars(p.epi);
#pragma unroll
        for (int r = 0; r < 32; ++r) {
            acc[r][0] -= acc[r][1] << 16;  // low-half sum = whole-word sum - 65536 * high-half sum
            // the row and the first of the two columns that acc[r] holds
            const int m = HW ? m0 + wp * 32 + (lane >> 4) * 16 + (r >> 1) : m0 + wp * 32 + r;
            const int n = HW ? n0 + 4 * (lane & 15) + 2 * (r & 1) : n0 + 2 * lane;
            if (m < M) {
                if (p.epi.out) {
                    // the layer's de-quantisation applied to the sums in registers (one split per tile here)
                    const int l = m % p.epi.L;
                    const float zw_box = __fmul_rn(ev.zw, p.epi.box[m]), zz_taps = __fmul_rn(ev.zz, p.epi.taps[l]);
                    float *orow = p.epi.out + (size_t)m * N;
                    if (n < N) orow[n] = epilogue_value(p.epi, ev, acc[r][0], zw_box, zz_taps, l, n, N);
                    if (n + 1 < N) orow[n + 1] = epilogue_value(p.epi, ev, acc[r][1], zw_box, zz_taps, l, n + 1, N);
                    continue;
                }
                uint32_t *crow = p.c + (size_t)m * N;
                if (HW && !partial && p.vec_c4) {
                    // the lane's four columns of this row in one 16-byte store (acc[r] and acc[r + 1] are one row)
                    if ((r & 1) == 0 && n < N) {
                        const uint32_t lo1 = acc[r + 1][0] - (acc[r + 1][1] << 16);
                        *reinterpret_cast<uint4 *>(crow + n) = make_uint4(acc[r][0], acc[r][1], lo1, acc[r + 1][1]);
                    }
                    continue;
                }
                if (partial) {
                    if (n < N) atomicAdd(crow + n, acc[r][0]);
                    if (n + 1 < N) atomicAdd(crow + n + 1, acc[r][1]);
                } else if (p.vec_c) {
                    if (n < N) *reinterpret_cast<uint2 *>(crow + n) = make_uint2(acc[r][0], acc[r][1]);
                } else {
                    if (n < N) crow[n] = acc[r][0];
                    if (n + 1 < N) crow[n + 1] = acc[r][1];
                }
            }
        }
    }
}

}  // namespace sf

static bool g_fwd_tma = true;  // bulk-tensor operand loads (false: 16-byte vector loads through registers)
void slab_fwd_set_tma(bool on) { g_fwd_tma = on; }

// the K split that best fills the last wave of the persistent grid (1 = every tile sums its whole K range)
int slab_fwd_ksplits(int M, int K, int N, int num_sms) {
    using C = sf::Cfg<8>;  // tile geometry does not depend on the bit-width
    const long tiles = (long)((M + C::RT - 1) / C::RT) * ((N + C::CT - 1) / C::CT);
    const int kchunks = (K + C::KC - 1) / C::KC;
    int ksplits = 1;
    double best = -1.0;
    for (int s = 1; s <= 16 && s <= kchunks; ++s) {
        const int per = ((kchunks + s - 1) / s) * C::KC;
        if ((K + per - 1) / per != s) continue;  // some split would get no work
        const long items = tiles * s;
        const long waves = (items + num_sms - 1) / num_sms;
        const double eff = (double)items / (double)(waves * num_sms) * (double)per / (double)(per + 6);
        if (eff > best + 1e-9) { best = eff; ksplits = s; }
    }
    return ksplits;
}

template <int BITS>
static int launch_fwd_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int M, int K, int N,
                           const ConvGeom &conv, const uint8_t *at, int at_pitch, const LayerEpilogue *epi, int num_sms,
                           cudaStream_t stream) {
    using C = sf::Cfg<BITS>;
    // operand chunks by bulk-tensor copies where the transposed copy exists and w keeps the copy engine's alignment
    // rules (base and row pitch multiples of 16 bytes); otherwise through registers
    CUtensorMap map_at{}, map_w{};
    const bool tma = at && g_fwd_tma && N % 16 == 0 &&
                     make_tensor_map_u8_2d(&map_at, at, (unsigned long long)at_pitch, (unsigned long long)K,
                                           (unsigned long long)at_pitch, 256, C::KC) &&
                     make_tensor_map_u8_2d(&map_w, w, (unsigned long long)N, (unsigned long long)K, (unsigned long long)N,
                                           C::CT, C::KC);
    auto kern = tma ? sf::slab_fwd_kernel<BITS, true, true>
                    : at ? sf::slab_fwd_kernel<BITS, true, false> : sf::slab_fwd_kernel<BITS, false, false>;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM)))
        return LUTGEMM_E_CUDA;
    sf::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.c = c; p.M = M; p.K = K; p.N = N;
    p.conv = conv;
    p.at = at;
    p.at_pitch = at_pitch;
    if (epi) p.epi = *epi;
    p.error_word = device_error_word();
    if (!p.error_word) return LUTGEMM_E_CUDA;
    p.tiles_r = (M + C::RT - 1) / C::RT;
    p.tiles_c = (N + C::CT - 1) / C::CT;
    const long tiles = (long)p.tiles_r * p.tiles_c;
    const long kchunks = (K + C::KC - 1) / C::KC;
    // K is cut where whole tiles would leave the last wave of the persistent grid badly filled (with a fused epilogue
    // every tile must hold complete sums: the caller only asks for it when no K split pays)
    p.share = !epi && slab_fwd_ksplits(M, K, N, num_sms) > 1;
    const long units = p.share ? tiles * kchunks : tiles;
    const int grid = (int)(units < num_sms ? units : num_sms);
    if (p.share && !cuda_ok(cudaMemsetAsync(c, 0, (size_t)M * N * sizeof(uint32_t), stream)))
        return LUTGEMM_E_CUDA;
    p.vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_c = (N % 2 == 0) && ((reinterpret_cast<uintptr_t>(c) & 7) == 0);
    p.vec_c4 = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    kern<<<grid, C::THREADS, C::SMEM, stream>>>(p, map_at, map_w);
    return launch_status();
}

int forward_slab(const uint8_t *a, const uint8_t *w, uint32_t *c, const uint16_t *lut, int bits, int M, int K, int N,
                 const ConvGeom &conv, const uint8_t *at, int at_pitch, const LayerEpilogue *epi, int num_sms,
                 cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_fwd_slab<4>(a, w, c, lut, M, K, N, conv, at, at_pitch, epi, num_sms, stream);
        case 6: return launch_fwd_slab<6>(a, w, c, lut, M, K, N, conv, at, at_pitch, epi, num_sms, stream);
        case 7: return launch_fwd_slab<7>(a, w, c, lut, M, K, N, conv, at, at_pitch, epi, num_sms, stream);
        case 8: return launch_fwd_slab<8>(a, w, c, lut, M, K, N, conv, at, at_pitch, epi, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
