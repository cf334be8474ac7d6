// Gradient LUT-GEMM kernels for sm_100a, fp32 column-gathered slab with a TALL tile (1024 rows x 32 columns).
//
//   grad_w:  gw[k,n] = 1/16 * sum_m T(a[m,k], w[k,n]) * gc[m,n]     rows r = m, columns c = n
//   grad_a:  ga[m,k] = 1/16 * sum_n gc[m,n] * T(a[m,k], w[k,n])     rows r = n, columns c = m
//
// Same scheme as lutgemm_slab_grad.cu (per k: gather a slab U_k[x][c] = T(x, cc[k,c]) once, then every row
// reads slab row rc[r,k] contiguously and multiplies it with its grad_out entries held in registers), but a
// lane owns ONE column and 64 rows per warp instead of two columns and 32 rows.  The register budget is
// the same (64 grad_out values per thread); the slab is half as wide, so its build - 2^b rows per k,
// whatever the tile height - is paid once per 1024 rows instead of once per 512: at 8 bits the shared-memory
// wavefronts per 32768 look-ups drop from 1024 + 768 to 1024 + 384.  The narrower slab also leaves room
// for two slab buffers at 8 bits (the row codes are staged 8 k at a time there), so slab k+1 is built
// while slab k is read and one CTA barrier per k suffices at every bit-width.
// Partial sums: one per lane, warp and k; the 16 warps are added in ascending order by one warp (rotating
// with k), row blocks by slab_reduce_blocks in ascending order: results are deterministic.
// grad_w takes its row codes from a transposed copy at[k][m] of the activation codes when the caller has one
// (lutgemm_api.cu makes it, or receives the forward pass's): the same coalesced 16-byte fetch as grad_a's
// weight rows instead of one 16-byte piece per activation row.
// Used when the reduction dimension fills 1024-row tiles well; otherwise the 512 x 64 kernel runs.
// Replaces ApproxGemmBackwardKernelForGA / ForGB, self_ops/src/approx_gemm_backward.cu:13-258, 261-492.
#include "lutgemm_common.cuh"
#include "lutgemm_kernels.h"


namespace lutgemm {
namespace sgt {

enum { kGw = 1, kGa = 2 };

template <int BITS>
struct Cfg {
    static constexpr int Q = 1 << BITS;
    static constexpr bool F32_TABLE = BITS <= 7;
    static constexpr int HALF = Q / 2;
    static constexpr int TT_STRIDE = F32_TABLE ? Q + 1 : HALF + 1;  // words per table row
    static constexpr int WARPS = 16, THREADS = 512, RW = 64, RT = WARPS * RW, CT = 32;
    static constexpr int KC = 16;                       // k per global fetch (16 codes per row in registers)
    static constexpr int SC = BITS == 8 ? 8 : 16;       // k per shared-memory stage
    static constexpr int U_STRIDE = 34;  // words per slab row: 32 floats + 2 (8-byte aligned rows, conflict-free stores)
    static constexpr int P_STRIDE = 33;
    static constexpr int TT_BYTES = Q * TT_STRIDE * 4;
    static constexpr int U_BYTES = Q * U_STRIDE * 4;
    static constexpr int RC_STAGE = SC * RT, CC_STAGE = SC * CT;
    static constexpr int P_BYTES = WARPS * P_STRIDE * 4;
    static constexpr int OFF_U = TT_BYTES;
    static constexpr int OFF_RC = OFF_U + 2 * U_BYTES;
    static constexpr int OFF_CC = OFF_RC + 2 * RC_STAGE;
    static constexpr int OFF_PART = OFF_CC + 2 * CC_STAGE;
    static constexpr int SMEM = OFF_PART + 2 * P_BYTES;
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
    int ga_bkl;
    const uint8_t *at;  // grad_w only, optional: transposed row codes at[k][m], rows at_pitch bytes apart
    int at_pitch;       // a multiple of 16; columns m >= M hold 0
};

// USE_AT (grad_w only): the row codes come from the transposed copy p.at; the other instantiation keeps the
// direct / implicit-im2col fetch, so neither carries the other's registers.
template <int BITS, int MODE, int PF, bool USE_AT>
__global__ void __launch_bounds__(512, 1) slab_grad_tall_kernel(const Args p) {
    using C = Cfg<BITS>;
    constexpr int RW = C::RW, WARPS = C::WARPS;
    constexpr int Q = C::Q, HALF = C::HALF, TTS = C::TT_STRIDE, RT = C::RT, CT = C::CT, KC = C::KC, SC = C::SC;
    constexpr int US = C::U_STRIDE, PS = C::P_STRIDE, THREADS = C::THREADS;
    constexpr int HALVES = KC / SC;  // shared-memory stages per fetched group of 16 k
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

    auto ga_index = [&](int m, int k) -> size_t {
        if (!p.ga_bkl) return (size_t)m * K + k;
        const int L = p.conv.Ho * p.conv.Wo, b = m / L;
        return ((size_t)b * K + k) * L + (m - b * L);
    };

    // ---- operand staging.  A group of 16 k is fetched into registers (two row-code vectors and one column-
    //      code vector per thread) and written to shared memory SC k at a time:
    //      rc_s[stage][kk][r] (1024 row codes per k), cc_s[stage][kk][c] (32 column codes per k) -------------
    uint4 prc[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)}, pcc = make_uint4(0, 0, 0, 0);
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
    auto fetch_group = [&](int r0, int c0, int group) {
        const int kbase = group * KC;
        if (MODE == kGw && USE_AT) {
            // row codes from the transposed copy at[k][m]: 16 rows per load, coalesced like the w operand
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int idx = tid + THREADS * j;  // (k, 16-row segment): RT / 16 = 64 segments per k
                const int gk = kbase + idx / (RT / 16), gm = r0 + (idx % (RT / 16)) * 16;
                prc[j] = (gk < K && gm < p.at_pitch) ? *reinterpret_cast<const uint4 *>(p.at + (size_t)gk * p.at_pitch + gm)
                                                     : make_uint4(0, 0, 0, 0);
            }
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else if (MODE == kGw) {
#pragma unroll
            for (int j = 0; j < 2; ++j) prc[j] = a_codes16(r0 + tid + THREADS * j, kbase);
            if (tid < KC * CT / 16) pcc = w_codes16(kbase + tid / (CT / 16), c0 + (tid % (CT / 16)) * 16);
        } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int idx = tid + THREADS * j;  // (k, 16-row segment): RT / 16 = 64 segments per k
                prc[j] = w_codes16(kbase + idx / (RT / 16), r0 + (idx % (RT / 16)) * 16);
            }
            if (tid < CT) pcc = a_codes16(c0 + tid, kbase);
        }
    };
    // writes the k range [half*SC, half*SC + SC) of the fetched group to `stage`
    auto store_stage = [&](int stage, int half) {
        uint8_t *rs = rc_s + stage * C::RC_STAGE;
        uint8_t *cs = cc_s + stage * C::CC_STAGE;
        const uint32_t tc[4] = {pcc.x & MASK4, pcc.y & MASK4, pcc.z & MASK4, pcc.w & MASK4};
        if (MODE == kGw && USE_AT) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int idx = tid + THREADS * j, kq = idx / (RT / 16);
                if (kq / SC == half || HALVES == 1)
                    *reinterpret_cast<uint4 *>(rs + (kq % SC) * RT + (idx % (RT / 16)) * 16) =
                        make_uint4(prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4);
            }
            if (tid < KC * CT / 16) {
                const int kq = tid / (CT / 16);
                if (kq / SC == half || HALVES == 1)
                    *reinterpret_cast<uint4 *>(cs + (kq % SC) * CT + (tid % (CT / 16)) * 16) =
                        make_uint4(tc[0], tc[1], tc[2], tc[3]);
            }
        } else if (MODE == kGw) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t tr[4] = {prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4};
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (q / SC == half || HALVES == 1)
                        rs[(q % SC) * RT + tid + THREADS * j] = (uint8_t)(tr[q >> 2] >> (8 * (q & 3)));
            }
            if (tid < KC * CT / 16) {
                const int kq = tid / (CT / 16);
                if (kq / SC == half || HALVES == 1)
                    *reinterpret_cast<uint4 *>(cs + (kq % SC) * CT + (tid % (CT / 16)) * 16) =
                        make_uint4(tc[0], tc[1], tc[2], tc[3]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int idx = tid + THREADS * j, kq = idx / (RT / 16);
                if (kq / SC == half || HALVES == 1)
                    *reinterpret_cast<uint4 *>(rs + (kq % SC) * RT + (idx % (RT / 16)) * 16) =
                        make_uint4(prc[j].x & MASK4, prc[j].y & MASK4, prc[j].z & MASK4, prc[j].w & MASK4);
            }
            if (tid < CT) {
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (q / SC == half || HALVES == 1) cs[(q % SC) * CT + tid] = (uint8_t)(tc[q >> 2] >> (8 * (q & 3)));
            }
        }
    };
    // build slab `buf` for the k at (stage, kk): warp wp fills the 64-bit column pair (2wp, 2wp+1).
    // Lanes run over x, so the table reads are contiguous and the 64-bit slab stores (row stride 34 words)
    // fall on distinct bank pairs within each half-warp.
    auto build = [&](int buf, int stage, int kk) {
        const uint32_t cw = *reinterpret_cast<const uint16_t *>(cc_s + stage * C::CC_STAGE + kk * CT + wp * 2);
        const uint32_t y0 = cw & 0xffu, y1 = cw >> 8;
        const uint32_t ub = u_addr + buf * C::U_BYTES + wp * 8;
        if constexpr (C::F32_TABLE) {
#pragma unroll
            for (int j = 0; j < (Q + 31) / 32; ++j) {
                const int x = lane + 32 * j;
                if (Q >= 32 || x < Q) {
                    const uint32_t r0 = lds_u32(tt_addr + (y0 * TTS + x) * 4);
                    const uint32_t r1 = lds_u32(tt_addr + (y1 * TTS + x) * 4);
                    asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(ub + x * (US * 4)), "r"(r0), "r"(r1) : "memory");
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
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + i * (US * 4)), "f"(f00), "f"(f01) : "memory");
                asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(ub + (i + HALF) * (US * 4)), "f"(f10), "f"(f11)
                             : "memory");
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
            if (p.direct && MODE == kGa) obase[ga_index(col, k)] = v * kGradFactor;
            else obase[(size_t)k * CDIM + col] = p.direct ? v * kGradFactor : v;
        }
    };

    const int items = p.tiles_r * p.tiles_c * p.ksplits;
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int tile = item / p.ksplits;
        const int kbeg = (item % p.ksplits) * p.k_per_split, kend = min(K, kbeg + p.k_per_split);
        const int tr = tile / p.tiles_c, tc = tile % p.tiles_c;
        const int r0 = tr * RT, c0 = tc * CT;

        // the grad_out block of this tile: g[r] for the warp's RW rows and the lane's column
        float g[RW];
        if (MODE == kGw) {
            const int n = c0 + lane;
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int m = r0 + wp * RW + r;
                g[r] = (m < M && n < N) ? p.gc[(size_t)m * N + n] : 0.f;
            }
        } else {
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
        }

        // kbeg is a multiple of 16, so the first stage is half 0 of its group
        fetch_group(r0, c0, kbeg / KC);
        __syncthreads();  // previous item (or the table staging) is done with every buffer
        store_stage((kbeg / SC) & 1, 0);
        __syncthreads();
        build(kbeg & 1, (kbeg / SC) & 1, 0);
        __syncthreads();

        float *obase = p.out + (p.direct ? (size_t)0 : (size_t)tr * K * CDIM);

        for (int k = kbeg; k < kend; ++k) {
            const int chunk = k / SC, kk = k % SC, stage = chunk & 1;
            const bool have_next_chunk = (chunk + 1) * SC < kend;
            // the registers are free for the next group once the last stage of the current one is written
            if (kk == 0 && have_next_chunk && (chunk + 1) % HALVES == 0) fetch_group(r0, c0, (chunk + 1) / HALVES);
            // Half of the warps (alternating groups of four, so that every scheduler has both kinds) run the
            // side work - building slab k+1 and adding up the partial sums of k-1 - before their gathers,
            // the other half after them, so that its dependent shared-memory chains overlap gather streams.
            const bool side_first = (wp >> 2) & 1;
            auto side_work = [&]() {
                if (k + 1 < kend) build((k + 1) & 1, ((k + 1) / SC) & 1, (k + 1) % SC);
                if (k > kbeg && wp == ((k - 1) & (WARPS - 1))) reduce_store(k - 1, obase, c0);
            };
            auto use_phase = [&]() {
                // use slab k: slab row rc[r,k], one fp32 column per lane, for this warp's RW rows
                const uint4 *rp = reinterpret_cast<const uint4 *>(rc_s + stage * C::RC_STAGE + kk * RT + wp * RW);
                const uint32_t ub = u_addr + (k & 1) * C::U_BYTES + lane * 4;
                float s[4] = {0.f, 0.f, 0.f, 0.f};
                // slab row address = base + 136 * code in one integer dot-product instruction
                auto row_addr = [&](uint32_t v, int i) { return byte_scaled_add<US * 4>(v, i, ub); };
                uint32_t rv[RW / 4];
#pragma unroll
                for (int q = 0; q < RW / 16; ++q) {
                    const uint4 t = rp[q];
                    rv[4 * q] = t.x; rv[4 * q + 1] = t.y; rv[4 * q + 2] = t.z; rv[4 * q + 3] = t.w;
                }
                float pf[PF];
#pragma unroll
                for (int r = 0; r < PF; ++r)
                    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(pf[r]) : "r"(row_addr(rv[r >> 2], r & 3)));
#pragma unroll
                for (int r = 0; r < RW; ++r) {
                    const float f = pf[r % PF];
                    if (r + PF < RW)
                        asm volatile("ld.shared.f32 %0, [%1];"
                                     : "=f"(pf[r % PF]) : "r"(row_addr(rv[(r + PF) >> 2], (r + PF) & 3)));
                    s[r & 3] = fmaf(f, g[r], s[r & 3]);
                }
                part_s[(k & 1) * (WARPS * PS) + wp * PS + lane] = (s[0] + s[1]) + (s[2] + s[3]);
            };
            if (side_first) { side_work(); use_phase(); } else { use_phase(); side_work(); }
            if (kk == SC - 2 && have_next_chunk) store_stage(stage ^ 1, (chunk + 1) % HALVES);
            __syncthreads();
        }
        if (wp == ((kend - 1) & (WARPS - 1))) reduce_store(kend - 1, obase, c0);
    }
}

}  // namespace sgt

int slab_tall_row_blocks(int rdim) { return (rdim + kSlabTallRows - 1) / kSlabTallRows; }

template <int BITS, int MODE>
static int launch_slab_grad_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *out, const int16_t *lut,
                                 int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                                 int at_pitch, int num_sms, cudaStream_t stream) {
    using C = sgt::Cfg<BITS>;
    static_assert(C::RT == kSlabTallRows, "tile height");
    static_assert(C::SMEM <= 232448, "shared memory budget");
    const bool use_at = MODE == sgt::kGw && at != nullptr;
    auto kern = use_at ? sgt::slab_grad_tall_kernel<BITS, MODE, 4, MODE == sgt::kGw>
                       : sgt::slab_grad_tall_kernel<BITS, MODE, 4, false>;
    if (!cuda_ok(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM)))
        return LUTGEMM_E_CUDA;
    const int RDIM = MODE == sgt::kGa ? N : M, CDIM = MODE == sgt::kGa ? M : N;
    sgt::Args p{};
    p.a = a; p.w = w; p.lut = lut; p.gc = gc; p.M = M; p.K = K; p.N = N;
    p.conv = conv;
    p.at = MODE == sgt::kGw ? at : nullptr;
    p.at_pitch = at_pitch;
    p.ga_bkl = (MODE == sgt::kGa && conv.enabled) ? 1 : 0;
    p.tiles_r = (RDIM + C::RT - 1) / C::RT;
    p.tiles_c = (CDIM + C::CT - 1) / C::CT;
    p.direct = p.tiles_r == 1;
    p.out = p.direct ? out : scratch;
    p.vec_a = !conv.enabled && (K % 16 == 0) && ((reinterpret_cast<uintptr_t>(a) & 15) == 0);
    p.vec_w = (N % 16 == 0) && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    p.vec_g = (N % 4 == 0) && ((reinterpret_cast<uintptr_t>(gc) & 15) == 0);
    // cut K so that the persistent grid's last wave is as full as possible (k ranges are multiples of 16)
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
        return slab_reduce_blocks(scratch, out, K, CDIM, p.tiles_r, MODE == sgt::kGa, p.ga_bkl ? conv.Ho * conv.Wo : 0,
                                  num_sms, stream);
    return LUTGEMM_OK;
}

int backward_gw_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *gw, const int16_t *lut_gw,
                          int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, const uint8_t *at,
                          int at_pitch, int num_sms, cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_slab_grad_tall<4, sgt::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 6: return launch_slab_grad_tall<6, sgt::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 7: return launch_slab_grad_tall<7, sgt::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
        case 8: return launch_slab_grad_tall<8, sgt::kGw>(gc, a, w, gw, lut_gw, M, K, N, conv, scratch, at, at_pitch, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

int backward_ga_slab_tall(const float *gc, const uint8_t *a, const uint8_t *w, float *ga, const int16_t *lut_ga,
                          int bits, int M, int K, int N, const ConvGeom &conv, float *scratch, int num_sms,
                          cudaStream_t stream) {
    switch (bits) {
        case 4: return launch_slab_grad_tall<4, sgt::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 6: return launch_slab_grad_tall<6, sgt::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 7: return launch_slab_grad_tall<7, sgt::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
        case 8: return launch_slab_grad_tall<8, sgt::kGa>(gc, a, w, ga, lut_ga, M, K, N, conv, scratch, nullptr, 0, num_sms, stream);
    }
    return LUTGEMM_E_BITS;
}

}  // namespace lutgemm
