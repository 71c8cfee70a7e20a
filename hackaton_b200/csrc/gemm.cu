// Fused NF4 dequant-GEMM for sm_100a: TMA -> producer-warp decode -> tcgen05.mma (TMEM).
//
// Forward  (TRANS_W = false): out[M, N_w] = act[M, K_w] . W^T (+ bias) (+ ext_a . ext_b^T)
// Backward (TRANS_W = true):  out[M, K_w] = act[M, N_w] . W          (+ ext_a . ext_b)
// replacing the reference's "decode the whole weight to fp16 in HBM, then cuBLAS"
// (solution/nf4.py:87-92 forward, 94-99 backward). W never exists in HBM as fp16 here.
//
// One CTA computes a (128*NACC) x 256 output tile over a range of 64-deep k-blocks. Roles:
//   warps 0..15  producers: read the packed-code tile from shared memory, fetch the block scales
//                (u8 absmax -> second-level table -> * absmax2 + offset, prefetched one k-block
//                ahead), expand codes through a register-resident fp16 table (byte permutes, no
//                shared-memory lookups) and write the fp16 weight tile in the 128-byte-swizzled
//                layout the MMA descriptor expects. After the main loop the same warps run the
//                epilogue (tcgen05.ld -> fp16 -> global, or fp32 partials for split-K).
//   warp 16      TMA: activation tiles (128-byte swizzle) and the code tile of each k-block into
//                a STAGES-deep ring of shared memory.
//   warp 17      allocates TMEM; one lane issues tcgen05.mma (M=128, N=256, K=16) and commits
//                each k-block to the ring's "empty" barrier.
// The weight tile is always stored as rows of n_w holding 64 consecutive k_w (128 bytes, chunk
// index XOR row%8). Forward reads it as a K-major B operand; backward as an MN-major one.
// With NACC = 2 both accumulators (two 128-row halves of the token tile) reuse each decoded
// weight tile, halving the decode work per flop.
//
// Split-K: when a problem has fewer tiles than SMs, gridDim.z CTAs share one tile, each over a
// slice of the k-blocks. They park fp32 partial tiles in a caller-provided workspace; the CTA
// that arrives last (a per-tile counter) adds the slices in a fixed order, applies the bias and
// writes fp16. The counters return to zero, so the workspace is reusable without clearing.
//
// The rank-16 LoRA term rides along as one extra K=16 MMA step after the main loop ("K
// extension", done by split 0): its two small operands are copied by the producers into the
// ring slot in the unswizzled core-matrix layout.
//
// Every barrier wait is bounded (ptx.cuh); on a timeout the CTA records a status code, lets its
// copies in flight land, frees TMEM and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "decode.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

constexpr int PRODUCER_WARPS = 16;
constexpr int PRODUCER_THREADS = PRODUCER_WARPS * 32;
constexpr int GEMM_THREADS = PRODUCER_THREADS + 64;
constexpr int TMA_WARP = PRODUCER_WARPS;
constexpr int MMA_WARP = PRODUCER_WARPS + 1;
constexpr int BK = 64;   // k-block depth = one quantisation block
constexpr int BN = 256;  // output-tile width

struct GemmParams {
    const void* absmax;
    const float* code2;
    const float* absmax2;
    const float* offset;
    const float* code16;
    const __half* bias;
    const __half* ext_a;
    const __half* ext_b;
    __half* out;
    int* status;
    float* ws_partials;      // split-K: [tile][split][128*NACC][BN] fp32
    unsigned int* ws_count;  // split-K: one arrival counter per tile, zero between launches
    long long ld_out;
    int m, n_w, k_w;
    int nested, nested_shift, nested_blocksize;
    int kb_per_split;
};

template <int NACC, int STAGES>
struct SmemLayout {
    static constexpr int A_BYTES = NACC * 128 * BK * 2;
    static constexpr int W_BYTES = BN * BK * 2;
    static constexpr int C_BYTES = BN * BK / 2;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES + C_BYTES;
    static constexpr int TABLE2_OFF = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFF = TABLE2_OFF + 1024;
    static constexpr int TOTAL = BAR_OFF + 256;
    static constexpr int DYNAMIC_BYTES = TOTAL + 1024;  // slack for 1024-byte alignment
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Adds the bias (if any), rounds eight fp32 values to fp16 and stores them at dst (columns
// col .. col+7 of a row that is n_out wide): one 16-byte store when allowed, else element-wise.
__device__ __forceinline__ void store8(__half* dst, float (&v)[8], int col, int n_out, bool vec_ok,
                                       const __half* bias) {
    if (bias != nullptr) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (col + e < n_out) v[e] += __half2float(bias[col + e]);
    }
    if (vec_ok && col + 8 <= n_out) {
        uint4 o;
        __half2 h;
        h = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        *reinterpret_cast<uint4*>(dst) = o;
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (col + e < n_out) dst[e] = __float2half_rn(v[e]);
    }
}

template <int NACC, bool TRANS_W, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap tm_act,
                const __grid_constant__ CUtensorMap tm_codes, const GemmParams p) {
    using L = SmemLayout<NACC, STAGES>;
    static_assert(BN * 2 == PRODUCER_THREADS, "one 16-byte code chunk per producer thread");
    constexpr uint32_t TMEM_COLS = NACC * BN;
    static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    float* table2 = reinterpret_cast<float*>(smem_gen + L::TABLE2_OFF);
    const uint32_t bar_base = smem_base + L::BAR_OFF;
    auto bar_full_tma = [&](int s) { return bar_base + 8u * s; };
    auto bar_full_w = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    const uint32_t bar_accum = bar_base + 8u * (3 * STAGES);
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFF + 8 * (3 * STAGES + 1));
    volatile int* abort_flag =
        reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFF + 8 * (3 * STAGES + 1) + 4);
    volatile int* last_flag =
        reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFF + 8 * (3 * STAGES + 1) + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * (128 * NACC);
    const int n0 = blockIdx.y * BN;          // first output column of this tile
    const int kc = TRANS_W ? p.n_w : p.k_w;  // contraction length
    const int nkb_total = (kc + BK - 1) / BK;
    const int kb_begin = blockIdx.z * p.kb_per_split;
    const int kb_end = min(kb_begin + p.kb_per_split, nkb_total);
    const int nkb = kb_end - kb_begin;       // k-blocks of this CTA (>= 1)
    const bool has_ext = p.ext_a != nullptr && blockIdx.z == 0;
    const int n_iter = nkb + (has_ext ? 1 : 0);
    const int blocks_per_row = p.k_w >> 6;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full_tma(s), 1);
            mbar_init(bar_full_w(s), PRODUCER_THREADS);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_accum, 1);
        *abort_flag = 0;
        *last_flag = 0;
        fence_barrier_init();
    }
    if (warp == TMA_WARP && lane == 0) {
        tma_prefetch_desc(&tm_act);
        tma_prefetch_desc(&tm_codes);
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    if (p.nested && threadIdx.x < 256) table2[threadIdx.x] = p.code2[threadIdx.x];
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    int fail = 0;

    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const uint32_t sa = smem_base + (uint32_t)s * L::STAGE_BYTES;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag)) { fail = 1; break; }
                if (it < nkb) {
                    const int kb = kb_begin + it;
                    mbar_arrive_expect_tx(bar_full_tma(s), L::A_BYTES + L::C_BYTES);
#pragma unroll
                    for (int a = 0; a < NACC; ++a)
                        tma_load_2d(sa + a * (128 * BK * 2), &tm_act, kb * BK, m0 + a * 128,
                                    bar_full_tma(s));
                    const uint32_t sc = sa + L::A_BYTES + L::W_BYTES;
                    if (TRANS_W)
                        tma_load_2d(sc, &tm_codes, n0 / 2, kb * BK, bar_full_tma(s));
                    else
                        tma_load_2d(sc, &tm_codes, kb * (BK / 2), n0, bar_full_tma(s));
                } else {
                    mbar_arrive(bar_full_tma(s));  // extension step: operands come from producers
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BN, 0u, TRANS_W ? 1u : 0u);
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                const uint32_t sa = smem_base + (uint32_t)s * L::STAGE_BYTES;
                const uint32_t sw = sa + L::A_BYTES;
                if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 2; break; }
                if (!mbar_wait(bar_full_w(s), ph, abort_flag)) { fail = 3; break; }
                tc_fence_after_sync();
                if (it < nkb) {
                    const uint64_t bdesc0 = TRANS_W ? make_smem_desc(sw, 64 * 128, 1024, LAYOUT_SW128)
                                                    : make_smem_desc(sw, 16, 1024, LAYOUT_SW128);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t bdesc =
                            bdesc0 + (uint64_t)(TRANS_W ? (16 * 128) >> 4 : 32 >> 4) * k;
#pragma unroll
                        for (int a = 0; a < NACC; ++a) {
                            const uint64_t adesc =
                                make_smem_desc(sa + a * (128 * BK * 2), 16, 1024, LAYOUT_SW128) +
                                (uint64_t)(32 >> 4) * k;
                            umma_f16(tmem_base + a * BN, adesc, bdesc, idesc,
                                     (it > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                } else {
                    // K extension: unswizzled core-matrix operands (layout type 0).
                    // A: [row/8][k-half][row%8][16 B]  -> LBO 128, SBO 256 (K-major).
                    // B forward:  same form over n_w rows (K-major).
                    // B backward: [r/8][k_w/8][r%8][16 B] -> LBO BN*16, SBO 128 (MN-major).
                    const uint64_t bdesc = TRANS_W ? make_smem_desc(sw, BN * 16, 128, LAYOUT_NONE)
                                                   : make_smem_desc(sw, 128, 256, LAYOUT_NONE);
#pragma unroll
                    for (int a = 0; a < NACC; ++a) {
                        const uint64_t adesc =
                            make_smem_desc(sa + a * (128 * BK * 2), 128, 256, LAYOUT_NONE);
                        umma_f16(tmem_base + a * BN, adesc, bdesc, idesc, it > 0 ? 1u : 0u);
                    }
                }
                umma_commit(bar_empty(s));
            }
            if (!fail) umma_commit(bar_accum);
        }
    } else {
        // ------------------------------------------------------------------ decode producers
        const int pt = threadIdx.x;  // 0..511: one 16-byte code chunk (32 weights) per k-block
        RegLut lut;
        {
            uint16_t bits[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) bits[i] = __half_as_ushort(__float2half_rn(p.code16[i]));
            lut = make_reg_lut(bits);
        }
        const float offset = p.nested ? *p.offset : 0.f;

        // Chunk geometry. Forward: the code tile is [256 rows][32 B]; chunk c covers row c/2,
        // half c%2 of the 64-wide k-block. Backward: the tile is [64 rows][128 B], 128-byte
        // swizzled by TMA; 8 consecutive lanes take 8 different rows of one chunk column so that
        // both the swizzled reads and the swizzled writes are bank-conflict free.
        int row, col;
        uint32_t src_off, dst_off[4];
        {
            uint32_t dst;
            int chunk0;
            if (!TRANS_W) {
                row = pt >> 1;
                col = pt & 1;
                src_off = (uint32_t)pt * 16u;
                dst = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
                chunk0 = col * 4;
            } else {
                row = ((pt >> 6) << 3) | (pt & 7);
                col = (pt >> 3) & 7;
                src_off = (uint32_t)row * 128u + (uint32_t)((col ^ (row & 7)) << 4);
                dst = (uint32_t)(col >> 1) * 8192u + (uint32_t)(row >> 3) * 1024u +
                      (uint32_t)(row & 7) * 128u;
                chunk0 = (col & 1) * 4;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
                dst_off[i] = smem_base + L::A_BYTES + dst + (uint32_t)(((chunk0 + i) ^ (row & 7)) << 4);
            src_off += smem_base + L::A_BYTES + L::W_BYTES;
        }

        // First-level scale index of this thread's chunk in k-block kb (32-bit: n_blocks < 2^31).
        //   forward : block (n0 + row) * bpr + kb            valid while n0 + row < N_w
        //   backward: block (kb*64 + row) * bpr + kw / 64    valid while kb*64 + row < N_w, kw < K_w
        uint32_t blk;
        uint32_t blk_step;
        bool col_ok;
        if (!TRANS_W) {
            blk = (uint32_t)(n0 + row) * (uint32_t)blocks_per_row + (uint32_t)kb_begin;
            blk_step = 1u;
            col_ok = n0 + row < p.n_w;
        } else {
            const int kw = n0 + col * 32;
            blk = (uint32_t)(kb_begin * BK + row) * (uint32_t)blocks_per_row + (uint32_t)(kw >> 6);
            blk_step = (uint32_t)BK * (uint32_t)blocks_per_row;
            col_ok = kw < p.k_w;
        }
        const uint8_t* absmax_u8 = static_cast<const uint8_t*>(p.absmax);
        const float* absmax_f32 = static_cast<const float*>(p.absmax);

        uint32_t raw_q = 0;   // u8 code (nested) or fp32 bits (flat) of the current k-block
        float raw_a2 = 0.f;   // second-level scale
        bool raw_ok = false;
        auto fetch_scale = [&](int it) {
            bool ok = col_ok;
            if (TRANS_W) ok = ok && ((kb_begin + it) * BK + row < p.n_w);
            raw_ok = ok;
            if (ok) {
                if (p.nested) {
                    raw_q = __ldg(absmax_u8 + blk);
                    const uint32_t b2 = p.nested_shift >= 0 ? (blk >> p.nested_shift)
                                                            : (blk / (uint32_t)p.nested_blocksize);
                    raw_a2 = __ldg(p.absmax2 + b2);
                } else {
                    raw_q = __float_as_uint(__ldg(absmax_f32 + blk));
                }
            }
            blk += blk_step;
        };
        if (nkb > 0) fetch_scale(0);

        uint32_t ph = 0;
        for (int it0 = 0; it0 < n_iter && !fail; it0 += STAGES, ph ^= 1u) {
#pragma unroll
            for (int s = 0; s < STAGES; ++s) {
                const int it = it0 + s;
                if (it >= n_iter) break;
                const uint32_t stage_off = (uint32_t)s * L::STAGE_BYTES;
                if (it < nkb) {
                    float sc;
                    if (!raw_ok)
                        sc = 0.f;  // rows / columns outside the weight contribute zeros
                    else if (p.nested)
                        sc = nested_scale(table2[raw_q], raw_a2, offset);
                    else
                        sc = __uint_as_float(raw_q);
                    const __half2 scale2 = __float2half2_rn(sc);
                    if (it + 1 < nkb) fetch_scale(it + 1);
                    if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                    const uint4 cw = lds128(src_off + stage_off);
                    sts128(dst_off[0] + stage_off, decode_word_reg(cw.x, lut, scale2));
                    sts128(dst_off[1] + stage_off, decode_word_reg(cw.y, lut, scale2));
                    sts128(dst_off[2] + stage_off, decode_word_reg(cw.z, lut, scale2));
                    sts128(dst_off[3] + stage_off, decode_word_reg(cw.w, lut, scale2));
                } else {
                    // K extension operands, unswizzled core-matrix layout (see the MMA branch).
                    if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                    const uint32_t abase = smem_base + stage_off;
                    const uint32_t wbase = abase + L::A_BYTES;
                    const uint4 zero = make_uint4(0, 0, 0, 0);
                    // ext_a rows m0 .. m0 + 128*NACC: two 16-byte halves per row
                    for (int c = pt; c < 128 * NACC * 2; c += PRODUCER_THREADS) {
                        const int r_all = c >> 1, half = c & 1;
                        const long long gm = (long long)m0 + r_all;
                        uint4 v = zero;
                        if (gm < p.m)
                            v = __ldg(reinterpret_cast<const uint4*>(p.ext_a + gm * 16) + half);
                        const int acc = r_all >> 7, r = r_all & 127;
                        sts128(abase + acc * (128 * BK * 2) + (r >> 3) * 256 + half * 128 +
                                   (r & 7) * 16, v);
                    }
                    if (!TRANS_W) {
                        for (int c = pt; c < BN * 2; c += PRODUCER_THREADS) {
                            const int r = c >> 1, half = c & 1;
                            const long long gn = (long long)n0 + r;
                            uint4 v = zero;
                            if (gn < p.n_w)
                                v = __ldg(reinterpret_cast<const uint4*>(p.ext_b + gn * 16) + half);
                            sts128(wbase + (r >> 3) * 256 + half * 128 + (r & 7) * 16, v);
                        }
                    } else {
                        // lora_a [16, K_w]: chunk (r, g) = 8 consecutive k_w of rank row r
                        for (int c = pt; c < 16 * (BN / 8); c += PRODUCER_THREADS) {
                            const int r = c / (BN / 8), g = c % (BN / 8);
                            const long long kw = (long long)n0 + g * 8;
                            uint4 v = zero;
                            if (kw < p.k_w)
                                v = __ldg(reinterpret_cast<const uint4*>(
                                    p.ext_b + (long long)r * p.k_w + kw));
                            sts128(wbase + (r >> 3) * (BN * 16) + g * 128 + (r & 7) * 16, v);
                        }
                    }
                }
                fence_proxy_async_smem();
                mbar_arrive(bar_full_w(s));
            }
        }

        // ------------------------------------------------------------------ epilogue
        if (!fail) {
            if (!mbar_wait(bar_accum, 0u, abort_flag)) fail = 5;
        }
        const int n_out = TRANS_W ? p.k_w : p.n_w;
        const bool split = gridDim.z > 1;
        const bool vec_ok = (p.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
        const unsigned tile_id = blockIdx.y * gridDim.x + blockIdx.x;
        constexpr size_t TILE_ELEMS = (size_t)128 * NACC * BN;
        if (!fail) {
            tc_fence_after_sync();
            const int q = warp & 3;     // TMEM lane quadrant this warp may read
            const int grp = warp >> 2;  // 0..3: which share of the column chunks
            constexpr int CHUNKS_PER_GRP = NACC * (BN / 32) / 4;
            float* part = split ? p.ws_partials + ((size_t)tile_id * gridDim.z + blockIdx.z) * TILE_ELEMS
                                : nullptr;
#pragma unroll 1
            for (int t = grp * CHUNKS_PER_GRP; t < (grp + 1) * CHUNKS_PER_GRP; ++t) {
                const int acc = t / (BN / 32), ch = t % (BN / 32);
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + ch * 32, r);
                tmem_ld_wait();
                const int trow = acc * 128 + q * 32 + lane;  // row within the tile
                const long long grow = (long long)m0 + trow;
                const int col0 = n0 + ch * 32;
                if (split) {
                    float4* dst = reinterpret_cast<float4*>(part + (size_t)trow * BN + ch * 32);
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        __stcg(dst + g, make_float4(__uint_as_float(r[4 * g]),
                                                    __uint_as_float(r[4 * g + 1]),
                                                    __uint_as_float(r[4 * g + 2]),
                                                    __uint_as_float(r[4 * g + 3])));
                } else if (grow < p.m && col0 < n_out) {
                    __half* dst = p.out + grow * p.ld_out + col0;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]);
                        store8(dst + g * 8, v, col0 + g * 8, n_out, vec_ok,
                               TRANS_W ? nullptr : p.bias);
                    }
                }
            }
        }
        if (split) {
            // Last-arriver reduction. Every thread publishes its partials, the 512 epilogue
            // threads meet (whether or not a wait timed out, so the barrier always fills), one of
            // them takes a ticket; the CTA holding the last ticket sums the slices in order.
            __threadfence();
            named_bar_sync(1, PRODUCER_THREADS);
            if (threadIdx.x == 0) {
                int last = 0;
                if (!*abort_flag) {
                    const unsigned ticket = atomicAdd(p.ws_count + tile_id, 1u);
                    last = (ticket == gridDim.z - 1) ? 1 : 0;
                }
                *last_flag = last;
            }
            named_bar_sync(1, PRODUCER_THREADS);
            if (*last_flag) {
                __threadfence();
                const float* base = p.ws_partials + (size_t)tile_id * gridDim.z * TILE_ELEMS;
                constexpr int UNITS = 128 * NACC * (BN / 8);  // 8-column groups in the tile
                const unsigned nz = gridDim.z;
                for (int u = threadIdx.x; u < UNITS; u += PRODUCER_THREADS) {
                    const int trow = u / (BN / 8), c8 = u % (BN / 8);
                    const long long grow = (long long)m0 + trow;
                    const int col = n0 + c8 * 8;
                    if (grow >= p.m || col >= n_out) continue;
                    const float4* src0 =
                        reinterpret_cast<const float4*>(base + (size_t)trow * BN + c8 * 8);
                    float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                    // slices are added in index order (deterministic); loads go out four slices
                    // at a time so that their latencies overlap
                    for (unsigned z0 = 0; z0 < nz; z0 += 4) {
                        float4 a[4], b[4];
#pragma unroll
                        for (unsigned j = 0; j < 4; ++j) {
                            if (z0 + j < nz) {
                                const float4* src = src0 + (size_t)(z0 + j) * (TILE_ELEMS / 4);
                                a[j] = __ldcg(src);
                                b[j] = __ldcg(src + 1);
                            } else {
                                a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                                b[j] = a[j];
                            }
                        }
#pragma unroll
                        for (unsigned j = 0; j < 4; ++j) {
                            v[0] += a[j].x; v[1] += a[j].y; v[2] += a[j].z; v[3] += a[j].w;
                            v[4] += b[j].x; v[5] += b[j].y; v[6] += b[j].z; v[7] += b[j].w;
                        }
                    }
                    store8(p.out + grow * p.ld_out + col, v, col, n_out, vec_ok,
                           TRANS_W ? nullptr : p.bias);
                }
                if (threadIdx.x == 0) p.ws_count[tile_id] = 0u;  // ready for the next launch
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    if (fail) {
        atomicCAS(p.status, 0, 100 + fail);
        // give copies and MMAs in flight time to land before shared memory / TMEM go away
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
                cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

static bool make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t inner,
                        uint64_t outer, uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tiling and split-K plan shared by the launcher and the workspace-size query.
GemmPlan plan_gemm(long long m, long long n_w, long long k_w, bool trans_w, int sm_count) {
    GemmPlan pl;
    pl.nacc = m > 128 ? 2 : 1;
    const long long n_out = trans_w ? k_w : n_w;
    const long long kc = trans_w ? n_w : k_w;
    pl.m_tiles = (int)((m + 128 * pl.nacc - 1) / (128 * pl.nacc));
    pl.n_tiles = (int)((n_out + BN - 1) / BN);
    const int nkb = (int)((kc + BK - 1) / BK);
    const long long tiles = (long long)pl.m_tiles * pl.n_tiles;
    int splits = 1;
    if (tiles * 2 <= sm_count && tiles <= (long long)(GEMM_COUNTER_BYTES / sizeof(unsigned)) &&
        nkb >= 8) {
        splits = (int)(sm_count / tiles);
        const int max_by_depth = nkb / 4;  // keep at least 4 k-blocks per slice
        if (splits > max_by_depth) splits = max_by_depth;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    pl.kb_per_split = (nkb + splits - 1) / splits;
    pl.splits = (nkb + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty slice
    pl.partial_bytes = pl.splits > 1
        ? (size_t)tiles * pl.splits * (size_t)(128 * pl.nacc * BN) * sizeof(float) : 0;
    // A fixed-size counter area (splitting only happens with fewer tiles than SMs, so 1024
    // counters always suffice): its extent never depends on the shape, so the bytes that must stay
    // zero are the same for every call that shares a workspace.
    pl.counter_bytes = pl.splits > 1 ? GEMM_COUNTER_BYTES : 0;
    return pl;
}

template <int NACC, bool TRANS_W, int STAGES>
static cudaError_t launch_cfg(const GemmArgs& a, const GemmPlan& pl, cudaStream_t stream,
                              const char** why) {
    using L = SmemLayout<NACC, STAGES>;
    auto kernel = nf4_gemm_kernel<NACC, TRANS_W, STAGES>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::DYNAMIC_BYTES);
    if (e != cudaSuccess) { *why = "cudaFuncSetAttribute(shared memory)"; return e; }

    const long long kc = TRANS_W ? a.n_w : a.k_w;
    CUtensorMap tm_act, tm_codes;
    if (!make_map_2d(&tm_act, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a.act, (uint64_t)kc, (uint64_t)a.m,
                     (uint64_t)a.ld_act * 2, BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)) {
        *why = "cuTensorMapEncodeTiled(activations)";
        return cudaErrorInvalidValue;
    }
    const bool ok = TRANS_W
        ? make_map_2d(&tm_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.codes, (uint64_t)a.k_w / 2,
                      (uint64_t)a.n_w, (uint64_t)a.k_w / 2, BN / 2, BK, CU_TENSOR_MAP_SWIZZLE_128B)
        : make_map_2d(&tm_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.codes, (uint64_t)a.k_w / 2,
                      (uint64_t)a.n_w, (uint64_t)a.k_w / 2, BK / 2, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (!ok) { *why = "cuTensorMapEncodeTiled(codes)"; return cudaErrorInvalidValue; }

    GemmParams p;
    p.absmax = a.absmax; p.code2 = a.code2; p.absmax2 = a.absmax2; p.offset = a.offset;
    p.code16 = a.code16; p.bias = a.bias; p.ext_a = a.ext_a; p.ext_b = a.ext_b; p.out = a.out;
    p.status = device_status_word();
    p.ld_out = a.ld_out; p.m = (int)a.m; p.n_w = (int)a.n_w; p.k_w = (int)a.k_w;
    p.nested = a.nested; p.nested_blocksize = a.nested_blocksize;
    p.nested_shift = -1;
    if (a.nested_blocksize > 0 && (a.nested_blocksize & (a.nested_blocksize - 1)) == 0) {
        int s = 0;
        while ((1 << s) < a.nested_blocksize) ++s;
        p.nested_shift = s;
    }
    if (p.status == nullptr) { *why = "device status word"; return cudaErrorInvalidValue; }
    int splits = pl.splits;
    p.kb_per_split = pl.kb_per_split;
    p.ws_count = nullptr;
    p.ws_partials = nullptr;
    if (splits > 1) {
        if (a.workspace == nullptr || a.workspace_bytes < pl.counter_bytes + pl.partial_bytes) {
            splits = 1;  // no scratch given: one CTA per tile walks the whole K range
            p.kb_per_split = (int)((kc + BK - 1) / BK);
        } else {
            p.ws_count = static_cast<unsigned int*>(a.workspace);
            p.ws_partials = reinterpret_cast<float*>(static_cast<char*>(a.workspace) + pl.counter_bytes);
        }
    }
    dim3 grid((unsigned)pl.m_tiles, (unsigned)pl.n_tiles, (unsigned)splits);
    kernel<<<grid, GEMM_THREADS, L::DYNAMIC_BYTES, stream>>>(tm_act, tm_codes, p);
    e = cudaGetLastError();
    if (e != cudaSuccess) *why = "kernel launch";
    return e;
}

cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream, const char** why) {
    *why = "";
    const GemmPlan pl = plan_gemm(a.m, a.n_w, a.k_w, a.trans_w, a.sm_count);
    if (pl.nacc == 2) {
        return a.trans_w ? launch_cfg<2, true, 3>(a, pl, stream, why)
                         : launch_cfg<2, false, 3>(a, pl, stream, why);
    }
    return a.trans_w ? launch_cfg<1, true, 4>(a, pl, stream, why)
                     : launch_cfg<1, false, 4>(a, pl, stream, why);
}

}  // namespace nf4
