// Fused NF4 dequant-GEMM for sm_100a: TMA -> producer-warp decode -> tcgen05.mma (TMEM).
//
// Forward  (TRANS_W = false): out[M, N_w] = act[M, K_w] . W^T (+ bias) (+ ext_a . ext_b^T)
// Backward (TRANS_W = true):  out[M, K_w] = act[M, N_w] . W          (+ ext_a . ext_b)
// replacing the reference's "decode the whole weight to fp16 in HBM, then cuBLAS"
// (solution/nf4.py:87-92 forward, 94-99 backward). W never exists in HBM as fp16 here.
//
// Persistent kernel. With CG = 2 the grid is a set of CTA pairs (clusters of two, one CTA per SM)
// driving tcgen05.mma.cta_group::2: a work unit is a (256*NACC) x 256 output tile over a slice of
// the 64-deep k-blocks; each CTA holds 128*NACC of its rows (activations in shared memory,
// accumulators in its own TMEM) and decodes only half of the weight tile, which the tensor cores
// of both SMs then read. With CG = 1 (token counts up to 128) a single CTA owns a 128 x 256 tile.
// Roles inside a CTA (18 warps):
//   warps 0..15  producers: read packed codes from shared memory, fetch the block scales (u8
//                absmax -> second-level table -> * absmax2 + offset, prefetched one k-block
//                ahead), expand codes through a register-resident fp16 table (byte permutes, no
//                shared-memory lookups) and write the fp16 weight tile in the 128-byte-swizzled
//                layout the MMA descriptor expects. At the end of a unit the same warps drain the
//                accumulators (tcgen05.ld), transpose them through shared memory and store whole
//                128-byte lines.
//   warp 16      TMA: this CTA's activation tiles (128-byte swizzle) and code tile of each
//                k-block into a STAGES-deep ring; it runs ahead into the next unit while the
//                producers are still in the epilogue of the current one.
//   warp 17      allocates TMEM; in the leader CTA one lane issues the MMAs (N = 256, K = 16) and
//                commits each k-block to the ring's "empty" barriers and each unit to
//                "accumulators full" (multicast to both CTAs of a pair).
// The weight tile is always stored as rows of n_w holding 64 consecutive k_w (128 bytes, chunk
// index XOR row%8). Forward reads it as a K-major B operand; backward as an MN-major one.
// With NACC = 2 two accumulators (two token sub-tiles) reuse each decoded weight tile.
//
// Synchronisation across a pair: the producers of both CTAs arrive (one lane per warp, release at
// cluster scope) on the leader's "weights ready" barrier; the peer's producers only get there
// after their own TMA barrier fired, so that one barrier also vouches for the peer's activation
// tile. Accumulator hand-back ("TMEM drained") works the same way.
//
// Split-K: when a problem has fewer tiles than the GPU has CTA slots, several units share a tile,
// each over a slice of the k-blocks, and write fp32 partial sums as plain row-major planes
// [slice][M][ldp] into caller-provided scratch; splitk_reduce_kernel then adds the planes in
// slice order (deterministic), applies the bias and writes fp16.
//
// The rank-16 LoRA term rides along as one extra K=16 MMA step after the main loop ("K
// extension", done by slice 0): its two small operands are copied by the producers into the
// ring slot in the unswizzled core-matrix layout.
//
// Every barrier wait is bounded (ptx.cuh); on a timeout the CTA records a status code, lets its
// copies in flight land, frees TMEM and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
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

// One weight of a group. Forward groups share the activations and stack their outputs along N
// (one output buffer each); backward groups share the output and stack along the contraction
// (one dY each). `first` is the group-wide index of the problem's first n-tile (forward) or
// first k-block (backward).
struct GemmProblem {
    const void* absmax;
    const float* code2;
    const float* absmax2;
    const float* offset;
    const float* code16;
    const __half* bias;   // forward only
    const __half* ext_a;  // rank-16 left factor [M, 16] (xa / u) or null
    const __half* ext_b;  // forward: lora_b [n_w, 16]; backward: lora_a [16, k_w]
    __half* out;          // forward: this problem's output; backward: only problem 0's is used
    float* ws;            // split-K planes [slice][m][ldp] (same remark)
    long long ld_out, ldp;
    int n_w;              // rows of this weight
    int first;
    int nested, nested_shift, nested_blocksize;
    int pad;
};

constexpr int MAXP = GEMM_MAX_GROUP;

struct GemmParams {
    GemmProblem prob[MAXP];
    int* status;
    int n_prob;
    int n_ext;               // backward: problems that carry a rank-16 extension
    int m, k_w;              // token rows; columns of every weight of the group
    int nkb_total;           // k-blocks of the whole contraction
    int m_tiles, n_tiles, splits, kb_per_split;
    int debug;               // bit 0: producers skip the decode, bit 1: phase trace (tuning only)
};

struct GemmMaps {
    CUtensorMap act[MAXP];    // forward: only [0]; backward: one dY per problem
    CUtensorMap codes[MAXP];
};

template <int CG, int NACC, int STAGES, int TABLES_>
struct SmemLayout {
    static constexpr int NB = BN / CG;                 // weight-tile columns decoded by one CTA
    static constexpr int A_BYTES = NACC * 128 * BK * 2;
    static constexpr int W_BYTES = NB * BK * 2;
    static constexpr int C_BYTES = NB * BK / 2;
    static constexpr int STAGE_BYTES = A_BYTES + W_BYTES + C_BYTES;
    static constexpr int TABLES = TABLES_;  // second-level tables kept in shared memory
    static constexpr int TABLE2_OFF = STAGES * STAGE_BYTES;
    static constexpr int BAR_OFF = TABLE2_OFF + 1024 * TABLES;
    static constexpr int TOTAL = BAR_OFF + 256;
    static constexpr int DYNAMIC_BYTES = TOTAL + 1024;  // slack for 1024-byte alignment
    static constexpr int WARPS_PER_W_SLOT = W_BYTES / 4096;  // 4 KB epilogue staging per warp
    static_assert(STAGES * WARPS_PER_W_SLOT >= PRODUCER_WARPS, "staging needs more weight slots");
    static_assert(DYNAMIC_BYTES <= 232448, "exceeds the 227 KB of shared memory per CTA");
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

__device__ __forceinline__ void sts128(uint32_t addr, const uint4& v) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                 ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Optional phase timestamps for tuning (NF4B200_DEBUG bit 1): producer thread 0 of each CTA records
// %globaltimer at fixed points of its first TRACE_UNITS units.
constexpr int TRACE_CTAS = 160, TRACE_UNITS = 4, TRACE_STAMPS = 8;
__device__ unsigned long long g_trace[TRACE_CTAS * TRACE_UNITS * TRACE_STAMPS];

#define NF4_TRACE(slot)                                                                       \
    do {                                                                                      \
        if ((p.debug & 2) && threadIdx.x == 0 && blockIdx.x < TRACE_CTAS &&                   \
            unit_iter < TRACE_UNITS)                                                          \
            g_trace[(blockIdx.x * TRACE_UNITS + unit_iter) * TRACE_STAMPS + (slot)] =         \
                globaltimer_ns();                                                             \
    } while (0)

// Second tuning aid: per-k-block event times of the first pair's first unit.
constexpr int TRACE2_EVENTS = 6, TRACE2_ITERS = 64;
__device__ unsigned long long g_trace2[2 * TRACE2_EVENTS * TRACE2_ITERS];
#define NF4_TRACE2(ev, it_)                                                                    \
    do {                                                                                       \
        if ((p.debug & 2) && blockIdx.x < 2 && unit_iter2 == 0 && (it_) < TRACE2_ITERS)         \
            g_trace2[(blockIdx.x * TRACE2_EVENTS + (ev)) * TRACE2_ITERS + (it_)] = globaltimer_ns(); \
    } while (0)

// One work unit of the persistent loop.
struct Unit {
    int m0, n0;         // tile origin (token row, output column inside the problem's output)
    int kb_begin, nkb;  // slice of (group-wide) k-blocks
    int n_iter;         // nkb + the K-extension steps this unit also runs
    int slice;
    int prob;           // forward: the problem this tile belongs to; backward: 0
};

// Problem that owns group-wide index idx (n-tile for forward, k-block for backward).
__device__ __forceinline__ int find_problem(const GemmParams& p, int idx) {
    if (p.n_prob == 1) return 0;
    int r = 0;
#pragma unroll
    for (int i = 1; i < MAXP; ++i)
        if (i < p.n_prob && idx >= p.prob[i].first) r = i;
    return r;
}

template <bool TRANS_W>
__device__ __forceinline__ Unit make_unit(int u, const GemmParams& p, int rows_per_tile) {
    Unit w;
    const int tile = u / p.splits;
    w.slice = u % p.splits;
    const int mt = tile % p.m_tiles, nt = tile / p.m_tiles;
    w.m0 = mt * rows_per_tile;
    w.prob = TRANS_W ? 0 : find_problem(p, nt);
    w.n0 = (nt - (TRANS_W ? 0 : p.prob[w.prob].first)) * BN;
    w.kb_begin = w.slice * p.kb_per_split;
    const int kb_end = min(w.kb_begin + p.kb_per_split, p.nkb_total);
    w.nkb = kb_end - w.kb_begin;
    int ext = 0;
    if (w.slice == 0) ext = TRANS_W ? p.n_ext : (p.prob[w.prob].ext_a != nullptr ? 1 : 0);
    w.n_iter = w.nkb + ext;
    return w;
}

// Backward: the e-th problem (in group order) that carries an extension.
__device__ __forceinline__ int ext_problem(const GemmParams& p, int e) {
    int seen = 0, r = 0;
#pragma unroll
    for (int i = 0; i < MAXP; ++i)
        if (i < p.n_prob && p.prob[i].ext_a != nullptr) {
            if (seen == e) r = i;
            ++seen;
        }
    return r;
}

template <int CG, int NACC, bool TRANS_W, int STAGES, int DW, int TABLES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
nf4_gemm_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ GemmParams p) {
    using L = SmemLayout<CG, NACC, STAGES, TABLES>;
    constexpr int NB = L::NB;
    // DW of the 16 producer warps decode (all 16 drain the accumulators); each decoding thread
    // expands WORDS 32-bit code words (8 weights each) per k-block
    constexpr int DECODE_THREADS = DW * 32;
    constexpr int WORDS = NB * BK / 8 / DECODE_THREADS;
    static_assert(WORDS == 2 || WORDS == 4, "producer work split");
    constexpr uint32_t TMEM_COLS = NACC * BN;
    static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");
    constexpr int ROWS_PER_TILE = 128 * CG * NACC;  // token rows of a unit (whole pair)
    constexpr uint32_t ARRIVALS = CG * PRODUCER_WARPS;  // "TMEM drained" arrivals (all warps)
    constexpr uint32_t W_ARRIVALS = CG * DW;             // "weights ready" arrivals

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    float* table2 = reinterpret_cast<float*>(smem_gen + L::TABLE2_OFF);
    const uint32_t bar_base = smem_base + L::BAR_OFF;
    auto bar_full_tma = [&](int s) { return bar_base + 8u * s; };
    auto bar_full_w = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto bar_empty = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
    const uint32_t bar_tmem_full = bar_base + 8u * (3 * STAGES);
    const uint32_t bar_tmem_empty = bar_base + 8u * (3 * STAGES + 1);
    volatile uint32_t* tmem_slot =
        reinterpret_cast<volatile uint32_t*>(smem_gen + L::BAR_OFF + 8 * (3 * STAGES + 2));
    volatile int* abort_flag =
        reinterpret_cast<volatile int*>(smem_gen + L::BAR_OFF + 8 * (3 * STAGES + 2) + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;  // 0 = leader of the pair
    const int pair = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_pairs = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int total_units = p.m_tiles * p.n_tiles * p.splits;
    const int blocks_per_row = p.k_w >> 6;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full_tma(s), 1);
            mbar_init(bar_full_w(s), W_ARRIVALS);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_tmem_full, 1);
        mbar_init(bar_tmem_empty, ARRIVALS);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == TMA_WARP && lane == 0) {
        tma_prefetch_desc(&maps.act[0]);
        tma_prefetch_desc(&maps.codes[0]);
    }
    if (warp == MMA_WARP) {
        if (CG == 2) {
            tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
            tmem_relinquish();
        }
    }
    if (threadIdx.x < 256) {
        for (int i = 0; i < L::TABLES && i < p.n_prob; ++i)
            if (p.prob[i].nested) table2[i * 256 + threadIdx.x] = p.prob[i].code2[threadIdx.x];
    }
    tc_fence_before_sync();
    __syncthreads();
    if (CG == 2) cluster_sync_all();  // the peer's barriers and TMEM exist before anyone uses them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // barriers that both CTAs arrive on live in the leader; everyone reaches them through the
    // cluster window
    const uint32_t lead_full_w0 = CG == 2 ? mapa_shared(bar_full_w(0), 0u) : bar_full_w(0);
    const uint32_t lead_tmem_empty = CG == 2 ? mapa_shared(bar_tmem_empty, 0u) : bar_tmem_empty;

    int fail = 0;

    if (warp == TMA_WARP) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t g = 0;  // ring position, running across units
            uint32_t unit_iter2 = 0;
            for (int u = pair; u < total_units && !fail; u += n_pairs, ++unit_iter2) {
                const Unit w = make_unit<TRANS_W>(u, p, ROWS_PER_TILE);
                for (int it = 0; it < w.n_iter; ++it, ++g) {
                    const int s = (int)(g % STAGES);
                    const uint32_t ph = (g / STAGES) & 1u;
                    const uint32_t sa = smem_base + (uint32_t)s * L::STAGE_BYTES;
                    const bool free_slot = CG == 2 ? mbar_wait_cluster(bar_empty(s), ph ^ 1u, abort_flag)
                                                   : mbar_wait(bar_empty(s), ph ^ 1u, abort_flag);
                    if (!free_slot) { fail = 1; break; }
                    NF4_TRACE2(0, it);
                    if (it < w.nkb) {
                        const int kbg = w.kb_begin + it;                 // group-wide k-block
                        const int pi = TRANS_W ? find_problem(p, kbg) : w.prob;
                        const int kb = TRANS_W ? kbg - p.prob[pi].first : kbg;
                        mbar_arrive_expect_tx(bar_full_tma(s), L::A_BYTES + L::C_BYTES);
#pragma unroll
                        for (int a = 0; a < NACC; ++a)
                            tma_load_2d(sa + a * (128 * BK * 2), &maps.act[TRANS_W ? pi : 0], kb * BK,
                                        w.m0 + a * (128 * CG) + (int)rank * 128, bar_full_tma(s));
                        const uint32_t sc = sa + L::A_BYTES + L::W_BYTES;
                        const int nb0 = w.n0 + (int)rank * NB;
                        if (TRANS_W)
                            tma_load_2d(sc, &maps.codes[pi], nb0 / 2, kb * BK, bar_full_tma(s));
                        else
                            tma_load_2d(sc, &maps.codes[pi], kb * (BK / 2), nb0, bar_full_tma(s));
                    } else {
                        mbar_arrive(bar_full_tma(s));  // extension step: producers bring operands
                    }
                }
            }
        }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer (leader)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BN, 0u, TRANS_W ? 1u : 0u, 128u * CG);
            uint32_t g = 0;
            uint32_t unit_iter = 0;
            long long wait_tma = 0, wait_w = 0;  // tuning: cycles the issuer spent on each barrier
            for (int u = pair; u < total_units && !fail; u += n_pairs, ++unit_iter) {
                const Unit w = make_unit<TRANS_W>(u, p, ROWS_PER_TILE);
                // the accumulators of the previous unit must have been drained (in both CTAs)
                if (!mbar_wait_cluster(bar_tmem_empty, (unit_iter & 1u) ^ 1u, abort_flag)) {
                    fail = 6;
                    break;
                }
                tc_fence_after_sync();
                for (int it = 0; it < w.n_iter; ++it, ++g) {
                    const int s = (int)(g % STAGES);
                    const uint32_t ph = (g / STAGES) & 1u;
                    const uint32_t sa = smem_base + (uint32_t)s * L::STAGE_BYTES;
                    const uint32_t sw = sa + L::A_BYTES;
                    const uint32_t unit_iter2 = unit_iter;
                    const long long c0 = (p.debug & 2) ? clock64() : 0;
                    if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 2; break; }
                    NF4_TRACE2(3, it);
                    const long long c1 = (p.debug & 2) ? clock64() : 0;
                    if (!mbar_wait_cluster(bar_full_w(s), ph, abort_flag)) { fail = 3; break; }
                    NF4_TRACE2(4, it);
                    if (p.debug & 2) {
                        const long long c2 = clock64();
                        wait_tma += c1 - c0;
                        wait_w += c2 - c1;
                    }
                    tc_fence_after_sync();
                    if (it < w.nkb) {
                        const uint64_t bdesc0 = TRANS_W
                            ? make_smem_desc(sw, 64 * 128, 1024, LAYOUT_SW128)
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
                                const uint32_t accum = (it > 0 || k > 0) ? 1u : 0u;
                                if (CG == 2) umma_f16_pair(tmem_base + a * BN, adesc, bdesc, idesc, accum);
                                else         umma_f16(tmem_base + a * BN, adesc, bdesc, idesc, accum);
                            }
                        }
                    } else {
                        // K extension: unswizzled core-matrix operands (layout type 0).
                        // A: [row/8][k-half][row%8][16 B]  -> LBO 128, SBO 256 (K-major).
                        // B forward:  same form over this CTA's NB n_w rows (K-major).
                        // B backward: [r/8][k_w/8][r%8][16 B] -> LBO NB*16, SBO 128 (MN-major).
                        const uint64_t bdesc = TRANS_W
                            ? make_smem_desc(sw, NB * 16, 128, LAYOUT_NONE)
                            : make_smem_desc(sw, 128, 256, LAYOUT_NONE);
#pragma unroll
                        for (int a = 0; a < NACC; ++a) {
                            const uint64_t adesc =
                                make_smem_desc(sa + a * (128 * BK * 2), 128, 256, LAYOUT_NONE);
                            const uint32_t accum = it > 0 ? 1u : 0u;
                            if (CG == 2) umma_f16_pair(tmem_base + a * BN, adesc, bdesc, idesc, accum);
                            else         umma_f16(tmem_base + a * BN, adesc, bdesc, idesc, accum);
                        }
                    }
                    if (CG == 2) umma_commit_pair(bar_empty(s), (uint16_t)3);
                    else         umma_commit(bar_empty(s));
                    NF4_TRACE2(5, it);
                }
                if (!fail) {
                    if (CG == 2) umma_commit_pair(bar_tmem_full, (uint16_t)3);
                    else         umma_commit(bar_tmem_full);
                }
                if ((p.debug & 2) && blockIdx.x < TRACE_CTAS && unit_iter == 0) {
                    g_trace[(blockIdx.x * TRACE_UNITS) * TRACE_STAMPS + 5] = (unsigned long long)wait_tma;
                    g_trace[(blockIdx.x * TRACE_UNITS) * TRACE_STAMPS + 6] = (unsigned long long)wait_w;
                    g_trace[(blockIdx.x * TRACE_UNITS) * TRACE_STAMPS + 7] = (unsigned long long)clock64();
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ decode producers
        const int pt = threadIdx.x;  // 0..511: WORDS code words (8 weights each) per k-block
        RegLut lut;
        int lut_prob = -1;  // problem whose 16-entry table is currently held in registers
        auto load_lut = [&](int pi) {
            uint16_t bits[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
                bits[i] = __half_as_ushort(__float2half_rn(__ldg(p.prob[pi].code16 + i)));
            lut = make_reg_lut(bits);
            lut_prob = pi;
        };
        load_lut(0);

        // Piece geometry (a piece = the 4*WORDS code bytes of one thread).
        // Forward: the code tile is [NB rows][32 B], pieces in memory order.
        // Backward: the tile is [64 rows][NB/2 B], swizzled by TMA (128-byte pattern for 128-byte
        // rows, 64-byte pattern for 64-byte rows); 8 consecutive lanes take 8 different rows of
        // one piece column, so the swizzled reads and the swizzled writes are bank-conflict free.
        int row, klocal;  // row of the tile; first k_w column (backward) / first k (forward)
        uint32_t src_off, dst_off[WORDS];
        {
            uint32_t dst;
            int chunk0;
            if (!TRANS_W) {
                constexpr int PPR = 8 / WORDS;  // pieces per row
                row = pt / PPR;
                const int part = pt % PPR;
                klocal = part * 8 * WORDS;
                src_off = (uint32_t)pt * (4u * WORDS);
                dst = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
                chunk0 = part * WORDS;
            } else {
                constexpr int PPR = (NB / 2) / (4 * WORDS);  // pieces per 64-row tile row
                row = ((pt / (8 * PPR)) << 3) | (pt & 7);
                const int e = (pt >> 3) % PPR;
                klocal = e * 8 * WORDS;
                const int byte = e * 4 * WORDS;              // offset of the piece inside its row
                if (CG == 1)
                    src_off = (uint32_t)row * 128u + (uint32_t)(((byte >> 4) ^ (row & 7)) << 4);
                else
                    src_off = (uint32_t)row * 64u +
                              (uint32_t)((((byte >> 4) ^ ((row >> 1) & 3)) << 4) + (byte & 15));
                dst = (uint32_t)(klocal >> 6) * 8192u + (uint32_t)(row >> 3) * 1024u +
                      (uint32_t)(row & 7) * 128u;
                chunk0 = (klocal & 63) >> 3;
            }
#pragma unroll
            for (int i = 0; i < WORDS; ++i)
                dst_off[i] = smem_base + L::A_BYTES + dst + (uint32_t)(((chunk0 + i) ^ (row & 7)) << 4);
            src_off += smem_base + L::A_BYTES + L::W_BYTES;
        }
        // epilogue geometry: TMEM lane quadrant, column share, private 4 KB staging area inside
        // the weight slots of the ring (free while the accumulators are drained)
        const int q = warp & 3;
        const int grp = warp >> 2;
        constexpr int CHUNKS_PER_GRP = NACC * (BN / 32) / 4;
        const uint32_t staging = smem_base + (uint32_t)(warp / L::WARPS_PER_W_SLOT) * L::STAGE_BYTES +
                                 L::A_BYTES + (uint32_t)(warp % L::WARPS_PER_W_SLOT) * 4096u;
        const bool split = p.splits > 1;

        uint32_t g = 0;
        uint32_t unit_iter = 0;
        for (int u = pair; u < total_units; u += n_pairs, ++unit_iter) {
            const Unit w = make_unit<TRANS_W>(u, p, ROWS_PER_TILE);
            NF4_TRACE(0);
            const int nb0 = w.n0 + (int)rank * NB;  // first weight-tile column of this CTA

            // First-level scale of this thread's piece in step `it` (32-bit indices: n_blocks < 2^31).
            //   forward : block (nb0 + row) * bpr + kb           valid while nb0 + row < N_w
            //   backward: block (kb*64 + row) * bpr + kw / 64    valid while kb*64 + row < N_w, kw < K_w
            // with kb counted inside the problem that owns the step. The raw first-level entry (u8
            // code or fp32 bits), the second-level scale and the offset are fetched one step ahead.
            const int kw = nb0 + klocal;  // backward: first k_w column of this thread's piece
            const uint32_t blk_base = TRANS_W
                ? (uint32_t)row * (uint32_t)blocks_per_row + (uint32_t)(kw >> 6)
                : (uint32_t)(nb0 + row) * (uint32_t)blocks_per_row;
            const uint32_t blk_per_kb = (uint32_t)BK * (uint32_t)blocks_per_row;
            uint32_t raw_q = 0;
            float raw_a2 = 0.f, raw_off = 0.f;
            int raw_prob = 0;
            bool raw_ok = false;
            auto fetch_scale = [&](int it) {
                const int kbg = w.kb_begin + it;
                const int pi = TRANS_W ? find_problem(p, kbg) : w.prob;
                const GemmProblem& pr = p.prob[pi];
                const int kb = TRANS_W ? kbg - pr.first : kbg;
                uint32_t blk;
                bool ok;
                if (!TRANS_W) {
                    blk = blk_base + (uint32_t)kb;
                    ok = nb0 + row < pr.n_w;
                } else {
                    blk = blk_base + (uint32_t)kb * blk_per_kb;
                    ok = kw < p.k_w && kb * BK + row < pr.n_w;
                }
                raw_ok = ok;
                raw_prob = pi;
                if (ok) {
                    if (pr.nested) {
                        raw_q = __ldg(static_cast<const uint8_t*>(pr.absmax) + blk);
                        const uint32_t b2 = pr.nested_shift >= 0
                            ? (blk >> pr.nested_shift) : (blk / (uint32_t)pr.nested_blocksize);
                        raw_a2 = __ldg(pr.absmax2 + b2);
                        raw_off = __ldg(pr.offset);
                    } else {
                        raw_q = __float_as_uint(__ldg(static_cast<const float*>(pr.absmax) + blk));
                    }
                }
            };
            if (!fail && warp < DW) fetch_scale(0);

            for (int it = 0; warp < DW && it < w.n_iter && !fail; ++it, ++g) {
                const int s = (int)(g % STAGES);
                const uint32_t ph = (g / STAGES) & 1u;
                const uint32_t stage_off = (uint32_t)s * L::STAGE_BYTES;
                if (it < w.nkb) {
                    float sc;
                    if (!raw_ok)
                        sc = 0.f;  // rows / columns outside the weight contribute zeros
                    else if (p.prob[raw_prob].nested)
                        sc = nested_scale(table2[(L::TABLES > 1 ? raw_prob * 256 : 0) + raw_q], raw_a2,
                                          raw_off);
                    else
                        sc = __uint_as_float(raw_q);
                    const __half2 scale2 = __float2half2_rn(sc);
                    if (raw_prob != lut_prob) load_lut(raw_prob);
                    if (it + 1 < w.nkb) fetch_scale(it + 1);
                    if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                    if (threadIdx.x == 0) { const uint32_t unit_iter2 = unit_iter; NF4_TRACE2(1, it); }
                    if (!(p.debug & 1)) {
                        if (WORDS == 4) {
                            const uint4 cw = lds128(src_off + stage_off);
                            sts128(dst_off[0] + stage_off, decode_word_reg(cw.x, lut, scale2));
                            sts128(dst_off[1] + stage_off, decode_word_reg(cw.y, lut, scale2));
                            sts128(dst_off[WORDS - 2] + stage_off, decode_word_reg(cw.z, lut, scale2));
                            sts128(dst_off[WORDS - 1] + stage_off, decode_word_reg(cw.w, lut, scale2));
                        } else {
                            const uint2 cw = lds64(src_off + stage_off);
                            sts128(dst_off[0] + stage_off, decode_word_reg(cw.x, lut, scale2));
                            sts128(dst_off[1] + stage_off, decode_word_reg(cw.y, lut, scale2));
                        }
                    }
                } else {
                    // K extension operands, unswizzled core-matrix layout (see the MMA branch).
                    if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                    const GemmProblem& pe = p.prob[TRANS_W ? ext_problem(p, it - w.nkb) : w.prob];
                    const uint32_t abase = smem_base + stage_off;
                    const uint32_t wbase = abase + L::A_BYTES;
                    const uint4 zero = make_uint4(0, 0, 0, 0);
                    // this CTA's ext_a rows: two 16-byte halves per row
                    for (int c = pt; c < 128 * NACC * 2; c += DECODE_THREADS) {
                        const int r_all = c >> 1, half = c & 1;
                        const int acc = r_all >> 7, r = r_all & 127;
                        const long long gm = (long long)w.m0 + acc * (128 * CG) + (int)rank * 128 + r;
                        uint4 v = zero;
                        if (gm < p.m)
                            v = __ldg(reinterpret_cast<const uint4*>(pe.ext_a + gm * 16) + half);
                        sts128(abase + acc * (128 * BK * 2) + (r >> 3) * 256 + half * 128 +
                                   (r & 7) * 16, v);
                    }
                    if (!TRANS_W) {
                        for (int c = pt; c < NB * 2; c += DECODE_THREADS) {
                            const int r = c >> 1, half = c & 1;
                            const long long gn = (long long)nb0 + r;
                            uint4 v = zero;
                            if (gn < pe.n_w)
                                v = __ldg(reinterpret_cast<const uint4*>(pe.ext_b + gn * 16) + half);
                            sts128(wbase + (r >> 3) * 256 + half * 128 + (r & 7) * 16, v);
                        }
                    } else {
                        // lora_a [16, K_w]: chunk (r, gq) = 8 consecutive k_w of rank row r
                        for (int c = pt; c < 16 * (NB / 8); c += DECODE_THREADS) {
                            const int r = c / (NB / 8), gq = c % (NB / 8);
                            const long long kwc = (long long)nb0 + gq * 8;
                            uint4 v = zero;
                            if (kwc < p.k_w)
                                v = __ldg(reinterpret_cast<const uint4*>(
                                    pe.ext_b + (long long)r * p.k_w + kwc));
                            sts128(wbase + (r >> 3) * (NB * 16) + gq * 128 + (r & 7) * 16, v);
                        }
                    }
                }
                // publish: every lane fences its writes towards the async proxy, one lane arrives
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    if (CG == 2) mbar_arrive_cluster(lead_full_w0 + 8u * s);
                    else         mbar_arrive(bar_full_w(s));
                }
                if (threadIdx.x == 0) { const uint32_t unit_iter2 = unit_iter; NF4_TRACE2(2, it); }
            }

            // -------------------------------------------------------------- epilogue of the unit
            NF4_TRACE(1);
            if (!fail) {
                if (!mbar_wait(bar_tmem_full, unit_iter & 1u, abort_flag)) fail = 5;
            }
            NF4_TRACE(2);
            const GemmProblem& po = p.prob[w.prob];  // backward: problem 0 carries the output
            const int n_out = TRANS_W ? p.k_w : po.n_w;
            const bool vec_ok = (po.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(po.out) & 15) == 0);
            if (!fail) {
                tc_fence_after_sync();
                const int lrow = lane;  // row of this lane inside its quadrant
                const int rd_row = lane >> 3, rd_chunk = lane & 7;
                auto release_tmem = [&]() {
                    // every accumulator value of this warp is in registers / staging
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if (CG == 2) mbar_arrive_cluster(lead_tmem_empty);
                        else         mbar_arrive(bar_tmem_empty);
                    }
                };
                if (!split) {
                    // two 32-column chunks -> one [32 rows x 64 cols] fp16 box, written out as
                    // whole 128-byte lines
#pragma unroll 1
                    for (int b = 0; b < CHUNKS_PER_GRP / 2; ++b) {
                        const int t0 = grp * CHUNKS_PER_GRP + 2 * b;
                        const int acc = t0 / (BN / 32), ch0 = t0 % (BN / 32);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t r[32];
                            tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN +
                                              (ch0 + h) * 32, r);
                            tmem_ld_wait();
                            if (!TRANS_W && po.bias != nullptr) {
                                const int cb = w.n0 + (ch0 + h) * 32;
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (cb + e < n_out)
                                        r[e] = __float_as_uint(__uint_as_float(r[e]) +
                                                               __half2float(po.bias[cb + e]));
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                uint4 o;
                                o.x = pack_half2(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                                o.y = pack_half2(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                                o.z = pack_half2(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                                o.w = pack_half2(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                                sts128(staging + lrow * 128 + (((h * 4 + i) ^ (lrow & 7)) << 4), o);
                            }
                        }
                        if (b == CHUNKS_PER_GRP / 2 - 1) release_tmem();
                        __syncwarp();
                        const long long grow0 =
                            (long long)w.m0 + acc * (128 * CG) + (int)rank * 128 + q * 32;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + rd_row;
                            const uint4 v = lds128(staging + rr * 128 + ((rd_chunk ^ (rr & 7)) << 4));
                            const long long grow = grow0 + rr;
                            const int colg = w.n0 + ch0 * 32 + rd_chunk * 8;
                            if (grow < p.m && colg < n_out && !(p.debug & 64)) {
                                __half* dst = po.out + grow * po.ld_out + colg;
                                if (vec_ok && colg + 8 <= n_out) {
                                    *reinterpret_cast<uint4*>(dst) = v;
                                } else {
                                    const __half* hv = reinterpret_cast<const __half*>(&v);
#pragma unroll
                                    for (int e = 0; e < 8; ++e)
                                        if (colg + e < n_out) dst[e] = hv[e];
                                }
                            }
                        }
                        __syncwarp();
                    }
                } else {
                    // fp32 partial sums of this slice: one [32 rows x 32 cols] box per chunk into
                    // the slice's row-major plane
                    float* plane = po.ws + (size_t)w.slice * ((size_t)p.m * (size_t)po.ldp);
#pragma unroll 1
                    for (int t = grp * CHUNKS_PER_GRP; t < (grp + 1) * CHUNKS_PER_GRP; ++t) {
                        const int acc = t / (BN / 32), ch = t % (BN / 32);
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + ch * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            sts128(staging + lrow * 128 + ((i ^ (lrow & 7)) << 4),
                                   make_uint4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]));
                        if (t == (grp + 1) * CHUNKS_PER_GRP - 1) release_tmem();
                        __syncwarp();
                        const long long grow0 =
                            (long long)w.m0 + acc * (128 * CG) + (int)rank * 128 + q * 32;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int rr = i * 4 + rd_row;
                            const uint4 v = lds128(staging + rr * 128 + ((rd_chunk ^ (rr & 7)) << 4));
                            const long long grow = grow0 + rr;
                            const int colg = w.n0 + ch * 32 + rd_chunk * 4;
                            if (grow < p.m && colg < n_out) {
                                float* dst = plane + grow * po.ldp + colg;  // ldp % 4 == 0
                                if (colg + 4 <= n_out) {
                                    __stcg(reinterpret_cast<uint4*>(dst), v);
                                } else {
                                    const float* fv = reinterpret_cast<const float*>(&v);
                                    for (int e = 0; e < 4; ++e)
                                        if (colg + e < n_out) dst[e] = fv[e];
                                }
                            }
                        }
                        __syncwarp();
                    }
                }
            }
            NF4_TRACE(3);
            // the staging areas live in weight slots: nobody may decode the next unit into them
            // before every warp has read its staging back
            named_bar_sync(1, PRODUCER_THREADS);
            NF4_TRACE(4);
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
    if (CG == 2) cluster_sync_all();  // the peer may still read this CTA's shared memory / barriers
    if (warp == MMA_WARP) {
        tc_fence_after_sync();
        if (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
        else         tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Adds the split-K planes in slice order, applies the bias and writes fp16: out[i][j] =
// fp16(sum_z ws[z][i][j] + bias[j]). Eight columns per thread, all slices' loads in flight at once.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, long long m, long long n_out, long long ldp,
                     int splits, const __half* __restrict__ bias, __half* __restrict__ out,
                     long long ld_out, int vec_ok) {
    const long long groups_per_row = (n_out + 7) / 8;
    const long long total = m * groups_per_row;
    const size_t plane = (size_t)m * (size_t)ldp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / groups_per_row;
        const long long col = (i % groups_per_row) * 8;
        const float* src = ws + row * ldp + col;
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (col + 8 <= n_out) {
            for (int z0 = 0; z0 < splits; z0 += 4) {
                float4 a[4], b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (z0 + j < splits) {
                        const float4* s4 = reinterpret_cast<const float4*>(src + (size_t)(z0 + j) * plane);
                        a[j] = __ldcs(s4);
                        b[j] = __ldcs(s4 + 1);
                    } else {
                        a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                        b[j] = a[j];
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[0] += a[j].x; v[1] += a[j].y; v[2] += a[j].z; v[3] += a[j].w;
                    v[4] += b[j].x; v[5] += b[j].y; v[6] += b[j].z; v[7] += b[j].w;
                }
            }
        } else {
            for (int z = 0; z < splits; ++z)
                for (int e = 0; e < 8; ++e)
                    if (col + e < n_out) v[e] += src[(size_t)z * plane + e];
        }
        if (bias != nullptr) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + e < n_out) v[e] += __half2float(bias[col + e]);
        }
        __half* dst = out + row * ld_out + col;
        if (vec_ok && col + 8 <= n_out) {
            uint4 o;
            o.x = pack_half2(v[0], v[1]); o.y = pack_half2(v[2], v[3]);
            o.z = pack_half2(v[4], v[5]); o.w = pack_half2(v[6], v[7]);
            *reinterpret_cast<uint4*>(dst) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (col + e < n_out) dst[e] = __float2half_rn(v[e]);
        }
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

static int debug_flags() {
    static int flags = -1;
    if (flags < 0) {
        const char* e = std::getenv("NF4B200_DEBUG");
        flags = e ? std::atoi(e) : 0;
    }
    return flags;
}

// Tiling and split-K plan shared by the launcher and the workspace-size query.
GemmPlan plan_gemm_group(long long m, const long long* n_w, int count, long long k_w, bool trans_w,
                         int sm_count) {
    GemmPlan pl;
    if (m <= 128)      { pl.cg = 1; pl.nacc = 1; }
    else if (m <= 256) { pl.cg = 2; pl.nacc = 1; }
    else               { pl.cg = 2; pl.nacc = 2; }
    if ((debug_flags() & 16) && m > 128 && count == 1) { pl.cg = 1; pl.nacc = 2; }  // tuning
    int force_splits = 0;
    if (const char* e = std::getenv("NF4B200_PLAN")) {  // tuning: "nacc,splits" for pair tiles
        int a = 0, b = 0;
        if (std::sscanf(e, "%d,%d", &a, &b) == 2 && m > 128) {
            if (a == 1 || a == 2) { pl.cg = 2; pl.nacc = a; }
            force_splits = b;
        }
    }
    const int rows = 128 * pl.cg * pl.nacc;
    pl.m_tiles = (int)((m + rows - 1) / rows);
    int n_tiles = 0, nkb = 0;
    size_t ws_floats = 0;
    for (int i = 0; i < count; ++i) {
        if (trans_w) {
            pl.first[i] = nkb;                          // first k-block of problem i
            nkb += (int)((n_w[i] + BK - 1) / BK);
        } else {
            pl.first[i] = n_tiles;                      // first n-tile of problem i
            n_tiles += (int)((n_w[i] + BN - 1) / BN);
            pl.ldp[i] = (n_w[i] + 3) / 4 * 4;
        }
    }
    if (trans_w) {
        n_tiles = (int)((k_w + BN - 1) / BN);
        pl.ldp[0] = (k_w + 3) / 4 * 4;
    } else {
        nkb = (int)((k_w + BK - 1) / BK);
    }
    pl.n_tiles = n_tiles;
    pl.nkb = nkb;
    const long long tiles = (long long)pl.m_tiles * pl.n_tiles;
    const int slots = sm_count / pl.cg;  // units that run at the same time
    int splits = 1;
    if (tiles * 2 <= slots && nkb >= 8) {
        splits = (int)(slots / tiles);
        const int max_by_depth = nkb / 4;  // keep at least 4 k-blocks per slice
        if (splits > max_by_depth) splits = max_by_depth;
        if (splits > 16) splits = 16;
        if (splits < 1) splits = 1;
    }
    if (force_splits > 0) splits = force_splits < nkb ? force_splits : nkb;
    pl.kb_per_split = (nkb + splits - 1) / splits;
    pl.splits = (nkb + pl.kb_per_split - 1) / pl.kb_per_split;  // no empty slice
    for (int i = 0; i < (trans_w ? 1 : count); ++i) {
        pl.ws_off[i] = ws_floats;
        if (pl.splits > 1) ws_floats += (size_t)pl.splits * (size_t)m * (size_t)pl.ldp[i];
    }
    pl.ws_bytes = ws_floats * sizeof(float);
    return pl;
}

GemmPlan plan_gemm(long long m, long long n_w, long long k_w, bool trans_w, int sm_count) {
    return plan_gemm_group(m, &n_w, 1, k_w, trans_w, sm_count);
}

template <int CG, int NACC, bool TRANS_W, int STAGES, int DW, int TABLES>
static cudaError_t launch_cfg(const GemmGroupArgs& ga, const GemmPlan& pl, cudaStream_t stream,
                              const char** why) {
    using L = SmemLayout<CG, NACC, STAGES, TABLES>;
    auto kernel = nf4_gemm_kernel<CG, NACC, TRANS_W, STAGES, DW, TABLES>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::DYNAMIC_BYTES);
    if (e != cudaSuccess) { *why = "cudaFuncSetAttribute(shared memory)"; return e; }

    const GemmArgs& a0 = ga.item[0];
    const long long m = a0.m, k_w = a0.k_w;
    GemmMaps maps;
    GemmParams p;
    p.n_prob = ga.count;
    p.n_ext = 0;
    for (int i = 0; i < ga.count; ++i) {
        const GemmArgs& a = ga.item[i];
        if (TRANS_W || i == 0) {
            const long long kc = TRANS_W ? a.n_w : k_w;
            if (!make_map_2d(&maps.act[i], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a.act, (uint64_t)kc,
                             (uint64_t)m, (uint64_t)a.ld_act * 2, BK, 128,
                             CU_TENSOR_MAP_SWIZZLE_128B)) {
                *why = "cuTensorMapEncodeTiled(activations)";
                return cudaErrorInvalidValue;
            }
        }
        const bool ok = TRANS_W
            ? make_map_2d(&maps.codes[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, a.codes, (uint64_t)k_w / 2,
                          (uint64_t)a.n_w, (uint64_t)k_w / 2, L::NB / 2, BK,
                          CG == 1 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)
            : make_map_2d(&maps.codes[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, a.codes, (uint64_t)k_w / 2,
                          (uint64_t)a.n_w, (uint64_t)k_w / 2, BK / 2, L::NB,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
        if (!ok) { *why = "cuTensorMapEncodeTiled(codes)"; return cudaErrorInvalidValue; }
        GemmProblem& q = p.prob[i];
        q.absmax = a.absmax; q.code2 = a.code2; q.absmax2 = a.absmax2; q.offset = a.offset;
        q.code16 = a.code16; q.bias = a.bias; q.ext_a = a.ext_a; q.ext_b = a.ext_b;
        q.out = a.out; q.ld_out = a.ld_out; q.ws = nullptr; q.ldp = pl.ldp[TRANS_W ? 0 : i];
        q.n_w = (int)a.n_w; q.first = pl.first[i];
        q.nested = a.nested; q.nested_blocksize = a.nested_blocksize;
        q.nested_shift = -1;
        if (a.nested_blocksize > 0 && (a.nested_blocksize & (a.nested_blocksize - 1)) == 0) {
            int sft = 0;
            while ((1 << sft) < a.nested_blocksize) ++sft;
            q.nested_shift = sft;
        }
        q.pad = 0;
        if (a.ext_a != nullptr) ++p.n_ext;
    }
    for (int i = ga.count; i < MAXP; ++i) {
        p.prob[i] = p.prob[0];
        maps.codes[i] = maps.codes[0];
    }
    if (!TRANS_W)
        for (int i = 1; i < MAXP; ++i) maps.act[i] = maps.act[0];
    else
        for (int i = ga.count; i < MAXP; ++i) maps.act[i] = maps.act[0];
    p.status = device_status_word();
    if (p.status == nullptr) { *why = "device status word"; return cudaErrorInvalidValue; }
    p.m = (int)m; p.k_w = (int)k_w;
    p.nkb_total = pl.nkb;
    p.m_tiles = pl.m_tiles;
    p.n_tiles = pl.n_tiles;
    p.splits = pl.splits;
    p.kb_per_split = pl.kb_per_split;
    p.debug = debug_flags();
    if (p.splits > 1) {
        if (a0.workspace == nullptr || a0.workspace_bytes < pl.ws_bytes) {
            p.splits = 1;  // no scratch given: one unit per tile walks the whole K range
            p.kb_per_split = pl.nkb;
        } else {
            for (int i = 0; i < (TRANS_W ? 1 : ga.count); ++i)
                p.prob[i].ws = static_cast<float*>(a0.workspace) + pl.ws_off[i];
        }
    }
    const long long units = (long long)p.m_tiles * p.n_tiles * p.splits;

    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = L::DYNAMIC_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = CG == 2 ? 1 : 0;

    // Units that can be resident at once: one CTA per SM; pairs must sit in one GPC, so ask the
    // runtime how many clusters fit (once per configuration).
    int slots = a0.sm_count / CG;
    if (CG == 2) {
        static int max_clusters = -1;
        if (max_clusters < 0) {
            cfg.gridDim = dim3((unsigned)(a0.sm_count / 2) * 2, 1, 1);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) == cudaSuccess && n > 0)
                max_clusters = n;
            else
                max_clusters = a0.sm_count / 2;
        }
        if (max_clusters < slots) slots = max_clusters;
    }
    const unsigned grid = (unsigned)(units < slots ? units : slots) * CG;
    cfg.gridDim = dim3(grid, 1, 1);
    e = cudaLaunchKernelEx(&cfg, kernel, maps, p);
    if (e != cudaSuccess) { *why = "kernel launch"; return e; }

    if (p.splits > 1) {
        for (int i = 0; i < (TRANS_W ? 1 : ga.count); ++i) {
            const GemmArgs& a = ga.item[i];
            const long long n_out = TRANS_W ? k_w : a.n_w;
            const long long total = m * ((n_out + 7) / 8);
            long long blocks = (total + 255) / 256;
            const long long cap = (long long)a0.sm_count * 8;
            if (blocks > cap) blocks = cap;
            const int vec_ok = (a.ld_out % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.out) & 15) == 0);
            splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
                p.prob[i].ws, m, n_out, p.prob[i].ldp, p.splits, TRANS_W ? nullptr : a.bias, a.out,
                a.ld_out, vec_ok);
            e = cudaGetLastError();
            if (e != cudaSuccess) { *why = "split-K reduce launch"; return e; }
        }
    }
    return e;
}

cudaError_t launch_gemm_group(const GemmGroupArgs& ga, cudaStream_t stream, const char** why) {
    *why = "";
    if (ga.count < 1 || ga.count > GEMM_MAX_GROUP) { *why = "group size"; return cudaErrorInvalidValue; }
    long long n_w[GEMM_MAX_GROUP];
    for (int i = 0; i < ga.count; ++i) n_w[i] = ga.item[i].n_w;
    const GemmArgs& a = ga.item[0];
    const GemmPlan pl = plan_gemm_group(a.m, n_w, ga.count, a.k_w, a.trans_w, a.sm_count);
    const bool dw8 = (debug_flags() & 32) != 0;  // tuning: 8 decoding warps with twice the work
    if (pl.cg == 2 && pl.nacc == 2) {
        if (dw8)
            return a.trans_w ? launch_cfg<2, 2, true, 4, 8, MAXP>(ga, pl, stream, why)
                             : launch_cfg<2, 2, false, 4, 8, MAXP>(ga, pl, stream, why);
        return a.trans_w ? launch_cfg<2, 2, true, 4, 16, MAXP>(ga, pl, stream, why)
                         : launch_cfg<2, 2, false, 4, 16, MAXP>(ga, pl, stream, why);
    }
    if (pl.cg == 2)
        return a.trans_w ? launch_cfg<2, 1, true, 6, 16, MAXP>(ga, pl, stream, why)
                         : launch_cfg<2, 1, false, 6, 16, MAXP>(ga, pl, stream, why);
    if (pl.nacc == 2)
        return a.trans_w ? launch_cfg<1, 2, true, 3, 16, 1>(ga, pl, stream, why)
                         : launch_cfg<1, 2, false, 3, 16, 1>(ga, pl, stream, why);
    if (ga.count > 1)  // small-M groups: one stage less makes room for every problem's table
        return a.trans_w ? launch_cfg<1, 1, true, 3, 16, MAXP>(ga, pl, stream, why)
                         : launch_cfg<1, 1, false, 3, 16, MAXP>(ga, pl, stream, why);
    return a.trans_w ? launch_cfg<1, 1, true, 4, 16, 1>(ga, pl, stream, why)
                     : launch_cfg<1, 1, false, 4, 16, 1>(ga, pl, stream, why);
}

cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream, const char** why) {
    GemmGroupArgs ga;
    ga.count = 1;
    ga.item[0] = a;
    return launch_gemm_group(ga, stream, why);
}

}  // namespace nf4

// Tuning aid, not part of the public ABI: copies the phase timestamps to the host.
extern "C" int nf4dbg_read_trace(unsigned long long* dst, int max_entries) {
    const int n = nf4::TRACE_CTAS * nf4::TRACE_UNITS * nf4::TRACE_STAMPS;
    if (max_entries < n) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -2;
    if (cudaMemcpyFromSymbol(dst, nf4::g_trace, sizeof(unsigned long long) * n) != cudaSuccess)
        return -3;
    return n;
}

extern "C" int nf4dbg_read_trace2(unsigned long long* dst, int max_entries) {
    const int n = 2 * nf4::TRACE2_EVENTS * nf4::TRACE2_ITERS;
    if (max_entries < n) return -1;
    if (cudaDeviceSynchronize() != cudaSuccess) return -2;
    if (cudaMemcpyFromSymbol(dst, nf4::g_trace2, sizeof(unsigned long long) * n) != cudaSuccess)
        return -3;
    return n;
}
