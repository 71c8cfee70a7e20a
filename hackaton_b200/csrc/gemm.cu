// Fused NF4 dequant-GEMM for sm_100a: TMA -> producer-warp decode -> tcgen05.mma (TMEM).
//
// Forward  (TRANS_W = false): out[M, N_w] = act[M, K_w] . W^T (+ bias) (+ ext_a . ext_b^T)
// Backward (TRANS_W = true):  out[M, K_w] = act[M, N_w] . W          (+ ext_a . ext_b)
// replacing the reference's "decode the whole weight to fp16 in HBM, then cuBLAS"
// (solution/nf4.py:87-92 forward, 94-99 backward). W never exists in HBM as fp16 here.
//
// One CTA computes a (128*NACC) x BN output tile. Roles (10 warps):
//   warp 0      TMA: activation tiles (128-byte swizzle) and the packed-code tile of each
//               64-deep k-block into a STAGES-deep ring of shared memory.
//   warp 1      allocates TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=16) and commits
//               each k-block to the ring's "empty" barrier.
//   warps 2..9  producers: read the code tile from shared memory, fetch the block scales
//               (u8 absmax -> second-level table -> * absmax2 + offset, prefetched one k-block
//               ahead), expand codes through a register-resident fp16 table and write the fp16
//               weight tile in the 128-byte-swizzled layout the MMA descriptor expects. After
//               the main loop the same warps run the epilogue (tcgen05.ld -> fp16 -> global).
// The weight tile is always stored as rows of n_w holding 64 consecutive k_w (128 bytes, chunk
// index XOR row%8). Forward reads it as a K-major B operand; backward as an MN-major one.
// With NACC = 2 both accumulators (two 128-row halves of the token tile) reuse each decoded
// weight tile, halving the decode work per flop.
//
// The rank-16 LoRA term rides along as one extra K=16 MMA step after the main loop ("K
// extension"): its two small operands are copied by the producers into the ring slot in the
// unswizzled core-matrix layout.
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

constexpr int GEMM_THREADS = 320;
constexpr int PRODUCER_THREADS = 256;
constexpr int BK = 64;  // k-block depth = one quantisation block

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
    long long ld_out;
    int m, n_w, k_w;
    int nested, nested_blocksize;
};

template <int NACC, int BN, int STAGES>
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

template <int NACC, int BN, bool TRANS_W, int STAGES>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
nf4_gemm_kernel(const __grid_constant__ CUtensorMap tm_act,
                const __grid_constant__ CUtensorMap tm_codes, const GemmParams p) {
    using L = SmemLayout<NACC, BN, STAGES>;
    constexpr int CHUNKS = BN * 2 / PRODUCER_THREADS;  // 16-byte code chunks per producer thread
    static_assert(CHUNKS >= 1, "tile too small for the producer count");
    static_assert(!TRANS_W || BN == 256, "backward tiles are 256 wide");
    constexpr uint32_t TMEM_COLS = NACC * BN;
    static_assert(TMEM_COLS == 128 || TMEM_COLS == 256 || TMEM_COLS == 512, "TMEM columns");

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

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * (128 * NACC);
    const int n0 = blockIdx.y * BN;  // first output column of this tile
    const int kc = TRANS_W ? p.n_w : p.k_w;  // contraction length
    const int nkb = (kc + BK - 1) / BK;
    const bool has_ext = p.ext_a != nullptr;
    const int n_iter = nkb + (has_ext ? 1 : 0);
    const int blocks_per_row = p.k_w / 64;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full_tma(s), 1);
            mbar_init(bar_full_w(s), PRODUCER_THREADS);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_accum, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_act);
        tma_prefetch_desc(&tm_codes);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), TMEM_COLS);
        tmem_relinquish();
    }
    if (p.nested && threadIdx.x >= 64) table2[threadIdx.x - 64] = p.code2[threadIdx.x - 64];
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    auto stage_a = [&](int s) { return smem_base + (uint32_t)s * L::STAGE_BYTES; };
    auto stage_w = [&](int s) { return smem_base + (uint32_t)s * L::STAGE_BYTES + L::A_BYTES; };
    auto stage_c = [&](int s) {
        return smem_base + (uint32_t)s * L::STAGE_BYTES + L::A_BYTES + L::W_BYTES;
    };

    int fail = 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag)) { fail = 1; break; }
                if (it < nkb) {
                    mbar_arrive_expect_tx(bar_full_tma(s), L::A_BYTES + L::C_BYTES);
#pragma unroll
                    for (int a = 0; a < NACC; ++a)
                        tma_load_2d(stage_a(s) + a * (128 * BK * 2), &tm_act, it * BK,
                                    m0 + a * 128, bar_full_tma(s));
                    if (TRANS_W)
                        tma_load_2d(stage_c(s), &tm_codes, n0 / 2, it * BK, bar_full_tma(s));
                    else
                        tma_load_2d(stage_c(s), &tm_codes, it * (BK / 2), n0, bar_full_tma(s));
                } else {
                    mbar_arrive(bar_full_tma(s));  // extension step: operands come from producers
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(BN, 0u, TRANS_W ? 1u : 0u);
            for (int it = 0; it < n_iter; ++it) {
                const int s = it % STAGES;
                const uint32_t ph = (it / STAGES) & 1;
                if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 2; break; }
                if (!mbar_wait(bar_full_w(s), ph, abort_flag)) { fail = 3; break; }
                tc_fence_after_sync();
                if (it < nkb) {
                    const uint64_t bdesc0 = TRANS_W
                        ? make_smem_desc(stage_w(s), 64 * 128, 1024, LAYOUT_SW128)
                        : make_smem_desc(stage_w(s), 16, 1024, LAYOUT_SW128);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k) {
                        const uint64_t bdesc = bdesc0 + (uint64_t)(TRANS_W ? (16 * 128) >> 4 : 32 >> 4) * k;
#pragma unroll
                        for (int a = 0; a < NACC; ++a) {
                            const uint64_t adesc =
                                make_smem_desc(stage_a(s) + a * (128 * BK * 2), 16, 1024,
                                               LAYOUT_SW128) +
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
                    const uint64_t bdesc =
                        TRANS_W ? make_smem_desc(stage_w(s), BN * 16, 128, LAYOUT_NONE)
                                : make_smem_desc(stage_w(s), 128, 256, LAYOUT_NONE);
#pragma unroll
                    for (int a = 0; a < NACC; ++a) {
                        const uint64_t adesc =
                            make_smem_desc(stage_a(s) + a * (128 * BK * 2), 128, 256, LAYOUT_NONE);
                        umma_f16(tmem_base + a * BN, adesc, bdesc, idesc, 1u);
                    }
                }
                umma_commit(bar_empty(s));
            }
            if (!fail) umma_commit(bar_accum);
        }
    } else {
        // ------------------------------------------------------------------ decode producers
        const int pt = threadIdx.x - 64;  // 0..255
        RegLut lut;
        {
            uint16_t bits[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) bits[i] = __half_as_ushort(__float2half_rn(p.code16[i]));
            lut = make_reg_lut(bits);
        }
        const float offset = p.nested ? *p.offset : 0.f;

        // Chunk geometry. Forward: the code tile is [BN rows][32 B]; chunk c covers row c/2,
        // half c%2 of the 64-wide k-block. Backward: the tile is [64 rows][128 B], 128-byte
        // swizzled by TMA; 8 consecutive lanes take 8 different rows of one chunk column so that
        // both the swizzled reads and the swizzled writes are bank-conflict free.
        int c_row[CHUNKS], c_col[CHUNKS];
        uint32_t c_src[CHUNKS], c_dst[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j) {
            const int c = pt + PRODUCER_THREADS * j;
            if (!TRANS_W) {
                const int row = c >> 1, half = c & 1;
                c_row[j] = row;
                c_col[j] = half;
                c_src[j] = (uint32_t)c * 16u;
                c_dst[j] = (uint32_t)(row >> 3) * 1024u + (uint32_t)(row & 7) * 128u;
            } else {
                const int row = ((c >> 6) << 3) | (c & 7), cc = (c >> 3) & 7;
                c_row[j] = row;
                c_col[j] = cc;
                c_src[j] = (uint32_t)row * 128u + (uint32_t)((cc ^ (row & 7)) << 4);
                c_dst[j] = (uint32_t)(cc >> 1) * 8192u + (uint32_t)(row >> 3) * 1024u +
                           (uint32_t)(row & 7) * 128u;
            }
        }

        // Scale prefetch registers: raw first-level entry (u8 code or fp32 bits) and the
        // second-level scale, loaded one k-block ahead.
        uint32_t raw_q[CHUNKS];
        float raw_a2[CHUNKS];
        bool raw_ok[CHUNKS];
        auto fetch_scale = [&](int kb, int j) {
            long long n, blk;
            bool ok;
            if (!TRANS_W) {
                n = (long long)n0 + c_row[j];
                blk = n * blocks_per_row + kb;
                ok = n < p.n_w;
            } else {
                n = (long long)kb * BK + c_row[j];
                const int kw = n0 + c_col[j] * 32;
                blk = n * blocks_per_row + (kw >> 6);
                ok = n < p.n_w && kw < p.k_w;
            }
            raw_q[j] = 0;
            raw_a2[j] = 0.f;
            raw_ok[j] = ok;
            if (ok) {
                if (p.nested) {
                    raw_q[j] = __ldg(static_cast<const uint8_t*>(p.absmax) + blk);
                    raw_a2[j] = __ldg(p.absmax2 + blk / p.nested_blocksize);
                } else {
                    raw_q[j] = __float_as_uint(__ldg(static_cast<const float*>(p.absmax) + blk));
                }
            }
        };
#pragma unroll
        for (int j = 0; j < CHUNKS; ++j) fetch_scale(0, j);

        for (int it = 0; it < n_iter; ++it) {
            const int s = it % STAGES;
            const uint32_t ph = (it / STAGES) & 1;
            if (it < nkb) {
                __half2 scale2[CHUNKS];
#pragma unroll
                for (int j = 0; j < CHUNKS; ++j) {
                    float sc;
                    if (!raw_ok[j])
                        sc = 0.f;  // rows / columns outside the weight contribute zeros
                    else if (p.nested)
                        sc = nested_scale(table2[raw_q[j]], raw_a2[j], offset);
                    else
                        sc = __uint_as_float(raw_q[j]);
                    scale2[j] = __float2half2_rn(sc);
                }
                if (it + 1 < nkb) {
#pragma unroll
                    for (int j = 0; j < CHUNKS; ++j) fetch_scale(it + 1, j);
                }
                if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                uint8_t* cbase = smem_gen + (stage_c(s) - smem_base);
                uint8_t* wbase = smem_gen + (stage_w(s) - smem_base);
#pragma unroll
                for (int j = 0; j < CHUNKS; ++j) {
                    const uint4 cw = *reinterpret_cast<const uint4*>(cbase + c_src[j]);
                    const uint32_t words[4] = {cw.x, cw.y, cw.z, cw.w};
                    const int sw = c_row[j] & 7;
                    const int chunk0 = TRANS_W ? (c_col[j] & 1) * 4 : c_col[j] * 4;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const uint4 v = decode_word_reg(words[i], lut, scale2[j]);
                        *reinterpret_cast<uint4*>(wbase + c_dst[j] + (((chunk0 + i) ^ sw) << 4)) = v;
                    }
                }
            } else {
                // K extension operands, unswizzled core-matrix layout (see the MMA branch).
                if (!mbar_wait(bar_full_tma(s), ph, abort_flag)) { fail = 4; break; }
                uint8_t* abase = smem_gen + (stage_a(s) - smem_base);
                uint8_t* wbase = smem_gen + (stage_w(s) - smem_base);
                const uint4 zero = make_uint4(0, 0, 0, 0);
                // ext_a rows m0 .. m0 + 128*NACC: two 16-byte halves per row
                for (int c = pt; c < 128 * NACC * 2; c += PRODUCER_THREADS) {
                    const int row = c >> 1, half = c & 1;
                    const long long gm = (long long)m0 + row;
                    uint4 v = zero;
                    if (gm < p.m)
                        v = __ldg(reinterpret_cast<const uint4*>(p.ext_a + gm * 16) + half);
                    const int acc = row >> 7, r = row & 127;
                    *reinterpret_cast<uint4*>(abase + acc * (128 * BK * 2) + (r >> 3) * 256 +
                                              half * 128 + (r & 7) * 16) = v;
                }
                if (!TRANS_W) {
                    for (int c = pt; c < BN * 2; c += PRODUCER_THREADS) {
                        const int row = c >> 1, half = c & 1;
                        const long long gn = (long long)n0 + row;
                        uint4 v = zero;
                        if (gn < p.n_w)
                            v = __ldg(reinterpret_cast<const uint4*>(p.ext_b + gn * 16) + half);
                        *reinterpret_cast<uint4*>(wbase + (row >> 3) * 256 + half * 128 +
                                                  (row & 7) * 16) = v;
                    }
                } else {
                    // lora_a [16, K_w]: chunk (r, g) = 8 consecutive k_w of rank row r
                    for (int c = pt; c < 16 * (BN / 8); c += PRODUCER_THREADS) {
                        const int r = c / (BN / 8), g = c % (BN / 8);
                        const long long kw = (long long)n0 + g * 8;
                        uint4 v = zero;
                        if (kw < p.k_w)
                            v = __ldg(reinterpret_cast<const uint4*>(p.ext_b + (long long)r * p.k_w + kw));
                        *reinterpret_cast<uint4*>(wbase + (r >> 3) * (BN * 16) + g * 128 +
                                                  (r & 7) * 16) = v;
                    }
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(bar_full_w(s));
        }

        // ------------------------------------------------------------------ epilogue
        if (!fail) {
            if (!mbar_wait(bar_accum, 0u, abort_flag)) fail = 5;
        }
        if (!fail) {
            tc_fence_after_sync();
            const int q = warp & 3;           // TMEM lane quadrant this warp may read
            const int grp = (warp - 2) >> 2;  // 0 or 1
            const int acc = NACC == 2 ? grp : 0;
            const int chunk_begin = NACC == 2 ? 0 : grp * (BN / 64);
            const int chunk_end = NACC == 2 ? BN / 32 : (grp + 1) * (BN / 64);
            const long long row = (long long)m0 + acc * 128 + q * 32 + lane;
            const int n_out = TRANS_W ? p.k_w : p.n_w;
            const bool vec_ok = (p.ld_out % 8 == 0) &&
                                ((reinterpret_cast<uintptr_t>(p.out) & 15) == 0);
            for (int ch = chunk_begin; ch < chunk_end; ++ch) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN + ch * 32, r);
                tmem_ld_wait();
                const int col0 = n0 + ch * 32;
                if (row < p.m && col0 < n_out) {
                    __half* dst = p.out + row * p.ld_out + col0;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        float v[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[g * 8 + e]);
                        const int col = col0 + g * 8;
                        if (!TRANS_W && p.bias != nullptr) {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (col + e < n_out) v[e] += __half2float(p.bias[col + e]);
                        }
                        if (vec_ok && col + 8 <= n_out) {
                            uint4 o;
                            __half2 h;
                            h = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
                            h = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
                            *reinterpret_cast<uint4*>(dst + g * 8) = o;
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                if (col + e < n_out) dst[g * 8 + e] = __float2half_rn(v[e]);
                        }
                    }
                }
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
    if (warp == 1) {
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

template <int NACC, int BN, bool TRANS_W, int STAGES>
static cudaError_t launch_cfg(const GemmArgs& a, cudaStream_t stream, const char** why) {
    using L = SmemLayout<NACC, BN, STAGES>;
    auto kernel = nf4_gemm_kernel<NACC, BN, TRANS_W, STAGES>;
    static std::once_flag once;
    static cudaError_t attr_err = cudaSuccess;
    std::call_once(once, [&] {
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        L::DYNAMIC_BYTES);
    });
    // the attribute is per device; set it again when another device is current (cheap)
    if (attr_err == cudaSuccess)
        attr_err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        L::DYNAMIC_BYTES);
    if (attr_err != cudaSuccess) { *why = "cudaFuncSetAttribute(shared memory)"; return attr_err; }

    const long long kc = TRANS_W ? a.n_w : a.k_w;
    const long long n_out = TRANS_W ? a.k_w : a.n_w;
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
    if (p.status == nullptr) { *why = "device status word"; return cudaErrorInvalidValue; }

    dim3 grid((unsigned)((a.m + 128 * NACC - 1) / (128 * NACC)), (unsigned)((n_out + BN - 1) / BN));
    kernel<<<grid, GEMM_THREADS, L::DYNAMIC_BYTES, stream>>>(tm_act, tm_codes, p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) *why = "kernel launch";
    return e;
}

cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream, const char** why) {
    *why = "";
    if (a.m > 128) {
        return a.trans_w ? launch_cfg<2, 256, true, 3>(a, stream, why)
                         : launch_cfg<2, 256, false, 3>(a, stream, why);
    }
    return a.trans_w ? launch_cfg<1, 256, true, 4>(a, stream, why)
                     : launch_cfg<1, 256, false, 4>(a, stream, why);
}

}  // namespace nf4
