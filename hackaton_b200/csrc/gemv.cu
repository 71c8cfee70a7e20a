// NF4 linear for a handful of token rows (the decode shapes of serving), both directions:
//   forward  (M <= 64): out_i[M, N_i] = act[M, K] . W_i^T (+ bias_i) (+ ext_a_i . ext_b_i^T)
//   backward (M <= 16): out[M, K]     = sum_i act_i[M, N_i] . W_i  (+ ext_a_i . ext_b_i)
// for a group of up to four weights that share K (forward: they also share the activations).
// At these sizes the work is reading the packed weights once (0.52 B per weight); a 128-row
// tensor-core tile would be 50-99 % padding and the persistent tcgen05 kernel's set-up and
// epilogue would dominate. So: no shared-memory ring, no TMEM. Warps stream the codes straight
// from global memory, expand them in registers with the same byte-permute table look-up as the
// big kernel (same rounding: fp16(table) * fp16(scale)) and multiply with warp-level mma.sync
// (m16n8k16, fp32 accumulate). Forward with up to 8 token rows: a byte -> fp16-pair table in
// shared memory instead, and the block scale applied to each k-block's fp32 sums.
//
// Forward: a CTA owns 16 weight rows of one member of the group, its warps split the 64-deep
// k-blocks. The contraction index is visited in a permuted order that A (weights) and B (tokens)
// share, so a thread's 16 consecutive weights and 16 consecutive activations feed four k16 steps
// without any shuffle. The warps' partial tiles are added through shared memory; bias and the
// rank-16 LoRA term are applied there.
//
// Backward: the contraction runs over weight rows, along which the codes are NOT contiguous. A
// warp owns one k-block (64 output columns) and a slab of weight rows; per step of 16 rows lane
// (g, t) decodes one 32-bit word (8 columns: word g of the k-block) of rows 2t, 2t+1, 2t+8, 2t+9
// and issues eight MMAs, one per column position c of its word: in MMA c the B operand's column
// g is "column c of word g", so the fragment a thread needs (two consecutive contraction rows of
// one column) is a byte-permute of two of its own decoded words. A (the upstream gradient,
// row-major over the contraction) is loaded as plain fragments. A thread ends up with 16
// consecutive output columns of tokens g and g + 8. Row slabs are summed in two steps: the
// warps of a CTA through shared memory, the CTAs of a k-block as fp32 planes in caller-provided
// scratch, which the last CTA of the k-block to finish (a ticket counter) adds in slab order
// (deterministic) and writes out as fp16.
//
// Both kernels ask for their slab of codes to be brought into L2 before they wait for the
// previous kernel of the stream (programmatic dependent launch): a prefetch reads no values, so
// it needs no ordering, and in a chain of small launches the weights of launch i + 1 travel
// from HBM while launch i runs.
//
// Both need the ready-made fp16 block-scale table (kernels.h, launch_prepare_scales) and
// N % 16 == 0; other calls take the tcgen05 kernel.
#include <cuda_fp16.h>

#include <atomic>

#include "decode.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

constexpr int GV_ROWS = 16;
#ifndef GV_BATCH_N
#define GV_BATCH_N 4
#endif
constexpr int GV_BATCH = GV_BATCH_N;
constexpr int GV_MAXP = GEMM_MAX_GROUP;

struct GemvProblem {
    const uint8_t* codes;
    const __half* scales16;  // [K / 64][N]
    const float* code16;
    const __half* bias;
    const __half* ext_a;     // forward: [M, 16] or null; backward: u [M, 16] or null
    const __half* ext_b;     // forward: lora_b [N, 16]; backward: lora_a [16, K]
    const __half* act;       // backward: this member's dY [M, N]
    __half* out;             // forward: this member's output
    long long ld_out, ld_act;
    int n_w;
    int first;               // forward: first CTA of this member; backward: first row slab
};

struct GemvParams {
    GemvProblem prob[GV_MAXP];
    const __half* act;       // forward: shared activations
    long long ld_act;
    float* planes;           // backward: [slabs][M][ldp] fp32
    long long ldp;
    int n_prob, m, k_w;
    int rows_per_slab;       // backward: weight rows per CTA (multiple of 16 * warps)
    int ticket_base;         // backward: first ticket of this launch, or -1 (reduction by a second kernel)
    int n_slabs;
    int prefetch;            // codes are 16-byte aligned: bulk L2 prefetch is legal
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// The same with a zero accumulator going in (first step of a k-block whose sums are scaled
// afterwards).
__device__ __forceinline__ void mma_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
    const float z = 0.f;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(z));
}

__device__ __forceinline__ uint32_t gv_lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// Forward decode by byte: a 256-entry table in shared memory maps a byte of codes to its two
// unscaled fp16 table values (first weight = high nibble in the low half), kept in PAIR_COPIES
// copies (lane l reads copy l % PAIR_COPIES) so that a warp's look-ups spread over the banks.
// One look-up per two weights instead of 27 register instructions per eight; the block scale
// is applied to the k-block's fp32 sums instead of to every weight (one rounding less). Used for
// up to 8 token rows (one token block): measured at M = 1, each group timed alone, 26.2 -> 24.0 us
// per layer forward, while with two token blocks (M = 16) the per-block scaling costs more than
// the look-ups save (gate/up 14.8 -> 19.0 us), so those keep the register look-up.
constexpr int PAIR_COPIES = 8;

__device__ __forceinline__ RegLut load_reg_lut(const float* code16) {
    uint16_t bits[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) bits[i] = __half_as_ushort(__float2half_rn(__ldg(code16 + i)));
    return make_reg_lut(bits);
}

__device__ __forceinline__ int gemv_find(const GemvParams& p, int idx) {
    int r = 0;
#pragma unroll
    for (int i = 1; i < GV_MAXP; ++i)
        if (i < p.n_prob && idx >= p.prob[i].first) r = i;
    return r;
}

// Asks for `bytes` starting at `ptr` (16-byte aligned, multiple of 16) to be brought into L2, in
// pieces the bulk-prefetch instruction takes.
__device__ __forceinline__ void prefetch_span(const uint8_t* ptr, long long bytes) {
    constexpr long long PIECE = 32768;
    for (long long off = 0; off < bytes; off += PIECE) {
        const long long n = bytes - off < PIECE ? bytes - off : PIECE;
        bulk_prefetch_l2(ptr + off, (uint32_t)n);
    }
}

// (the 4-warp instantiation for one token block is capped at 64 registers: eight CTAs per SM, so
// the 1120 CTAs of a gate/up group are one wave)
template <int NT, int GV_WARPS>  // token blocks of 8 (M <= 8 * NT); warps that split K
__global__ void __launch_bounds__(GV_WARPS * 32, (GV_WARPS == 4 && NT == 1) ? 8 : 1)
nf4_gemv_kernel(const __grid_constant__ GemvParams p) {
    constexpr int GV_THREADS = GV_WARPS * 32;
    const int pi = gemv_find(p, (int)blockIdx.x);
    const GemvProblem& pr = p.prob[pi];
    const int r0 = ((int)blockIdx.x - pr.first) * GV_ROWS;
    const size_t row_bytes = (size_t)p.k_w >> 1;
    // The CTA's 16 rows of codes are one contiguous span: on its way to L2 while the previous
    // kernel of the stream is still running.
    if (threadIdx.x == 0 && p.prefetch)
        prefetch_span(pr.codes + (size_t)r0 * row_bytes, (long long)(GV_ROWS * row_bytes));
    grid_dep_wait();
    grid_dep_launch();
    __shared__ float red[GV_WARPS][NT * 8][GV_ROWS + 1];
    constexpr bool PAIR = NT == 1;
    __shared__ uint32_t pair_table[PAIR ? 256 * PAIR_COPIES : 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r_lo = r0 + g, r_hi = r0 + g + 8;  // n_w % 16 == 0: both inside the weight

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int nkb = p.k_w >> 6;
#ifdef GV_INTERLEAVE
    // warps take the k-blocks in turn: at any moment the warps of a CTA read neighbouring 32-byte
    // pieces of the same 128-byte lines
    const int kb_begin = warp, kb_end = nkb;
    constexpr int KB_STEP = GV_WARPS;
#else
    const int kb_begin = nkb * warp / GV_WARPS, kb_end = nkb * (warp + 1) / GV_WARPS;
    constexpr int KB_STEP = 1;
#endif
    const uint8_t* c_lo = pr.codes + (size_t)r_lo * row_bytes + t * 8;
    const uint8_t* c_hi = pr.codes + (size_t)r_hi * row_bytes + t * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // k-blocks in batches of GV_BATCH: all of a batch's code and scale loads are issued before the
    // first one is used, so a warp pays the memory latency once per batch, not once per k-block.
    // The first batch goes out before the table look-up is built, so that the table's own loads
    // share its round trip instead of preceding it.
    uint2 q_lo[GV_BATCH], q_hi[GV_BATCH];
    __half s_lo[GV_BATCH], s_hi[GV_BATCH];
    auto issue = [&](int kb0) {
#pragma unroll
        for (int b = 0; b < GV_BATCH; ++b) {
            const int kb = min(kb0 + b * KB_STEP, kb_end - 1);  // (tail: re-reads the last block, unused)
            // this thread's 16 weights of rows r_lo and r_hi: k = kb*64 + 16t .. + 15
            q_lo[b] = __ldg(reinterpret_cast<const uint2*>(c_lo + (size_t)kb * 32));
            q_hi[b] = __ldg(reinterpret_cast<const uint2*>(c_hi + (size_t)kb * 32));
            s_lo[b] = __ldg(pr.scales16 + (size_t)kb * pr.n_w + r_lo);
            s_hi[b] = __ldg(pr.scales16 + (size_t)kb * pr.n_w + r_hi);
        }
    };
    if (kb_begin < kb_end) issue(kb_begin);
    RegLut lut = {};
    uint32_t pair_base = 0;
    if constexpr (PAIR) {
        // (red is free until the fold: it holds the 16 fp16 table values while the pairs are built)
        unsigned short* t16 = reinterpret_cast<unsigned short*>(&red[0][0][0]);
        if (threadIdx.x < 16)
            t16[threadIdx.x] = __half_as_ushort(__float2half_rn(__ldg(pr.code16 + threadIdx.x)));
        __syncthreads();
        for (int i = threadIdx.x; i < 256 * PAIR_COPIES; i += GV_THREADS) {
            const int e = i / PAIR_COPIES;
            pair_table[i] = (uint32_t)t16[e >> 4] | ((uint32_t)t16[e & 15] << 16);
        }
        __syncthreads();
        pair_base = (uint32_t)__cvta_generic_to_shared(pair_table) + (lane % PAIR_COPIES) * 4;
    } else {
        lut = load_reg_lut(pr.code16);
    }
    auto pairs = [&](uint32_t w, uint32_t (&o)[8], int at) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            o[at + i] = gv_lds32(pair_base + ((w >> (8 * i)) & 0xFFu) * (4u * PAIR_COPIES));
    };

    for (int kb0 = kb_begin; kb0 < kb_end; kb0 += GV_BATCH * KB_STEP) {
        if (kb0 != kb_begin) issue(kb0);
#pragma unroll
        for (int b = 0; b < GV_BATCH; ++b) {
            const int kb = kb0 + b * KB_STEP;
            if (kb >= kb_end) break;
            uint32_t wl[8], wh[8];
            const float f_lo = __half2float(s_lo[b]), f_hi = __half2float(s_hi[b]);
            if constexpr (PAIR) {
                pairs(q_lo[b].x, wl, 0); pairs(q_lo[b].y, wl, 4);
                pairs(q_hi[b].x, wh, 0); pairs(q_hi[b].y, wh, 4);
            } else {
                const uint4 a = decode_word_reg(q_lo[b].x, lut, __half2half2(s_lo[b]));
                const uint4 c = decode_word_reg(q_lo[b].y, lut, __half2half2(s_lo[b]));
                wl[0] = a.x; wl[1] = a.y; wl[2] = a.z; wl[3] = a.w;
                wl[4] = c.x; wl[5] = c.y; wl[6] = c.z; wl[7] = c.w;
                const uint4 d = decode_word_reg(q_hi[b].x, lut, __half2half2(s_hi[b]));
                const uint4 e = decode_word_reg(q_hi[b].y, lut, __half2half2(s_hi[b]));
                wh[0] = d.x; wh[1] = d.y; wh[2] = d.z; wh[3] = d.w;
                wh[4] = e.x; wh[5] = e.y; wh[6] = e.z; wh[7] = e.w;
            }
            const long long kcol = (long long)kb * 64 + t * 16;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                // the same 16 k of token nt*8 + g: k16 step j takes words 2j, 2j+1 of both operands
                const int token = nt * 8 + g;
                uint4 x0 = zero, x1 = zero;
                if (token < p.m) {
                    const uint4* xp =
                        reinterpret_cast<const uint4*>(p.act + (long long)token * p.ld_act + kcol);
                    x0 = __ldg(xp);
                    x1 = __ldg(xp + 1);
                }
                if constexpr (PAIR) {
                // unscaled sums of this k-block, then the rows' block scales (d0, d1: row g; d2, d3: g + 8)
                float blk[4];
                mma_16816_first(blk, wl[0], wh[0], wl[1], wh[1], x0.x, x0.y);
                mma_16816(blk, wl[2], wh[2], wl[3], wh[3], x0.z, x0.w);
                mma_16816(blk, wl[4], wh[4], wl[5], wh[5], x1.x, x1.y);
                mma_16816(blk, wl[6], wh[6], wl[7], wh[7], x1.z, x1.w);
                acc[nt][0] = fmaf(f_lo, blk[0], acc[nt][0]);
                acc[nt][1] = fmaf(f_lo, blk[1], acc[nt][1]);
                acc[nt][2] = fmaf(f_hi, blk[2], acc[nt][2]);
                acc[nt][3] = fmaf(f_hi, blk[3], acc[nt][3]);
                } else {
                mma_16816(acc[nt], wl[0], wh[0], wl[1], wh[1], x0.x, x0.y);
                mma_16816(acc[nt], wl[2], wh[2], wl[3], wh[3], x0.z, x0.w);
                mma_16816(acc[nt], wl[4], wh[4], wl[5], wh[5], x1.x, x1.y);
                mma_16816(acc[nt], wl[6], wh[6], wl[7], wh[7], x1.z, x1.w);
                }
            }
        }
    }
    __syncthreads();   // (the pair table build used `red`; every warp is past its look-ups)

    // accumulator fragment: d0,d1 -> (weight row g, tokens 2t, 2t+1); d2,d3 -> (row g+8, same)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        red[warp][nt * 8 + 2 * t][g] = acc[nt][0];
        red[warp][nt * 8 + 2 * t + 1][g] = acc[nt][1];
        red[warp][nt * 8 + 2 * t][g + 8] = acc[nt][2];
        red[warp][nt * 8 + 2 * t + 1][g + 8] = acc[nt][3];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < NT * 8 * GV_ROWS; e += GV_THREADS) {
        const int token = e / GV_ROWS, r = e % GV_ROWS;  // 16 consecutive rows: 32 bytes of out
        if (token >= p.m) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GV_WARPS; ++w) v += red[w][token][r];
        if (pr.ext_a != nullptr) {
            const __half2* xa = reinterpret_cast<const __half2*>(pr.ext_a + (long long)token * 16);
            const __half2* lb = reinterpret_cast<const __half2*>(pr.ext_b + (long long)(r0 + r) * 16);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 a = __half22float2(__ldg(xa + j)), b = __half22float2(__ldg(lb + j));
                s = fmaf(a.x, b.x, s);
                s = fmaf(a.y, b.y, s);
            }
            v += s;
        }
        if (pr.bias != nullptr) v += __half2float(__ldg(pr.bias + r0 + r));
        pr.out[(long long)token * pr.ld_out + r0 + r] = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------------------------ backward

constexpr int GB_BATCH = 4;   // 16-row steps whose loads are in flight together

// One ticket per k-block of a launch in flight: the CTA that takes the last ticket of its k-block
// adds the slabs' planes and writes the result, so small problems need no second kernel. The
// tickets start at zero (module load) and the last arriver puts its ticket back to zero. Launches
// get their span of tickets in turn; TICKET_LAUNCHES launches may be in flight at once.
constexpr int TICKET_LAUNCHES = 64, TICKET_SPAN = 512;
__device__ unsigned g_gemv_tickets[TICKET_LAUNCHES * TICKET_SPAN];

// grid = (k-blocks, row slabs over the whole group); a CTA's warps take the 16-row steps of its
// slab in turn. The slab's sums go to an fp32 plane; the split-K reduction kernel adds the planes.
template <int GB_WARPS>
__global__ void __launch_bounds__(GB_WARPS * 32)
nf4_gemv_bwd_kernel(const __grid_constant__ GemvParams p) {
    const int kb = (int)blockIdx.x;
    const int slab = (int)blockIdx.y;
    const int pi = gemv_find(p, slab);
    const GemvProblem& pr = p.prob[pi];
    const int row0 = (slab - pr.first) * p.rows_per_slab;          // first row of the slab
    const int row_end = min(row0 + p.rows_per_slab, pr.n_w);
    const size_t row_bytes = (size_t)p.k_w >> 1;
    grid_dep_wait();
    grid_dep_launch();
    __shared__ float red[GB_WARPS][16][64 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const RegLut lut = load_reg_lut(pr.code16);
    float acc[8][4];
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[c][0] = acc[c][1] = acc[c][2] = acc[c][3] = 0.f;

    // this lane's word of the k-block: columns kb*64 + 8g .. + 7
    const uint8_t* cbase = pr.codes + (size_t)kb * 32 + (size_t)g * 4;
    const __half* sbase = pr.scales16 + (size_t)kb * pr.n_w;
    const __half* a_lo = pr.act + (long long)g * pr.ld_act;        // token g
    const __half* a_hi = pr.act + (long long)(g + 8) * pr.ld_act;  // token g + 8
    const bool lo_ok = g < p.m, hi_ok = g + 8 < p.m;

    const int n_steps = (row_end - row0 + 15) / 16;   // n_w % 16 == 0: whole steps
    for (int s0 = warp * GB_BATCH; s0 < n_steps; s0 += GB_WARPS * GB_BATCH) {
        uint32_t code[GB_BATCH][4];
        uint32_t sc[GB_BATCH][2], av[GB_BATCH][4];
#pragma unroll
        for (int b = 0; b < GB_BATCH; ++b) {
            const int st = min(s0 + b, n_steps - 1);              // (tail: re-read, unused)
            const int n = row0 + st * 16 + 2 * t;                 // rows n, n+1, n+8, n+9
            const uint8_t* c0 = cbase + (size_t)n * row_bytes;
            code[b][0] = __ldg(reinterpret_cast<const uint32_t*>(c0));
            code[b][1] = __ldg(reinterpret_cast<const uint32_t*>(c0 + row_bytes));
            code[b][2] = __ldg(reinterpret_cast<const uint32_t*>(c0 + 8 * row_bytes));
            code[b][3] = __ldg(reinterpret_cast<const uint32_t*>(c0 + 9 * row_bytes));
            sc[b][0] = __ldg(reinterpret_cast<const uint32_t*>(sbase + n));      // scales of n, n+1
            sc[b][1] = __ldg(reinterpret_cast<const uint32_t*>(sbase + n + 8));  // of n+8, n+9
            av[b][0] = lo_ok ? __ldg(reinterpret_cast<const uint32_t*>(a_lo + n)) : 0u;
            av[b][1] = hi_ok ? __ldg(reinterpret_cast<const uint32_t*>(a_hi + n)) : 0u;
            av[b][2] = lo_ok ? __ldg(reinterpret_cast<const uint32_t*>(a_lo + n + 8)) : 0u;
            av[b][3] = hi_ok ? __ldg(reinterpret_cast<const uint32_t*>(a_hi + n + 8)) : 0u;
        }
#pragma unroll
        for (int b = 0; b < GB_BATCH; ++b) {
            if (s0 + b >= n_steps) break;
            uint32_t w[4][4];   // w[row][pair]: columns (2j, 2j+1) of the word, scaled
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const uint32_t s32 = sc[b][r >> 1];
                const uint32_t dup = (r & 1) ? __byte_perm(s32, 0u, 0x3232u) : __byte_perm(s32, 0u, 0x1010u);
                const uint4 d = decode_word_reg(code[b][r], lut, *reinterpret_cast<const __half2*>(&dup));
                w[r][0] = d.x; w[r][1] = d.y; w[r][2] = d.z; w[r][3] = d.w;
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t sel = (c & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(w[0][c >> 1], w[1][c >> 1], sel);  // rows n, n+1
                const uint32_t b1 = __byte_perm(w[2][c >> 1], w[3][c >> 1], sel);  // rows n+8, n+9
                mma_16816(acc[c], av[b][0], av[b][1], av[b][2], av[b][3], b0, b1);
            }
        }
    }

    // acc[c]: d0,d1 -> (token g, words 2t, 2t+1); d2,d3 -> (token g+8, same); column of (word j,
    // position c) = 8j + c
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        red[warp][g][16 * t + c] = acc[c][0];
        red[warp][g][16 * t + 8 + c] = acc[c][1];
        red[warp][g + 8][16 * t + c] = acc[c][2];
        red[warp][g + 8][16 * t + 8 + c] = acc[c][3];
    }
    __syncthreads();
    const size_t plane_elems = (size_t)p.m * (size_t)p.ldp;
    float* plane = p.planes + (size_t)slab * plane_elems;
    for (int e = threadIdx.x; e < 16 * 64; e += GB_WARPS * 32) {
        const int token = e >> 6, col = e & 63;
        if (token >= p.m) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GB_WARPS; ++w) v += red[w][token][col];
        const int kcol = kb * 64 + col;
        if (pr.ext_a != nullptr && slab == pr.first) {   // u . lora_a, once per member
            float s = 0.f;
#pragma unroll
            for (int r = 0; r < 16; ++r)
                s = fmaf(__half2float(__ldg(pr.ext_a + (long long)token * 16 + r)),
                         __half2float(__ldg(pr.ext_b + (long long)r * p.k_w + kcol)), s);
            v += s;
        }
        __stcg(plane + (size_t)token * p.ldp + kcol, v);
    }
    if (p.ticket_base < 0) return;   // a reduction kernel follows
    // Last arriver of this k-block: every thread makes its plane writes visible device-wide, then
    // one thread takes the ticket.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned* ticket = g_gemv_tickets + p.ticket_base + kb;
        const unsigned old = atomicAdd(ticket, 1u);
        is_last = old == (unsigned)(p.n_slabs - 1) ? 1 : 0;
        if (is_last) *ticket = 0u;   // (nobody else touches it any more in this launch)
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    __half* out = p.prob[0].out;
    for (int e = threadIdx.x; e < 16 * 64; e += GB_WARPS * 32) {
        const int token = e >> 6, col = e & 63;
        if (token >= p.m) continue;
        const size_t off = (size_t)token * p.ldp + (size_t)(kb * 64 + col);
        float v = 0.f;
        for (int z = 0; z < p.n_slabs; ++z) v += __ldcg(p.planes + (size_t)z * plane_elems + off);
        out[(long long)token * p.prob[0].ld_out + kb * 64 + col] = __float2half_rn(v);
    }
}

// ------------------------------------------------------------------------------------ host side

static bool gemv_common_ok(const GemmArgs& a) {
    return a.scales16 != nullptr && a.n_w % GV_ROWS == 0 && a.k_w % 64 == 0 &&
           (reinterpret_cast<uintptr_t>(a.codes) & 7) == 0;
}

bool gemv_eligible(const GemmArgs& a) {
    // measured against the tensor-core kernel: always ahead up to 16 rows; up to 64 rows only for
    // the small projections (the activations are re-read through L1/L2 once per 16 weight rows)
    const bool small_enough = a.m <= 16 || (a.m <= 64 && a.n_w * a.k_w <= (1ll << 22));
    return !a.trans_w && a.m >= 1 && small_enough && gemv_common_ok(a) && a.ld_act % 8 == 0 &&
           (reinterpret_cast<uintptr_t>(a.act) & 15) == 0;
}

bool gemv_bwd_eligible(const GemmArgs& a) {
    return a.trans_w && a.m >= 1 && a.m <= 16 && gemv_common_ok(a) && a.ld_act % 2 == 0 &&
           (reinterpret_cast<uintptr_t>(a.act) & 3) == 0 &&
           (reinterpret_cast<uintptr_t>(a.scales16) & 3) == 0;
}

static void fill_problem(GemvProblem& q, const GemmArgs& a) {
    q.codes = a.codes; q.scales16 = a.scales16; q.code16 = a.code16; q.bias = a.bias;
    q.ext_a = a.ext_a; q.ext_b = a.ext_b; q.act = a.act; q.out = a.out;
    q.ld_out = a.ld_out; q.ld_act = a.ld_act; q.n_w = (int)a.n_w; q.first = 0;
}

template <int NT, int WARPS>
static cudaError_t launch_gemv_t(const GemvParams& p, unsigned ctas, cudaStream_t stream) {
    return launch_pdl(nf4_gemv_kernel<NT, WARPS>, dim3(ctas), dim3(WARPS * 32), 0, stream, p);
}

cudaError_t launch_gemv_group(const GemmGroupArgs& ga, cudaStream_t stream) {
    const GemmArgs& a = ga.item[0];
    GemvParams p = {};
    p.n_prob = ga.count;
    p.act = a.act; p.ld_act = a.ld_act;
    p.m = (int)a.m; p.k_w = (int)a.k_w;
    p.prefetch = 1;
    long long ctas = 0;
    for (int i = 0; i < ga.count; ++i) {
        fill_problem(p.prob[i], ga.item[i]);
        p.prob[i].first = (int)ctas;
        ctas += ga.item[i].n_w / GV_ROWS;
        if ((reinterpret_cast<uintptr_t>(ga.item[i].codes) & 15) != 0 || ((a.k_w / 2) * GV_ROWS) % 16 != 0)
            p.prefetch = 0;
    }
    for (int i = ga.count; i < GV_MAXP; ++i) p.prob[i] = p.prob[0];
    // Warps per CTA: with many row groups, small CTAs so that all of them are resident at once
    // (a second round of CTAs costs as much as the first); with few row groups and long rows,
    // 16 warps to spread K.
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    const int warps = ctas >= 3ll * sms ? 4 : (a.k_w >= 4096 && ctas < 2ll * sms ? 16 : 8);
    const unsigned grid = (unsigned)ctas;
    if (a.m <= 8) {
        if (warps == 4) return launch_gemv_t<1, 4>(p, grid, stream);
        if (warps == 16) return launch_gemv_t<1, 16>(p, grid, stream);
        return launch_gemv_t<1, 8>(p, grid, stream);
    }
    if (a.m <= 16) {
        if (warps == 4) return launch_gemv_t<2, 4>(p, grid, stream);
        if (warps == 16) return launch_gemv_t<2, 16>(p, grid, stream);
        return launch_gemv_t<2, 8>(p, grid, stream);
    }
    if (a.m <= 32) return launch_gemv_t<4, 8>(p, grid, stream);
    return launch_gemv_t<8, 8>(p, grid, stream);
}

cudaError_t launch_gemv(const GemmArgs& a, cudaStream_t stream) {
    GemmGroupArgs ga;
    ga.count = 1;
    ga.item[0] = a;
    return launch_gemv_group(ga, stream);
}

// Row slabs of the streaming backward: enough CTAs (k-blocks x slabs) for about three per SM, slabs
// of whole 16-row steps for every warp.
constexpr int GB_WARPS_PER_CTA = 8;

StreamBwdPlan plan_stream_bwd(long long m, const long long* n_w, int count, long long k_w, int sm_count) {
    StreamBwdPlan pl = {};
    const long long nkb = k_w / 64;
    long long total_rows = 0;
    for (int i = 0; i < count; ++i) total_rows += n_w[i];
    const int sms = sm_count > 0 ? sm_count : 148;
    long long want = (3ll * sms + nkb - 1) / nkb;              // slabs wanted over the group
    if (want < 1) want = 1;
    const long long unit = 16ll * GB_WARPS_PER_CTA;             // one step per warp at least
    long long rows = (total_rows + want - 1) / want;
    rows = (rows + unit - 1) / unit * unit;
    pl.rows_per_slab = (int)rows;
    int slabs = 0;
    for (int i = 0; i < count; ++i) {
        pl.first[i] = slabs;
        slabs += (int)((n_w[i] + rows - 1) / rows);
    }
    pl.slabs = slabs;
    pl.ldp = (k_w + 3) / 4 * 4;
    pl.ws_bytes = (size_t)slabs * (size_t)m * (size_t)pl.ldp * sizeof(float);
    return pl;
}

cudaError_t launch_gemv_bwd_group(const GemmGroupArgs& ga, cudaStream_t stream, const char** why) {
    const GemmArgs& a = ga.item[0];
    long long n_w[GEMM_MAX_GROUP];
    for (int i = 0; i < ga.count; ++i) n_w[i] = ga.item[i].n_w;
    const StreamBwdPlan pl = plan_stream_bwd(a.m, n_w, ga.count, a.k_w, a.sm_count);
    if (a.workspace == nullptr || a.workspace_bytes < pl.ws_bytes) {
        *why = "small-M backward: workspace too small";
        return cudaErrorInvalidValue;
    }
    GemvParams p = {};
    p.n_prob = ga.count;
    p.m = (int)a.m; p.k_w = (int)a.k_w;
    p.planes = static_cast<float*>(a.workspace);
    p.ldp = pl.ldp;
    p.rows_per_slab = pl.rows_per_slab;
    p.n_slabs = pl.slabs;
    const long long nkb = a.k_w / 64;
    static std::atomic<unsigned> cursor{0};
    p.ticket_base = nkb <= TICKET_SPAN
        ? (int)((cursor.fetch_add(1u, std::memory_order_relaxed) % TICKET_LAUNCHES) * TICKET_SPAN)
        : -1;
    for (int i = 0; i < ga.count; ++i) {
        fill_problem(p.prob[i], ga.item[i]);
        p.prob[i].first = pl.first[i];
    }
    for (int i = ga.count; i < GV_MAXP; ++i) p.prob[i] = p.prob[0];
    cudaError_t e = launch_pdl(nf4_gemv_bwd_kernel<GB_WARPS_PER_CTA>,
                               dim3((unsigned)(a.k_w / 64), (unsigned)pl.slabs), dim3(GB_WARPS_PER_CTA * 32),
                               0, stream, p);
    if (e != cudaSuccess) { *why = "small-M backward kernel launch"; return e; }
    if (p.ticket_base >= 0) return e;
    e = launch_splitk_reduce(p.planes, a.m, a.k_w, pl.ldp, pl.slabs, nullptr, a.out, a.ld_out,
                             a.sm_count, stream);
    if (e != cudaSuccess) *why = "small-M backward reduce launch";
    return e;
}

}  // namespace nf4
