// Forward NF4 linear for a handful of token rows (M <= 64, the decode shapes of serving):
//   out[M, N] = act[M, K] . W^T (+ bias) (+ ext_a . ext_b^T)
// At these sizes the work is reading the packed weights once (0.52 B per weight); a 128-row
// tensor-core tile would be 50-99 % padding and the persistent tcgen05 kernel's set-up and
// epilogue would dominate. So: no shared-memory ring, no TMEM. A CTA owns 16 weight rows, its
// 4, 8 or 16 warps (more for long rows, fewer when there are many CTAs) split the 64-deep k-blocks; every warp streams its rows' codes straight from global
// memory (one 32-byte sector per row and k-block), expands them in registers with the same
// byte-permute table look-up as the big kernel (same rounding: fp16(table) * fp16(scale)), and
// multiplies with warp-level mma.sync (m16n8k16: 16 weight rows x 8 tokens x 16 k, fp32
// accumulate). The contraction index is visited in a permuted order that A and B share, so a
// thread's 16 consecutive weights and 16 consecutive activations feed four k16 steps without any
// shuffle. The warps' partial tiles are added through shared memory; bias and the rank-16 LoRA
// term are applied there. Needs the ready-made fp16 block-scale table (kernels.h,
// launch_prepare_scales) and N % 16 == 0; other calls take the tcgen05 kernel.
#include <cuda_fp16.h>

#include "decode.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

constexpr int GV_ROWS = 16;
constexpr int GV_BATCH = 4;

struct GemvParams {
    const uint8_t* codes;
    const __half* scales16;  // [K / 64][N]
    const float* code16;
    const __half* act;
    const __half* bias;
    const __half* ext_a;     // [M, 16] or null
    const __half* ext_b;     // [N, 16]
    __half* out;
    long long ld_act, ld_out;
    int m, n_w, k_w;
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int NT, int GV_WARPS>  // token blocks of 8 (M <= 8 * NT); warps that split K
__global__ void __launch_bounds__(GV_WARPS * 32)
nf4_gemv_kernel(const GemvParams p) {
    constexpr int GV_THREADS = GV_WARPS * 32;
    grid_dep_wait();
    grid_dep_launch();
    __shared__ float red[GV_WARPS][NT * 8][GV_ROWS + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int r0 = blockIdx.x * GV_ROWS;
    const int r_lo = r0 + g, r_hi = r0 + g + 8;  // n_w % 16 == 0: both inside the weight

    RegLut lut;
    {
        uint16_t bits[16];
#pragma unroll
        for (int i = 0; i < 16; ++i)
            bits[i] = __half_as_ushort(__float2half_rn(__ldg(p.code16 + i)));
        lut = make_reg_lut(bits);
    }

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

    const int nkb = p.k_w >> 6;
    const int kb_begin = nkb * warp / GV_WARPS, kb_end = nkb * (warp + 1) / GV_WARPS;
    const size_t row_bytes = (size_t)p.k_w >> 1;
    const uint8_t* c_lo = p.codes + (size_t)r_lo * row_bytes + t * 8;
    const uint8_t* c_hi = p.codes + (size_t)r_hi * row_bytes + t * 8;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // k-blocks in batches of GV_BATCH: all of a batch's code and scale loads are issued before the
    // first one is used, so a warp pays the HBM latency once per batch, not once per k-block
    for (int kb0 = kb_begin; kb0 < kb_end; kb0 += GV_BATCH) {
        uint2 q_lo[GV_BATCH], q_hi[GV_BATCH];
        __half s_lo[GV_BATCH], s_hi[GV_BATCH];
#pragma unroll
        for (int b = 0; b < GV_BATCH; ++b) {
            const int kb = min(kb0 + b, kb_end - 1);  // (tail: re-reads the last block, unused)
            // this thread's 16 weights of rows r_lo and r_hi: k = kb*64 + 16t .. + 15
            q_lo[b] = __ldg(reinterpret_cast<const uint2*>(c_lo + (size_t)kb * 32));
            q_hi[b] = __ldg(reinterpret_cast<const uint2*>(c_hi + (size_t)kb * 32));
            s_lo[b] = __ldg(p.scales16 + (size_t)kb * p.n_w + r_lo);
            s_hi[b] = __ldg(p.scales16 + (size_t)kb * p.n_w + r_hi);
        }
#pragma unroll
        for (int b = 0; b < GV_BATCH; ++b) {
            const int kb = kb0 + b;
            if (kb >= kb_end) break;
            uint32_t wl[8], wh[8];
            {
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
                mma_16816(acc[nt], wl[0], wh[0], wl[1], wh[1], x0.x, x0.y);
                mma_16816(acc[nt], wl[2], wh[2], wl[3], wh[3], x0.z, x0.w);
                mma_16816(acc[nt], wl[4], wh[4], wl[5], wh[5], x1.x, x1.y);
                mma_16816(acc[nt], wl[6], wh[6], wl[7], wh[7], x1.z, x1.w);
            }
        }
    }

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
        if (p.ext_a != nullptr) {
            const __half2* xa = reinterpret_cast<const __half2*>(p.ext_a + (long long)token * 16);
            const __half2* lb = reinterpret_cast<const __half2*>(p.ext_b + (long long)(r0 + r) * 16);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 a = __half22float2(__ldg(xa + j)), b = __half22float2(__ldg(lb + j));
                s = fmaf(a.x, b.x, s);
                s = fmaf(a.y, b.y, s);
            }
            v += s;
        }
        if (p.bias != nullptr) v += __half2float(__ldg(p.bias + r0 + r));
        p.out[(long long)token * p.ld_out + r0 + r] = __float2half_rn(v);
    }
}

bool gemv_eligible(const GemmArgs& a) {
    // measured against the tensor-core kernel: always ahead up to 16 rows; up to 64 rows only for
    // the small projections (the activations are re-read through L1/L2 once per 16 weight rows)
    const bool small_enough = a.m <= 16 || (a.m <= 64 && a.n_w * a.k_w <= (1ll << 22));
    return !a.trans_w && a.m >= 1 && small_enough && a.scales16 != nullptr && a.n_w % GV_ROWS == 0 &&
           a.k_w % 64 == 0 && a.ld_act % 8 == 0 && (reinterpret_cast<uintptr_t>(a.act) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(a.codes) & 7) == 0;
}

template <int NT, int WARPS>
static cudaError_t launch_gemv_t(const GemvParams& p, cudaStream_t stream) {
    return launch_pdl(nf4_gemv_kernel<NT, WARPS>, dim3((unsigned)(p.n_w / GV_ROWS)), dim3(WARPS * 32), 0,
                      stream, p);
}

cudaError_t launch_gemv(const GemmArgs& a, cudaStream_t stream) {
    GemvParams p;
    p.codes = a.codes; p.scales16 = a.scales16; p.code16 = a.code16; p.act = a.act;
    p.bias = a.bias; p.ext_a = a.ext_a; p.ext_b = a.ext_b; p.out = a.out;
    p.ld_act = a.ld_act; p.ld_out = a.ld_out;
    p.m = (int)a.m; p.n_w = (int)a.n_w; p.k_w = (int)a.k_w;
    // Warps per CTA: with many row groups, small CTAs so that all of them are resident at once
    // (a second round of CTAs costs as much as the first); with few row groups and long rows,
    // 16 warps to spread K.
    const long long ctas = a.n_w / GV_ROWS;
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    const int warps = ctas >= 3ll * sms ? 4 : (a.k_w >= 4096 && ctas < 2ll * sms ? 16 : 8);
    if (a.m <= 8) {
        if (warps == 4) return launch_gemv_t<1, 4>(p, stream);
        if (warps == 16) return launch_gemv_t<1, 16>(p, stream);
        return launch_gemv_t<1, 8>(p, stream);
    }
    if (a.m <= 16) {
        if (warps == 4) return launch_gemv_t<2, 4>(p, stream);
        if (warps == 16) return launch_gemv_t<2, 16>(p, stream);
        return launch_gemv_t<2, 8>(p, stream);
    }
    if (a.m <= 32) return launch_gemv_t<4, 8>(p, stream);
    return launch_gemv_t<8, 8>(p, stream);
}

}  // namespace nf4
