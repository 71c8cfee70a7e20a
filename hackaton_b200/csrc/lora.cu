// Rank-16 side products of the LoRA update (peft's lora_A / lora_B linears; third-party in the
// reference, configured at README.md:91 and task/task.yaml:18-21).
//
//   lora_down: out[M,16] = scaling * in[M,C] . P      feeds the GEMM kernels' K-extension step
//   lora_grad: out[C,16] += z[M,C]^T . s[M,16]        weight gradients dA, dB (fp32)
//
// Both are skinny (16 wide) and bound by reading `in` / `z` once (2 B per element): 16-byte
// coalesced loads, the small operand staged in shared memory as fp32, fp32 accumulation.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

// ------------------------------------------------------------------------------------ lora_down
// Tensor-core version (mma.sync m16n8k16, fp16 in / fp32 accumulate: the op is bound by reading
// `in` once, the legacy warp-level MMA is ample). A block owns 16 rows; its LD_WARPS warps split
// the columns, each walking 32 columns per step:
//   lane (g = lane/4, t = lane%4) loads 8 contiguous halves in[g][c0 + 8t ..] and in[g+8][...]
//   (one 16-byte load each) and the matching 8 halves of P for outputs j = g and j = 8 + g.
// The contraction index may be visited in any order as long as A and B agree, so halves 0..3 of
// those 8 feed the first k16 step (a0a1 | a4a5) and halves 4..7 the second: no shuffles, no
// shared-memory staging. The warps' 16x16 partial tiles are added through shared memory.
constexpr int LD_WARPS = 8;
constexpr int LD_ROWS = 16;
constexpr int LD_THREADS = LD_WARPS * 32;
constexpr int LD_BATCH = 3;   // chunks in flight per warp (16 registers each; two blocks per SM)

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <bool RANK_MAJOR>  // P is row-major [16, C] (true) or row-major [C, 16] (false)
__device__ __forceinline__ void lora_down_block(const __half* __restrict__ in, long long m,
                                                long long c, long long ld_in,
                                                const __half* __restrict__ p, float scaling,
                                                __half* __restrict__ out) {
    __shared__ float part[LD_WARPS][16][17];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long row0 = (long long)blockIdx.x * LD_ROWS;
    const long long r_lo = row0 + g, r_hi = row0 + g + 8;
    float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};  // outputs j 0..7, 8..15

    const long long chunks = (c + 31) / 32;   // c % 8 == 0 on this path
    const long long ch_begin = chunks * warp / LD_WARPS, ch_end = chunks * (warp + 1) / LD_WARPS;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    // LD_BATCH chunks per round: every load of the round is issued before the first MMA, so a
    // warp pays one memory round trip per round instead of one per chunk.
    for (long long ch0 = ch_begin; ch0 < ch_end; ch0 += LD_BATCH) {
        uint4 a_lo[LD_BATCH], a_hi[LD_BATCH], b_lo[LD_BATCH], b_hi[LD_BATCH];
#pragma unroll
        for (int q = 0; q < LD_BATCH; ++q) {
            const long long col = (ch0 + q) * 32 + t * 8;
            const bool col_ok = ch0 + q < ch_end && col < c;
            a_lo[q] = a_hi[q] = b_lo[q] = b_hi[q] = zero;
            if (col_ok) {
                if (r_lo < m) a_lo[q] = __ldg(reinterpret_cast<const uint4*>(in + r_lo * ld_in + col));
                if (r_hi < m) a_hi[q] = __ldg(reinterpret_cast<const uint4*>(in + r_hi * ld_in + col));
                if (RANK_MAJOR) {
                    b_lo[q] = __ldg(reinterpret_cast<const uint4*>(p + (long long)g * c + col));
                    b_hi[q] = __ldg(reinterpret_cast<const uint4*>(p + (long long)(g + 8) * c + col));
                } else {
                    __half lo[8], hi[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        lo[e] = __ldg(p + (col + e) * 16 + g);
                        hi[e] = __ldg(p + (col + e) * 16 + g + 8);
                    }
                    b_lo[q] = *reinterpret_cast<const uint4*>(lo);
                    b_hi[q] = *reinterpret_cast<const uint4*>(hi);
                }
            }
        }
#pragma unroll
        for (int q = 0; q < LD_BATCH; ++q) {
            // k16 step 0: halves 0,1 | 2,3 ; step 1: halves 4,5 | 6,7
            mma16816(d0, a_lo[q].x, a_hi[q].x, a_lo[q].y, a_hi[q].y, b_lo[q].x, b_lo[q].y);
            mma16816(d1, a_lo[q].x, a_hi[q].x, a_lo[q].y, a_hi[q].y, b_hi[q].x, b_hi[q].y);
            mma16816(d0, a_lo[q].z, a_hi[q].z, a_lo[q].w, a_hi[q].w, b_lo[q].z, b_lo[q].w);
            mma16816(d1, a_lo[q].z, a_hi[q].z, a_lo[q].w, a_hi[q].w, b_hi[q].z, b_hi[q].w);
        }
    }
    // accumulator layout: d[0],d[1] -> (row g, cols 2t, 2t+1); d[2],d[3] -> (row g+8, same cols)
    part[warp][g][2 * t] = d0[0];         part[warp][g][2 * t + 1] = d0[1];
    part[warp][g + 8][2 * t] = d0[2];     part[warp][g + 8][2 * t + 1] = d0[3];
    part[warp][g][8 + 2 * t] = d1[0];     part[warp][g][8 + 2 * t + 1] = d1[1];
    part[warp][g + 8][8 + 2 * t] = d1[2]; part[warp][g + 8][8 + 2 * t + 1] = d1[3];
    __syncthreads();
    if (threadIdx.x < LD_ROWS * 8) {
        const int r = threadIdx.x >> 3, jp = (threadIdx.x & 7) * 2;
        const long long gr = row0 + r;
        if (gr < m) {
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int w = 0; w < LD_WARPS; ++w) { a += part[w][r][jp]; b += part[w][r][jp + 1]; }
            *reinterpret_cast<__half2*>(out + gr * 16 + jp) = __floats2half2_rn(a * scaling, b * scaling);
        }
    }
}

template <bool RANK_MAJOR>
__global__ void __launch_bounds__(LD_THREADS)
lora_down_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                 const __half* __restrict__ p, float scaling, __half* __restrict__ out) {
    grid_dep_wait();    // (programmatic dependent launch: the predecessor's results)
    grid_dep_launch();
    lora_down_block<RANK_MAJOR>(in, m, c, ld_in, p, scaling, out);
}

// Several lora_down problems with the same row count in one launch: blockIdx.y picks the problem.
template <bool RANK_MAJOR>
__global__ void __launch_bounds__(LD_THREADS)
lora_down_batch_kernel(const __grid_constant__ LoraDownBatch b) {
    grid_dep_wait();
    grid_dep_launch();
    const LoraDownArgs& a = b.item[blockIdx.y];
    lora_down_block<RANK_MAJOR>(a.in, a.m, a.c, a.ld_in, a.p, a.scaling, a.out);
}

// Layout-agnostic variant (any strides, any alignment): one thread per output element.
__global__ void __launch_bounds__(256)
lora_down_generic_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                         const __half* __restrict__ p, long long p_stride_r, long long p_stride_c,
                         float scaling, __half* __restrict__ out) {
    grid_dep_wait();    // (programmatic dependent launch: the predecessor's results)
    grid_dep_launch();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m * 16) return;
    const long long row = i / 16;
    const int j = (int)(i % 16);
    float acc = 0.f;
    for (long long cc = 0; cc < c; ++cc)
        acc = fmaf(__half2float(in[row * ld_in + cc]), __half2float(p[cc * p_stride_c + j * p_stride_r]),
                   acc);
    out[row * 16 + j] = __float2half_rn(acc * scaling);
}

cudaError_t launch_lora_down(const LoraDownArgs& a, cudaStream_t stream) {
    if (a.m <= 0) return cudaSuccess;
    const bool aligned = (a.ld_in % 8 == 0) && (a.c % 8 == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.in) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.p) & 15) == 0);
    const unsigned blocks = (unsigned)((a.m + LD_ROWS - 1) / LD_ROWS);
    if (aligned && a.p_stride_c == 1 && a.p_stride_r == a.c) {
        return launch_pdl(lora_down_kernel<true>, dim3(blocks), dim3(LD_THREADS), 0, stream, a.in, a.m,
                          a.c, a.ld_in, a.p, a.scaling, a.out);
    } else if (aligned && a.p_stride_r == 1 && a.p_stride_c == 16) {
        return launch_pdl(lora_down_kernel<false>, dim3(blocks), dim3(LD_THREADS), 0, stream, a.in,
                          a.m, a.c, a.ld_in, a.p, a.scaling, a.out);
    } else {
        const long long total = a.m * 16;
        return launch_pdl(lora_down_generic_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                          stream, a.in, a.m, a.c, a.ld_in, a.p, a.p_stride_r, a.p_stride_c,
                          a.scaling, a.out);
    }
}

cudaError_t launch_lora_down_batch(const LoraDownBatch& b, cudaStream_t stream) {
    // one launch when every problem has the same row count and the same (fast-path) layout of P
    bool one_launch = b.count > 1;
    bool rank_major = false;
    for (int i = 0; i < b.count; ++i) {
        const LoraDownArgs& a = b.item[i];
        const bool aligned = (a.ld_in % 8 == 0) && (a.c % 8 == 0) &&
                             ((reinterpret_cast<uintptr_t>(a.in) & 15) == 0) &&
                             ((reinterpret_cast<uintptr_t>(a.p) & 15) == 0);
        const bool rm = a.p_stride_c == 1 && a.p_stride_r == a.c;
        const bool cm = a.p_stride_r == 1 && a.p_stride_c == 16;
        if (!aligned || !(rm || cm) || a.m <= 0 || a.m != b.item[0].m) one_launch = false;
        if (i == 0) rank_major = rm;
        else if (rm != rank_major) one_launch = false;
    }
    if (!one_launch) {
        for (int i = 0; i < b.count; ++i) {
            cudaError_t e = launch_lora_down(b.item[i], stream);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    dim3 grid((unsigned)((b.item[0].m + LD_ROWS - 1) / LD_ROWS), (unsigned)b.count);
    if (rank_major)
        return launch_pdl(lora_down_batch_kernel<true>, grid, dim3(LD_THREADS), 0, stream, b);
    return launch_pdl(lora_down_batch_kernel<false>, grid, dim3(LD_THREADS), 0, stream, b);
}

// ------------------------------------------------------------------------------------ lora_grad
// Block: 8 warps over one tile of 128 columns (lane l owns columns 4l .. 4l+3) and 128 rows
// (warp w takes rows w, w+8, ...). Each lane keeps 4 x 16 fp32 sums; the 8 warps are folded
// through shared memory and one warp adds the block's result to the output atomically.
constexpr int LG_COLS = 128;
constexpr int LG_ROWS = 128;
constexpr int LG_WARPS = 8;
constexpr int LG_THREADS = LG_WARPS * 32;

__global__ void __launch_bounds__(LG_THREADS)
lora_grad_kernel(const __half* __restrict__ z, long long m, long long c, long long ld_z,
                 const __half* __restrict__ s, float* __restrict__ out, long long o_stride_r,
                 long long o_stride_c, int vec_ok) {
    grid_dep_wait();    // (programmatic dependent launch: the predecessor's results)
    grid_dep_launch();
    __shared__ __align__(16) float s_s[LG_ROWS][16];                 // 8 KB
    __shared__ __align__(16) float red[LG_WARPS / 2][64][32 + 1];    // 33 KB: [warp][value][lane]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long c0 = (long long)blockIdx.x * LG_COLS + lane * 4;
    const long long m0 = (long long)blockIdx.y * LG_ROWS;
    for (int i = threadIdx.x; i < LG_ROWS * 16; i += LG_THREADS) {
        const long long gm = m0 + i / 16;
        s_s[i / 16][i % 16] = gm < m ? __half2float(s[gm * 16 + i % 16]) : 0.f;
    }
    __syncthreads();
    float acc[4][16];
#pragma unroll
    for (int e = 0; e < 4; ++e)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[e][j] = 0.f;
    const int rows = (int)((m - m0 < LG_ROWS) ? (m - m0) : LG_ROWS);
    if (c0 < c) {
#pragma unroll 4
        for (int r = warp; r < rows; r += LG_WARPS) {
            const __half* src = z + (m0 + r) * ld_z + c0;
            float x[4] = {0.f, 0.f, 0.f, 0.f};
            if (vec_ok && c0 + 4 <= c) {
                const uint2 v = __ldg(reinterpret_cast<const uint2*>(src));
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
                const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
                x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (c0 + e < c) x[e] = __half2float(src[e]);
            }
            const float4* sr = reinterpret_cast<const float4*>(&s_s[r][0]);
#pragma unroll
            for (int jq = 0; jq < 4; ++jq) {
                const float4 sv = sr[jq];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[e][4 * jq + 0] = fmaf(x[e], sv.x, acc[e][4 * jq + 0]);
                    acc[e][4 * jq + 1] = fmaf(x[e], sv.y, acc[e][4 * jq + 1]);
                    acc[e][4 * jq + 2] = fmaf(x[e], sv.z, acc[e][4 * jq + 2]);
                    acc[e][4 * jq + 3] = fmaf(x[e], sv.w, acc[e][4 * jq + 3]);
                }
            }
        }
    }
    // fold 8 -> 4 -> 2 -> 1 warps
#pragma unroll
    for (int half = LG_WARPS / 2; half >= 1; half >>= 1) {
        __syncthreads();
        if (warp >= half && warp < 2 * half) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int j = 0; j < 16; ++j) red[warp - half][e * 16 + j][lane] = acc[e][j];
        }
        __syncthreads();
        if (warp < half) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[e][j] += red[warp][e * 16 + j][lane];
        }
    }
    if (warp == 0 && c0 < c) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (c0 + e < c) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    atomicAdd(out + (c0 + e) * o_stride_c + j * o_stride_r, acc[e][j]);
            }
        }
    }
}

// Tensor-core version of lora_grad: D[j][c] = sum_m s[m][j] * z[m][c] with mma.sync m16n8k16.
// The contraction runs over the slow (row) index of both operands, so 32-token chunks of z
// ([32 x 128]) and s ([32 x 16]) are staged in shared memory with 16-byte loads and read back
// transposed with ldmatrix.trans. 8 warps, each owning 16 of the block's 128 columns; chunk i+1 is
// fetched into registers while chunk i is multiplied.
// (128 rows per block: a layer's four gradients at 2048 tokens are 608 blocks, one wave at five
// blocks per SM, each walking four chunks; 256 rows measured 9.9 us, 128 rows 8.3, 64 rows 10.4)
constexpr int LGM_COLS = 128, LGM_CHUNK = 32, LGM_ROWS = 128, LGM_THREADS = 256;
constexpr int LGM_ZP = LGM_COLS + 8;   // padded row pitches (halves): conflict-free ldmatrix
constexpr int LGM_SP = 16 + 8;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void lora_grad_mma_block(const __half* __restrict__ z, long long m,
                                                    long long c, long long ld_z,
                                                    const __half* __restrict__ s,
                                                    float* __restrict__ out, long long o_stride_r,
                                                    long long o_stride_c) {
    __shared__ __align__(16) __half zt[2][LGM_CHUNK][LGM_ZP];
    __shared__ __align__(16) __half st[2][LGM_CHUNK][LGM_SP];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const long long c0 = (long long)blockIdx.x * LGM_COLS;
    const long long m0 = (long long)blockIdx.y * LGM_ROWS;
    const long long m_end = (m0 + LGM_ROWS < m) ? m0 + LGM_ROWS : m;
    const int n_chunks = (int)((m_end - m0 + LGM_CHUNK - 1) / LGM_CHUNK);

    // staging assignment: z chunk = 32 rows x 16 uint4 -> 2 per thread; s chunk = 32 rows x 2 uint4
    const int zr = threadIdx.x >> 4, zc = (threadIdx.x & 15) * 8;   // rows zr and zr + 16
    const int sr = threadIdx.x >> 1, sc = (threadIdx.x & 1) * 8;    // threads 0..63
    uint4 zreg[2], sreg;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    auto fetch = [&](int chunk) {
        const long long r0 = m0 + (long long)chunk * LGM_CHUNK;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const long long r = r0 + zr + 16 * h;
            zreg[h] = (r < m_end && c0 + zc < c)
                ? __ldg(reinterpret_cast<const uint4*>(z + r * ld_z + c0 + zc)) : zero;
        }
        if (threadIdx.x < 64) {
            const long long r = r0 + sr;
            sreg = r < m_end ? __ldg(reinterpret_cast<const uint4*>(s + r * 16 + sc)) : zero;
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int h = 0; h < 2; ++h)
            *reinterpret_cast<uint4*>(&zt[buf][zr + 16 * h][zc]) = zreg[h];
        if (threadIdx.x < 64) *reinterpret_cast<uint4*>(&st[buf][sr][sc]) = sreg;
    };

    float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};  // columns 16w+0..7, +8..15
    fetch(0);
    stash(0);
    __syncthreads();
    for (int ch = 0; ch < n_chunks; ++ch) {
        const int buf = ch & 1;
        if (ch + 1 < n_chunks) fetch(ch + 1);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            // A (16 j x 16 k) from st[k][j]: matrices (j0-7,k0-7), (j8-15,k0-7), (j0-7,k8-15), (j8-15,k8-15)
            const int q = lane >> 3, i = lane & 7;
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(
                                  &st[buf][ks * 16 + (q >> 1) * 8 + i][(q & 1) * 8]),
                              a0, a1, a2, a3);
            // B (16 k x 8 n) x 2 n-tiles from zt[k][n]: (k0-7,n0), (k8-15,n0), (k0-7,n0+8), (k8-15,n0+8)
            ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(
                                  &zt[buf][ks * 16 + (q & 1) * 8 + i][warp * 16 + (q >> 1) * 8]),
                              b0, b1, b2, b3);
            mma16816(d0, a0, a1, a2, a3, b0, b1);
            mma16816(d1, a0, a1, a2, a3, b2, b3);
        }
        if (ch + 1 < n_chunks) stash(buf ^ 1);
        __syncthreads();
    }
    // d[0],d[1] -> (j = g, columns 2t, 2t+1 of the n-tile); d[2],d[3] -> (j = g + 8, same columns)
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
        const float* d = nt == 0 ? d0 : d1;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const long long col = c0 + warp * 16 + nt * 8 + 2 * t + (e & 1);
            const int j = g + (e >> 1) * 8;
            if (col < c) atomicAdd(out + col * o_stride_c + j * o_stride_r, d[e]);
        }
    }
}

__global__ void __launch_bounds__(LGM_THREADS)
lora_grad_mma_kernel(const __half* __restrict__ z, long long m, long long c, long long ld_z,
                     const __half* __restrict__ s, float* __restrict__ out, long long o_stride_r,
                     long long o_stride_c) {
    grid_dep_wait();    // (programmatic dependent launch: the predecessor's results)
    grid_dep_launch();
    lora_grad_mma_block(z, m, c, ld_z, s, out, o_stride_r, o_stride_c);
}

// Several lora_grad problems in one launch: blockIdx.z picks the problem; the grid is sized for
// the widest one, blocks outside a narrower problem leave at once.
__global__ void __launch_bounds__(LGM_THREADS)
lora_grad_batch_kernel(const __grid_constant__ LoraGradBatch b) {
    grid_dep_wait();
    grid_dep_launch();
    const LoraGradArgs& a = b.item[blockIdx.z];
    if ((long long)blockIdx.x * LGM_COLS >= a.c || (long long)blockIdx.y * LGM_ROWS >= a.m) return;
    lora_grad_mma_block(a.z, a.m, a.c, a.ld_z, a.s, a.out, a.o_stride_r, a.o_stride_c);
}

static bool lora_grad_aligned(const LoraGradArgs& a) {
    return (a.ld_z % 8 == 0) && (a.c % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.z) & 15) == 0) &&
           ((reinterpret_cast<uintptr_t>(a.s) & 15) == 0);
}

cudaError_t launch_lora_grad_batch(const LoraGradBatch& b, cudaStream_t stream) {
    bool one_launch = b.count > 1;
    long long max_c = 0, max_m = 0;
    for (int i = 0; i < b.count; ++i) {
        const LoraGradArgs& a = b.item[i];
        if (a.m <= 0 || a.c <= 0 || !lora_grad_aligned(a)) one_launch = false;
        max_c = a.c > max_c ? a.c : max_c;
        max_m = a.m > max_m ? a.m : max_m;
    }
    if (!one_launch) {
        for (int i = 0; i < b.count; ++i) {
            cudaError_t e = launch_lora_grad(b.item[i], stream);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    dim3 grid((unsigned)((max_c + LGM_COLS - 1) / LGM_COLS), (unsigned)((max_m + LGM_ROWS - 1) / LGM_ROWS),
              (unsigned)b.count);
    return launch_pdl(lora_grad_batch_kernel, grid, dim3(LGM_THREADS), 0, stream, b);
}

cudaError_t launch_lora_grad(const LoraGradArgs& a, cudaStream_t stream) {
    if (a.m <= 0 || a.c <= 0) return cudaSuccess;
    const bool aligned = (a.ld_z % 8 == 0) && (a.c % 8 == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.z) & 15) == 0) &&
                         ((reinterpret_cast<uintptr_t>(a.s) & 15) == 0);
    if (aligned) {
        dim3 grid_mma((unsigned)((a.c + LGM_COLS - 1) / LGM_COLS),
                      (unsigned)((a.m + LGM_ROWS - 1) / LGM_ROWS));
        return launch_pdl(lora_grad_mma_kernel, grid_mma, dim3(LGM_THREADS), 0, stream, a.z, a.m, a.c,
                          a.ld_z, a.s, a.out, a.o_stride_r, a.o_stride_c);
    }
    dim3 grid((unsigned)((a.c + LG_COLS - 1) / LG_COLS), (unsigned)((a.m + LG_ROWS - 1) / LG_ROWS));
    const int vec_ok = (a.ld_z % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.z) & 7) == 0);
    return launch_pdl(lora_grad_kernel, grid, dim3(LG_THREADS), 0, stream, a.z, a.m, a.c, a.ld_z, a.s,
                      a.out, a.o_stride_r, a.o_stride_c, vec_ok);
}

}  // namespace nf4
