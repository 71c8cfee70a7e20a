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
// A block of 4 warps owns LD_ROWS rows; each warp takes a quarter of the columns for all of them
// (lane l owns 8 columns at a time), then the four partial results are added through shared
// memory. P (at most a few hundred KB, shared by every block) is read straight from global memory
// with 16-byte loads and lives in L1/L2.
constexpr int LD_WARPS = 4;
constexpr int LD_ROWS_PER_WARP = 4;   // rows whose sums one warp carries (= rows per block)
constexpr int LD_ROWS = LD_ROWS_PER_WARP;
constexpr int LD_THREADS = LD_WARPS * 32;

template <bool RANK_MAJOR>  // P is row-major [16, C] (true) or row-major [C, 16] (false)
__global__ void __launch_bounds__(LD_THREADS)
lora_down_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                 const __half* __restrict__ p, float scaling, __half* __restrict__ out) {
    __shared__ float part[LD_WARPS][LD_ROWS_PER_WARP][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row0 = (long long)blockIdx.x * LD_ROWS;
    float acc[LD_ROWS_PER_WARP][16];
#pragma unroll
    for (int r = 0; r < LD_ROWS_PER_WARP; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[r][j] = 0.f;

    // this warp's column range: a quarter of the columns, in multiples of 8 (c % 8 == 0 here)
    const long long groups = c / 8;
    const long long g_begin = groups * warp / LD_WARPS, g_end = groups * (warp + 1) / LD_WARPS;
    for (long long gc = (g_begin + lane) * 8; gc < g_end * 8; gc += 256) {
        float x[LD_ROWS_PER_WARP][8];
#pragma unroll
        for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
            const long long gr = row0 + r;
            if (gr < m) {
                unpack8(__ldg(reinterpret_cast<const uint4*>(in + gr * ld_in + gc)), x[r]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[r][e] = 0.f;
            }
        }
        if (RANK_MAJOR) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                float pv[8];
                unpack8(__ldg(reinterpret_cast<const uint4*>(p + (long long)j * c + gc)), pv);
#pragma unroll
                for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
                    float a = acc[r][j];
#pragma unroll
                    for (int e = 0; e < 8; ++e) a = fmaf(x[r][e], pv[e], a);
                    acc[r][j] = a;
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float pa[8], pb[8];
                const uint4* src = reinterpret_cast<const uint4*>(p + (gc + e) * 16);
                unpack8(__ldg(src), pa);
                unpack8(__ldg(src + 1), pb);
#pragma unroll
                for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[r][j] = fmaf(x[r][e], pa[j], acc[r][j]);
                        acc[r][8 + j] = fmaf(x[r][e], pb[j], acc[r][8 + j]);
                    }
                }
            }
        }
    }
    // butterfly over the 32 lanes, fold the four warps, lanes 0..7 of warp 0..3 write the rows
#pragma unroll
    for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = acc[r][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) part[warp][r][j] = v;
        }
    }
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

// Layout-agnostic variant (any strides, any alignment): one thread per output element.
__global__ void __launch_bounds__(256)
lora_down_generic_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                         const __half* __restrict__ p, long long p_stride_r, long long p_stride_c,
                         float scaling, __half* __restrict__ out) {
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
        lora_down_kernel<true><<<blocks, LD_THREADS, 0, stream>>>(a.in, a.m, a.c, a.ld_in, a.p,
                                                                   a.scaling, a.out);
    } else if (aligned && a.p_stride_r == 1 && a.p_stride_c == 16) {
        lora_down_kernel<false><<<blocks, LD_THREADS, 0, stream>>>(a.in, a.m, a.c, a.ld_in, a.p,
                                                                    a.scaling, a.out);
    } else {
        const long long total = a.m * 16;
        lora_down_generic_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
            a.in, a.m, a.c, a.ld_in, a.p, a.p_stride_r, a.p_stride_c, a.scaling, a.out);
    }
    return cudaGetLastError();
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

cudaError_t launch_lora_grad(const LoraGradArgs& a, cudaStream_t stream) {
    if (a.m <= 0 || a.c <= 0) return cudaSuccess;
    dim3 grid((unsigned)((a.c + LG_COLS - 1) / LG_COLS), (unsigned)((a.m + LG_ROWS - 1) / LG_ROWS));
    const int vec_ok = (a.ld_z % 4 == 0) && ((reinterpret_cast<uintptr_t>(a.z) & 7) == 0);
    lora_grad_kernel<<<grid, LG_THREADS, 0, stream>>>(a.z, a.m, a.c, a.ld_z, a.s, a.out,
                                                      a.o_stride_r, a.o_stride_c, vec_ok);
    return cudaGetLastError();
}

}  // namespace nf4
