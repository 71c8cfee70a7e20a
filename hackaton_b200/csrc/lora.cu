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
// Block: 4 warps x 2 rows. Columns are walked in chunks of 512; P's chunk sits in shared memory
// as fp32 [16][512]. Lane l owns columns l*8 + 256*t of the chunk.
constexpr int LD_WARPS = 4;
constexpr int LD_ROWS_PER_WARP = 2;
constexpr int LD_ROWS = LD_WARPS * LD_ROWS_PER_WARP;
constexpr int LD_THREADS = LD_WARPS * 32;
constexpr int LD_CHUNK = 512;

__global__ void __launch_bounds__(LD_THREADS)
lora_down_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                 const __half* __restrict__ p, long long p_stride_r, long long p_stride_c,
                 float scaling, __half* __restrict__ out, int vec_ok, int p_vec) {
    __shared__ __align__(16) float p_s[16][LD_CHUNK];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row0 = (long long)blockIdx.x * LD_ROWS + warp * LD_ROWS_PER_WARP;
    float acc[LD_ROWS_PER_WARP][16];
#pragma unroll
    for (int r = 0; r < LD_ROWS_PER_WARP; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[r][j] = 0.f;

    for (long long c0 = 0; c0 < c; c0 += LD_CHUNK) {
        __syncthreads();
        // stage P[c0 .. c0+512) as fp32 [16][512] with 16-byte loads along the source's
        // contiguous axis (element-wise when the layout or alignment does not allow them)
        if (p_vec && p_stride_c == 1) {           // row-major [16, C]
            for (int i = threadIdx.x; i < 16 * (LD_CHUNK / 8); i += LD_THREADS) {
                const int j = i / (LD_CHUNK / 8), cc = (i % (LD_CHUNK / 8)) * 8;
                const long long gc = c0 + cc;
                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (gc + 8 <= c) {
                    unpack8(__ldg(reinterpret_cast<const uint4*>(p + j * p_stride_r + gc)), f);
                } else {
                    for (int e = 0; e < 8; ++e)
                        if (gc + e < c) f[e] = __half2float(p[j * p_stride_r + gc + e]);
                }
                *reinterpret_cast<float4*>(&p_s[j][cc]) = make_float4(f[0], f[1], f[2], f[3]);
                *reinterpret_cast<float4*>(&p_s[j][cc + 4]) = make_float4(f[4], f[5], f[6], f[7]);
            }
        } else if (p_vec && p_stride_r == 1 && p_stride_c == 16) {   // row-major [C, 16]
            for (int i = threadIdx.x; i < LD_CHUNK * 2; i += LD_THREADS) {
                const int cc = i >> 1, h = i & 1;
                const long long gc = c0 + cc;
                float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                if (gc < c) unpack8(__ldg(reinterpret_cast<const uint4*>(p + gc * 16 + h * 8)), f);
#pragma unroll
                for (int e = 0; e < 8; ++e) p_s[h * 8 + e][cc] = f[e];
            }
        } else {
            for (int i = threadIdx.x; i < 16 * LD_CHUNK; i += LD_THREADS) {
                int cc, j;
                if (p_stride_c == 1) { j = i / LD_CHUNK; cc = i % LD_CHUNK; }
                else                 { cc = i / 16;      j = i % 16; }
                const long long gc = c0 + cc;
                p_s[j][cc] = gc < c ? __half2float(p[gc * p_stride_c + j * p_stride_r]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int t = 0; t < LD_CHUNK / 256; ++t) {
            const int cc = lane * 8 + 256 * t;
            const long long gc = c0 + cc;
            float x[LD_ROWS_PER_WARP][8];
#pragma unroll
            for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
                const long long gr = row0 + r;
#pragma unroll
                for (int e = 0; e < 8; ++e) x[r][e] = 0.f;
                if (gr < m && gc < c) {
                    const __half* src = in + gr * ld_in + gc;
                    if (vec_ok && gc + 8 <= c) {
                        unpack8(__ldg(reinterpret_cast<const uint4*>(src)), x[r]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e)
                            if (gc + e < c) x[r][e] = __half2float(src[e]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const float4 pa = *reinterpret_cast<const float4*>(&p_s[j][cc]);
                const float4 pb = *reinterpret_cast<const float4*>(&p_s[j][cc + 4]);
#pragma unroll
                for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
                    float a = acc[r][j];
                    a = fmaf(x[r][0], pa.x, a); a = fmaf(x[r][1], pa.y, a);
                    a = fmaf(x[r][2], pa.z, a); a = fmaf(x[r][3], pa.w, a);
                    a = fmaf(x[r][4], pb.x, a); a = fmaf(x[r][5], pb.y, a);
                    a = fmaf(x[r][6], pb.z, a); a = fmaf(x[r][7], pb.w, a);
                    acc[r][j] = a;
                }
            }
        }
    }
    // butterfly over the 32 lanes, then lanes 0..7 write one half2 each per row
#pragma unroll
    for (int r = 0; r < LD_ROWS_PER_WARP; ++r) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = acc[r][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            acc[r][j] = v * scaling;
        }
        const long long gr = row0 + r;
        if (gr < m && lane < 8) {
            float a = 0.f, b = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (lane == j) { a = acc[r][2 * j]; b = acc[r][2 * j + 1]; }
            *reinterpret_cast<__half2*>(out + gr * 16 + 2 * lane) = __floats2half2_rn(a, b);
        }
    }
}

cudaError_t launch_lora_down(const LoraDownArgs& a, cudaStream_t stream) {
    if (a.m <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((a.m + LD_ROWS - 1) / LD_ROWS);
    const int vec_ok = (a.ld_in % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.in) & 15) == 0);
    const int p_vec = ((reinterpret_cast<uintptr_t>(a.p) & 15) == 0) &&
                      (a.p_stride_c != 1 || a.p_stride_r % 8 == 0);
    lora_down_kernel<<<blocks, LD_THREADS, 0, stream>>>(a.in, a.m, a.c, a.ld_in, a.p, a.p_stride_r,
                                                        a.p_stride_c, a.scaling, a.out, vec_ok,
                                                        p_vec);
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
