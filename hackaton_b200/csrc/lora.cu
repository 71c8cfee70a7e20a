// Rank-16 side products of the LoRA update (peft's lora_A / lora_B linears; third-party in the
// reference, configured at README.md:91 and task/task.yaml:18-21).
//
//   lora_down: out[M,16] = scaling * in[M,C] . P      feeds the GEMM kernels' K-extension step
//   lora_grad: out[C,16] += z[M,C]^T . s[M,16]        weight gradients dA, dB (fp32)
//
// Both are skinny (16 wide) and bound by reading `in` / `z` once from HBM (2 B per element);
// plain SIMT with shared-memory staging, fp32 accumulation.
#include <cuda_fp16.h>

#include "kernels.h"

namespace nf4 {

constexpr int LD_ROWS = 16;      // rows of `in` per block
constexpr int LD_THREADS = 128;  // 8 threads per row, 2 outputs each
constexpr int LD_CHUNK = 128;    // columns staged per step

__global__ void __launch_bounds__(LD_THREADS)
lora_down_kernel(const __half* __restrict__ in, long long m, long long c, long long ld_in,
                 const __half* __restrict__ p, long long p_stride_r, long long p_stride_c,
                 float scaling, __half* __restrict__ out) {
    __shared__ float in_s[LD_ROWS][LD_CHUNK + 1];
    __shared__ float p_s[LD_CHUNK][16 + 1];
    const long long row0 = (long long)blockIdx.x * LD_ROWS;
    const int r = threadIdx.x >> 3;
    const int j0 = (threadIdx.x & 7) * 2;
    float acc0 = 0.f, acc1 = 0.f;
    for (long long c0 = 0; c0 < c; c0 += LD_CHUNK) {
        for (int i = threadIdx.x; i < LD_ROWS * LD_CHUNK; i += LD_THREADS) {
            const int rr = i / LD_CHUNK, cc = i % LD_CHUNK;
            const long long gr = row0 + rr, gc = c0 + cc;
            in_s[rr][cc] = (gr < m && gc < c) ? __half2float(in[gr * ld_in + gc]) : 0.f;
        }
        for (int i = threadIdx.x; i < LD_CHUNK * 16; i += LD_THREADS) {
            // walk P along its contiguous direction
            int cc, j;
            if (p_stride_c == 1) { j = i / LD_CHUNK; cc = i % LD_CHUNK; }
            else                 { cc = i / 16;      j = i % 16; }
            const long long gc = c0 + cc;
            p_s[cc][j] = gc < c ? __half2float(p[gc * p_stride_c + j * p_stride_r]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int cc = 0; cc < LD_CHUNK; ++cc) {
            const float v = in_s[r][cc];
            acc0 = fmaf(v, p_s[cc][j0], acc0);
            acc1 = fmaf(v, p_s[cc][j0 + 1], acc1);
        }
        __syncthreads();
    }
    const long long gr = row0 + r;
    if (gr < m) {
        const __half2 h = __floats2half2_rn(acc0 * scaling, acc1 * scaling);
        *reinterpret_cast<__half2*>(out + gr * 16 + j0) = h;
    }
}

cudaError_t launch_lora_down(const LoraDownArgs& a, cudaStream_t stream) {
    if (a.m <= 0) return cudaSuccess;
    const unsigned blocks = (unsigned)((a.m + LD_ROWS - 1) / LD_ROWS);
    lora_down_kernel<<<blocks, LD_THREADS, 0, stream>>>(a.in, a.m, a.c, a.ld_in, a.p, a.p_stride_r,
                                                        a.p_stride_c, a.scaling, a.out);
    return cudaGetLastError();
}

constexpr int LG_COLS = 64;    // columns of z per block
constexpr int LG_ROWS = 256;   // rows (contraction) per block
constexpr int LG_THREADS = 256;

__global__ void __launch_bounds__(LG_THREADS)
lora_grad_kernel(const __half* __restrict__ z, long long m, long long c, long long ld_z,
                 const __half* __restrict__ s, float* __restrict__ out, long long o_stride_r,
                 long long o_stride_c) {
    __shared__ float s_s[LG_ROWS][16];
    const long long c0 = (long long)blockIdx.x * LG_COLS;
    const long long m0 = (long long)blockIdx.y * LG_ROWS;
    for (int i = threadIdx.x; i < LG_ROWS * 16; i += LG_THREADS) {
        const long long gm = m0 + i / 16;
        s_s[i / 16][i % 16] = gm < m ? __half2float(s[gm * 16 + i % 16]) : 0.f;
    }
    __syncthreads();
    const int cl = threadIdx.x % LG_COLS;
    const int j0 = (threadIdx.x / LG_COLS) * 4;
    const long long gc = c0 + cl;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    if (gc < c) {
        const long long rows = (m - m0 < LG_ROWS) ? (m - m0) : LG_ROWS;
        for (int r = 0; r < rows; ++r) {
            const float v = __half2float(z[(m0 + r) * ld_z + gc]);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(v, s_s[r][j0 + j], acc[j]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
            atomicAdd(out + gc * o_stride_c + (j0 + j) * o_stride_r, acc[j]);
    }
}

cudaError_t launch_lora_grad(const LoraGradArgs& a, cudaStream_t stream) {
    if (a.m <= 0 || a.c <= 0) return cudaSuccess;
    dim3 grid((unsigned)((a.c + LG_COLS - 1) / LG_COLS), (unsigned)((a.m + LG_ROWS - 1) / LG_ROWS));
    lora_grad_kernel<<<grid, LG_THREADS, 0, stream>>>(a.z, a.m, a.c, a.ld_z, a.s, a.out,
                                                      a.o_stride_r, a.o_stride_c);
    return cudaGetLastError();
}

}  // namespace nf4
