// Elementwise SwiGLU on contiguous fp16 arrays, forward and backward: the same arithmetic as the
// reference's silu_mul_kernel (solution/kernels.py:39-57): fp16 values widened to fp32, one
// rounding at the end.
//   forward : hidden = gate * sigmoid(gate) * up
//   backward: d_up   = d_hidden * gate * sigmoid(gate)
//             d_gate = d_hidden * up * sig * (1 + gate * (1 - sig))
// Pure streaming work (forward 6 B, backward 10 B per element): 16-byte loads and stores, eight
// elements per thread and step, a grid of a few CTAs per SM that strides over the array. The
// forward is only used where the product cannot be formed in the gate/up GEMM's epilogue
// (gemm.cu, EPI = 1); the backward always runs.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"
#include "swiglu.cuh"

namespace nf4 {

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __half* __restrict__ gate, const __half* __restrict__ up,
                  __half* __restrict__ hidden, long long n, int vec) {
    grid_dep_wait();
    grid_dep_launch();
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n8 = vec ? n / 8 : 0;
    for (long long i = tid; i < n8; i += stride) {
        const uint4 g = __ldcs(reinterpret_cast<const uint4*>(gate) + i);
        const uint4 u = __ldcs(reinterpret_cast<const uint4*>(up) + i);
        uint4 h;
        h.x = swiglu2(g.x, u.x); h.y = swiglu2(g.y, u.y);
        h.z = swiglu2(g.z, u.z); h.w = swiglu2(g.w, u.w);
        reinterpret_cast<uint4*>(hidden)[i] = h;
    }
    for (long long i = n8 * 8 + tid; i < n; i += stride) {
        const float g = __half2float(gate[i]), u = __half2float(up[i]);
        hidden[i] = __float2half_rn(g * sigmoid_fast(g) * u);
    }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __half* __restrict__ d_hidden, const __half* __restrict__ gate,
                  const __half* __restrict__ up, __half* __restrict__ d_gate,
                  __half* __restrict__ d_up, long long n, int vec) {
    grid_dep_wait();
    grid_dep_launch();
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n8 = vec ? n / 8 : 0;
    for (long long i = tid; i < n8; i += stride) {
        const uint4 d = __ldcs(reinterpret_cast<const uint4*>(d_hidden) + i);
        const uint4 g = __ldcs(reinterpret_cast<const uint4*>(gate) + i);
        const uint4 u = __ldcs(reinterpret_cast<const uint4*>(up) + i);
        uint4 dg, du;
        swiglu_bwd2(d.x, g.x, u.x, dg.x, du.x);
        swiglu_bwd2(d.y, g.y, u.y, dg.y, du.y);
        swiglu_bwd2(d.z, g.z, u.z, dg.z, du.z);
        swiglu_bwd2(d.w, g.w, u.w, dg.w, du.w);
        reinterpret_cast<uint4*>(d_gate)[i] = dg;
        reinterpret_cast<uint4*>(d_up)[i] = du;
    }
    for (long long i = n8 * 8 + tid; i < n; i += stride) {
        float dg, du;
        swiglu_bwd1(__half2float(d_hidden[i]), __half2float(gate[i]), __half2float(up[i]), dg, du);
        d_gate[i] = __float2half_rn(dg);
        d_up[i] = __float2half_rn(du);
    }
}

static unsigned stream_grid(long long n, int sm_count) {
    const int sms = sm_count > 0 ? sm_count : 148;
    long long blocks = (n / 8 + 255) / 256;
    if (blocks < 1) blocks = 1;
    const long long cap = (long long)sms * 8;
    return (unsigned)(blocks < cap ? blocks : cap);
}

static int all_aligned16(const void* a, const void* b, const void* c, const void* d = nullptr,
                         const void* e = nullptr) {
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
                           reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(d) |
                           reinterpret_cast<uintptr_t>(e);
    return (bits & 15) == 0 ? 1 : 0;
}

cudaError_t launch_swiglu_fwd(const __half* gate, const __half* up, __half* hidden, long long n,
                              int sm_count, cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    return launch_pdl(swiglu_fwd_kernel, dim3(stream_grid(n, sm_count)), dim3(256), 0, stream, gate,
                      up, hidden, n, all_aligned16(gate, up, hidden));
}

cudaError_t launch_swiglu_bwd(const __half* d_hidden, const __half* gate, const __half* up,
                              __half* d_gate, __half* d_up, long long n, int sm_count,
                              cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    return launch_pdl(swiglu_bwd_kernel, dim3(stream_grid(n, sm_count)), dim3(256), 0, stream,
                      d_hidden, gate, up, d_gate, d_up, n,
                      all_aligned16(d_hidden, gate, up, d_gate, d_up));
}

}  // namespace nf4
