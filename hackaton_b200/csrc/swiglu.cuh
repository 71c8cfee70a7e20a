// SwiGLU arithmetic shared by the elementwise kernels (swiglu.cu) and the GEMM epilogues (gemm.cu):
// the reference's silu_mul_kernel (solution/kernels.py:39-57) on pairs of fp16 values, fp32
// inside, one rounding.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace nf4 {

__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

__device__ __forceinline__ uint32_t swiglu2(uint32_t g2, uint32_t u2) {
    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&g2));
    const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&u2));
    const __half2 h = __floats2half2_rn(g.x * sigmoid_fast(g.x) * u.x, g.y * sigmoid_fast(g.y) * u.y);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__device__ __forceinline__ void swiglu_bwd1(float d, float g, float u, float& dg, float& du) {
    const float sig = sigmoid_fast(g);
    du = d * g * sig;
    dg = d * u * sig * (1.f + g * (1.f - sig));
}

__device__ __forceinline__ void swiglu_bwd2(uint32_t d2, uint32_t g2, uint32_t u2, uint32_t& dg2,
                                            uint32_t& du2) {
    const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&d2));
    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&g2));
    const float2 u = __half22float2(*reinterpret_cast<const __half2*>(&u2));
    float a0, a1, b0, b1;
    swiglu_bwd1(d.x, g.x, u.x, a0, b0);
    swiglu_bwd1(d.y, g.y, u.y, a1, b1);
    const __half2 hg = __floats2half2_rn(a0, a1), hu = __floats2half2_rn(b0, b1);
    dg2 = *reinterpret_cast<const uint32_t*>(&hg);
    du2 = *reinterpret_cast<const uint32_t*>(&hu);
}

}  // namespace nf4
