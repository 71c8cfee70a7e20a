// RMSNorm on the fp32 residual stream, one pass each way, with the residual add folded in: the
// arithmetic of the reference's rmsnorm_kernel (solution/rmsnorm.py:17-49) in its four modes
//   0  forward            y = w * (x * rstd),            rstd = 1 / sqrt(mean(x^2) + eps)
//   1  backward           dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w, xhat = x * rstd
//   2  add + forward      s = x + delta (delta fp16), s stored, then mode 0 on s
//   3  backward + the gradient that reaches the sum directly: dx += d_total
// x, w, s, dx, d_total fp32; y (and dy) fp32 or fp16 (the projections that follow read fp16).
// One warp owns one row: the row is read once into registers with 16-byte loads that are all in
// flight together (hidden = 128 * NV floats; NV = 12 and 28 are the Qwen2.5 1.5B / 7B widths),
// two warp reductions by shuffles, outputs written once. HBM bound: 6 to 14 bytes per element.
// Any other width takes the generic kernel, which walks the row twice (the second time out of
// L1 / L2). Inputs are read through the read-only path (ld.global.nc), which lets the compiler
// issue a row's loads ahead of its stores: outputs must not overlap inputs.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

constexpr int RN_WARPS = 8;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float4 load4_any(const void* base, long long idx4, int half) {
    if (half) {
        const uint2 raw = __ldg(reinterpret_cast<const uint2*>(base) + idx4);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    return __ldg(reinterpret_cast<const float4*>(base) + idx4);
}

__device__ __forceinline__ void store4_any(void* base, long long idx4, int half, float4 v) {
    if (half) {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&a);
        raw.y = *reinterpret_cast<const uint32_t*>(&b);
        reinterpret_cast<uint2*>(base)[idx4] = raw;
    } else {
        reinterpret_cast<float4*>(base)[idx4] = v;
    }
}

template <int NV>
__global__ void __launch_bounds__(RN_WARPS * 32, NV <= 16 ? 2 : 1)
rmsnorm_rows_kernel(const RmsNormArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const long long base4 = row * (long long)(NV * 32);  // in units of 4 elements
    float4 x[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) x[i] = __ldg(reinterpret_cast<const float4*>(a.x) + base4 + i * 32 + lane);
    if (a.mode == 2) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 d = load4_any(a.delta, base4 + i * 32 + lane, 1);
            x[i].x += d.x; x[i].y += d.y; x[i].z += d.z; x[i].w += d.w;
            reinterpret_cast<float4*>(a.total)[base4 + i * 32 + lane] = x[i];
        }
    }
    const float inv_h = 1.f / (float)(NV * 128);
    if ((a.mode & 1) == 0) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NV; ++i)
            ss += x[i].x * x[i].x + x[i].y * x[i].y + x[i].z * x[i].z + x[i].w * x[i].w;
        ss = warp_sum(ss);
        const float rstd = 1.f / sqrtf(ss * inv_h + a.eps);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.w) + i * 32 + lane);
            store4_any(a.y, base4 + i * 32 + lane, a.y_half,
                       make_float4(w.x * (x[i].x * rstd), w.y * (x[i].y * rstd),
                                   w.z * (x[i].z * rstd), w.w * (x[i].w * rstd)));
        }
        if (lane == 0) a.rstd[row] = rstd;
    } else {
        const float rstd = a.rstd[row];
        float dot = 0.f;
        if (a.y_half && NV <= 16) {
            // fp16 dy of a narrow row stays in registers (2 per 4 elements) next to xhat
            uint2 dyr[NV];
#pragma unroll
            for (int i = 0; i < NV; ++i) dyr[i] = __ldg(reinterpret_cast<const uint2*>(a.dy) + base4 + i * 32 + lane);
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const float4 w = __ldg(reinterpret_cast<const float4*>(a.w) + i * 32 + lane);
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&dyr[i].x));
                const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&dyr[i].y));
                x[i].x *= rstd; x[i].y *= rstd; x[i].z *= rstd; x[i].w *= rstd;  // xhat
                dot += lo.x * w.x * x[i].x + lo.y * w.y * x[i].y + hi.x * w.z * x[i].z + hi.y * w.w * x[i].w;
            }
            const float mean_gx = warp_sum(dot) * inv_h;
#pragma unroll
            for (int i = 0; i < NV; ++i) {
                const float4 w = __ldg(reinterpret_cast<const float4*>(a.w) + i * 32 + lane);
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&dyr[i].x));
                const float2 hi = __half22float2(*reinterpret_cast<const __half2*>(&dyr[i].y));
                float4 dx = make_float4(rstd * (lo.x * w.x - x[i].x * mean_gx), rstd * (lo.y * w.y - x[i].y * mean_gx),
                                        rstd * (hi.x * w.z - x[i].z * mean_gx), rstd * (hi.y * w.w - x[i].w * mean_gx));
                if (a.mode == 3) {
                    const float4 t = __ldg(reinterpret_cast<const float4*>(a.d_total) + base4 + i * 32 + lane);
                    dx.x += t.x; dx.y += t.y; dx.z += t.z; dx.w += t.w;
                }
                reinterpret_cast<float4*>(a.dx)[base4 + i * 32 + lane] = dx;
            }
            return;
        }
        // otherwise the row of dy is read twice (the second time out of L1 / L2): keeping it next
        // to xhat would need up to 2 * NV float4 registers per thread
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.w) + i * 32 + lane);
            const float4 dy = load4_any(a.dy, base4 + i * 32 + lane, a.y_half);
            x[i].x *= rstd; x[i].y *= rstd; x[i].z *= rstd; x[i].w *= rstd;  // xhat
            dot += dy.x * w.x * x[i].x + dy.y * w.y * x[i].y + dy.z * w.z * x[i].z + dy.w * w.w * x[i].w;
        }
        const float mean_gx = warp_sum(dot) * inv_h;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(a.w) + i * 32 + lane);
            const float4 dy = load4_any(a.dy, base4 + i * 32 + lane, a.y_half);
            float4 dx = make_float4(rstd * (dy.x * w.x - x[i].x * mean_gx), rstd * (dy.y * w.y - x[i].y * mean_gx),
                                    rstd * (dy.z * w.z - x[i].z * mean_gx), rstd * (dy.w * w.w - x[i].w * mean_gx));
            if (a.mode == 3) {
                const float4 t = __ldg(reinterpret_cast<const float4*>(a.d_total) + base4 + i * 32 + lane);
                dx.x += t.x; dx.y += t.y; dx.z += t.z; dx.w += t.w;
            }
            reinterpret_cast<float4*>(a.dx)[base4 + i * 32 + lane] = dx;
        }
    }
}

// Any width: scalar accesses, the row is walked twice.
__global__ void __launch_bounds__(RN_WARPS * 32)
rmsnorm_generic_kernel(const RmsNormArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * RN_WARPS + (threadIdx.x >> 5);
    if (row >= a.rows) return;
    const long long base = row * a.hidden;
    const float* xs = a.x + base;
    if (a.mode == 2) {
        const __half* d = static_cast<const __half*>(a.delta) + base;
        for (int c = lane; c < a.hidden; c += 32) a.total[base + c] = xs[c] + __half2float(d[c]);
        __syncwarp();
        xs = a.total + base;
    }
    const float inv_h = 1.f / (float)a.hidden;
    if ((a.mode & 1) == 0) {
        float ss = 0.f;
        for (int c = lane; c < a.hidden; c += 32) ss += xs[c] * xs[c];
        const float rstd = 1.f / sqrtf(warp_sum(ss) * inv_h + a.eps);
        for (int c = lane; c < a.hidden; c += 32) {
            const float v = a.w[c] * (xs[c] * rstd);
            if (a.y_half) static_cast<__half*>(a.y)[base + c] = __float2half_rn(v);
            else          static_cast<float*>(a.y)[base + c] = v;
        }
        if (lane == 0) a.rstd[row] = rstd;
    } else {
        const float rstd = a.rstd[row];
        float dot = 0.f;
        for (int c = lane; c < a.hidden; c += 32) {
            const float dy = a.y_half ? __half2float(static_cast<const __half*>(a.dy)[base + c])
                                      : static_cast<const float*>(a.dy)[base + c];
            dot += dy * a.w[c] * (xs[c] * rstd);
        }
        const float mean_gx = warp_sum(dot) * inv_h;
        for (int c = lane; c < a.hidden; c += 32) {
            const float dy = a.y_half ? __half2float(static_cast<const __half*>(a.dy)[base + c])
                                      : static_cast<const float*>(a.dy)[base + c];
            float dx = rstd * (dy * a.w[c] - xs[c] * rstd * mean_gx);
            if (a.mode == 3) dx += a.d_total[base + c];
            a.dx[base + c] = dx;
        }
    }
}

cudaError_t launch_rmsnorm(const RmsNormArgs& a, cudaStream_t stream) {
    if (a.rows <= 0 || a.hidden <= 0) return cudaSuccess;
    const dim3 grid((unsigned)((a.rows + RN_WARPS - 1) / RN_WARPS)), block(RN_WARPS * 32);
    const uintptr_t bits = reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w) |
                           reinterpret_cast<uintptr_t>(a.y) | reinterpret_cast<uintptr_t>(a.dy) |
                           reinterpret_cast<uintptr_t>(a.dx) | reinterpret_cast<uintptr_t>(a.delta) |
                           reinterpret_cast<uintptr_t>(a.total) | reinterpret_cast<uintptr_t>(a.d_total);
    const bool vec = (bits & 15) == 0;
    if (vec && a.hidden == 12 * 128) return launch_pdl(rmsnorm_rows_kernel<12>, grid, block, 0, stream, a);
    if (vec && a.hidden == 28 * 128) return launch_pdl(rmsnorm_rows_kernel<28>, grid, block, 0, stream, a);
    return launch_pdl(rmsnorm_generic_kernel, grid, block, 0, stream, a);
}

}  // namespace nf4
