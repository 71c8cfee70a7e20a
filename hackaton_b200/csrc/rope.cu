// Rotary embedding + grouped-query expansion on the packed q / k / v projections, forward and
// backward in one launch each: the arithmetic of the reference's qkv_kernel
// (solution/attention.py:36-146).
//   forward : q, k rotated (fp32 arithmetic, one rounding to fp16); every k and v head written
//             REP = heads / kv_heads times, so that the attention that follows sees `heads` heads;
//             output rows either packed (N, heads, D) or padded (B, heads, T, D)
//   backward: the copies' gradients summed (fp32), the inverse rotation for q and k, written
//             packed (N, heads * D) in the projections' type
// with y1 = x1*c1 - x2*s1, y2 = x2*c2 + x1*s2 over the two halves of a head (c1/c2, s1/s2: the two
// halves of the cos / sin rows of the token's position).
// A work item is one (token, slot) pair, slot = q heads, then k heads, then v heads; HALF / 4
// threads share it, each with 4 consecutive elements of both halves (8- or 16-byte accesses).
// Pure streaming: HBM bound.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

template <bool F32>
__device__ __forceinline__ float4 rope_load4(const void* p, long long idx) {
    if (F32) return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx));
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(p) + idx));
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <bool F32>
__device__ __forceinline__ void rope_store4(void* p, long long idx, float4 v) {
    if (F32) {
        *reinterpret_cast<float4*>(static_cast<float*>(p) + idx) = v;
    } else {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<const uint32_t*>(&a);
        raw.y = *reinterpret_cast<const uint32_t*>(&b);
        *reinterpret_cast<uint2*>(static_cast<__half*>(p) + idx) = raw;
    }
}

__device__ __forceinline__ float4 fma4(float4 a, float4 b, float4 c, float4 d, float sign) {
    // a * b + sign * c * d, element by element
    return make_float4(a.x * b.x + sign * (c.x * d.x), a.y * b.y + sign * (c.y * d.y),
                       a.z * b.z + sign * (c.z * d.z), a.w * b.w + sign * (c.w * d.w));
}

template <bool F32, bool BACKWARD>
__global__ void __launch_bounds__(256)
qkv_rotate_kernel(const RopeArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    const int half = a.dim / 2, lps = half / 4;  // threads per work item
    const int slots = a.heads + 2 * a.kv_heads;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long item = gid / lps;
    if (item >= a.tokens * slots) return;
    const int j = (int)(gid % lps) * 4;
    const long long tok = item / slots;
    const int slot = (int)(item % slots);
    const int b = a.b_idx[tok], t = a.t_idx[tok];
    const int rep = a.heads / a.kv_heads;
    // row (in units of heads) of output head h: packed (N, H, D) or padded (B, H, T, D)
    const long long head_base = a.padded ? (long long)b * a.heads * a.seq + t : tok * a.heads;
    const long long head_step = a.padded ? a.seq : 1;

    float4 c1, c2, s1, s2;
    if (slot < a.heads + a.kv_heads) {
        const long long cb = (long long)b * a.cos_stride_b + (long long)t * a.cos_stride_t;
        c1 = __ldg(reinterpret_cast<const float4*>(a.cos + cb + j));
        c2 = __ldg(reinterpret_cast<const float4*>(a.cos + cb + half + j));
        s1 = __ldg(reinterpret_cast<const float4*>(a.sin + cb + j));
        s2 = __ldg(reinterpret_cast<const float4*>(a.sin + cb + half + j));
    }

    if (!BACKWARD) {
        if (slot < a.heads) {
            const long long xi = tok * (long long)(a.heads * a.dim) + slot * a.dim + j;
            const float4 x1 = rope_load4<F32>(a.q, xi), x2 = rope_load4<F32>(a.q, xi + half);
            const long long yi = (head_base + slot * head_step) * a.dim + j;
            rope_store4<false>(a.qo, yi, fma4(x1, c1, x2, s1, -1.f));
            rope_store4<false>(a.qo, yi + half, fma4(x2, c2, x1, s2, 1.f));
        } else {
            const bool is_k = slot < a.heads + a.kv_heads;
            const int head = slot - a.heads - (is_k ? 0 : a.kv_heads);
            const void* src = is_k ? a.k : a.v;
            void* dst = is_k ? a.ko : a.vo;
            const long long xi = tok * (long long)(a.kv_heads * a.dim) + head * a.dim + j;
            const float4 x1 = rope_load4<F32>(src, xi), x2 = rope_load4<F32>(src, xi + half);
            const float4 y1 = is_k ? fma4(x1, c1, x2, s1, -1.f) : x1;
            const float4 y2 = is_k ? fma4(x2, c2, x1, s2, 1.f) : x2;
            for (int r = 0; r < rep; ++r) {
                const long long yi = (head_base + (head * rep + r) * head_step) * a.dim + j;
                rope_store4<false>(dst, yi, y1);
                rope_store4<false>(dst, yi + half, y2);
            }
        }
    } else {
        // here q / k / v are the gradients of the rotated heads (fp16), qo / ko / vo the
        // gradients of the projections
        if (slot < a.heads) {
            const long long yi = (head_base + slot * head_step) * a.dim + j;
            const float4 d1 = rope_load4<false>(a.q, yi), d2 = rope_load4<false>(a.q, yi + half);
            const long long xi = tok * (long long)(a.heads * a.dim) + slot * a.dim + j;
            rope_store4<F32>(a.qo, xi, fma4(d1, c1, d2, s2, 1.f));
            rope_store4<F32>(a.qo, xi + half, fma4(d2, c2, d1, s1, -1.f));
        } else {
            const bool is_k = slot < a.heads + a.kv_heads;
            const int head = slot - a.heads - (is_k ? 0 : a.kv_heads);
            const void* src = is_k ? a.k : a.v;
            void* dst = is_k ? a.ko : a.vo;
            float4 d1 = make_float4(0.f, 0.f, 0.f, 0.f), d2 = d1;
            for (int r = 0; r < rep; ++r) {
                const long long yi = (head_base + (head * rep + r) * head_step) * a.dim + j;
                const float4 u = rope_load4<false>(src, yi), w = rope_load4<false>(src, yi + half);
                d1.x += u.x; d1.y += u.y; d1.z += u.z; d1.w += u.w;
                d2.x += w.x; d2.y += w.y; d2.z += w.z; d2.w += w.w;
            }
            const long long xi = tok * (long long)(a.kv_heads * a.dim) + head * a.dim + j;
            rope_store4<F32>(dst, xi, is_k ? fma4(d1, c1, d2, s2, 1.f) : d1);
            rope_store4<F32>(dst, xi + half, is_k ? fma4(d2, c2, d1, s1, -1.f) : d2);
        }
    }
}

cudaError_t launch_qkv_rotate(const RopeArgs& a, cudaStream_t stream) {
    if (a.tokens <= 0) return cudaSuccess;
    const int lps = a.dim / 8;
    const long long threads = a.tokens * (a.heads + 2 * a.kv_heads) * lps;
    const dim3 grid((unsigned)((threads + 255) / 256)), block(256);
    if (a.proj_f32)
        return a.backward ? launch_pdl(qkv_rotate_kernel<true, true>, grid, block, 0, stream, a)
                          : launch_pdl(qkv_rotate_kernel<true, false>, grid, block, 0, stream, a);
    return a.backward ? launch_pdl(qkv_rotate_kernel<false, true>, grid, block, 0, stream, a)
                      : launch_pdl(qkv_rotate_kernel<false, false>, grid, block, 0, stream, a);
}

}  // namespace nf4
