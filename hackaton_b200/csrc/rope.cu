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
// A work item is one (token, slot) pair, slot = q heads, then k heads, then v heads; HALF / 8
// threads share it, each with 8 consecutive elements of both halves (16-byte accesses for fp16).
// Pure streaming: HBM bound.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

struct F8 {
    float v[8];
};

template <bool F32>
__device__ __forceinline__ F8 rope_load8(const void* p, long long idx) {
    F8 r;
    if (F32) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx));
        const float4 b = __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(p) + idx + 4));
        r.v[0] = a.x; r.v[1] = a.y; r.v[2] = a.z; r.v[3] = a.w;
        r.v[4] = b.x; r.v[5] = b.y; r.v[6] = b.z; r.v[7] = b.w;
    } else {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(p) + idx));
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            r.v[2 * i] = f.x;
            r.v[2 * i + 1] = f.y;
        }
    }
    return r;
}

template <bool F32>
__device__ __forceinline__ void rope_store8(void* p, long long idx, const F8& r) {
    if (F32) {
        float* d = static_cast<float*>(p) + idx;
        *reinterpret_cast<float4*>(d) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
        *reinterpret_cast<float4*>(d + 4) = make_float4(r.v[4], r.v[5], r.v[6], r.v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(r.v[2 * i], r.v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(static_cast<__half*>(p) + idx) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// a * b + sign * c * d, element by element
__device__ __forceinline__ F8 fma8(const F8& a, const F8& b, const F8& c, const F8& d, float sign) {
    F8 r;
#pragma unroll
    for (int i = 0; i < 8; ++i) r.v[i] = a.v[i] * b.v[i] + sign * (c.v[i] * d.v[i]);
    return r;
}

constexpr int ROPE_MAX_REP = 4;  // copies whose loads are issued together in the backward

template <bool F32, bool BACKWARD>
__global__ void __launch_bounds__(256, 4)
qkv_rotate_kernel(const RopeArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    // threads per work item: dim / 16 (a power of two), 8 elements of each half per thread.
    // 32-bit index arithmetic (the launcher checks that the thread count fits).
    const int half = a.dim / 2;
    const unsigned slots = (unsigned)(a.heads + 2 * a.kv_heads);
    const unsigned gid = blockIdx.x * blockDim.x + threadIdx.x;
    // Forward: a token's 16 slots side by side. Backward: every token's q heads first, then every
    // token's k / v heads, so that a CTA holds either light items (q) or heavy ones (k / v read
    // `rep` copies) and no warp idles in a CTA that waits for its one heavy warp (measured:
    // 62 -> 54 us; the same order made the forward 4 % slower).
    const unsigned item = gid >> a.lps_shift;
    if (item >= (unsigned)a.tokens * slots) return;
    const unsigned q_items = (unsigned)a.tokens * (unsigned)a.heads;
    unsigned tok_u, slot_u;
    if (!BACKWARD) {
        tok_u = item / slots;
        slot_u = item - tok_u * slots;
    } else if (item < q_items) {
        tok_u = item / (unsigned)a.heads;
        slot_u = item - tok_u * (unsigned)a.heads;
    } else {
        const unsigned r = item - q_items, kv2 = 2u * (unsigned)a.kv_heads;
        tok_u = r / kv2;
        slot_u = (unsigned)a.heads + (r - tok_u * kv2);
    }
    const int j = (int)(gid & ((1u << a.lps_shift) - 1u)) * 8;
    const long long tok = tok_u;
    const int slot = (int)slot_u;
    const int b = a.b_idx[tok], t = a.t_idx[tok];
    const int rep = a.heads / a.kv_heads;
    // row (in units of heads) of output head h: packed (N, H, D) or padded (B, H, T, D)
    const long long head_base = a.padded ? (long long)b * a.heads * a.seq + t : tok * a.heads;
    const long long head_step = a.padded ? a.seq : 1;

    // cos / sin of the token's position (L1 / L2 hits: 16 work items share a row); fetched where
    // they are used, so that in the backward they do not sit in registers next to the copies
    const long long cb = (long long)b * a.cos_stride_b + (long long)t * a.cos_stride_t;
    F8 c1, c2, s1, s2;
    auto load_angles = [&]() {
        c1 = rope_load8<true>(a.cos, cb + j);
        c2 = rope_load8<true>(a.cos, cb + half + j);
        s1 = rope_load8<true>(a.sin, cb + j);
        s2 = rope_load8<true>(a.sin, cb + half + j);
    };
    if (!BACKWARD && slot < a.heads + a.kv_heads) load_angles();

    if (!BACKWARD) {
        if (slot < a.heads) {
            const long long xi = tok * (long long)(a.heads * a.dim) + slot * a.dim + j;
            const F8 x1 = rope_load8<F32>(a.q, xi), x2 = rope_load8<F32>(a.q, xi + half);
            const long long yi = (head_base + slot * head_step) * a.dim + j;
            rope_store8<false>(a.qo, yi, fma8(x1, c1, x2, s1, -1.f));
            rope_store8<false>(a.qo, yi + half, fma8(x2, c2, x1, s2, 1.f));
        } else {
            const bool is_k = slot < a.heads + a.kv_heads;
            const int head = slot - a.heads - (is_k ? 0 : a.kv_heads);
            const void* src = is_k ? a.k : a.v;
            void* dst = is_k ? a.ko : a.vo;
            const long long xi = tok * (long long)(a.kv_heads * a.dim) + head * a.dim + j;
            const F8 x1 = rope_load8<F32>(src, xi), x2 = rope_load8<F32>(src, xi + half);
            const F8 y1 = is_k ? fma8(x1, c1, x2, s1, -1.f) : x1;
            const F8 y2 = is_k ? fma8(x2, c2, x1, s2, 1.f) : x2;
            for (int r = 0; r < rep; ++r) {
                const long long yi = (head_base + (head * rep + r) * head_step) * a.dim + j;
                rope_store8<false>(dst, yi, y1);
                rope_store8<false>(dst, yi + half, y2);
            }
        }
    } else {
        // here q / k / v are the gradients of the rotated heads (fp16), qo / ko / vo the
        // gradients of the projections
        if (slot < a.heads) {
            const long long yi = (head_base + slot * head_step) * a.dim + j;
            const F8 d1 = rope_load8<false>(a.q, yi), d2 = rope_load8<false>(a.q, yi + half);
            load_angles();
            const long long xi = tok * (long long)(a.heads * a.dim) + slot * a.dim + j;
            rope_store8<F32>(a.qo, xi, fma8(d1, c1, d2, s2, 1.f));
            rope_store8<F32>(a.qo, xi + half, fma8(d2, c2, d1, s1, -1.f));
        } else {
            const bool is_k = slot < a.heads + a.kv_heads;
            const int head = slot - a.heads - (is_k ? 0 : a.kv_heads);
            const void* src = is_k ? a.k : a.v;
            void* dst = is_k ? a.ko : a.vo;
            F8 d1, d2;
#pragma unroll
            for (int i = 0; i < 8; ++i) d1.v[i] = d2.v[i] = 0.f;
            for (int r0 = 0; r0 < rep; r0 += ROPE_MAX_REP) {
                // the copies' loads go out together (raw fp16), the sums follow in copy order
                uint4 u[ROPE_MAX_REP], w[ROPE_MAX_REP];
#pragma unroll
                for (int r = 0; r < ROPE_MAX_REP; ++r) {
                    u[r] = w[r] = make_uint4(0u, 0u, 0u, 0u);
                    if (r0 + r < rep) {
                        const long long yi = (head_base + (head * rep + r0 + r) * head_step) * a.dim + j;
                        u[r] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(src) + yi));
                        w[r] = __ldg(reinterpret_cast<const uint4*>(static_cast<const __half*>(src) + yi + half));
                    }
                }
#pragma unroll
                for (int r = 0; r < ROPE_MAX_REP; ++r) {
                    if (r0 + r < rep) {
                        const uint32_t uu[4] = {u[r].x, u[r].y, u[r].z, u[r].w};
                        const uint32_t ww[4] = {w[r].x, w[r].y, w[r].z, w[r].w};
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&uu[i]));
                            const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&ww[i]));
                            d1.v[2 * i] += f.x; d1.v[2 * i + 1] += f.y;
                            d2.v[2 * i] += g.x; d2.v[2 * i + 1] += g.y;
                        }
                    }
                }
            }
            const long long xi = tok * (long long)(a.kv_heads * a.dim) + head * a.dim + j;
            if (is_k) load_angles();
            rope_store8<F32>(dst, xi, is_k ? fma8(d1, c1, d2, s2, 1.f) : d1);
            rope_store8<F32>(dst, xi + half, is_k ? fma8(d2, c2, d1, s1, -1.f) : d2);
        }
    }
}

cudaError_t launch_qkv_rotate(const RopeArgs& a_in, cudaStream_t stream) {
    if (a_in.tokens <= 0) return cudaSuccess;
    RopeArgs a = a_in;
    const int lps = a.dim / 16;
    a.lps_shift = 0;
    while ((1 << a.lps_shift) < lps) ++a.lps_shift;
    const long long threads = a.tokens * (a.heads + 2 * a.kv_heads) * lps;
    if ((1 << a.lps_shift) != lps || threads >= (1ll << 31)) return cudaErrorInvalidValue;
    const dim3 grid((unsigned)((threads + 255) / 256)), block(256);
    if (a.proj_f32)
        return a.backward ? launch_pdl(qkv_rotate_kernel<true, true>, grid, block, 0, stream, a)
                          : launch_pdl(qkv_rotate_kernel<true, false>, grid, block, 0, stream, a);
    return a.backward ? launch_pdl(qkv_rotate_kernel<false, true>, grid, block, 0, stream, a)
                      : launch_pdl(qkv_rotate_kernel<false, false>, grid, block, 0, stream, a);
}

}  // namespace nf4
