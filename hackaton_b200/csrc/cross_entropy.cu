// Cross-entropy over the vocabulary straight from the fp16 (or fp32) logits: the two passes of
// the reference's ce_kernel (solution/kernels.py:106-170).
//   statistics: one pass per row keeps a running max, sum of exp and sum of exp * logit (online
//     log-sum-exp): lse, loss = lse - logit[target] (0 for target < 0), optionally the entropy of
//     the softmax (lse - E[x]) and the first index of the maximum. No fp32 copy of the logits.
//   gradient:   grad = scale * (softmax - onehot(target)), 0 for rows with target < 0; may be
//     written over the logits themselves (every element is read before it is replaced).
// One CTA of 256 threads per row (a row of Qwen2.5's 151,936 logits is 297 KB), 16-byte loads.
// A thread rescales its running sums once per 8 logits (when their maximum beats the running
// one), not once per logit, and works in the base-2 domain (one FMA + one ex2 per logit). HBM bound: 2 bytes per logit for the statistics, 4 for the gradient.
#include <cuda_fp16.h>

#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

constexpr int CE_THREADS = 256;
constexpr float CE_NEG = -1.0e30f;  // finite "minus infinity", as in the reference (kernels.py:36)

// Running statistics of the logits seen so far, kept in the base-2 domain so that a logit costs
// one fused multiply-add and one ex2: maximum m (and m2 = m * log2(e)), s = sum 2^(t) with
// t = x * log2(e) - m2, d = sum 2^(t) * t (relative to the maximum, so that the entropy
// ln(s) - d / (s * log2(e)) does not come out of the difference of two numbers as large as the
// logits), first index of the maximum.
struct CeState {
    float m, m2, s, d;
    int idx;
};

constexpr float CE_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float ex2f(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ CeState ce_merge(const CeState& a, const CeState& b) {
    CeState r;
    const bool a_wins = a.m > b.m || (a.m == b.m && a.idx <= b.idx);
    r.m = fmaxf(a.m, b.m);
    r.m2 = fmaxf(a.m2, b.m2);
    const float ta = a.m2 - r.m2, tb = b.m2 - r.m2;  // <= 0
    const float fa = ex2f(ta), fb = ex2f(tb);
    r.s = a.s * fa + b.s * fb;
    r.d = fa * (a.d + a.s * ta) + fb * (b.d + b.s * tb);
    r.idx = a.m == b.m ? min(a.idx, b.idx) : (a_wins ? a.idx : b.idx);
    return r;
}

template <bool F32>
__device__ __forceinline__ void ce_load8(const void* row, long long i, float (&x)[8]) {
    if (F32) {
        const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(row) + i);
        const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(row) + i + 4);
        x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
    } else {
        const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __half*>(row) + i);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
            x[2 * e] = f.x;
            x[2 * e + 1] = f.y;
        }
    }
}

template <bool F32>
__device__ __forceinline__ float ce_load1(const void* row, long long i) {
    return F32 ? static_cast<const float*>(row)[i] : __half2float(static_cast<const __half*>(row)[i]);
}

template <bool F32>
__global__ void __launch_bounds__(CE_THREADS)
ce_stats_kernel(const CeArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    __shared__ CeState part[CE_THREADS / 32];
    const long long row = blockIdx.x;
    const void* base = F32 ? static_cast<const void*>(static_cast<const float*>(a.logits) + row * a.vocab)
                           : static_cast<const void*>(static_cast<const __half*>(a.logits) + row * a.vocab);
    CeState st = {CE_NEG, CE_NEG * CE_LOG2E, 0.f, 0.f, 0};
    const bool vec = a.vec != 0;
    const long long n8 = vec ? a.vocab / 8 : 0;
#pragma unroll 4
    for (long long v = threadIdx.x; v < n8; v += CE_THREADS) {
        float x[8];
        ce_load8<F32>(base, v * 8, x);
        float lm = x[0];
#pragma unroll
        for (int e = 1; e < 8; ++e) lm = fmaxf(lm, x[e]);
        if (lm > st.m) {  // rare after the first few vectors: only then look for the position
            int li = 7;
#pragma unroll
            for (int e = 6; e >= 0; --e)
                if (x[e] == lm) li = e;
            const float lm2 = lm * CE_LOG2E, t = st.m2 - lm2;
            const float r = ex2f(t);
            st.d = r * (st.d + st.s * t);
            st.s *= r;
            st.m = lm;
            st.m2 = lm2;
            st.idx = (int)(v * 8) + li;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float t = fmaf(x[e], CE_LOG2E, -st.m2);
            const float w = ex2f(t);
            st.s += w;
            st.d = fmaf(w, t, st.d);
        }
    }
    for (long long i = n8 * 8 + threadIdx.x; i < a.vocab; i += CE_THREADS) {
        const float x = ce_load1<F32>(base, i);
        if (x > st.m) {
            const float x2 = x * CE_LOG2E, t = st.m2 - x2;
            const float r = ex2f(t);
            st.d = r * (st.d + st.s * t);
            st.s *= r;
            st.m = x;
            st.m2 = x2;
            st.idx = (int)i;
        }
        const float t = fmaf(x, CE_LOG2E, -st.m2);
        const float w = ex2f(t);
        st.s += w;
        st.d = fmaf(w, t, st.d);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        CeState other;
        other.m = __shfl_xor_sync(0xffffffffu, st.m, o);
        other.m2 = __shfl_xor_sync(0xffffffffu, st.m2, o);
        other.s = __shfl_xor_sync(0xffffffffu, st.s, o);
        other.d = __shfl_xor_sync(0xffffffffu, st.d, o);
        other.idx = __shfl_xor_sync(0xffffffffu, st.idx, o);
        st = ce_merge(st, other);
    }
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = st;
    __syncthreads();
    if (threadIdx.x == 0) {
        CeState t = part[0];
        for (int w = 1; w < CE_THREADS / 32; ++w) t = ce_merge(t, part[w]);
        // A target beyond the vocabulary (a tokenizer / padding mismatch) is treated like an
        // ignored row, its logit is never read, and the device status word records it.
        const long long target = a.targets[row];
        const bool valid = target >= 0 && target < a.vocab;
        if (target >= a.vocab && a.status != nullptr) atomicCAS(a.status, 0, STATUS_CE_TARGET_RANGE);
        const float ln_s = logf(t.s);
        const float lse = t.m + ln_s;
        const float picked = ce_load1<F32>(base, valid ? target : 0);
        a.lse[row] = valid ? lse : 0.f;
        a.loss[row] = valid ? lse - picked : 0.f;
        if (a.entropy != nullptr) a.entropy[row] = ln_s - t.d / (t.s * CE_LOG2E);  // = lse - E[x]
        if (a.argmax != nullptr) a.argmax[row] = t.idx;
    }
}

template <bool F32>
__global__ void __launch_bounds__(CE_THREADS)
ce_grad_kernel(const CeArgs a) {
    grid_dep_wait();
    grid_dep_launch();
    const long long row = blockIdx.x;
    const long long target = a.targets[row];
    const float lse = a.lse[row];
    // ignored rows and rows whose target lies beyond the vocabulary get exact zeros (their lse
    // is 0: exp may overflow)
    const bool valid = target >= 0 && target < a.vocab;
    const float scale = *a.scale;
    const void* base = F32 ? static_cast<const void*>(static_cast<const float*>(a.logits) + row * a.vocab)
                           : static_cast<const void*>(static_cast<const __half*>(a.logits) + row * a.vocab);
    void* out = F32 ? static_cast<void*>(static_cast<float*>(a.grad) + row * a.vocab)
                    : static_cast<void*>(static_cast<__half*>(a.grad) + row * a.vocab);
    const long long n8 = a.vec ? a.vocab / 8 : 0;
    // four vectors per thread and step: their loads go out before the first store (the output may
    // be the input array, so the compiler has to keep loads behind earlier stores)
    for (long long v0 = threadIdx.x; v0 < n8; v0 += 4 * CE_THREADS) {
        float x[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (v0 + u * CE_THREADS < n8) ce_load8<F32>(base, (v0 + u * CE_THREADS) * 8, x[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long v = v0 + u * CE_THREADS;
            if (v >= n8) break;
            float g[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float hot = (v * 8 + e == target) ? 1.f : 0.f;
                g[e] = valid ? (__expf(x[u][e] - lse) - hot) * scale : 0.f;
            }
            if (F32) {
                float* o = static_cast<float*>(out) + v * 8;
                *reinterpret_cast<float4*>(o) = make_float4(g[0], g[1], g[2], g[3]);
                *reinterpret_cast<float4*>(o + 4) = make_float4(g[4], g[5], g[6], g[7]);
            } else {
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const __half2 h = __floats2half2_rn(g[2 * e], g[2 * e + 1]);
                    w[e] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(static_cast<__half*>(out) + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
    }
    for (long long i = n8 * 8 + threadIdx.x; i < a.vocab; i += CE_THREADS) {
        const float x = ce_load1<F32>(base, i);
        const float g = valid ? (__expf(x - lse) - (i == target ? 1.f : 0.f)) * scale : 0.f;
        if (F32) static_cast<float*>(out)[i] = g;
        else     static_cast<__half*>(out)[i] = __float2half_rn(g);
    }
}

cudaError_t launch_ce(const CeArgs& a_in, cudaStream_t stream) {
    if (a_in.rows <= 0 || a_in.vocab <= 0) return cudaSuccess;
    CeArgs a = a_in;
    const int elem = a.f32 ? 4 : 2;
    // 16-byte accesses need every row to start on a 16-byte boundary
    a.vec = ((reinterpret_cast<uintptr_t>(a.logits) | reinterpret_cast<uintptr_t>(a.grad)) % 16 == 0 &&
             (a.vocab * elem) % 16 == 0) ? 1 : 0;
    const dim3 grid((unsigned)a.rows), block(CE_THREADS);
    if (a.grad != nullptr)
        return a.f32 ? launch_pdl(ce_grad_kernel<true>, grid, block, 0, stream, a)
                     : launch_pdl(ce_grad_kernel<false>, grid, block, 0, stream, a);
    return a.f32 ? launch_pdl(ce_stats_kernel<true>, grid, block, 0, stream, a)
                 : launch_pdl(ce_stats_kernel<false>, grid, block, 0, stream, a);
}

}  // namespace nf4
