// Standalone NF4 decode: packed codes + (flat fp32 | double-quantised) scales -> fp16/bf16/fp32.
//
// Replaces the reference's `nf4_dequant_kernel` (solution/nf4.py:28-44) and, for nested states,
// the one-off `_flatten_quant_states` pre-pass (solution/packed.py:57-79): the two-level scale
// is decoded here, in the same kernel. Arithmetic is the reference's, so results are bit-equal:
// scale = code2[u8] * absmax2[i / 256] (fp32), then + offset (fp32, separately rounded);
// value = table[code] * scale (fp32), rounded once to the output type.
//
// HBM bound: 0.5159 B read + 2 B written per weight (fp16 out, nested scales). One lane per
// 32-bit word of codes (8 weights), eight words in flight per thread: 128-byte coalesced loads,
// one wave of resident CTAs in a grid-stride loop. 16-bit outputs leave through a 32 KB staging
// area and one bulk copy per tile, fp32 outputs with 512-byte coalesced stores.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "decode.cuh"
#include "kernels.h"
#include "ptx.cuh"

namespace nf4 {

template <typename T>
struct Pack8;
template <>
struct Pack8<__half> {
    __device__ static uint4 pack(const float (&v)[8]) {
        uint4 o;
        __half2 h;
        h = __floats2half2_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2half2_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        return o;
    }
    __device__ static void store(__half* dst, const float (&v)[8]) {
        __stcs(reinterpret_cast<uint4*>(dst), pack(v));
    }
};
template <>
struct Pack8<__nv_bfloat16> {
    __device__ static uint4 pack(const float (&v)[8]) {
        uint4 o;
        __nv_bfloat162 h;
        h = __floats2bfloat162_rn(v[0], v[1]); o.x = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(v[2], v[3]); o.y = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(v[4], v[5]); o.z = *reinterpret_cast<uint32_t*>(&h);
        h = __floats2bfloat162_rn(v[6], v[7]); o.w = *reinterpret_cast<uint32_t*>(&h);
        return o;
    }
    __device__ static void store(__nv_bfloat16* dst, const float (&v)[8]) {
        __stcs(reinterpret_cast<uint4*>(dst), pack(v));
    }
};
template <>
struct Pack8<float> {
    __device__ static uint4 pack(const float (&)[8]) { return make_uint4(0u, 0u, 0u, 0u); }  // (unused)
    __device__ static void store(float* dst, const float (&v)[8]) {
        __stcs(reinterpret_cast<float4*>(dst), make_float4(v[0], v[1], v[2], v[3]));
        __stcs(reinterpret_cast<float4*>(dst) + 1, make_float4(v[4], v[5], v[6], v[7]));
    }
};

constexpr int DEQ_THREADS = 256;
constexpr int DEQ_WORDS_PER_THREAD = 8;   // 32-bit code words (8 weights each) in flight per thread

// The 16-entry table is kept once per lane (entry e of lane l at [e * 32 + l]): every look-up of a
// warp then goes to 32 different banks whatever the codes are.
// SHIFTS: block sizes are powers of two (the bitsandbytes layout: 64 and 256), so the block of a
// word and the second-level block of a block are shifts; other sizes take the dividing variant.
// Bulk copy shared -> global (asynchronous, tracked by the thread's bulk group), and the wait
// until the copies of this thread have read their source.
__device__ __forceinline__ void bulk_store(void* gdst, uint32_t smem_src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
                 "r"(smem_src), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// STAGED (16-bit outputs): a tile is expanded into 32 KB of shared
// memory and leaves as one bulk copy, so all that is left to do after the dependency wait is one
// instruction per CTA.
template <typename T, bool NESTED, bool SHIFTS, bool STAGED>
__global__ void __launch_bounds__(DEQ_THREADS)
nf4_dequant_kernel(const uint32_t* __restrict__ codes, const void* __restrict__ absmax,
                   const float* __restrict__ code2, const float* __restrict__ absmax2,
                   const float* __restrict__ offset_ptr, const float* __restrict__ code16,
                   T* __restrict__ out, long long n_words, int words_per_block,
                   int nested_blocksize, int block_shift, int nested_shift) {
    const long long tile = (long long)DEQ_THREADS * DEQ_WORDS_PER_THREAD;
    // Programmatic dependent launch: everything this kernel reads (codes, scales, tables) belongs
    // to the weight and is never written by a kernel of the stream, so the first tile's loads and
    // the table set-up run while the predecessor is still draining; the dependency wait comes
    // before the first store (the output buffer may be one the predecessor still reads or writes).
    grid_dep_launch();
    __shared__ float table[16 * 32];
    __shared__ float table2[256];
    __shared__ __align__(128) uint4 stage[STAGED ? DEQ_THREADS * DEQ_WORDS_PER_THREAD : 1];
    const float* my_table = table + (threadIdx.x & 31);

    uint32_t word[DEQ_WORDS_PER_THREAD];
    float raw[DEQ_WORDS_PER_THREAD];      // flat: the scale; nested: the second-level scale
    uint32_t q8[DEQ_WORDS_PER_THREAD];    // nested: the 8-bit first-level code
    auto issue = [&](long long base) {
#pragma unroll
        for (int j = 0; j < DEQ_WORDS_PER_THREAD; ++j) {
            const long long w = base + j * DEQ_THREADS + threadIdx.x;
            word[j] = 0;
            raw[j] = 0.f;
            q8[j] = 0;
            if (w < n_words) {
                word[j] = __ldcs(codes + w);
                const long long blk = SHIFTS ? (w >> block_shift) : (w / words_per_block);
                if (NESTED) {
                    q8[j] = __ldg(static_cast<const uint8_t*>(absmax) + blk);
                    const long long blk2 = SHIFTS ? (blk >> nested_shift) : (blk / nested_blocksize);
                    raw[j] = __ldg(absmax2 + blk2);
                } else {
                    raw[j] = __ldg(static_cast<const float*>(absmax) + blk);
                }
            }
        }
    };
    // the first tile's loads go out before the tables are built: their round trips overlap
    long long base = (long long)blockIdx.x * tile;
    if (base < n_words) issue(base);
    for (int i = threadIdx.x; i < 16 * 32; i += DEQ_THREADS) table[i] = code16[i >> 5];
    if (NESTED) table2[threadIdx.x] = code2[threadIdx.x];
    const float offset = NESTED ? *offset_ptr : 0.f;
    __syncthreads();
    bool waited = false;

    while (base < n_words) {
        if (STAGED) {
            if (waited) {   // (not the first tile: the previous bulk copy still reads the staging area)
                if (threadIdx.x == 0) bulk_store_wait_read();
                __syncthreads();
            }
#pragma unroll
            for (int j = 0; j < DEQ_WORDS_PER_THREAD; ++j) {
                const long long w = base + j * DEQ_THREADS + threadIdx.x;
                if (w < n_words) {
                    const float scale = NESTED ? nested_scale(table2[q8[j]], raw[j], offset) : raw[j];
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t byte = (word[j] >> (8 * k)) & 0xFFu;
                        v[2 * k] = __fmul_rn(my_table[(byte >> 4) << 5], scale);
                        v[2 * k + 1] = __fmul_rn(my_table[(byte & 15u) << 5], scale);
                    }
                    stage[j * DEQ_THREADS + threadIdx.x] = Pack8<T>::pack(v);
                }
            }
            fence_proxy_async_smem();   // generic-proxy writes, then an async-proxy read
            __syncthreads();
            if (!waited) { grid_dep_wait(); waited = true; }
            if (threadIdx.x == 0) {
                const long long n = n_words - base < tile ? n_words - base : tile;
                bulk_store(out + base * 8, (uint32_t)__cvta_generic_to_shared(stage), (uint32_t)(n * 16));
            }
        } else {
            if (!waited) { grid_dep_wait(); waited = true; }
#pragma unroll
            for (int j = 0; j < DEQ_WORDS_PER_THREAD; ++j) {
                const long long w = base + j * DEQ_THREADS + threadIdx.x;
                if (w < n_words) {
                    const float scale = NESTED ? nested_scale(table2[q8[j]], raw[j], offset) : raw[j];
                    float v[8];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t byte = (word[j] >> (8 * k)) & 0xFFu;
                        v[2 * k] = __fmul_rn(my_table[(byte >> 4) << 5], scale);
                        v[2 * k + 1] = __fmul_rn(my_table[(byte & 15u) << 5], scale);
                    }
                    Pack8<T>::store(out + w * 8, v);
                }
            }
        }
        base += (long long)gridDim.x * tile;
        if (base < n_words) issue(base);
    }
    // the staging area must outlive the last bulk copy's read
    if (STAGED && threadIdx.x == 0) bulk_store_wait_read();
}

static int exact_log2(long long v) {
    if (v <= 0 || (v & (v - 1)) != 0) return -1;
    int s = 0;
    while ((1ll << s) < v) ++s;
    return s;
}

template <typename T, bool STAGED>
static cudaError_t launch_t(const DequantArgs& a, cudaStream_t stream) {
    const long long n_words = a.n / 8;
    const long long tile = (long long)DEQ_THREADS * DEQ_WORDS_PER_THREAD;
    long long blocks = (n_words + tile - 1) / tile;
    // One wave: as many CTAs as are resident at once (8 per SM at 256 threads, 6 with the 32 KB
    // staging area), each walking the words in grid-stride order; a second, partly filled wave
    // would cost as much as the first.
    const long long cap = (long long)a.sm_count * (STAGED ? 6 : 8);
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const int wpb = a.blocksize / 8;
    const int bshift = exact_log2(wpb);
    const int nshift = a.nested ? exact_log2(a.nested_blocksize) : 0;
    const bool shifts = bshift >= 0 && nshift >= 0;
    const dim3 grid((unsigned)blocks), block(DEQ_THREADS);
    const uint32_t* codes = static_cast<const uint32_t*>(a.codes);
    T* out = static_cast<T*>(a.out);
    if (a.nested) {
        if (shifts)
            return launch_pdl(nf4_dequant_kernel<T, true, true, STAGED>, grid, block, 0, stream, codes,
                              a.absmax, a.code2, a.absmax2, a.offset, a.code16, out, n_words, wpb,
                              a.nested_blocksize, bshift, nshift);
        return launch_pdl(nf4_dequant_kernel<T, true, false, STAGED>, grid, block, 0, stream, codes,
                          a.absmax, a.code2, a.absmax2, a.offset, a.code16, out, n_words, wpb,
                          a.nested_blocksize, 0, 0);
    }
    const float* none = nullptr;
    if (shifts)
        return launch_pdl(nf4_dequant_kernel<T, false, true, STAGED>, grid, block, 0, stream, codes,
                          a.absmax, none, none, none, a.code16, out, n_words, wpb, 1, bshift, 0);
    return launch_pdl(nf4_dequant_kernel<T, false, false, STAGED>, grid, block, 0, stream, codes,
                      a.absmax, none, none, none, a.code16, out, n_words, wpb, 1, 0, 0);
}

cudaError_t launch_dequant(const DequantArgs& a, cudaStream_t stream) {
    // (the C entry point has checked that `out` is 16-byte aligned, which the bulk copies need)
    switch (a.out_dtype) {
        case 0: return launch_t<__half, true>(a, stream);
        case 1: return launch_t<__nv_bfloat16, true>(a, stream);
        case 2: return launch_t<float, false>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

// Block-scale table for the fused GEMM: out[kb][row] = fp16(scale of block row * bpr + kb), i.e. the
// (double-)dequantised absmax rounded to fp16 exactly as the GEMM's decode step rounds it, stored
// k-block-major so that the scales a tile needs are contiguous in both directions.
__global__ void __launch_bounds__(256)
prepare_scales_kernel(const void* __restrict__ absmax, const float* __restrict__ code2,
                      const float* __restrict__ absmax2, const float* __restrict__ offset,
                      long long n_rows, long long bpr, int nested, int nested_blocksize,
                      __half* __restrict__ out, int* status) {
    grid_dep_wait();    // (programmatic dependent launch: the predecessor's results)
    grid_dep_launch();
    bool out_of_range = false;
    const long long total = n_rows * bpr;
    const float off = nested ? __ldg(offset) : 0.f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long kb = i / n_rows, row = i % n_rows;  // consecutive threads: consecutive rows
        const long long blk = row * bpr + kb;
        float sc;
        if (nested)
            sc = nested_scale(__ldg(code2 + __ldg(static_cast<const uint8_t*>(absmax) + blk)),
                              __ldg(absmax2 + blk / nested_blocksize), off);
        else
            sc = __ldg(static_cast<const float*>(absmax) + blk);
        const __half h = __float2half_rn(sc);
        out[i] = h;
        // The fused GEMM multiplies in fp16: a scale that rounds to inf, to zero or into the
        // subnormals loses the block there (the standalone decode multiplies in fp32 and is fine).
        const float back = fabsf(__half2float(h));
        if (sc != 0.f && (back > 65504.f || back < 6.103515625e-5f)) out_of_range = true;
    }
    if (out_of_range && status != nullptr) atomicCAS(status, 0, STATUS_SCALE_RANGE);
}

cudaError_t launch_prepare_scales(const void* absmax, const float* code2, const float* absmax2,
                                  const float* offset, long long n_rows, long long bpr, int nested,
                                  int nested_blocksize, __half* out, int sm_count,
                                  cudaStream_t stream) {
    const long long total = n_rows * bpr;
    long long blocks = (total + 255) / 256;
    const long long cap = (long long)sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return launch_pdl(prepare_scales_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, absmax,
                      code2, absmax2, offset, n_rows, bpr, nested, nested_blocksize, out,
                      device_status_word());
}

}  // namespace nf4
