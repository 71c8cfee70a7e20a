// NF4 nibble expansion helpers shared by the kernels.
//
// Storage (reference solution/nf4.py:7-14, 33-44): byte k of a little-endian 32-bit word holds
// weight 2k in its high nibble and weight 2k+1 in its low nibble, so a word carries 8
// consecutive weights.
//
// Two decoders live here:
//  * exact:     table[code] * scale in fp32, one rounding to the output type. This is the
//               arithmetic of the reference kernel and is what the standalone dequant uses.
//  * register:  a 16-entry fp16 table held in eight registers and indexed with byte-permute
//               instructions, scaled by a half2 multiply. No shared-memory traffic; used inside
//               the GEMM main loop where results only need fp16-GEMM tolerance.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define NF4_HD __host__ __device__ __forceinline__
#else
#define NF4_HD inline
#endif

namespace nf4 {

// prmt.b32 in its generic mode: each selector nibble picks one of the 8 bytes of {a (0-3),
// b (4-7)}; with the nibble's bit 3 set, the byte's sign bit is replicated over the result byte.
NF4_HD uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
#if defined(__CUDA_ARCH__)
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
#else
    uint64_t src = ((uint64_t)b << 32) | a;
    uint32_t d = 0;
    for (int i = 0; i < 4; ++i) {
        uint32_t nib = (sel >> (4 * i)) & 0xF;
        uint32_t byte = (uint32_t)(src >> (8 * (nib & 7))) & 0xFF;
        if (nib & 8) byte = (byte & 0x80) ? 0xFF : 0x00;
        d |= byte << (8 * i);
    }
    return d;
#endif
}

// fp16 table split into byte planes: lo[j] holds the low bytes of entries 4j..4j+3, hi[j] the
// high bytes.
struct RegLut {
    uint32_t lo[4];
    uint32_t hi[4];
};

NF4_HD RegLut make_reg_lut(const uint16_t (&table_f16_bits)[16]) {
    RegLut l;
    for (int j = 0; j < 4; ++j) {
        l.lo[j] = 0;
        l.hi[j] = 0;
        for (int e = 0; e < 4; ++e) {
            uint32_t v = table_f16_bits[4 * j + e];
            l.lo[j] |= (v & 0xFF) << (8 * e);
            l.hi[j] |= (v >> 8) << (8 * e);
        }
    }
    return l;
}

// Eight unscaled fp16 table values for one word, as four packed pairs in weight order.
NF4_HD void lookup_word(uint32_t w, const RegLut& L, uint32_t (&out)[4]) {
    const uint32_t sel_lo = w & 0x77777777u;  // nibbles 0..3 (bit 3 cleared) in the low 16 bits
    const uint32_t sel_hi = sel_lo >> 16;     // nibbles 4..7
    // Per-nibble "code >= 8" byte masks. Odd nibbles have bit 3 on a byte's sign bit already.
    const uint32_t m_odd = prmt(w, 0u, 0xBA98u);        // nibbles 1,3,5,7
    const uint32_t m_even = prmt(w << 4, 0u, 0xBA98u);  // nibbles 0,2,4,6
    const uint32_t m_lo = prmt(m_even, m_odd, 0x5140u);  // nibbles 0,1,2,3
    const uint32_t m_hi = prmt(m_even, m_odd, 0x7362u);  // nibbles 4,5,6,7
    {
        const uint32_t la = prmt(L.lo[0], L.lo[1], sel_lo), lb = prmt(L.lo[2], L.lo[3], sel_lo);
        const uint32_t ha = prmt(L.hi[0], L.hi[1], sel_lo), hb = prmt(L.hi[2], L.hi[3], sel_lo);
        const uint32_t lo = (la & ~m_lo) | (lb & m_lo);
        const uint32_t hi = (ha & ~m_lo) | (hb & m_lo);
        out[0] = prmt(lo, hi, 0x4051u);  // weights 0,1 = nibbles 1,0
        out[1] = prmt(lo, hi, 0x6273u);  // weights 2,3 = nibbles 3,2
    }
    {
        const uint32_t la = prmt(L.lo[0], L.lo[1], sel_hi), lb = prmt(L.lo[2], L.lo[3], sel_hi);
        const uint32_t ha = prmt(L.hi[0], L.hi[1], sel_hi), hb = prmt(L.hi[2], L.hi[3], sel_hi);
        const uint32_t lo = (la & ~m_hi) | (lb & m_hi);
        const uint32_t hi = (ha & ~m_hi) | (hb & m_hi);
        out[2] = prmt(lo, hi, 0x4051u);  // weights 4,5 = nibbles 5,4
        out[3] = prmt(lo, hi, 0x6273u);  // weights 6,7 = nibbles 7,6
    }
}

#if defined(__CUDACC__)
// Eight scaled fp16 weights of one word: table lookup in registers, one half2 multiply per pair.
__device__ __forceinline__ uint4 decode_word_reg(uint32_t w, const RegLut& L, __half2 scale2) {
    uint32_t t[4];
    lookup_word(w, L, t);
    uint4 o;
    __half2 v;
    v = __hmul2(*reinterpret_cast<__half2*>(&t[0]), scale2); o.x = *reinterpret_cast<uint32_t*>(&v);
    v = __hmul2(*reinterpret_cast<__half2*>(&t[1]), scale2); o.y = *reinterpret_cast<uint32_t*>(&v);
    v = __hmul2(*reinterpret_cast<__half2*>(&t[2]), scale2); o.z = *reinterpret_cast<uint32_t*>(&v);
    v = __hmul2(*reinterpret_cast<__half2*>(&t[3]), scale2); o.w = *reinterpret_cast<uint32_t*>(&v);
    return o;
}

// Second-level scale decode (reference solution/packed.py:74-77): a product and a sum that are
// rounded separately; the intrinsics stop the compiler from fusing them into one FMA.
__device__ __forceinline__ float nested_scale(float code2_value, float absmax2, float offset) {
    return __fadd_rn(__fmul_rn(code2_value, absmax2), offset);
}
#endif

}  // namespace nf4
