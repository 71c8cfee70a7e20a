/*
 * Plain C restatement of the reference's NF4 decode and frozen-weight linear.
 * TEST INFRASTRUCTURE: loaded only by the tests, the smoke check and the CPU-baseline leg of the
 * benchmark; the product library never links or calls it.
 *
 * Parity: the flat decode is pinned by golden vectors produced with the reference's own kernel
 * (tests/golden/); the nested-absmax decode restates bitsandbytes' published arithmetic and is
 * "parity unpinned" (bitsandbytes is not available to run against).
 *
 * Layout (reference solution/nf4.py:7-14, 33-44): flat element i lives in byte i/2; the even
 * element is the high nibble; `blocksize` consecutive elements share one scale;
 * value = table[code] * scale in fp32, rounded once to fp16.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static inline uint16_t f32_to_f16_bits(float f) {
    _Float16 h = (_Float16)f; /* round to nearest even */
    uint16_t u;
    memcpy(&u, &h, sizeof u);
    return u;
}

static inline float f16_bits_to_f32(uint16_t u) {
    _Float16 h;
    memcpy(&h, &u, sizeof u);
    return (float)h;
}

/* solution/packed.py:74-77: code2[u8] * absmax2[i / nested_blocksize], then += offset.
 * `volatile` keeps the product a separately rounded fp32 value (no fused multiply-add). */
void oracle_flatten_absmax(const uint8_t *absmax_u8, const float *code2, const float *absmax2,
                           float offset, int64_t n_blocks, int nested_blocksize, float *out) {
    for (int64_t i = 0; i < n_blocks; ++i) {
        volatile float prod = code2[absmax_u8[i]] * absmax2[i / nested_blocksize];
        out[i] = prod + offset;
    }
}

/* solution/nf4.py:33-44 with flat fp32 scales; out holds fp16 bit patterns. */
void oracle_dequant_flat_f16(const uint8_t *packed, const float *absmax, const float *code16,
                             int64_t n, int blocksize, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        uint8_t byte = packed[i >> 1];
        int code = (i & 1) ? (byte & 15) : (byte >> 4);
        out[i] = f32_to_f16_bits(code16[code] * absmax[i / blocksize]);
    }
}

/* Double-quantised layout: nested scales decoded on the fly, then the flat decode. */
void oracle_dequant_nested_f16(const uint8_t *packed, const uint8_t *absmax_u8,
                               const float *code2, const float *absmax2, float offset,
                               const float *code16, int64_t n, int blocksize,
                               int nested_blocksize, uint16_t *out) {
    for (int64_t i = 0; i < n; ++i) {
        int64_t blk = i / blocksize;
        volatile float prod = code2[absmax_u8[blk]] * absmax2[blk / nested_blocksize];
        float scale = prod + offset;
        uint8_t byte = packed[i >> 1];
        int code = (i & 1) ? (byte & 15) : (byte >> 4);
        out[i] = f32_to_f16_bits(code16[code] * scale);
    }
}

/* solution/nf4.py:87-92: Y[M,N] = X[M,K] W[N,K]^T (+ bias), fp32 accumulate, fp16 result.
 * Straightforward loops: meant for small checks, not for timing. */
void oracle_linear_fwd_f16(const uint16_t *x, const uint16_t *w, const uint16_t *bias,
                           int64_t M, int64_t N, int64_t K, uint16_t *y) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k)
                acc += f16_bits_to_f32(x[m * K + k]) * f16_bits_to_f32(w[n * K + k]);
            if (bias) acc += f16_bits_to_f32(bias[n]);
            y[m * N + n] = f32_to_f16_bits(acc);
        }
}

/* solution/nf4.py:94-99: dX[M,K] = dY[M,N] W[N,K], fp32 accumulate, fp16 result. */
void oracle_linear_bwd_f16(const uint16_t *dy, const uint16_t *w, int64_t M, int64_t N,
                           int64_t K, uint16_t *dx) {
    for (int64_t m = 0; m < M; ++m)
        for (int64_t k = 0; k < K; ++k) {
            float acc = 0.f;
            for (int64_t n = 0; n < N; ++n)
                acc += f16_bits_to_f32(dy[m * N + n]) * f16_bits_to_f32(w[n * K + k]);
            dx[m * K + k] = f32_to_f16_bits(acc);
        }
}
