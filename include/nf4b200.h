/*
 * nf4b200 — C ABI of the B200 (sm_100a) NF4 dequant / fused dequant-GEMM / LoRA kernels.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer owned by the caller and
 * borrowed for the duration of the enqueue. `stream` is a cudaStream_t passed as void*. Calls
 * are asynchronous with respect to the host; they allocate no device memory. All functions
 * return 0 on success or a negative NF4B200_E* code; nf4b200_last_error() then gives a message
 * for the calling thread. There is no CPU fallback: on a device that is not compute capability
 * 10.x every compute entry point returns NF4B200_EARCH.
 *
 * "Replaces" comments cite the reference project (mergentlegen/hackaton) by file:line.
 */
#ifndef NF4B200_H
#define NF4B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NF4B200_OK 0
#define NF4B200_EINVAL (-1)  /* bad argument: shape, alignment, dtype, null pointer */
#define NF4B200_EARCH (-2)   /* device is not sm_100 */
#define NF4B200_ECUDA (-3)   /* a CUDA runtime / driver call failed */
#define NF4B200_EDEVICE (-4) /* a kernel recorded a problem in the device status word */

enum { NF4B200_F16 = 0, NF4B200_BF16 = 1, NF4B200_F32 = 2 };

/*
 * One NF4 weight W[n_rows, n_cols] in bitsandbytes layout: the fields of bitsandbytes'
 * QuantState that the reference reads (solution/nf4.py:55-76, solution/packed.py:71-79).
 * Flat element i = row * n_cols + col lives in byte i / 2 (even element = high nibble);
 * `blocksize` consecutive flat elements share one scale.
 */
typedef struct nf4b200_weight {
    const void* codes;      /* uint8 [n_rows * n_cols / 2], 16-byte aligned */
    const void* absmax;     /* nested != 0: uint8 [n_blocks]; nested == 0: float [n_blocks] */
    const float* code2;     /* nested: float [256], second-level table; else NULL */
    const float* absmax2;   /* nested: float [ceil(n_blocks / nested_blocksize)]; else NULL */
    const float* offset;    /* nested: pointer to one float on the device; else NULL */
    const float* code16;    /* float [16]: the 4-bit table (quant_state.code) */
    int64_t n_rows;         /* N, output features */
    int64_t n_cols;         /* K, input features */
    int32_t blocksize;      /* weights per first-level scale (64) */
    int32_t nested_blocksize; /* scales per second-level scale (256) */
    int32_t nested;         /* 1: double-quantised scales, 0: flat fp32 scales */
    int32_t reserved;
    const void* scales16;   /* optional: table made by nf4b200_prepare_scales, else NULL */
} nf4b200_weight;

/* Device / build facts. */
typedef struct nf4b200_props {
    int32_t cc_major, cc_minor, sm_count, supported;
    int64_t smem_per_block_optin;
} nf4b200_props;

int nf4b200_query(int device, nf4b200_props* out);

/* Message for the last non-zero status returned on this thread ("" if none). */
const char* nf4b200_last_error(void);

/*
 * Caps the number of SMs the fused GEMM kernels of this process occupy (their persistent grids
 * otherwise take every SM); 0 restores "all". For callers that run communication kernels next to
 * the GEMMs (tensor-parallel shards: the collective of projection i overlaps the GEMM of
 * projection i+1 only if some SMs are left for it). Affects later calls, including
 * nf4b200_workspace_bytes*. No counterpart in the reference (single GPU).
 */
int nf4b200_set_sm_limit(int sms);

/*
 * Optional set-up step for the fused GEMM entry points. Writes the block scales of `w` (the
 * (double-)dequantised absmax, rounded to fp16 exactly as the GEMM's decode rounds them) as an
 * fp16 table [n_cols / 64][n_rows] into `scales16` (nf4b200_scales16_bytes(...) bytes, 16-byte
 * aligned, n_rows % 8 == 0). A weight descriptor whose `scales16` field points at that table makes
 * nf4b200_linear_fwd / _bwd_dx (and the group forms) fetch ready-made scales with one small TMA
 * copy per 64-deep step instead of gathering absmax / absmax2 themselves; results are bit-identical
 * either way. The table must be rebuilt if absmax / absmax2 / offset change. The reference has no
 * counterpart: its kernel re-derives the scales on every call (solution/nf4.py:40-52).
 * `w->scales16` is ignored by this call and by nf4b200_dequant.
 */
int64_t nf4b200_scales16_bytes(int64_t n_rows, int64_t n_cols); /* 0 if the shape is not eligible */
int nf4b200_prepare_scales(const nf4b200_weight* w, void* scales16, void* stream);

/*
 * Reads and clears the device-side status word of the current device (synchronises the device).
 * 0 = no kernel reported anything since the last call. Otherwise the call returns NF4B200_EDEVICE
 * and *status_out holds the first code recorded: 100..199 a bounded wait of the fused GEMM ran
 * out; 200 cross-entropy met a target index beyond the vocabulary (that row was treated as
 * ignored, nothing was read out of bounds); 300 nf4b200_prepare_scales met a block scale outside
 * fp16's normal range (the fused GEMM multiplies table and scale in fp16 and cannot represent
 * that block; the standalone decode can); 400 the self-test below.
 */
int nf4b200_device_status(int* status_out);

/*
 * Self-test of the failure-reporting path: launches one small kernel that waits, with the same
 * bounded wait the fused GEMM uses, on a barrier nothing ever signals; after limit_ns
 * (1 ns .. 1 s) the kernel gives up, records a status and ends by itself. The next
 * nf4b200_device_status then returns NF4B200_EDEVICE (status 400) and the context stays usable.
 * The reference has no counterpart (its Triton kernels contain no waits).
 */
int nf4b200_selftest_wait(int64_t limit_ns, void* stream);

/*
 * Standalone decode: out[n_rows, n_cols] = table[code] * scale, one rounding to out_dtype.
 * Replaces nf4_dequant_kernel / dequantize_nf4 (solution/nf4.py:28-44, 67-77) and, for nested
 * weights, the scale pre-pass _flatten_quant_states (solution/packed.py:57-79).
 * Needs n_rows * n_cols % 8 == 0 and blocksize % 8 == 0 (as solution/nf4.py:61-63).
 * Stream order: the kernel is launched as a programmatic dependent of its predecessor in the
 * stream and reads the weight's arrays (codes, absmax, code2, absmax2, offset, table) before it
 * waits for that predecessor; `out` is written after the wait. This is ordinary stream order
 * unless the predecessor is itself a kernel that releases its dependents early
 * (cudaTriggerProgrammaticLaunchCompletion) and is what writes those arrays: such a producer must
 * be separated from this call by another kernel or an event. No kernel of this library writes them.
 */
int nf4b200_dequant(const nf4b200_weight* w, void* out, int out_dtype, void* stream);

/*
 * Forward of the frozen-weight linear, decode fused into the GEMM:
 *   y[m, n_rows] = x[m, n_cols] . W^T (+ bias) (+ xa[m, rank] . lora_b[n_rows, rank]^T)
 * fp16 in, fp32 accumulate (tcgen05 / TMEM), fp16 out. Replaces NF4Linear.forward
 * (solution/nf4.py:87-92): dequantize_nf4 + torch.nn.functional.linear.
 * x: fp16, row stride ldx elements (ldx % 8 == 0, 16-byte aligned base). y likewise with ldy.
 * bias: fp16 [n_rows] or NULL. LoRA (rank 16): xa = scaling * x . A^T as fp16 [m, 16]
 * (see nf4b200_lora_down), lora_b fp16 [n_rows, 16]; pass NULL for both to skip it.
 * Needs n_cols % 64 == 0, blocksize == 64.
 * workspace: split-K scratch of at least nf4b200_workspace_bytes(...) bytes, 256-byte aligned, or
 * NULL (then one CTA walks the whole K range of its tile: correct, slower on shapes with few
 * tiles). See nf4b200_workspace_bytes for its rules.
 */
int nf4b200_linear_fwd(const nf4b200_weight* w, const void* x, int64_t m, int64_t ldx,
                       const void* bias, const void* xa, const void* lora_b, void* y, int64_t ldy,
                       void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same forward as nf4b200_linear_fwd for callers that have no device memory to lend: hosts
 * whose memory pool is fixed at start-up, plug-ins that must not allocate inside another
 * component's stream-ordered region, processes at their memory limit. The split-K scratch is a
 * fixed array of NF4B200_STATIC_SCRATCH_BYTES inside the library image (each GPU that loads the
 * library holds it until the process exits); this entry point allocates nothing. Shapes that need
 * more scratch than that are refused with NF4B200_EINVAL and a message naming both sizes.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); with
 * CUDA's lazy module loading that look-up is also the moment the driver places the library's
 * device image, the array included, on that GPU, so it is the one call that can still fail for
 * lack of memory. Make it once per device at start-up (any small shape that needs scratch will
 * do), outside any stream capture; later calls allocate nothing. All calls on a device share the
 * array: calls that can overlap on the GPU would race on it. It has no counterpart in the
 * reference.
 */
#define NF4B200_STATIC_SCRATCH_BYTES (32u << 20)
int nf4b200_linear_fwd_static(const nf4b200_weight* w, const void* x, int64_t m, int64_t ldx,
                              const void* bias, const void* xa, const void* lora_b, void* y,
                              int64_t ldy, void* stream);

/*
 * Linear with a plain fp16 weight [n_rows, n_cols] (row stride ldw elements), through the same
 * tcgen05 / TMEM pipeline as the NF4 linear with the weight tiles brought by TMA instead of
 * decoded: the lm_head products of the chunked loss, which the reference leaves to cuBLAS
 * (solution/lm_loss.py:31-40: F.linear(hidden, weight) and torch.mm(grad_logits, weight)).
 *   transposed == 0:  y[m, n_rows] = x[m, n_cols] . W^T (+ bias)
 *   transposed != 0:  y[m, n_cols] = x[m, n_rows] . W
 * fp16 in, fp32 accumulate, fp16 out; n_rows and n_cols multiples of 8, rows of x / y / W 16-byte
 * aligned. workspace: nf4b200_workspace_bytes(n_rows, n_cols, m, transposed) bytes or NULL, as for
 * nf4b200_linear_fwd.
 */
int nf4b200_fp16_linear(const void* weight, int64_t n_rows, int64_t n_cols, int64_t ldw,
                        const void* x, int64_t m, int64_t ldx, int transposed, const void* bias,
                        void* y, int64_t ldy, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Input gradient of the same linear, decode fused:
 *   dx[m, n_cols] = dy[m, n_rows] . W (+ u[m, rank] . lora_a[rank, n_cols])
 * Replaces NF4Linear.backward (solution/nf4.py:94-99): a second dequantize_nf4 + torch.matmul.
 * u = scaling * dy . B as fp16 [m, 16] (nf4b200_lora_down), lora_a fp16 [16, n_cols]; NULL to skip.
 */
int nf4b200_linear_bwd_dx(const nf4b200_weight* w, const void* dy, int64_t m, int64_t lddy,
                          const void* u, const void* lora_a, void* dx, int64_t lddx,
                          void* workspace, size_t workspace_bytes, void* stream);

/*
 * Bytes of split-K scratch that nf4b200_linear_fwd (backward == 0) or nf4b200_linear_bwd_dx
 * (backward == 1) can use for a weight [n_rows, n_cols] and m rows on the current device; 0 when
 * the shape has enough tiles to fill the GPU without splitting. The scratch holds fp32 partial
 * sums between the GEMM kernel and the reduction kernel of one call; its contents need no
 * initialisation and mean nothing afterwards, so one buffer serves any number of calls on one
 * stream. Calls that may overlap on the GPU (different streams) need separate buffers. The
 * reference has no counterpart: it lets cuBLAS pick its own workspace (solution/nf4.py:92,99).
 */
int64_t nf4b200_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m, int backward);

/*
 * Grouped launches for projections that sit side by side in the model (the call sites of
 * solution/patches.py:32-41 and :98-99: q/k/v share the post-norm hidden state, gate/up share the
 * MLP input). `count` weights (1..4) with the same n_cols go through one kernel launch:
 *   forward : y[i][m, n_rows_i] = x . W_i^T (+ bias[i]) (+ xa[i] . lora_b[i]^T)   one x, one y each
 *   backward: dx[m, n_cols] = sum_i dy[i][m, n_rows_i] . W_i (+ u[i] . lora_a[i])  one dx for all
 * which is what autograd needs, since the inputs' gradients of such projections are summed anyway.
 * The arrays bias / xa / lora_b / u / lora_a may be NULL or hold NULL entries. The scratch rules
 * are those of nf4b200_workspace_bytes. The reference launches one decode + one cuBLAS call per
 * projection (solution/nf4.py:87-99) and has no grouped counterpart.
 */
int nf4b200_linear_fwd_group(int count, const nf4b200_weight* const* w, const void* x, int64_t m,
                             int64_t ldx, const void* const* bias, const void* const* xa,
                             const void* const* lora_b, void* const* y, const int64_t* ldy,
                             void* workspace, size_t workspace_bytes, void* stream);
int nf4b200_linear_bwd_dx_group(int count, const nf4b200_weight* const* w, const void* const* dy,
                                int64_t m, const int64_t* lddy, const void* const* u,
                                const void* const* lora_a, void* dx, int64_t lddx, void* workspace,
                                size_t workspace_bytes, void* stream);
int64_t nf4b200_workspace_bytes_group(int count, const int64_t* n_rows, int64_t n_cols, int64_t m,
                                      int backward);
/*
 * Kernels that one nf4b200_linear_fwd_group / nf4b200_linear_bwd_dx_group call of this shape
 * launches with more than 64 token rows: the fused GEMM, plus one reduction per output when the
 * plan cuts the contraction into K-slices. with_scale_tables: every weight of the group carries
 * the table of nf4b200_prepare_scales (the 128-wide tiles need it). Negative: an error code.
 * (No counterpart in the reference; a benchmark's launch count reads it instead of guessing.)
 */
int nf4b200_launches_group(int count, const int64_t* n_rows, int64_t n_cols, int64_t m, int backward,
                           int with_scale_tables);

/*
 * SwiGLU, the step that follows the gate / up projections in the MLP (the reference's
 * silu_mul_kernel and SiluMul, solution/kernels.py:39-96; call site solution/patches.py:39-41:
 * `silu_mul(gate_proj(x16), up_proj(x16))`).
 *
 * nf4b200_gate_up_swiglu_fwd: gate = x . Wg^T, up = x . Wu^T, hidden = silu(gate) * up, all
 *   [m, n_rows] fp16 without padding between rows. With more than 256 token rows this is ONE
 *   kernel: each CTA pair expands 128 rows of Wg and the same 128 rows of Wu, so that a token's
 *   gate and up values meet in one accumulator row and the product is formed while the tile is
 *   drained; gate and up are rounded to fp16 first, so `hidden` holds what the two-step path
 *   gives. gate_out and up_out may both be NULL (inference: only `hidden` is written, half the
 *   output bytes of the plain grouped launch); training keeps them for the backward pass like
 *   the reference does. With fewer rows it runs the grouped GEMM and nf4b200_swiglu_fwd; scratch
 *   as nf4b200_gate_up_swiglu_workspace_bytes says (keep = 1 when gate_out / up_out are given).
 * nf4b200_swiglu_fwd / nf4b200_swiglu_bwd: the elementwise form on n contiguous fp16 values:
 *   hidden = gate * sigmoid(gate) * up;  d_up = d_hidden * gate * sig;
 *   d_gate = d_hidden * up * sig * (1 + gate * (1 - sig)); fp32 arithmetic, one rounding.
 */
int nf4b200_gate_up_swiglu_fwd(const nf4b200_weight* gate_w, const nf4b200_weight* up_w,
                               const void* x, int64_t m, int64_t ldx, void* gate_out, void* up_out,
                               void* hidden, void* workspace, size_t workspace_bytes, void* stream);
int64_t nf4b200_gate_up_swiglu_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m, int keep);
/*
 * Backward of the projection that consumes the product (down_proj: d_hidden = dy . W_down) with the
 * SwiGLU backward applied to every tile as it is drained: d_gate and d_up ([m, n_cols], no
 * padding) are written instead of d_hidden, from the gate / up arrays the forward kept. One
 * kernel when the plan has 512-row tiles and no K-slices (the training shapes); otherwise the dX
 * GEMM writes d_hidden into the scratch and nf4b200_swiglu_bwd follows
 * (nf4b200_linear_bwd_dx_swiglu_workspace_bytes). The reference runs SiluMul.backward
 * (solution/kernels.py:78-91) as a separate kernel after NF4Linear.backward (solution/nf4.py:94-102).
 */
int nf4b200_linear_bwd_dx_swiglu(const nf4b200_weight* w, const void* dy, int64_t m, int64_t lddy,
                                 const void* gate, const void* up, void* d_gate, void* d_up,
                                 void* workspace, size_t workspace_bytes, void* stream);
int64_t nf4b200_linear_bwd_dx_swiglu_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m);
int nf4b200_swiglu_fwd(const void* gate, const void* up, void* hidden, int64_t n, void* stream);
int nf4b200_swiglu_bwd(const void* d_hidden, const void* gate, const void* up, void* d_gate,
                       void* d_up, int64_t n, void* stream);

/*
 * RMSNorm on the fp32 residual stream, optionally with the residual add in the same pass: the
 * reference's rmsnorm_kernel (solution/rmsnorm.py:17-49; modes 0-3) behind `rms_norm`
 * (solution/rmsnorm.py:99-101) and `add_rms_norm` (:147-150), the producers of the fp16 X that
 * q/k/v and gate/up read (solution/packed.py:88-115).
 *   fwd: s = x (+ delta, fp16; then `total` receives s, fp32); rstd[r] = 1/sqrt(mean(s^2) + eps);
 *        y = weight * (s * rstd), stored as fp32 or fp16 (y_dtype: NF4B200_F32 / NF4B200_F16).
 *   bwd: x is the tensor that was normalised (the input, or `total`);
 *        dx = rstd * (g - xhat * mean(g * xhat)) with g = dy * weight, xhat = x * rstd,
 *        plus d_total (fp32, the gradient that reaches the sum directly) when it is not NULL.
 * x, weight, total, rstd, dx, d_total are fp32; rows are contiguous ([rows, hidden]). The
 * gradient of `weight`, which the task never needs (frozen norms), is left to the caller, as in
 * the reference (solution/rmsnorm.py:93-95).
 */
int nf4b200_rmsnorm_fwd(const void* x, const void* delta, const void* weight, void* total, void* y,
                        int y_dtype, void* rstd, int64_t rows, int64_t hidden, float eps,
                        void* stream);
int nf4b200_rmsnorm_bwd(const void* x, const void* weight, const void* rstd, const void* dy,
                        int dy_dtype, const void* d_total, void* dx, int64_t rows, int64_t hidden,
                        void* stream);

/*
 * Rotary embedding + grouped-query expansion on the packed q / k / v projections: the step after
 * the q/k/v GEMM (the reference's qkv_kernel / QKVRotate, solution/attention.py:36-192).
 *   backward == 0: q [tokens, heads*dim], k, v [tokens, kv_heads*dim] (proj_dtype: fp16 or fp32)
 *     -> q_out, k_out, v_out fp16, every k / v head written heads/kv_heads times; rows packed
 *     (tokens, heads, dim) or, with `padded`, (batch, heads, seq, dim) at (b_idx, t_idx) (the
 *     caller zero-fills the padded outputs first). y1 = x1*c1 - x2*s1, y2 = x2*c2 + x1*s2 over the
 *     two halves of a head, fp32 arithmetic, one rounding.
 *   backward != 0: q, k, v are the fp16 gradients of those outputs (same layout); q_out, k_out,
 *     v_out receive the projections' gradients (proj_dtype), copies summed, rotation inverted.
 * cos / sin: fp32 [1 or batch, seq, dim] with element strides (cos_stride_b = 0 for a broadcast
 * batch dimension); b_idx, t_idx: int32 [tokens].
 */
int nf4b200_qkv_rotate(const void* q, const void* k, const void* v, void* q_out, void* k_out,
                       void* v_out, const void* cos, const void* sin, int64_t cos_stride_b,
                       int64_t cos_stride_t, const void* b_idx, const void* t_idx, int64_t tokens,
                       int64_t seq, int heads, int kv_heads, int dim, int padded, int backward,
                       int proj_dtype, void* stream);

/*
 * Cross-entropy over the vocabulary from the lm_head's logits, the other large tensor of the step:
 * the reference's ce_kernel (solution/kernels.py:106-170) behind `ce_stats` / `ce_grad`
 * (:173-204), `fused_cross_entropy` (:207-238) and the chunked lm_head + loss
 * (solution/lm_loss.py:27-62).
 *   nf4b200_ce_stats: per row, in one pass over [rows, vocab] logits (fp16 or fp32): lse =
 *     logsumexp (0 for rows with target < 0), loss = lse - logit[target] (0 for those rows);
 *     entropy (= lse - E[x], may be NULL) and argmax (int64, first maximal index, may be NULL).
 *   nf4b200_ce_grad: grad = scale[0] * (exp(logit - lse) - onehot(target)), 0 for rows with
 *     target < 0, in the logits' type; `grad` may be `logits` (in place).
 * targets: int64 [rows]; lse, loss, entropy, scale: fp32 on the device.
 */
int nf4b200_ce_stats(const void* logits, int logits_dtype, const void* targets, void* lse, void* loss,
                     void* entropy, void* argmax, int64_t rows, int64_t vocab, void* stream);
int nf4b200_ce_grad(const void* logits, int logits_dtype, const void* targets, const void* lse,
                    const void* scale, void* grad, int64_t rows, int64_t vocab, void* stream);

/*
 * Rank-16 projection used by both passes of the LoRA update (peft's lora_A / lora_B linears;
 * third-party in the reference, configured at README.md:91 and task/task.yaml:18-21):
 *   out[m, 16] = scaling * in[m, c] . P        (fp16 in, fp32 accumulate, fp16 out)
 * P[c][j] is read at p[c * p_stride_c + j * p_stride_r]: (p_stride_r, p_stride_c) = (c, 1) for
 * a row-major [16, c] matrix (lora_A, forward), (1, 16) for a row-major [c, 16] matrix (lora_B,
 * backward).
 */
int nf4b200_lora_down(const void* in, int64_t m, int64_t c, int64_t ld_in, const void* p,
                      int64_t p_stride_r, int64_t p_stride_c, float scaling, void* out,
                      void* stream);

/*
 * Rank-16 weight gradients (contraction over the m rows, fp32 accumulate, fp32 out):
 *   out[c][j] (at out + c * o_stride_c + j * o_stride_r) = sum_m z[m, c] * s[m, j]
 * dA[16, K] = u^T . x  -> z = x, s = u, strides (o_stride_r, o_stride_c) = (K, 1);
 * dB[N, 16] = dy^T . xa -> z = dy, s = xa, strides (1, 16).
 * `out` must be zeroed by the caller (partial sums are added atomically).
 */
int nf4b200_lora_grad(const void* z, int64_t m, int64_t c, int64_t ld_z, const void* s,
                      float* out, int64_t o_stride_r, int64_t o_stride_c, void* stream);

/*
 * The two calls above for several problems (up to 8) in one launch each, with arrays in place of
 * the per-problem arguments: a layer with LoRA on q_proj and v_proj needs lora_down for both
 * adapters on the same hidden state, and four weight gradients per backward pass, each far too
 * small to fill the GPU. lora_down_batch: all problems share the row count m. Problems that do
 * not fit one launch (different layouts of p, unaligned pointers) are launched one by one; the
 * results do not depend on the route. No counterpart in the reference (peft runs one small GEMM
 * per adapter matrix).
 */
int nf4b200_lora_down_batch(int count, const void* const* in, int64_t m, const int64_t* c,
                            const int64_t* ld_in, const void* const* p, const int64_t* p_stride_r,
                            const int64_t* p_stride_c, const float* scaling, void* const* out,
                            void* stream);
int nf4b200_lora_grad_batch(int count, const void* const* z, const int64_t* m, const int64_t* c,
                            const int64_t* ld_z, const void* const* s, float* const* out,
                            const int64_t* o_stride_r, const int64_t* o_stride_c, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NF4B200_H */
