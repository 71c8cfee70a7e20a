// Internal launch interface between the C-ABI layer (capi.cu) and the kernels.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nf4 {

// True unless NF4B200_PDL=0: kernels are launched with programmatic stream serialization allowed, so
// that a kernel's set-up overlaps the tail of its predecessor (every kernel of the library calls
// griddepcontrol.wait before its first global-memory access).
bool pdl_enabled();

// <<<grid, block, smem, stream>>> with that attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

struct DequantArgs {
    const void* codes;
    const void* absmax;
    const float* code2;
    const float* absmax2;
    const float* offset;
    const float* code16;
    void* out;
    long long n;  // number of weights
    int blocksize;
    int nested_blocksize;
    int nested;
    int out_dtype;  // 0 fp16, 1 bf16, 2 fp32
    int sm_count;
};

cudaError_t launch_dequant(const DequantArgs& a, cudaStream_t stream);

// fp16 block-scale table [n_cols / 64][n_rows] of a blocksize-64 weight (see dequant.cu).
cudaError_t launch_prepare_scales(const void* absmax, const float* code2, const float* absmax2,
                                  const float* offset, long long n_rows, long long bpr, int nested,
                                  int nested_blocksize, __half* out, int sm_count,
                                  cudaStream_t stream);

// Fused dequant-GEMM. trans_w == false: out[M, N_w] = act[M, K_w] . W^T (forward).
// trans_w == true: out[M, K_w] = act[M, N_w] . W (input gradient).
struct GemmArgs {
    const uint8_t* codes;
    const void* absmax;
    const float* code2;
    const float* absmax2;
    const float* offset;
    const float* code16;
    const __half* scales16;  // optional ready-made block scales [k_w / 64][n_w] (fp16), or null
    const __half* dense_w;   // instead of the NF4 fields: a plain fp16 weight [n_w, k_w], or null
    long long ld_w;          // its row pitch in elements
    long long n_w, k_w;
    int nested;
    int nested_blocksize;
    const __half* act;
    long long m, ld_act;
    __half* out;
    long long ld_out;
    const __half* bias;   // forward only, may be null
    const __half* ext_a;  // [M, 16] fp16 rank-16 left factor (xa or u), may be null
    const __half* ext_b;  // forward: lora_b [N_w, 16]; backward: lora_a [16, K_w]
    bool trans_w;
    int sm_count;
    void* workspace;          // split-K scratch (counters, then fp32 partial tiles); may be null
    size_t workspace_bytes;
};

constexpr int GEMM_MAX_GROUP = 4;  // weights that one grouped launch can take

// Tiling and split-K plan of one GEMM call.
struct GemmPlan {
    int cg;            // CTAs cooperating on one tile (1, or 2 = CTA pair)
    int nacc;          // 128-row accumulators per CTA (1 or 2)
    int bn;            // output-tile width: 256, or 128 (pair kernel with two accumulators only)
    int m_tiles, n_tiles;
    int splits;        // units sharing one tile along K
    int kb_per_split;  // 64-deep k-blocks per unit
    int nkb;           // k-blocks of the whole contraction
    int first[GEMM_MAX_GROUP];        // first n-tile (forward) / k-block (backward) per problem
    long long ldp[GEMM_MAX_GROUP];    // row pitch (floats) of each output's split-K planes
    size_t ws_off[GEMM_MAX_GROUP];    // offset (floats) of each output's planes in the scratch
    size_t ws_bytes;   // split-K scratch: per output, splits planes of m x ldp floats (0: no split)
};

struct GemmArgs;
// A group of up to GEMM_MAX_GROUP weights with the same number of columns. Forward: shared
// activations (item[0].act), one output per item. Backward: one dY per item (item[i].act), the
// products are summed into item[0].out. m, trans_w, sm_count and the workspace come from item[0].
// narrow_ok = false keeps the 128-wide tiles out of the plan (they need every weight's scale table).
GemmPlan plan_gemm_group(long long m, const long long* n_w, int count, long long k_w, bool trans_w,
                         int sm_count, bool narrow_ok = true);
GemmPlan plan_gemm(long long m, long long n_w, long long k_w, bool trans_w, int sm_count);

struct GemmGroupArgs {
    int count;
    GemmArgs item[GEMM_MAX_GROUP];
};

// Returns cudaSuccess or the failing CUDA error; `why` receives a short reason on failure.
cudaError_t launch_gemm(const GemmArgs& a, cudaStream_t stream, const char** why);
cudaError_t launch_gemm_group(const GemmGroupArgs& a, cudaStream_t stream, const char** why);

// gate / up pair with hidden = silu(gate) * up formed in the GEMM epilogue (item[0] = gate,
// item[1] = up; their `out` may both be null when only `hidden` is wanted). The caller checks
// swiglu_fused_eligible first and otherwise runs launch_gemm_group + launch_swiglu_fwd.
struct SwigluArgs {
    __half* hidden;        // forward epilogue: the product
    const __half* gate;    // backward epilogue: saved gate / up, outputs d_gate / d_up
    const __half* up;
    __half* d_gate;
    __half* d_up;
    long long ld;          // row pitch of all of them
};
bool swiglu_fused_eligible(const GemmGroupArgs& ga);
// dX GEMM (a.trans_w) whose result is d_hidden of a SwiGLU: writes d_gate / d_up instead, from
// the saved gate / up (epi.gate, epi.up, epi.d_gate, epi.d_up: [m, k_w], pitch epi.ld).
bool swiglu_bwd_fused_eligible(const GemmArgs& a);
cudaError_t launch_bwd_dx_swiglu(const GemmArgs& a, const SwigluArgs& epi, cudaStream_t stream,
                                 const char** why);
cudaError_t launch_gate_up_swiglu(const GemmGroupArgs& ga, __half* hidden, long long ld_hidden,
                                  cudaStream_t stream, const char** why);
// Elementwise SwiGLU on contiguous fp16 arrays (swiglu.cu): hidden = silu(gate) * up, and its
// backward d_gate = d_hidden * up * sig * (1 + gate * (1 - sig)), d_up = d_hidden * gate * sig.
cudaError_t launch_swiglu_fwd(const __half* gate, const __half* up, __half* hidden, long long n,
                              int sm_count, cudaStream_t stream);
cudaError_t launch_swiglu_bwd(const __half* d_hidden, const __half* gate, const __half* up,
                              __half* d_gate, __half* d_up, long long n, int sm_count,
                              cudaStream_t stream);

// RMSNorm / add + RMSNorm on the fp32 stream (rmsnorm.cu); mode as in the reference kernel:
// 0 forward, 1 backward, 2 add then forward, 3 backward plus the sum's own gradient.
struct RmsNormArgs {
    const float* x;        // [rows, hidden]: the input (modes 0, 1, 3: the tensor that was normalised)
    const float* w;        // [hidden]
    void* y;               // modes 0, 2: output, fp32 or fp16 (y_half)
    float* rstd;           // [rows]: written by 0 / 2, read by 1 / 3
    const void* dy;        // modes 1, 3: gradient of y, same type as y
    float* dx;             // modes 1, 3
    const void* delta;     // mode 2: fp16 [rows, hidden], added to x
    float* total;          // mode 2: x + delta
    const float* d_total;  // mode 3: gradient of the sum, added to dx
    long long rows;
    int hidden;
    int mode;
    int y_half;
    float eps;
};
cudaError_t launch_rmsnorm(const RmsNormArgs& a, cudaStream_t stream);

// Rotary embedding + grouped-query expansion of the packed q / k / v projections (rope.cu).
struct RopeArgs {
    const void* q;          // forward: projections [tokens, heads*dim] / [tokens, kv_heads*dim]
    const void* k;          //          (fp16, or fp32 when proj_f32);
    const void* v;          // backward: gradients of the rotated heads (fp16, output layout)
    void* qo;               // forward: rotated heads, fp16, packed (N, H, D) or padded (B, H, T, D)
    void* ko;               // backward: gradients of the projections (their type)
    void* vo;
    const float* cos;       // [1 or B, T, dim] fp32
    const float* sin;
    const int* b_idx;       // [tokens]: sequence of each packed token
    const int* t_idx;       // [tokens]: its position
    long long tokens;
    long long cos_stride_b, cos_stride_t;  // in elements (0 for a broadcast batch dimension)
    int seq, heads, kv_heads, dim;
    int padded, backward, proj_f32;
    int lps_shift;          // set by the launcher: log2(threads per work item)
};
cudaError_t launch_qkv_rotate(const RopeArgs& a, cudaStream_t stream);

// Cross-entropy over the vocabulary (cross_entropy.cu). grad == null: statistics pass (lse and
// loss always; entropy / argmax when not null); grad != null: gradient pass.
struct CeArgs {
    const void* logits;          // [rows, vocab] fp16, or fp32 when f32
    const long long* targets;    // [rows], negative = ignored row
    float* lse;                  // [rows]: written by the statistics pass, read by the gradient pass
    float* loss;                 // [rows]
    float* entropy;              // [rows] or null
    long long* argmax;           // [rows] or null
    const float* scale;          // gradient pass: one fp32 number on the device
    void* grad;                  // gradient pass: [rows, vocab] in the logits' type (may be `logits`)
    long long rows, vocab;
    int f32;
    int vec;                     // set by the launcher
    int* status;                 // device status word (a target beyond the vocabulary is recorded there)
};
cudaError_t launch_ce(const CeArgs& a, cudaStream_t stream);

// Weight-streaming kernels for a handful of token rows (gemv.cu); launch_gemm* route eligible
// calls to them: forward for M <= 64 (a whole group in one launch), backward for M <= 16.
bool gemv_eligible(const GemmArgs& a);
bool gemv_bwd_eligible(const GemmArgs& a);
cudaError_t launch_gemv(const GemmArgs& a, cudaStream_t stream);
cudaError_t launch_gemv_group(const GemmGroupArgs& ga, cudaStream_t stream);
cudaError_t launch_gemv_bwd_group(const GemmGroupArgs& ga, cudaStream_t stream, const char** why);
// Row slabs of the streaming backward and the fp32 planes they need as scratch.
struct StreamBwdPlan {
    int rows_per_slab, slabs;
    int first[GEMM_MAX_GROUP];   // first slab of each member
    long long ldp;
    size_t ws_bytes;
};
StreamBwdPlan plan_stream_bwd(long long m, const long long* n_w, int count, long long k_w, int sm_count);
// out[m, n_out] = fp16(sum of `splits` fp32 planes [m][ldp] (+ bias)): the split-K reduction (gemm.cu).
cudaError_t launch_splitk_reduce(const float* planes, long long m, long long n_out, long long ldp,
                                 int splits, const __half* bias, __half* out, long long ld_out,
                                 int sm_count, cudaStream_t stream);

struct LoraDownArgs {
    const __half* in;
    long long m, c, ld_in;
    const __half* p;
    long long p_stride_r, p_stride_c;
    float scaling;
    __half* out;
};
cudaError_t launch_lora_down(const LoraDownArgs& a, cudaStream_t stream);

constexpr int LORA_MAX_BATCH = 8;
struct LoraDownBatch {
    LoraDownArgs item[LORA_MAX_BATCH];
    int count;
};
// One launch when the problems share row count and layout of P; separate launches otherwise.
cudaError_t launch_lora_down_batch(const LoraDownBatch& b, cudaStream_t stream);

struct LoraGradArgs {
    const __half* z;
    long long m, c, ld_z;
    const __half* s;
    float* out;
    long long o_stride_r, o_stride_c;
    int sm_count;
};
cudaError_t launch_lora_grad(const LoraGradArgs& a, cudaStream_t stream);

struct LoraGradBatch {
    LoraGradArgs item[LORA_MAX_BATCH];
    int count;
};
// One launch when every problem is on the tensor-core path; separate launches otherwise.
cudaError_t launch_lora_grad_batch(const LoraGradBatch& b, cudaStream_t stream);

// Records a message for nf4b200_last_error() on this thread and returns `code`.
int set_error(int code, const char* fmt, ...);

// Device-side status word: 0, or the first code a kernel recorded since it was last read:
//   100 + role   a bounded wait of the fused GEMM ran out (role = which wait)
//   200          cross-entropy: a target index beyond the vocabulary (row treated as ignored)
//   300          scale table: a block scale outside fp16's normal range (inf, subnormal or zero)
//   400          the self-test kernel's bounded wait ran out (what nf4b200_selftest_wait asks for)
constexpr int STATUS_CE_TARGET_RANGE = 200;
constexpr int STATUS_SCALE_RANGE = 300;
constexpr int STATUS_SELFTEST_WAIT = 400;
int* device_status_word();   // device address of the word for the current device
cudaError_t launch_selftest_wait(unsigned long long limit_ns, cudaStream_t stream);  // selftest.cu
cudaError_t read_and_clear_device_status(int* out);

}  // namespace nf4
