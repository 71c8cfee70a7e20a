// C-ABI entry points (declared in include/nf4b200.h): argument validation, device checks and
// dispatch to the kernels. No C++ exception crosses this boundary; errors come back as status
// codes plus a thread-local message.
#include <cuda_runtime.h>

#include <atomic>

#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/nf4b200.h"
#include "kernels.h"

namespace {

thread_local char g_error[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

constexpr int MAX_DEVICES = 64;

struct DeviceInfo {
    bool known = false;
    int major = 0, minor = 0, sms = 0;
    size_t smem_optin = 0;
    int* status_word = nullptr;
};
std::mutex g_mutex;
DeviceInfo g_devices[MAX_DEVICES];

__device__ int g_status_word;  // written by kernels whose bounded wait ran out

// Facts about the current device, looked up once per device.
int current_device(DeviceInfo** info) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(NF4B200_EINVAL, "device index %d", dev);
    std::lock_guard<std::mutex> lock(g_mutex);
    DeviceInfo& d = g_devices[dev];
    if (!d.known) {
        cudaDeviceProp prop;
        e = cudaGetDeviceProperties(&prop, dev);
        if (e != cudaSuccess)
            return fail(NF4B200_ECUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
        d.major = prop.major;
        d.minor = prop.minor;
        d.sms = prop.multiProcessorCount;
        d.smem_optin = prop.sharedMemPerBlockOptin;
        if (d.major == 10) {
            void* ptr = nullptr;
            e = cudaGetSymbolAddress(&ptr, g_status_word);
            if (e != cudaSuccess)
                return fail(NF4B200_ECUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            d.status_word = static_cast<int*>(ptr);
        }
        d.known = true;
    }
    *info = &d;
    return NF4B200_OK;
}

int require_sm100(DeviceInfo** info) {
    int rc = current_device(info);
    if (rc != NF4B200_OK) return rc;
    if ((*info)->major != 10)
        return fail(NF4B200_EARCH,
                    "nf4b200 kernels are built for sm_100a only; current device is sm_%d%d and "
                    "there is no fallback path",
                    (*info)->major, (*info)->minor);
    return NF4B200_OK;
}

// SMs the fused GEMM kernels may occupy (nf4b200_set_sm_limit); 0 = all of them.
std::atomic<int> g_sm_limit{0};

int gemm_sms(const DeviceInfo* d) {
    const int limit = g_sm_limit.load(std::memory_order_relaxed);
    return (limit > 0 && limit < d->sms) ? limit : d->sms;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_weight(const nf4b200_weight* w, bool for_gemm) {
    if (!w) return fail(NF4B200_EINVAL, "weight descriptor is NULL");
    if (!w->codes || !w->absmax || !w->code16)
        return fail(NF4B200_EINVAL, "weight: codes, absmax and code16 must be non-NULL");
    if (w->n_rows <= 0 || w->n_cols <= 0)
        return fail(NF4B200_EINVAL, "weight shape %lld x %lld", (long long)w->n_rows,
                    (long long)w->n_cols);
    const long long n = (long long)w->n_rows * w->n_cols;
    if (n % 8 != 0) return fail(NF4B200_EINVAL, "weight element count %lld is not a multiple of 8", n);
    if (w->blocksize <= 0 || w->blocksize % 8 != 0)
        return fail(NF4B200_EINVAL, "blocksize %d is not a positive multiple of 8", w->blocksize);
    if (n % w->blocksize != 0)
        return fail(NF4B200_EINVAL, "weight element count %lld is not a multiple of blocksize %d", n,
                    w->blocksize);
    if ((reinterpret_cast<uintptr_t>(w->codes) & 3u) != 0)
        return fail(NF4B200_EINVAL, "codes pointer is not 4-byte aligned");
    if (w->nested) {
        if (!w->code2 || !w->absmax2 || !w->offset)
            return fail(NF4B200_EINVAL, "nested weight: code2, absmax2 and offset must be non-NULL");
        if (w->nested_blocksize <= 0)
            return fail(NF4B200_EINVAL, "nested_blocksize %d", w->nested_blocksize);
    }
    if (for_gemm) {
        if (w->blocksize != 64)
            return fail(NF4B200_EINVAL, "fused GEMM needs blocksize 64, got %d", w->blocksize);
        if (w->n_cols % 64 != 0)
            return fail(NF4B200_EINVAL, "fused GEMM needs n_cols %% 64 == 0, got %lld",
                        (long long)w->n_cols);
        if (!aligned16(w->codes)) return fail(NF4B200_EINVAL, "codes pointer is not 16-byte aligned");
        if (w->n_rows > 0x7FFFFFFF || w->n_cols > 0x7FFFFFFF)
            return fail(NF4B200_EINVAL, "weight dimension exceeds 2^31");
        if (w->scales16 != nullptr) {
            if (!aligned16(w->scales16))
                return fail(NF4B200_EINVAL, "scales16 is not 16-byte aligned");
            if (w->n_rows % 8 != 0)
                return fail(NF4B200_EINVAL, "scales16 needs n_rows %% 8 == 0, got %lld",
                            (long long)w->n_rows);
        }
    }
    return NF4B200_OK;
}

int check_act(const char* name, const void* p, int64_t m, int64_t ld, int64_t cols) {
    if (!p) return fail(NF4B200_EINVAL, "%s is NULL", name);
    if (m <= 0 || m > 0x7FFFFFFF) return fail(NF4B200_EINVAL, "%s: row count %lld", name, (long long)m);
    if (ld < cols) return fail(NF4B200_EINVAL, "%s: row stride %lld < %lld columns", name,
                               (long long)ld, (long long)cols);
    if (ld % 8 != 0) return fail(NF4B200_EINVAL, "%s: row stride %lld is not a multiple of 8", name,
                                 (long long)ld);
    if (!aligned16(p)) return fail(NF4B200_EINVAL, "%s is not 16-byte aligned", name);
    return NF4B200_OK;
}

void fill_gemm(nf4::GemmArgs& g, const nf4b200_weight* w, int sms) {
    g.codes = static_cast<const uint8_t*>(w->codes);
    g.absmax = w->absmax;
    g.code2 = w->code2;
    g.absmax2 = w->absmax2;
    g.offset = w->offset;
    g.code16 = w->code16;
    g.scales16 = static_cast<const __half*>(w->scales16);
    g.dense_w = nullptr;
    g.ld_w = 0;
    g.n_w = w->n_rows;
    g.k_w = w->n_cols;
    g.nested = w->nested ? 1 : 0;
    g.nested_blocksize = w->nested ? w->nested_blocksize : 1;
    g.sm_count = sms;
}

int set_workspace(nf4::GemmArgs& g, void* workspace, size_t bytes) {
    if (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
        return fail(NF4B200_EINVAL, "workspace is not 256-byte aligned");
    g.workspace = workspace;
    g.workspace_bytes = workspace ? bytes : 0;
    return NF4B200_OK;
}

}  // namespace

namespace nf4 {

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

int* device_status_word() {
    DeviceInfo* d = nullptr;
    if (current_device(&d) != NF4B200_OK) return nullptr;
    return d->status_word;
}

cudaError_t read_and_clear_device_status(int* out) {
    int* word = device_status_word();
    if (!word) return cudaErrorInvalidDevice;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return e;
    e = cudaMemcpy(out, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    if (*out != 0) e = cudaMemset(word, 0, sizeof(int));
    return e;
}

}  // namespace nf4

extern "C" {

const char* nf4b200_last_error(void) { return g_error; }

int nf4b200_query(int device, nf4b200_props* out) {
    if (!out) return fail(NF4B200_EINVAL, "props pointer is NULL");
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "cudaGetDeviceProperties(%d): %s", device, cudaGetErrorString(e));
    out->cc_major = prop.major;
    out->cc_minor = prop.minor;
    out->sm_count = prop.multiProcessorCount;
    out->supported = prop.major == 10 ? 1 : 0;
    out->smem_per_block_optin = (int64_t)prop.sharedMemPerBlockOptin;
    return NF4B200_OK;
}

int nf4b200_device_status(int* status_out) {
    if (!status_out) return fail(NF4B200_EINVAL, "status pointer is NULL");
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    cudaError_t e = nf4::read_and_clear_device_status(status_out);
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "device status: %s", cudaGetErrorString(e));
    if (*status_out != 0) {
        const int st = *status_out;
        const char* what = st == nf4::STATUS_CE_TARGET_RANGE
                               ? "cross-entropy saw a target index beyond the vocabulary; the row was treated as ignored"
                           : st == nf4::STATUS_SCALE_RANGE
                               ? "a block scale is outside fp16's normal range; the fused GEMM cannot represent it"
                           : st == nf4::STATUS_SELFTEST_WAIT ? "the self-test kernel's bounded wait ran out"
                                                             : "a kernel gave up a bounded wait";
        return fail(NF4B200_EDEVICE, "%s (status %d)", what, st);
    }
    return NF4B200_OK;
}

int nf4b200_selftest_wait(int64_t limit_ns, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (limit_ns <= 0 || limit_ns > 1000000000ll)
        return fail(NF4B200_EINVAL, "selftest_wait: limit of %lld ns (allowed: 1 ns .. 1 s)", (long long)limit_ns);
    cudaError_t e = nf4::launch_selftest_wait((unsigned long long)limit_ns, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "selftest_wait launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_dequant(const nf4b200_weight* w, void* out, int out_dtype, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    rc = check_weight(w, false);
    if (rc != NF4B200_OK) return rc;
    if (!out) return fail(NF4B200_EINVAL, "out is NULL");
    if (out_dtype < 0 || out_dtype > 2) return fail(NF4B200_EINVAL, "out_dtype %d", out_dtype);
    if (!aligned16(out)) return fail(NF4B200_EINVAL, "out is not 16-byte aligned");
    nf4::DequantArgs a;
    a.codes = w->codes; a.absmax = w->absmax; a.code2 = w->code2; a.absmax2 = w->absmax2;
    a.offset = w->offset; a.code16 = w->code16; a.out = out;
    a.n = (long long)w->n_rows * w->n_cols;
    a.blocksize = w->blocksize;
    a.nested_blocksize = w->nested ? w->nested_blocksize : 1;
    a.nested = w->nested ? 1 : 0;
    a.out_dtype = out_dtype;
    a.sm_count = d->sms;
    cudaError_t e = nf4::launch_dequant(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "dequant launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_set_sm_limit(int sms) {
    if (sms < 0) return fail(NF4B200_EINVAL, "set_sm_limit: %d", sms);
    if (sms != 0 && sms < 2) sms = 2;
    g_sm_limit.store(sms, std::memory_order_relaxed);
    return NF4B200_OK;
}

int64_t nf4b200_scales16_bytes(int64_t n_rows, int64_t n_cols) {
    if (n_rows <= 0 || n_cols <= 0 || n_cols % 64 != 0 || n_rows % 8 != 0) return 0;
    return n_rows * (n_cols / 64) * 2;
}

int nf4b200_prepare_scales(const nf4b200_weight* w, void* scales16, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    nf4b200_weight tmp;
    if (w) { tmp = *w; tmp.scales16 = nullptr; }
    if ((rc = check_weight(w ? &tmp : nullptr, true)) != NF4B200_OK) return rc;
    if (w->n_rows % 8 != 0)
        return fail(NF4B200_EINVAL, "prepare_scales needs n_rows %% 8 == 0, got %lld",
                    (long long)w->n_rows);
    if (!scales16 || !aligned16(scales16))
        return fail(NF4B200_EINVAL, "scales16 must be a 16-byte aligned device pointer");
    cudaError_t e = nf4::launch_prepare_scales(
        w->absmax, w->code2, w->absmax2, w->offset, w->n_rows, w->n_cols / 64, w->nested ? 1 : 0,
        w->nested ? w->nested_blocksize : 1, static_cast<__half*>(scales16), d->sms,
        static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "prepare_scales launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_linear_fwd(const nf4b200_weight* w, const void* x, int64_t m, int64_t ldx,
                       const void* bias, const void* xa, const void* lora_b, void* y, int64_t ldy,
                       void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if ((rc = check_weight(w, true)) != NF4B200_OK) return rc;
    if ((rc = check_act("x", x, m, ldx, w->n_cols)) != NF4B200_OK) return rc;
    if (!y) return fail(NF4B200_EINVAL, "y is NULL");
    if (ldy < w->n_rows) return fail(NF4B200_EINVAL, "y: row stride %lld < %lld columns",
                                     (long long)ldy, (long long)w->n_rows);
    if ((xa == nullptr) != (lora_b == nullptr))
        return fail(NF4B200_EINVAL, "xa and lora_b must both be given or both be NULL");
    if (xa && (!aligned16(xa) || !aligned16(lora_b)))
        return fail(NF4B200_EINVAL, "xa / lora_b are not 16-byte aligned");
    nf4::GemmArgs g;
    fill_gemm(g, w, gemm_sms(d));
    g.act = static_cast<const __half*>(x); g.m = m; g.ld_act = ldx;
    g.out = static_cast<__half*>(y); g.ld_out = ldy;
    g.bias = static_cast<const __half*>(bias);
    g.ext_a = static_cast<const __half*>(xa);
    g.ext_b = static_cast<const __half*>(lora_b);
    g.trans_w = false;
    if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    const char* why = "";
    cudaError_t e = nf4::launch_gemm(g, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "linear_fwd: %s: %s", why, cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_fp16_linear(const void* weight, int64_t n_rows, int64_t n_cols, int64_t ldw,
                        const void* x, int64_t m, int64_t ldx, int transposed, const void* bias,
                        void* y, int64_t ldy, void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (!weight || !aligned16(weight)) return fail(NF4B200_EINVAL, "fp16_linear: weight is NULL or not 16-byte aligned");
    if (n_rows <= 0 || n_cols <= 0 || n_rows > 0x7FFFFFFF || n_cols > 0x7FFFFFFF)
        return fail(NF4B200_EINVAL, "fp16_linear: weight shape %lld x %lld", (long long)n_rows, (long long)n_cols);
    if (ldw < n_cols || ldw % 8 != 0)
        return fail(NF4B200_EINVAL, "fp16_linear: weight row stride %lld (needs >= %lld columns, multiple of 8)",
                    (long long)ldw, (long long)n_cols);
    if (n_cols % 8 != 0 || n_rows % 8 != 0)
        return fail(NF4B200_EINVAL, "fp16_linear: weight dimensions must be multiples of 8");
    const int64_t in_cols = transposed ? n_rows : n_cols, out_cols = transposed ? n_cols : n_rows;
    if ((rc = check_act("x", x, m, ldx, in_cols)) != NF4B200_OK) return rc;
    if (!y) return fail(NF4B200_EINVAL, "y is NULL");
    if (ldy < out_cols) return fail(NF4B200_EINVAL, "y: row stride %lld < %lld columns", (long long)ldy,
                                    (long long)out_cols);
    if (transposed && bias) return fail(NF4B200_EINVAL, "fp16_linear: bias only with transposed = 0");
    nf4::GemmArgs g = {};
    g.dense_w = static_cast<const __half*>(weight);
    g.ld_w = ldw;
    g.n_w = n_rows; g.k_w = n_cols;
    g.nested_blocksize = 1;
    g.sm_count = gemm_sms(d);
    g.act = static_cast<const __half*>(x); g.m = m; g.ld_act = ldx;
    g.out = static_cast<__half*>(y); g.ld_out = ldy;
    g.bias = static_cast<const __half*>(bias);
    g.trans_w = transposed != 0;
    if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    const char* why = "";
    cudaError_t e = nf4::launch_gemm(g, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "fp16_linear: %s: %s", why, cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_linear_bwd_dx(const nf4b200_weight* w, const void* dy, int64_t m, int64_t lddy,
                          const void* u, const void* lora_a, void* dx, int64_t lddx,
                          void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if ((rc = check_weight(w, true)) != NF4B200_OK) return rc;
    if ((rc = check_act("dy", dy, m, lddy, w->n_rows)) != NF4B200_OK) return rc;
    if (!dx) return fail(NF4B200_EINVAL, "dx is NULL");
    if (lddx < w->n_cols) return fail(NF4B200_EINVAL, "dx: row stride %lld < %lld columns",
                                      (long long)lddx, (long long)w->n_cols);
    if ((u == nullptr) != (lora_a == nullptr))
        return fail(NF4B200_EINVAL, "u and lora_a must both be given or both be NULL");
    if (u && (!aligned16(u) || !aligned16(lora_a)))
        return fail(NF4B200_EINVAL, "u / lora_a are not 16-byte aligned");
    nf4::GemmArgs g;
    fill_gemm(g, w, gemm_sms(d));
    g.act = static_cast<const __half*>(dy); g.m = m; g.ld_act = lddy;
    g.out = static_cast<__half*>(dx); g.ld_out = lddx;
    g.bias = nullptr;
    g.ext_a = static_cast<const __half*>(u);
    g.ext_b = static_cast<const __half*>(lora_a);
    g.trans_w = true;
    if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    const char* why = "";
    cudaError_t e = nf4::launch_gemm(g, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "linear_bwd_dx: %s: %s", why, cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_linear_fwd_group(int count, const nf4b200_weight* const* w, const void* x, int64_t m,
                             int64_t ldx, const void* const* bias, const void* const* xa,
                             const void* const* lora_b, void* const* y, const int64_t* ldy,
                             void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::GEMM_MAX_GROUP)
        return fail(NF4B200_EINVAL, "group of %d weights (1..%d allowed)", count, nf4::GEMM_MAX_GROUP);
    if (!w || !y || !ldy) return fail(NF4B200_EINVAL, "fwd_group: NULL array");
    nf4::GemmGroupArgs ga;
    ga.count = count;
    for (int i = 0; i < count; ++i) {
        if ((rc = check_weight(w[i], true)) != NF4B200_OK) return rc;
        if (w[i]->n_cols != w[0]->n_cols)
            return fail(NF4B200_EINVAL, "fwd_group: weights must have the same number of columns");
        if (!y[i]) return fail(NF4B200_EINVAL, "fwd_group: y[%d] is NULL", i);
        if (ldy[i] < w[i]->n_rows)
            return fail(NF4B200_EINVAL, "fwd_group: y[%d] row stride %lld < %lld columns", i,
                        (long long)ldy[i], (long long)w[i]->n_rows);
        const void* xa_i = xa ? xa[i] : nullptr;
        const void* lb_i = lora_b ? lora_b[i] : nullptr;
        if ((xa_i == nullptr) != (lb_i == nullptr))
            return fail(NF4B200_EINVAL, "fwd_group: xa[%d] and lora_b[%d] must both be given or NULL", i, i);
        if (xa_i && (!aligned16(xa_i) || !aligned16(lb_i)))
            return fail(NF4B200_EINVAL, "fwd_group: xa / lora_b are not 16-byte aligned");
        nf4::GemmArgs& g = ga.item[i];
        fill_gemm(g, w[i], gemm_sms(d));
        g.act = static_cast<const __half*>(x); g.m = m; g.ld_act = ldx;
        g.out = static_cast<__half*>(y[i]); g.ld_out = ldy[i];
        g.bias = static_cast<const __half*>(bias ? bias[i] : nullptr);
        g.ext_a = static_cast<const __half*>(xa_i);
        g.ext_b = static_cast<const __half*>(lb_i);
        g.trans_w = false;
        if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    }
    if ((rc = check_act("x", x, m, ldx, w[0]->n_cols)) != NF4B200_OK) return rc;
    const char* why = "";
    cudaError_t e = nf4::launch_gemm_group(ga, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "linear_fwd_group: %s: %s", why, cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_linear_bwd_dx_group(int count, const nf4b200_weight* const* w, const void* const* dy,
                                int64_t m, const int64_t* lddy, const void* const* u,
                                const void* const* lora_a, void* dx, int64_t lddx, void* workspace,
                                size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::GEMM_MAX_GROUP)
        return fail(NF4B200_EINVAL, "group of %d weights (1..%d allowed)", count, nf4::GEMM_MAX_GROUP);
    if (!w || !dy || !lddy || !dx) return fail(NF4B200_EINVAL, "bwd_group: NULL argument");
    nf4::GemmGroupArgs ga;
    ga.count = count;
    for (int i = 0; i < count; ++i) {
        if ((rc = check_weight(w[i], true)) != NF4B200_OK) return rc;
        if (w[i]->n_cols != w[0]->n_cols)
            return fail(NF4B200_EINVAL, "bwd_group: weights must have the same number of columns");
        if ((rc = check_act("dy", dy[i], m, lddy[i], w[i]->n_rows)) != NF4B200_OK) return rc;
        const void* u_i = u ? u[i] : nullptr;
        const void* la_i = lora_a ? lora_a[i] : nullptr;
        if ((u_i == nullptr) != (la_i == nullptr))
            return fail(NF4B200_EINVAL, "bwd_group: u[%d] and lora_a[%d] must both be given or NULL", i, i);
        if (u_i && (!aligned16(u_i) || !aligned16(la_i)))
            return fail(NF4B200_EINVAL, "bwd_group: u / lora_a are not 16-byte aligned");
        nf4::GemmArgs& g = ga.item[i];
        fill_gemm(g, w[i], gemm_sms(d));
        g.act = static_cast<const __half*>(dy[i]); g.m = m; g.ld_act = lddy[i];
        g.out = static_cast<__half*>(dx); g.ld_out = lddx;
        g.bias = nullptr;
        g.ext_a = static_cast<const __half*>(u_i);
        g.ext_b = static_cast<const __half*>(la_i);
        g.trans_w = true;
        if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    }
    if (lddx < w[0]->n_cols)
        return fail(NF4B200_EINVAL, "bwd_group: dx row stride %lld < %lld columns", (long long)lddx,
                    (long long)w[0]->n_cols);
    const char* why = "";
    cudaError_t e = nf4::launch_gemm_group(ga, static_cast<cudaStream_t>(stream), &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "linear_bwd_dx_group: %s: %s", why, cudaGetErrorString(e));
    return NF4B200_OK;
}

int64_t nf4b200_workspace_bytes_group(int count, const int64_t* n_rows, int64_t n_cols, int64_t m,
                                      int backward) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::GEMM_MAX_GROUP || !n_rows || n_cols <= 0 || m <= 0)
        return fail(NF4B200_EINVAL, "workspace_bytes_group: bad arguments");
    long long rows[nf4::GEMM_MAX_GROUP];
    for (int i = 0; i < count; ++i) {
        if (n_rows[i] <= 0) return fail(NF4B200_EINVAL, "workspace_bytes_group: bad shape");
        rows[i] = n_rows[i];
    }
    const nf4::GemmPlan pl = nf4::plan_gemm_group(m, rows, count, n_cols, backward != 0, gemm_sms(d));
    return (int64_t)pl.ws_bytes;
}

int nf4b200_launches_group(int count, const int64_t* n_rows, int64_t n_cols, int64_t m, int backward,
                           int with_scale_tables) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::GEMM_MAX_GROUP || !n_rows || n_cols <= 0 || m <= 0)
        return fail(NF4B200_EINVAL, "launches_group: bad arguments");
    long long rows[nf4::GEMM_MAX_GROUP];
    for (int i = 0; i < count; ++i) {
        if (n_rows[i] <= 0) return fail(NF4B200_EINVAL, "launches_group: bad shape");
        rows[i] = n_rows[i];
    }
    const nf4::GemmPlan pl = nf4::plan_gemm_group(m, rows, count, n_cols, backward != 0, gemm_sms(d),
                                                  with_scale_tables != 0);
    // one GEMM; with K-slices, one reduction per output (forward: per weight; backward: one dX)
    return 1 + (pl.splits > 1 ? (backward ? 1 : count) : 0);
}

// Bytes of one temporary [m, n_rows] fp16 array, rounded so that the next one stays aligned.
static size_t swiglu_tmp_bytes(int64_t m, int64_t n_rows) {
    return ((size_t)m * (size_t)n_rows * 2 + 255) / 256 * 256;
}

int64_t nf4b200_gate_up_swiglu_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m, int keep) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (n_rows <= 0 || n_cols <= 0 || m <= 0)
        return fail(NF4B200_EINVAL, "gate_up_swiglu_workspace_bytes: bad shape");
    if (m > 256) return 0;  // epilogue-fused kernel: no scratch
    long long rows[2] = {n_rows, n_rows};
    const nf4::GemmPlan pl = nf4::plan_gemm_group(m, rows, 2, n_cols, false, gemm_sms(d));
    const size_t gemm_ws = (pl.ws_bytes + 255) / 256 * 256;
    return (int64_t)(gemm_ws + (keep ? 0 : 2 * swiglu_tmp_bytes(m, n_rows)));
}

int nf4b200_gate_up_swiglu_fwd(const nf4b200_weight* gate_w, const nf4b200_weight* up_w,
                               const void* x, int64_t m, int64_t ldx, void* gate_out, void* up_out,
                               void* hidden, void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if ((rc = check_weight(gate_w, true)) != NF4B200_OK) return rc;
    if ((rc = check_weight(up_w, true)) != NF4B200_OK) return rc;
    if (gate_w->n_rows != up_w->n_rows || gate_w->n_cols != up_w->n_cols)
        return fail(NF4B200_EINVAL, "gate_up_swiglu: gate and up weights differ in shape");
    if ((gate_out == nullptr) != (up_out == nullptr))
        return fail(NF4B200_EINVAL, "gate_up_swiglu: gate_out and up_out must both be given or NULL");
    const int64_t n = gate_w->n_rows;
    if (n % 8 != 0) return fail(NF4B200_EINVAL, "gate_up_swiglu: %lld output columns (multiple of 8 needed)", (long long)n);
    if (!hidden || !aligned16(hidden) || (gate_out && (!aligned16(gate_out) || !aligned16(up_out))))
        return fail(NF4B200_EINVAL, "gate_up_swiglu: outputs must be 16-byte aligned and hidden not NULL");
    if ((rc = check_act("x", x, m, ldx, gate_w->n_cols)) != NF4B200_OK) return rc;
    nf4::GemmGroupArgs ga;
    ga.count = 2;
    const nf4b200_weight* ws[2] = {gate_w, up_w};
    void* outs[2] = {gate_out, up_out};
    for (int i = 0; i < 2; ++i) {
        nf4::GemmArgs& g = ga.item[i];
        fill_gemm(g, ws[i], gemm_sms(d));
        g.act = static_cast<const __half*>(x); g.m = m; g.ld_act = ldx;
        g.out = static_cast<__half*>(outs[i]); g.ld_out = n;
        g.bias = nullptr; g.ext_a = nullptr; g.ext_b = nullptr;
        g.trans_w = false;
        if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const char* why = "";
    if (nf4::swiglu_fused_eligible(ga)) {
        cudaError_t e = nf4::launch_gate_up_swiglu(ga, static_cast<__half*>(hidden), n, st, &why);
        if (e != cudaSuccess)
            return fail(NF4B200_ECUDA, "gate_up_swiglu: %s: %s", why, cudaGetErrorString(e));
        return NF4B200_OK;
    }
    // few token rows: grouped GEMM, then the elementwise kernel; without gate_out / up_out the two
    // arrays live at the end of the scratch
    if (!gate_out) {
        const size_t tmp = swiglu_tmp_bytes(m, n);
        if (!workspace || workspace_bytes < 2 * tmp)
            return fail(NF4B200_EINVAL, "gate_up_swiglu: workspace too small for the two temporaries "
                                        "(nf4b200_gate_up_swiglu_workspace_bytes)");
        uint8_t* base = static_cast<uint8_t*>(workspace) + (workspace_bytes - 2 * tmp) / 256 * 256;
        for (int i = 0; i < 2; ++i) {
            ga.item[i].out = reinterpret_cast<__half*>(base + i * tmp);
            ga.item[i].workspace_bytes = (size_t)(base - static_cast<uint8_t*>(workspace));
        }
    }
    cudaError_t e = nf4::launch_gemm_group(ga, st, &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "gate_up_swiglu: %s: %s", why, cudaGetErrorString(e));
    e = nf4::launch_swiglu_fwd(ga.item[0].out, ga.item[1].out, static_cast<__half*>(hidden), m * n,
                               gemm_sms(d), st);
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "swiglu_fwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int64_t nf4b200_linear_bwd_dx_swiglu_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (n_rows <= 0 || n_cols <= 0 || m <= 0)
        return fail(NF4B200_EINVAL, "linear_bwd_dx_swiglu_workspace_bytes: bad shape");
    const nf4::GemmPlan pl = nf4::plan_gemm(m, n_rows, n_cols, true, gemm_sms(d));
    if (pl.cg == 2 && pl.nacc == 2 && pl.splits == 1 && pl.bn == 256 && n_cols % 8 == 0) return 0;
    return (int64_t)((pl.ws_bytes + 255) / 256 * 256 + swiglu_tmp_bytes(m, n_cols));
}

int nf4b200_linear_bwd_dx_swiglu(const nf4b200_weight* w, const void* dy, int64_t m, int64_t lddy,
                                 const void* gate, const void* up, void* d_gate, void* d_up,
                                 void* workspace, size_t workspace_bytes, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if ((rc = check_weight(w, true)) != NF4B200_OK) return rc;
    if ((rc = check_act("dy", dy, m, lddy, w->n_rows)) != NF4B200_OK) return rc;
    if (!gate || !up || !d_gate || !d_up)
        return fail(NF4B200_EINVAL, "linear_bwd_dx_swiglu: NULL argument");
    if (!aligned16(gate) || !aligned16(up) || !aligned16(d_gate) || !aligned16(d_up))
        return fail(NF4B200_EINVAL, "linear_bwd_dx_swiglu: gate / up / d_gate / d_up must be 16-byte aligned");
    const int64_t k = w->n_cols;
    if (k % 8 != 0)
        return fail(NF4B200_EINVAL, "linear_bwd_dx_swiglu: %lld columns (multiple of 8 needed)", (long long)k);
    nf4::GemmArgs g;
    fill_gemm(g, w, gemm_sms(d));
    g.act = static_cast<const __half*>(dy); g.m = m; g.ld_act = lddy;
    g.out = nullptr; g.ld_out = k;
    g.bias = nullptr; g.ext_a = nullptr; g.ext_b = nullptr;
    g.trans_w = true;
    if ((rc = set_workspace(g, workspace, workspace_bytes)) != NF4B200_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const char* why = "";
    if (nf4::swiglu_bwd_fused_eligible(g)) {
        nf4::SwigluArgs epi = {};
        epi.gate = static_cast<const __half*>(gate); epi.up = static_cast<const __half*>(up);
        epi.d_gate = static_cast<__half*>(d_gate); epi.d_up = static_cast<__half*>(d_up);
        epi.ld = k;
        cudaError_t e = nf4::launch_bwd_dx_swiglu(g, epi, st, &why);
        if (e != cudaSuccess)
            return fail(NF4B200_ECUDA, "linear_bwd_dx_swiglu: %s: %s", why, cudaGetErrorString(e));
        return NF4B200_OK;
    }
    // other plans (few rows, K-slices): d_hidden into the end of the scratch, then the
    // elementwise kernel
    const size_t tmp = swiglu_tmp_bytes(m, k);
    if (!workspace || workspace_bytes < tmp)
        return fail(NF4B200_EINVAL, "linear_bwd_dx_swiglu: workspace too small "
                                    "(nf4b200_linear_bwd_dx_swiglu_workspace_bytes)");
    uint8_t* base = static_cast<uint8_t*>(workspace) + (workspace_bytes - tmp) / 256 * 256;
    g.out = reinterpret_cast<__half*>(base);
    g.workspace_bytes = (size_t)(base - static_cast<uint8_t*>(workspace));
    cudaError_t e = nf4::launch_gemm(g, st, &why);
    if (e != cudaSuccess)
        return fail(NF4B200_ECUDA, "linear_bwd_dx_swiglu: %s: %s", why, cudaGetErrorString(e));
    e = nf4::launch_swiglu_bwd(g.out, static_cast<const __half*>(gate), static_cast<const __half*>(up),
                               static_cast<__half*>(d_gate), static_cast<__half*>(d_up), m * k,
                               gemm_sms(d), st);
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "swiglu_bwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_rmsnorm_fwd(const void* x, const void* delta, const void* weight, void* total, void* y,
                        int y_dtype, void* rstd, int64_t rows, int64_t hidden, float eps,
                        void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (rows < 0 || hidden <= 0 || hidden > 0x7FFFFFFF)
        return fail(NF4B200_EINVAL, "rmsnorm_fwd: bad shape %lld x %lld", (long long)rows, (long long)hidden);
    if (rows > 0 && (!x || !weight || !y || !rstd))
        return fail(NF4B200_EINVAL, "rmsnorm_fwd: NULL argument");
    if ((delta == nullptr) != (total == nullptr))
        return fail(NF4B200_EINVAL, "rmsnorm_fwd: delta and total must both be given or both be NULL");
    if (y_dtype != NF4B200_F16 && y_dtype != NF4B200_F32)
        return fail(NF4B200_EINVAL, "rmsnorm_fwd: y must be fp16 or fp32");
    nf4::RmsNormArgs a = {};
    a.x = static_cast<const float*>(x); a.w = static_cast<const float*>(weight);
    a.y = y; a.rstd = static_cast<float*>(rstd);
    a.delta = delta; a.total = static_cast<float*>(total);
    a.rows = rows; a.hidden = (int)hidden; a.mode = delta ? 2 : 0;
    a.y_half = y_dtype == NF4B200_F16 ? 1 : 0; a.eps = eps;
    cudaError_t e = nf4::launch_rmsnorm(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "rmsnorm_fwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_rmsnorm_bwd(const void* x, const void* weight, const void* rstd, const void* dy,
                        int dy_dtype, const void* d_total, void* dx, int64_t rows, int64_t hidden,
                        void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (rows < 0 || hidden <= 0 || hidden > 0x7FFFFFFF)
        return fail(NF4B200_EINVAL, "rmsnorm_bwd: bad shape %lld x %lld", (long long)rows, (long long)hidden);
    if (rows > 0 && (!x || !weight || !rstd || !dy || !dx))
        return fail(NF4B200_EINVAL, "rmsnorm_bwd: NULL argument");
    if (dy_dtype != NF4B200_F16 && dy_dtype != NF4B200_F32)
        return fail(NF4B200_EINVAL, "rmsnorm_bwd: dy must be fp16 or fp32");
    nf4::RmsNormArgs a = {};
    a.x = static_cast<const float*>(x); a.w = static_cast<const float*>(weight);
    a.rstd = const_cast<float*>(static_cast<const float*>(rstd));
    a.dy = dy; a.dx = static_cast<float*>(dx); a.d_total = static_cast<const float*>(d_total);
    a.rows = rows; a.hidden = (int)hidden; a.mode = d_total ? 3 : 1;
    a.y_half = dy_dtype == NF4B200_F16 ? 1 : 0; a.eps = 0.f;
    cudaError_t e = nf4::launch_rmsnorm(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "rmsnorm_bwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_qkv_rotate(const void* q, const void* k, const void* v, void* q_out, void* k_out,
                       void* v_out, const void* cos, const void* sin, int64_t cos_stride_b,
                       int64_t cos_stride_t, const void* b_idx, const void* t_idx, int64_t tokens,
                       int64_t seq, int heads, int kv_heads, int dim, int padded, int backward,
                       int proj_dtype, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (tokens < 0 || seq <= 0 || seq > 0x7FFFFFFF || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0)
        return fail(NF4B200_EINVAL, "qkv_rotate: bad shape (tokens %lld, seq %lld, heads %d, kv heads %d)",
                    (long long)tokens, (long long)seq, heads, kv_heads);
    if (dim != 64 && dim != 128 && dim != 256)
        return fail(NF4B200_EINVAL, "qkv_rotate: head size %d (64, 128 or 256)", dim);
    if (proj_dtype != NF4B200_F16 && proj_dtype != NF4B200_F32)
        return fail(NF4B200_EINVAL, "qkv_rotate: projections must be fp16 or fp32");
    if (tokens > 0 && (!q || !k || !v || !q_out || !k_out || !v_out || !cos || !sin || !b_idx || !t_idx))
        return fail(NF4B200_EINVAL, "qkv_rotate: NULL argument");
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(q_out) || !aligned16(k_out) ||
        !aligned16(v_out) || !aligned16(cos) || !aligned16(sin))
        return fail(NF4B200_EINVAL, "qkv_rotate: arrays must be 16-byte aligned");
    if (cos_stride_b % 4 != 0 || cos_stride_t % 4 != 0 || cos_stride_t < dim)
        return fail(NF4B200_EINVAL, "qkv_rotate: cos / sin strides %lld, %lld", (long long)cos_stride_b,
                    (long long)cos_stride_t);
    nf4::RopeArgs a = {};
    a.q = q; a.k = k; a.v = v; a.qo = q_out; a.ko = k_out; a.vo = v_out;
    a.cos = static_cast<const float*>(cos); a.sin = static_cast<const float*>(sin);
    a.b_idx = static_cast<const int*>(b_idx); a.t_idx = static_cast<const int*>(t_idx);
    a.tokens = tokens; a.cos_stride_b = cos_stride_b; a.cos_stride_t = cos_stride_t;
    a.seq = (int)seq; a.heads = heads; a.kv_heads = kv_heads; a.dim = dim;
    a.padded = padded ? 1 : 0; a.backward = backward ? 1 : 0;
    a.proj_f32 = proj_dtype == NF4B200_F32 ? 1 : 0;
    cudaError_t e = nf4::launch_qkv_rotate(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "qkv_rotate: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_ce_stats(const void* logits, int logits_dtype, const void* targets, void* lse, void* loss,
                     void* entropy, void* argmax, int64_t rows, int64_t vocab, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (rows < 0 || vocab <= 0 || vocab > 0x7FFFFFFF)
        return fail(NF4B200_EINVAL, "ce_stats: bad shape %lld x %lld", (long long)rows, (long long)vocab);
    if (logits_dtype != NF4B200_F16 && logits_dtype != NF4B200_F32)
        return fail(NF4B200_EINVAL, "ce_stats: logits must be fp16 or fp32");
    if (rows > 0 && (!logits || !targets || !lse || !loss))
        return fail(NF4B200_EINVAL, "ce_stats: NULL argument");
    nf4::CeArgs a = {};
    a.logits = logits; a.targets = static_cast<const long long*>(targets);
    a.lse = static_cast<float*>(lse); a.loss = static_cast<float*>(loss);
    a.entropy = static_cast<float*>(entropy); a.argmax = static_cast<long long*>(argmax);
    a.rows = rows; a.vocab = vocab; a.f32 = logits_dtype == NF4B200_F32 ? 1 : 0;
    a.status = nf4::device_status_word();
    cudaError_t e = nf4::launch_ce(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "ce_stats: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_ce_grad(const void* logits, int logits_dtype, const void* targets, const void* lse,
                    const void* scale, void* grad, int64_t rows, int64_t vocab, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (rows < 0 || vocab <= 0 || vocab > 0x7FFFFFFF)
        return fail(NF4B200_EINVAL, "ce_grad: bad shape %lld x %lld", (long long)rows, (long long)vocab);
    if (logits_dtype != NF4B200_F16 && logits_dtype != NF4B200_F32)
        return fail(NF4B200_EINVAL, "ce_grad: logits must be fp16 or fp32");
    if (rows > 0 && (!logits || !targets || !lse || !scale || !grad))
        return fail(NF4B200_EINVAL, "ce_grad: NULL argument");
    nf4::CeArgs a = {};
    a.logits = logits; a.targets = static_cast<const long long*>(targets);
    a.lse = const_cast<float*>(static_cast<const float*>(lse));
    a.scale = static_cast<const float*>(scale); a.grad = grad;
    a.rows = rows; a.vocab = vocab; a.f32 = logits_dtype == NF4B200_F32 ? 1 : 0;
    a.status = nf4::device_status_word();
    cudaError_t e = nf4::launch_ce(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "ce_grad: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_swiglu_fwd(const void* gate, const void* up, void* hidden, int64_t n, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (n < 0 || (n > 0 && (!gate || !up || !hidden)))
        return fail(NF4B200_EINVAL, "swiglu_fwd: NULL argument or negative size");
    cudaError_t e = nf4::launch_swiglu_fwd(static_cast<const __half*>(gate), static_cast<const __half*>(up),
                                           static_cast<__half*>(hidden), n, d->sms,
                                           static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "swiglu_fwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_swiglu_bwd(const void* d_hidden, const void* gate, const void* up, void* d_gate,
                       void* d_up, int64_t n, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (n < 0 || (n > 0 && (!d_hidden || !gate || !up || !d_gate || !d_up)))
        return fail(NF4B200_EINVAL, "swiglu_bwd: NULL argument or negative size");
    cudaError_t e = nf4::launch_swiglu_bwd(
        static_cast<const __half*>(d_hidden), static_cast<const __half*>(gate),
        static_cast<const __half*>(up), static_cast<__half*>(d_gate), static_cast<__half*>(d_up), n,
        d->sms, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "swiglu_bwd: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int64_t nf4b200_workspace_bytes(int64_t n_rows, int64_t n_cols, int64_t m, int backward) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (n_rows <= 0 || n_cols <= 0 || m <= 0)
        return fail(NF4B200_EINVAL, "workspace_bytes: bad shape");
    const nf4::GemmPlan pl = nf4::plan_gemm(m, n_rows, n_cols, backward != 0, gemm_sms(d));
    return (int64_t)pl.ws_bytes;
}

int nf4b200_lora_down(const void* in, int64_t m, int64_t c, int64_t ld_in, const void* p,
                      int64_t p_stride_r, int64_t p_stride_c, float scaling, void* out,
                      void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (!in || !p || !out) return fail(NF4B200_EINVAL, "lora_down: NULL pointer");
    if (m <= 0 || c <= 0 || ld_in < c) return fail(NF4B200_EINVAL, "lora_down: bad shape");
    if ((reinterpret_cast<uintptr_t>(out) & 3u) != 0)
        return fail(NF4B200_EINVAL, "lora_down: out is not 4-byte aligned");
    nf4::LoraDownArgs a{static_cast<const __half*>(in), m, c, ld_in, static_cast<const __half*>(p),
                        p_stride_r, p_stride_c, scaling, static_cast<__half*>(out)};
    cudaError_t e = nf4::launch_lora_down(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "lora_down launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_lora_grad(const void* z, int64_t m, int64_t c, int64_t ld_z, const void* s, float* out,
                      int64_t o_stride_r, int64_t o_stride_c, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (!z || !s || !out) return fail(NF4B200_EINVAL, "lora_grad: NULL pointer");
    if (m <= 0 || c <= 0 || ld_z < c) return fail(NF4B200_EINVAL, "lora_grad: bad shape");
    nf4::LoraGradArgs a{static_cast<const __half*>(z), m, c, ld_z, static_cast<const __half*>(s),
                        out, o_stride_r, o_stride_c, d->sms};
    cudaError_t e = nf4::launch_lora_grad(a, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "lora_grad launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_lora_down_batch(int count, const void* const* in, int64_t m, const int64_t* c,
                            const int64_t* ld_in, const void* const* p, const int64_t* p_stride_r,
                            const int64_t* p_stride_c, const float* scaling, void* const* out,
                            void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::LORA_MAX_BATCH)
        return fail(NF4B200_EINVAL, "lora_down_batch: count %d not in 1..%d", count, nf4::LORA_MAX_BATCH);
    if (!in || !c || !ld_in || !p || !p_stride_r || !p_stride_c || !scaling || !out)
        return fail(NF4B200_EINVAL, "lora_down_batch: NULL array");
    nf4::LoraDownBatch b;
    b.count = count;
    for (int i = 0; i < count; ++i) {
        if (!in[i] || !p[i] || !out[i]) return fail(NF4B200_EINVAL, "lora_down_batch: NULL pointer");
        if (m <= 0 || c[i] <= 0 || ld_in[i] < c[i])
            return fail(NF4B200_EINVAL, "lora_down_batch: bad shape in problem %d", i);
        if ((reinterpret_cast<uintptr_t>(out[i]) & 3u) != 0)
            return fail(NF4B200_EINVAL, "lora_down_batch: out is not 4-byte aligned");
        b.item[i] = nf4::LoraDownArgs{static_cast<const __half*>(in[i]), m, c[i], ld_in[i],
                                      static_cast<const __half*>(p[i]), p_stride_r[i],
                                      p_stride_c[i], scaling[i], static_cast<__half*>(out[i])};
    }
    for (int i = count; i < nf4::LORA_MAX_BATCH; ++i) b.item[i] = b.item[0];
    cudaError_t e = nf4::launch_lora_down_batch(b, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "lora_down_batch launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

int nf4b200_lora_grad_batch(int count, const void* const* z, const int64_t* m, const int64_t* c,
                            const int64_t* ld_z, const void* const* s, float* const* out,
                            const int64_t* o_stride_r, const int64_t* o_stride_c, void* stream) {
    DeviceInfo* d = nullptr;
    int rc = require_sm100(&d);
    if (rc != NF4B200_OK) return rc;
    if (count < 1 || count > nf4::LORA_MAX_BATCH)
        return fail(NF4B200_EINVAL, "lora_grad_batch: count %d not in 1..%d", count, nf4::LORA_MAX_BATCH);
    if (!z || !m || !c || !ld_z || !s || !out || !o_stride_r || !o_stride_c)
        return fail(NF4B200_EINVAL, "lora_grad_batch: NULL array");
    nf4::LoraGradBatch b;
    b.count = count;
    for (int i = 0; i < count; ++i) {
        if (!z[i] || !s[i] || !out[i]) return fail(NF4B200_EINVAL, "lora_grad_batch: NULL pointer");
        if (m[i] <= 0 || c[i] <= 0 || ld_z[i] < c[i])
            return fail(NF4B200_EINVAL, "lora_grad_batch: bad shape in problem %d", i);
        b.item[i] = nf4::LoraGradArgs{static_cast<const __half*>(z[i]), m[i], c[i], ld_z[i],
                                      static_cast<const __half*>(s[i]), out[i], o_stride_r[i],
                                      o_stride_c[i], d->sms};
    }
    for (int i = count; i < nf4::LORA_MAX_BATCH; ++i) b.item[i] = b.item[0];
    cudaError_t e = nf4::launch_lora_grad_batch(b, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(NF4B200_ECUDA, "lora_grad_batch launch: %s", cudaGetErrorString(e));
    return NF4B200_OK;
}

}  // extern "C"
