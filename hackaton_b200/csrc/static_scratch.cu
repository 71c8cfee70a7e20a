// Forward NF4 linear for callers that cannot hand the library any scratch memory.
//
// Some hosts of this library own no allocator on the device side: an inference server whose memory
// pool is fully carved up at start-up, a plug-in running inside someone else's stream-ordered
// region, code that runs after the process has hit its memory budget. For them the split-K scratch
// of nf4b200_linear_fwd lives in a fixed array that is part of the library image: every GPU that
// loads the library carries NF4B200_STATIC_SCRATCH_BYTES of it until the process exits.
//
// The array is shared by every call on the device and keeps whatever the previous call left in
// it. Nothing in it has to start at zero: a call writes every partial sum before its reduction
// kernel reads it. Two calls that overlap on the GPU (different streams, or a replayed graph next
// to a live call) would write the same bytes: that is a race the caller must rule out.
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/nf4b200.h"
#include "kernels.h"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[NF4B200_STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mutex;
void* g_scratch_ptr[MAX_DEVICES] = {};  // device address of the array, per device

// In host code `g_static_scratch` is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
cudaError_t scratch_for_current_device(void** out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int nf4b200_linear_fwd_static(const nf4b200_weight* w, const void* x, int64_t m,
                                         int64_t ldx, const void* bias, const void* xa,
                                         const void* lora_b, void* y, int64_t ldy, void* stream) {
    if (!w) return nf4::set_error(NF4B200_EINVAL, "weight descriptor is NULL");
    const int64_t need = nf4b200_workspace_bytes(w->n_rows, w->n_cols, m, 0);
    if (need < 0) return (int)need;  // message already set
    if (need > (int64_t)NF4B200_STATIC_SCRATCH_BYTES)
        return nf4::set_error(NF4B200_EINVAL,
                              "nf4b200_linear_fwd_static: this shape needs %lld bytes of scratch, the "
                              "built-in array holds %lld; use nf4b200_linear_fwd with a workspace",
                              (long long)need, (long long)NF4B200_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (need > 0) {
        const cudaError_t e = scratch_for_current_device(&scratch);
        if (e != cudaSuccess)
            return nf4::set_error(NF4B200_ECUDA, "cudaGetSymbolAddress(static scratch): %s",
                                  cudaGetErrorString(e));
    }
    return nf4b200_linear_fwd(w, x, m, ldx, bias, xa, lora_b, y, ldy, scratch,
                              scratch ? (size_t)NF4B200_STATIC_SCRATCH_BYTES : 0, stream);
}
