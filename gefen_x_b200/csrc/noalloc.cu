// Allocation-free gradient-norm / clip-coefficient entry point (see noalloc.h).
//
// Same two kernels as the regular path (per-CTA sums of squares, then one CTA that
// adds them in fp64 and writes the coefficient); only the home of the partial sums
// differs: a file-scope device array instead of a caller-allocated tensor.
#include "noalloc.h"

#include <stdint.h>
#include <stdio.h>

#include "update.h"

namespace {

constexpr int kMaxPartials = 65536;
constexpr long long kElemsPerPartial = 16384;
constexpr int kMaxDevices = 64;

// Scratch shared by every call on this device.  In host code this name is only a
// handle for cudaGetSymbolAddress; kernels receive the resolved device address.
static __device__ __align__(256) float g_noalloc_partials[kMaxPartials];

float* g_partials_by_device[kMaxDevices] = {nullptr};
thread_local char g_last_error[256] = "";

int fail(int code, const char* msg) {
    snprintf(g_last_error, sizeof(g_last_error), "%s", msg);
    return code;
}

// Resolve the device address of the scratch array for the current device (once per device).
float* scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (g_partials_by_device[dev] == nullptr) {
        float* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_partials);
        if (e != cudaSuccess || ptr == nullptr) return nullptr;
        g_partials_by_device[dev] = ptr;
    }
    return g_partials_by_device[dev];
}

}  // namespace

extern "C" int gefenx_clip_coef_noalloc(const void* grad, long long numel, int dtype, float max_norm,
                                        float* coef_out, cudaStream_t stream) {
    if (grad == nullptr || coef_out == nullptr) return fail(1, "gefenx_clip_coef_noalloc: null pointer");
    if (reinterpret_cast<uintptr_t>(grad) % 16 != 0)
        return fail(1, "gefenx_clip_coef_noalloc: grad must be 16-byte aligned");
    if (dtype < 0 || dtype > 2) return fail(1, "gefenx_clip_coef_noalloc: dtype must be 0 (fp32), 1 (bf16) or 2 (fp16)");
    if (numel < 0) return fail(1, "gefenx_clip_coef_noalloc: negative element count");
    if (numel > GEFENX_NOALLOC_MAX_ELEMS) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "gefenx_clip_coef_noalloc: %lld elements exceed the static scratch limit of %lld",
                 numel, (long long)GEFENX_NOALLOC_MAX_ELEMS);
        return 2;
    }
    // the scratch array is resolved for the current device: both buffers must live there
    {
        int dev = -1;
        cudaPointerAttributes ga{}, ca{};
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaPointerGetAttributes(&ga, grad) != cudaSuccess ||
            cudaPointerGetAttributes(&ca, coef_out) != cudaSuccess) {
            cudaGetLastError();
            return fail(1, "gefenx_clip_coef_noalloc: could not identify the device of grad / coef_out");
        }
        const bool g_ok = (ga.type == cudaMemoryTypeDevice || ga.type == cudaMemoryTypeManaged) && ga.device == dev;
        const bool c_ok = (ca.type == cudaMemoryTypeDevice || ca.type == cudaMemoryTypeManaged) && ca.device == dev;
        if (!g_ok || !c_ok)
            return fail(1, "gefenx_clip_coef_noalloc: grad and coef_out must be device memory of the current device");
    }
    float* partials = scratch_for_current_device();
    if (partials == nullptr)
        return fail(3, "gefenx_clip_coef_noalloc: could not resolve the device scratch array");
    long long need = (numel + kElemsPerPartial - 1) / kElemsPerPartial;
    if (need < 1) need = 1;
    const int n_partials = (int)need;
    // the array still holds the previous call's sums: clear the part this call accumulates into
    if (cudaMemsetAsync(partials, 0, sizeof(float) * n_partials, stream) != cudaSuccess)
        return fail(4, "gefenx_clip_coef_noalloc: clearing the scratch failed");
    if (numel > 0) {
        const void* src[1] = {grad};
        if (gx::launch_reduce_sources(nullptr, src, 1, numel, 1.0f, partials, n_partials, dtype, stream) !=
            cudaSuccess)
            return fail(4, "gefenx_clip_coef_noalloc: sum-of-squares launch failed");
    }
    if (gx::launch_clip_coef(partials, n_partials, max_norm, coef_out, stream) != cudaSuccess)
        return fail(4, "gefenx_clip_coef_noalloc: coefficient launch failed");
    g_last_error[0] = 0;
    return 0;
}

extern "C" const char* gefenx_noalloc_last_error(void) { return g_last_error; }
