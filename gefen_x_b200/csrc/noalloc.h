// Allocation-free C entry point for the gradient-norm / clip-coefficient reduction.
//
// This entry point has no counterpart in the reference: it exists for callers of
// this library that are not allowed to allocate device memory at the point where
// they need the clipping coefficient -- code running inside a memory pool that has
// been frozen (for example between the steps of a job whose allocator is locked to
// avoid fragmentation), plugins loaded into a host process that owns the CUDA
// context and forbids cudaMalloc from guests, and tools that must keep working when
// the device is already full.  Such callers pass their own input and output
// buffers; the per-CTA partial sums, which the regular path keeps in a tensor that
// torch allocates, live instead in a fixed array inside the library's device image.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest input, in elements, that one call accepts (one partial sum per 16384 elements,
// 65536 partial sums = 256 KiB of static device memory per GPU that loads the library).
#define GEFENX_NOALLOC_MAX_ELEMS (65536LL * 16384LL)

// coef_out[0] = min(1, max_norm / (||grad||_2 + 1e-6)), coef_out[1] = ||grad||_2.
//   grad      device pointer to `numel` elements of `dtype` (0 = fp32, 1 = bf16, 2 = fp16),
//             16-byte aligned
//   coef_out  device pointer to two floats (written by the call)
//   stream    stream to run on
//             and on the device that is current when the call is made
// Returns 0 on success; 1 for a null / misaligned pointer, a bad dtype, or a `grad` / `coef_out`
// that does not live on the current device (the scratch array is per device: with another device
// current the call would clear and fill the wrong GPU's array); 2 when numel
// exceeds GEFENX_NOALLOC_MAX_ELEMS (nothing is launched); 3 when the device-side array
// could not be resolved; 4 when a launch failed.  `gefenx_noalloc_last_error()` returns a
// text for the last non-zero code of the calling thread.
//
// The call allocates nothing: no cudaMalloc / cudaFree and no allocating library routine.
// The first call on a device resolves the address of the static array for that device
// (with that device current); make that first call before any stream capture.  One thing
// outside this code's control happens on that first call: with lazy module loading (the CUDA
// default) the driver loads the library's device image when it is first touched, and that
// loading takes device memory (the image itself, this array included).  So make the first
// call on every device while allocation is still allowed -- before the pool is frozen, before
// the device is filled -- or set CUDA_MODULE_LOADING=EAGER; later calls touch no allocator.  Every
// call uses the same array, which keeps the previous call's partial sums until the next
// call clears the part it is going to use, so two calls whose kernels can overlap on the
// GPU (different streams, no dependency) race: serialise them.
int gefenx_clip_coef_noalloc(const void* grad, long long numel, int dtype, float max_norm,
                             float* coef_out, cudaStream_t stream);

const char* gefenx_noalloc_last_error(void);

#ifdef __cplusplus
}  // extern "C"
#endif
