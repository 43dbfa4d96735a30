// Host-visible declarations of the first-step analysis kernels (quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gx {

// counts[bins] (uint64) += histogram of x / absmax(block) over [-1, 1].
cudaError_t launch_histogram(const void* x, int dtype, long long numel, int period, int bins,
                             unsigned long long* counts, int sm_count, cudaStream_t st);

// partials[n_div * ctas_per_div] (fp64) = per-CTA sums of the within-block
// variance of x^2 (or of x when `squared`) for every divisor in divisors_dev.
cudaError_t launch_period_errors(const void* x, int dtype, long long numel,
                                 const long long* divisors_dev, int n_div, bool squared,
                                 double* partials, int ctas_per_div, cudaStream_t st);

// idx[i] <- map[idx[i]] in place (map: 256 bytes on the device; idx 16-byte aligned)
cudaError_t launch_remap_indices(uint8_t* idx, const uint8_t* map, long long numel, int sm_count,
                                 cudaStream_t st);

// out[i] = codebook[idx[i]] * mag[i / period] (dense momentum), out dtype: 0 fp32, 1 bf16, 2 fp16
cudaError_t launch_dequantize(const uint8_t* idx, const float* mag, const float* codebook, long long numel,
                              long long period, void* out, int dtype, int sm_count, cudaStream_t st);

}  // namespace gx
