// Host-visible declaration of the e4m3 row quantisation (fp8_quant.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gx {

// y = alpha * x + beta * x2 (x2 may be null: y = x), rounded to bf16; per row r:
//   scale[r] = max(absmax(y[r, :]) / 448, 1e-12),  q[r, c] = e4m3(y[r, c] / scale[r])
// x, x2: bf16 [rows, cols] with row strides ldx / ldx2 (elements, multiples of 8, 16-byte aligned
// bases); q: [rows, cols] bytes, contiguous; y_out (may be null): bf16 [rows, cols] contiguous,
// not aliasing x or x2.  cols must be a multiple of 8.
cudaError_t launch_quantize_rows_e4m3(const void* x, long long ldx, const void* x2, long long ldx2,
                                      float alpha, float beta, long long rows, long long cols,
                                      uint8_t* q, float* scale, void* y_out, int sm_count,
                                      cudaStream_t st);

// The row-wise quantisation of x^T without materialising x^T: q_t [cols, rows] bytes (contiguous),
// scale_t[cols]; x: bf16 [rows, cols] with row stride ldx; rows % 4 == 0, cols % 8 == 0;
// colmax_zeroed: cols zero-initialised 32-bit words of scratch.
cudaError_t launch_quantize_cols_e4m3_t(const void* x, long long ldx, long long rows, long long cols,
                                        unsigned int* colmax_zeroed, uint8_t* q_t, float* scale_t,
                                        cudaStream_t st);

}  // namespace gx
