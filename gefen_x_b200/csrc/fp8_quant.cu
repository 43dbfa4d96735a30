// Row-wise e4m3 quantisation for the fp8 Newton-Schulz products.
//
// One CTA walks a row twice: the first pass takes the absolute maximum of
// y = alpha * x + beta * x2 (rounded to bf16), the second divides by
// scale = absmax / 448, converts to e4m3 (round to nearest even, saturating) and
// stores eight bytes per thread.  The second pass re-reads the row the CTA has just read,
// so it is served by the caches.  With `x2` the kernel is also the elementwise combine of the
// iteration (b G + c G G, or a X + U X) and can write y back as bf16, so neither the fp32
// temporaries nor the separate abs / amax / divide / clamp / cast passes of the torch
// statement exist.  The reference quantises with that chain of torch ops and relies on a
// tracing compiler to fuse it (reference src/gefen/gefen_muon.py:124-131, 174-186).
#include <cuda_fp8.h>

#include "common.cuh"
#include "fp8_quant.h"

namespace gx {
namespace {

constexpr int kThreads = 256;
constexpr float kE4m3Max = 448.0f;
constexpr float kMinScale = 1e-12f;

using bf16 = __nv_bfloat16;

__device__ __forceinline__ void load_combined(const bf16* __restrict__ xr, const bf16* __restrict__ x2r,
                                              long long c, float alpha, float beta, float (&y)[8]) {
    Vec8<bf16>::load(xr + c, y);
    if (x2r != nullptr) {
        float z[8];
        Vec8<bf16>::load(x2r + c, z);
#pragma unroll
        for (int e = 0; e < 8; ++e) y[e] = round_to<bf16>(fmaf(beta, z[e], __fmul_rn(alpha, y[e])));
    }
}

__global__ void __launch_bounds__(kThreads) quantize_rows_e4m3_kernel(
    const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ x2, long long ldx2, float alpha,
    float beta, long long rows, long long cols, uint8_t* __restrict__ q, float* __restrict__ scale,
    bf16* y_out) {
    __shared__ float red[kThreads / 32];
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        const bf16* xr = x + r * ldx;
        const bf16* x2r = x2 ? x2 + r * ldx2 : nullptr;
        float amax = 0.f;
        for (long long c = (long long)threadIdx.x * 8; c < cols; c += kThreads * 8) {
            float y[8];
            load_combined(xr, x2r, c, alpha, beta, y);
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(y[e]));
        }
        amax = warp_max(amax);
        __syncthreads();                       // `red` of the previous row has been read by everyone
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) amax = fmaxf(amax, red[i]);
        // absmax * (1 / 448): what dividing a tensor by the scalar 448 computes in torch on CUDA
        const float s = fmaxf(__fmul_rn(amax, 1.0f / kE4m3Max), kMinScale);
        if (threadIdx.x == 0) scale[r] = s;
        uint8_t* qr = q + r * cols;
        bf16* yr = y_out ? y_out + r * cols : nullptr;
        for (long long c = (long long)threadIdx.x * 8; c < cols; c += kThreads * 8) {
            float y[8];
            load_combined(xr, x2r, c, alpha, beta, y);
            uint32_t w[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float2 lo = make_float2(__fdiv_rn(y[4 * h], s), __fdiv_rn(y[4 * h + 1], s));
                const float2 hi = make_float2(__fdiv_rn(y[4 * h + 2], s), __fdiv_rn(y[4 * h + 3], s));
                const uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
                const uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
                w[h] = a | (b << 16);
            }
            *reinterpret_cast<uint2*>(qr + c) = make_uint2(w[0], w[1]);
            if (yr) Vec8<bf16>::store(yr + c, y);
        }
    }
}

// ---- column-wise quantisation with a transposed result --------------------------------------
// q_t[c, r] = e4m3(x[r, c] / scale_t[c]),  scale_t[c] = max(absmax(x[:, c]) / 448, 1e-12):
// the row-wise quantisation of x^T without materialising x^T (the column-major fp8 operand of
// U X).  Two kernels: column maxima (atomic max on the bit patterns of non-negative floats),
// then 128 x 64 tiles transposed through shared memory as packed bytes.

constexpr int kColsPerCta = kThreads * 8;     // col_absmax: 8 columns per thread
constexpr int kRowsPerCta = 32;

__global__ void __launch_bounds__(kThreads) col_absmax_kernel(const bf16* __restrict__ x, long long ldx,
                                                              long long rows, long long cols,
                                                              unsigned int* __restrict__ colmax) {
    const long long c = (long long)blockIdx.x * kColsPerCta + (long long)threadIdx.x * 8;
    if (c >= cols) return;
    const long long r0 = (long long)blockIdx.y * kRowsPerCta;
    const long long r1 = min(rows, r0 + kRowsPerCta);
    float m[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) m[e] = 0.f;
#pragma unroll 4
    for (long long r = r0; r < r1; ++r) {
        float y[8];
        Vec8<bf16>::load(x + r * ldx + c, y);
#pragma unroll
        for (int e = 0; e < 8; ++e) m[e] = fmaxf(m[e], fabsf(y[e]));
    }
#pragma unroll
    for (int e = 0; e < 8; ++e)
        if (m[e] > 0.f) atomicMax(colmax + c + e, __float_as_uint(m[e]));
}

constexpr int kTileRows = 128, kTileCols = 64, kPitchWords = kTileRows / 4 + 1;

__global__ void __launch_bounds__(kThreads) transpose_quant_kernel(const bf16* __restrict__ x, long long ldx,
                                                                   long long rows, long long cols,
                                                                   const unsigned int* __restrict__ colmax,
                                                                   uint8_t* __restrict__ q_t,
                                                                   float* __restrict__ scale_t) {
    __shared__ uint32_t tile[kTileCols * kPitchWords];       // tile[c][r / 4]: four rows per word
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // thread -> (row group of 4, column vector of 8): lanes vary the row group fastest so that the
    // shared-memory words of one store instruction fall into 32 different banks
    const int rg = (lane & 7) + 8 * (warp & 3);              // 0..31
    const int v = (lane >> 3) + 4 * (warp >> 2);             // 0..7
    const long long c0 = (long long)blockIdx.x * kTileCols, r0 = (long long)blockIdx.y * kTileRows;
    const long long c = c0 + v * 8, r = r0 + rg * 4;
    if (c < cols && r < rows) {                              // rows % 4 == 0 and cols % 8 == 0
        float s[8];
#pragma unroll
        for (int e = 0; e < 8; ++e)
            s[e] = fmaxf(__fmul_rn(__uint_as_float(colmax[c + e]), 1.0f / kE4m3Max), kMinScale);
        if (blockIdx.y == 0 && rg == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) scale_t[c + e] = s[e];
        }
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float y[8];
            Vec8<bf16>::load(x + (r + i) * ldx + c, y);
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
                const uint32_t p = __nv_cvt_float2_to_fp8x2(make_float2(__fdiv_rn(y[e], s[e]), __fdiv_rn(y[e + 1], s[e + 1])),
                                                            __NV_SATFINITE, __NV_E4M3);
                w[e] |= (p & 0xffu) << (8 * i);
                w[e + 1] |= (p >> 8) << (8 * i);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) tile[(v * 8 + e) * kPitchWords + rg] = w[e];
    }
    __syncthreads();
    // one warp writes the 128 bytes of one column's row segment per store
#pragma unroll
    for (int k = 0; k < kTileCols / 8; ++k) {
        const int cc = warp + 8 * k;
        const long long gc = c0 + cc, gr = r0 + lane * 4;
        if (gc < cols && gr < rows)
            *reinterpret_cast<uint32_t*>(q_t + gc * rows + gr) = tile[cc * kPitchWords + lane];
    }
}

}  // namespace

cudaError_t launch_quantize_rows_e4m3(const void* x, long long ldx, const void* x2, long long ldx2,
                                      float alpha, float beta, long long rows, long long cols,
                                      uint8_t* q, float* scale, void* y_out, int sm_count,
                                      cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    auto misaligned = [](const void* p, int a) { return reinterpret_cast<uintptr_t>(p) % a != 0; };
    if (cols % 8 || ldx % 8 || (x2 && ldx2 % 8)) return cudaErrorInvalidValue;
    if (misaligned(x, 16) || (x2 && misaligned(x2, 16)) || misaligned(q, 8) || (y_out && misaligned(y_out, 16)))
        return cudaErrorInvalidValue;
    const int grid = (int)max(1LL, min(rows, (long long)sm_count * 8));
    quantize_rows_e4m3_kernel<<<grid, kThreads, 0, st>>>((const bf16*)x, ldx, (const bf16*)x2, ldx2, alpha, beta,
                                                        rows, cols, q, scale, (bf16*)y_out);
    return cudaGetLastError();
}

cudaError_t launch_quantize_cols_e4m3_t(const void* x, long long ldx, long long rows, long long cols,
                                        unsigned int* colmax_zeroed, uint8_t* q_t, float* scale_t,
                                        cudaStream_t st) {
    if (rows <= 0 || cols <= 0) return cudaSuccess;
    if (cols % 8 || rows % 4 || ldx % 8 || reinterpret_cast<uintptr_t>(x) % 16 ||
        reinterpret_cast<uintptr_t>(q_t) % 4)
        return cudaErrorInvalidValue;
    dim3 g1((unsigned)((cols + kColsPerCta - 1) / kColsPerCta), (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta));
    col_absmax_kernel<<<g1, kThreads, 0, st>>>((const bf16*)x, ldx, rows, cols, colmax_zeroed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    dim3 g2((unsigned)((cols + kTileCols - 1) / kTileCols), (unsigned)((rows + kTileRows - 1) / kTileRows));
    transpose_quant_kernel<<<g2, kThreads, 0, st>>>((const bf16*)x, ldx, rows, cols, colmax_zeroed, q_t, scale_t);
    return cudaGetLastError();
}

}  // namespace gx
