// Row kernels of the GEMM-composed causal attention (ops/attention.py): the score and
// probability matrices are produced and consumed by the tcgen05 GEMM (gemm_sm100.cu); these
// kernels do the masked softmax of the forward pass and the probability / score-gradient
// recomputation of the backward pass, one warp per score row, 16-byte accesses, fp32 math.
//
// The reference has no attention kernel: its benchmark model calls
// F.scaled_dot_product_attention (reference benchmarks/training_matrix/tiny_qwen.py:168).
#include "attention.h"
#include "common.cuh"

namespace gx {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr float kLog2e = 1.4426950408889634f;

// scores: [rows, n_keys] raw q.k products (bf16), overwritten with the probabilities
// p = exp(scale * s - lse) for keys <= query position (row % seq_q) + key_offset, 0 beyond;
// lse[row] = log(sum_j exp(scale * s_j)) over the visible keys.
__global__ void __launch_bounds__(kThreads) causal_softmax_kernel(__nv_bfloat16* __restrict__ scores,
                                                                  float* __restrict__ lse, long long rows,
                                                                  int n_keys, int seq_q, float scale) {
    const int lane = threadIdx.x & 31;
    const float sl = scale * kLog2e;
    for (long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * kWarps) {
        __nv_bfloat16* r = scores + row * n_keys;
        const int last = (int)(row % seq_q) + (n_keys - seq_q);   // last visible key
        // pass 1: maximum over the visible keys
        float m = -INFINITY;
        for (int c = lane * 8; c <= last; c += 256) {
            float v[8];
            Vec8<__nv_bfloat16>::load(r + c, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) m = fmaxf(m, (c + e <= last) ? v[e] : -INFINITY);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        // pass 2 (row is in L1/L2): sum of exponentials
        float sum = 0.f;
        for (int c = lane * 8; c <= last; c += 256) {
            float v[8];
            Vec8<__nv_bfloat16>::load(r + c, v);
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += (c + e <= last) ? exp2f((v[e] - m) * sl) : 0.f;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        if (lane == 0) lse[row] = m * scale + logf(sum);
        // pass 3: probabilities (zeros beyond the diagonal)
        for (int c = lane * 8; c < n_keys; c += 256) {
            float v[8];
            if (c <= last) {
                Vec8<__nv_bfloat16>::load(r + c, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = (c + e <= last) ? exp2f((v[e] - m) * sl) * inv : 0.f;
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
            }
            Vec8<__nv_bfloat16>::store(r + c, v);
        }
    }
}

// delta[row] = sum_d dout[row, d] * out[row, d]
__global__ void __launch_bounds__(kThreads) row_dot_kernel(const __nv_bfloat16* __restrict__ a,
                                                           const __nv_bfloat16* __restrict__ b,
                                                           float* __restrict__ out, long long rows, int d) {
    const int lane = threadIdx.x & 31;
    for (long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * kWarps) {
        float acc = 0.f;
        for (int c = lane * 8; c < d; c += 256) {
            float x[8], y[8];
            Vec8<__nv_bfloat16>::load(a + row * d + c, x);
            Vec8<__nv_bfloat16>::load(b + row * d + c, y);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc += x[e] * y[e];
        }
        acc = warp_sum(acc);
        if (lane == 0) out[row] = acc;
    }
}

// Backward: scores (raw q.k) -> p = exp(scale * s - lse) (masked), dprob -> ds = p * (dp - delta) * scale,
// both in place.
__global__ void __launch_bounds__(kThreads) attn_bwd_rows_kernel(__nv_bfloat16* __restrict__ scores,
                                                                 __nv_bfloat16* __restrict__ dprob,
                                                                 const float* __restrict__ lse,
                                                                 const float* __restrict__ delta, long long rows,
                                                                 int n_keys, int seq_q, float scale) {
    const int lane = threadIdx.x & 31;
    const float sl = scale * kLog2e;
    for (long long row = (long long)blockIdx.x * kWarps + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * kWarps) {
        __nv_bfloat16* r = scores + row * n_keys;
        __nv_bfloat16* g = dprob + row * n_keys;
        const int last = (int)(row % seq_q) + (n_keys - seq_q);
        const float l2 = lse[row] * kLog2e, dl = delta[row];
        for (int c = lane * 8; c < n_keys; c += 256) {
            float v[8], w[8];
            if (c <= last) {
                Vec8<__nv_bfloat16>::load(r + c, v);
                Vec8<__nv_bfloat16>::load(g + c, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float p = (c + e <= last) ? exp2f(v[e] * sl - l2) : 0.f;
                    v[e] = p;
                    w[e] = p * (w[e] - dl) * scale;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) { v[e] = 0.f; w[e] = 0.f; }
            }
            Vec8<__nv_bfloat16>::store(r + c, v);
            Vec8<__nv_bfloat16>::store(g + c, w);
        }
    }
}

inline int grid_rows(long long rows) {
    long long g = (rows + kWarps - 1) / kWarps;
    return (int)(g < 148 * 8 ? (g < 1 ? 1 : g) : 148 * 8);
}

}  // namespace

cudaError_t launch_causal_softmax(void* scores, float* lse, long long rows, int n_keys, int seq_q,
                                  float scale, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (n_keys % 8 || seq_q <= 0 || n_keys < seq_q) return cudaErrorInvalidValue;
    causal_softmax_kernel<<<grid_rows(rows), kThreads, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(scores), lse,
                                                                rows, n_keys, seq_q, scale);
    return cudaGetLastError();
}

cudaError_t launch_row_dot(const void* a, const void* b, float* out, long long rows, int d, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (d % 8) return cudaErrorInvalidValue;
    row_dot_kernel<<<grid_rows(rows), kThreads, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(a),
                                                         reinterpret_cast<const __nv_bfloat16*>(b), out, rows, d);
    return cudaGetLastError();
}

cudaError_t launch_attn_bwd_rows(void* scores, void* dprob, const float* lse, const float* delta,
                                 long long rows, int n_keys, int seq_q, float scale, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (n_keys % 8 || seq_q <= 0 || n_keys < seq_q) return cudaErrorInvalidValue;
    attn_bwd_rows_kernel<<<grid_rows(rows), kThreads, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(scores),
                                                               reinterpret_cast<__nv_bfloat16*>(dprob), lse, delta,
                                                               rows, n_keys, seq_q, scale);
    return cudaGetLastError();
}

}  // namespace gx
