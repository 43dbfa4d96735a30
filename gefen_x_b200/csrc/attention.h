// Host-visible declarations of the attention row kernels (attention.cu).
#pragma once
#include <cuda_runtime.h>

namespace gx {

// scores [rows, n_keys] bf16 (raw q.k) -> probabilities in place; lse[rows]; the query position
// of a row is row % seq_q and key j is visible when j <= position + (n_keys - seq_q).
cudaError_t launch_causal_softmax(void* scores, float* lse, long long rows, int n_keys, int seq_q,
                                  float scale, cudaStream_t st);
// out[row] = sum_d a[row, d] * b[row, d] (bf16 inputs, d % 8 == 0)
cudaError_t launch_row_dot(const void* a, const void* b, float* out, long long rows, int d, cudaStream_t st);
// scores -> probabilities, dprob -> score gradients, both in place
cudaError_t launch_attn_bwd_rows(void* scores, void* dprob, const float* lse, const float* delta,
                                 long long rows, int n_keys, int seq_q, float scale, cudaStream_t st);

}  // namespace gx
