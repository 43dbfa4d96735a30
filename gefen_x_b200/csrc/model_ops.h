// Host-visible declarations of the memory-bound model kernels (model_ops.cu).
#pragma once
#include <cuda_runtime.h>

namespace gx {

cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int d,
                               float eps, int dtype, cudaStream_t st);
// number of rows the backward kernel writes into dw_partial for this problem
int rmsnorm_bwd_partials(long long rows, int d);
// `res` (optional, same shape as dx) is added to dx: the gradient of the residual path.
cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* dw_partial, int n_partial, long long rows, int d, int dtype,
                               cudaStream_t st, const void* res = nullptr);
// out[c] = sum over the n_rows rows of part [n_rows, d] (fp32), fixed order.
cudaError_t launch_colsum(const float* part, int n_rows, int d, float* out, cudaStream_t st);
// dst / src: [tokens, n_heads, head_dim] with dst_stride / src_stride elements between tokens
// (dst may alias src)
cudaError_t launch_rope(void* dst, const void* src, long long dst_stride, long long src_stride,
                        const float* cs, const float* sn, long long tokens, int seq_len,
                        int n_heads, int head_dim, bool inverse, bool interleaved, int dtype,
                        cudaStream_t st);
cudaError_t launch_swiglu_fwd(const void* gate_up, void* out, long long rows, int f, int dtype,
                              cudaStream_t st);
cudaError_t launch_swiglu_bwd(const void* gate_up, const void* dout, void* dgate_up, long long rows,
                              int f, int dtype, cudaStream_t st);
cudaError_t launch_xent_fwd_bwd(void* logits, const long long* targets, float* loss_rows, long long rows,
                                int v, float grad_scale, long long ignore_index, int dtype,
                                cudaStream_t st);

}  // namespace gx
