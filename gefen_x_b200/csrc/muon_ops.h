// Muon epilogue on the orthogonalised update: NorMuon row normalisation, the cautious mask and the
// parameter update as three launches over the matrix instead of a chain of elementwise torch ops.
#pragma once
#include <cuda_runtime.h>

namespace gx {

struct MuonEpilogue {
    void* update;              // [rows, cols] orthogonalised update (dtype), overwritten with the final update
    const void* grad;          // [rows, cols] gradient (dtype); cautious mask only, may be null
    void* param;               // [rows, cols] parameter (dtype) to step in the same pass, may be null
    float* v;                  // [rows] NorMuon second moment (updated), null without NorMuon
    float* row_sq;             // [rows] scratch: sum of squares per row
    int* agree;                // [rows] scratch: elements whose sign agrees with the gradient
    float* row_scale;          // [rows] scratch: factor of each row
    float* glob;               // [2] scratch: {cautious rescale, unused}
    const float* scal;         // device scalars {1 - beta2^t, lr * ratio, 1 - lr * weight_decay}
    long long rows;
    int cols;
    int normuon, cautious;
    float beta2, eps;
};

// dtype: 0 fp32, 1 bf16, 2 fp16.  Three kernels on `st`: row statistics, one CTA that turns them into
// row factors (fixed-order sums), and the pass that writes the update (and the parameter).
cudaError_t launch_muon_epilogue(const MuonEpilogue& e, int dtype, int sm_count, cudaStream_t st);

}  // namespace gx
