// Host-visible declarations of the multi-tensor Gefen update kernels.
//
// One launch serves every tensor of a plan: the device reads an array of
// TensorDesc records (pointers, geometry, hyper-parameters) and a prefix table
// that maps a work-tile number to its tensor.  The reference launches its
// kernels once per parameter (reference src/gefen/gefen.py:5783-5820); here the
// step of a whole model is a fixed handful of launches.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gx {

constexpr int kDescMaxSrc = 8;

// dtype codes shared with the bindings
enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2 };

struct alignas(16) TensorDesc {
    void* p;                          // parameter (shard), element type = launch dtype
    const void* g[kDescMaxSrc];       // gradient sources, summed: g = round(sum_s g[s] * src_scale)
    uint8_t* idx;                     // momentum codebook indices [numel]
    float* mag;                       // momentum magnitude per block [nb]
    float* mag_new;                   // scratch [nb] (zero before the statistics pass)
    float* v0;                        // block path: vmean [nb]; factored: v_row [rows]
    float* v1;                        // factored: v_col [cols]
    float* row_sq;                    // scratch [rows]  (zero before the statistics pass)
    float* col_sq;                    // scratch [cols]  (zero before the statistics pass)
    float* rfac;                      // scratch [rows]
    float* cfac;                      // scratch [cols]
    const float* scal;                // device scalars [lr, s2, 1/bc1, 1-lr*wd]
    // cross-shard exchange of the factored statistics (Shard(0) row shards)
    float* xchg_local;                // this rank's two slots [2][cols + 1] in symmetric memory (epoch parity)
    const float* xchg_peer[kDescMaxSrc];  // every rank's slot (own included), rank order
    uint32_t* flag_local;             // [world] arrival flags in this rank's memory
    uint32_t* flag_peer[kDescMaxSrc]; // the same array on every rank
    long long numel;
    long long nb;                     // number of blocks = numel / period
    int rows, cols;                   // local 2-D view (factored path)
    int period;
    int total_rows;                   // rows of the whole matrix (== rows when unsharded)
    int n_src;
    int blk_mode;                     // 0: period==cols, 1: cols%period==0, 2: period%cols==0, 3: general
    int tcols, trows;                 // thread tiling of a CTA: tcols*trows == 256
    int n_col_tiles;
    int rows_per_tile;
    int mode;                         // block path: 0 thread/block, 1 warp/block, 2 CTA/block
    int vec;                          // 1: 8-wide vector path allowed, 0: scalar path
    int world, rank;                  // exchange participants (world <= 1: no exchange)
    int row_only;                     // 1: second moment per row only (block path as [nb, period]);
                                      // 2 / 3: momentum emit (Muon): no second moment, p receives the dense
                                      // new momentum (3: with the Nesterov look-ahead)
    int g_multimem;                   // 1: g[0] is an NVLS multicast address (bf16): every 16 bytes are read with
                                      // multimem.ld_reduce, which returns the sum over all ranks; n_src == 1
    float beta1, omb1, beta2, omb2, eps, src_scale;
};

struct LaunchCommon {
    const TensorDesc* descs;
    const int* tile_start;            // [n_tensors + 1] prefix of work tiles (fast == 4: followed by the
                                      // prefix of the 16-wide tiles)
    int n_tensors;
    int total_tiles;
    const float* codebook;            // [256]
    const float* thresholds;          // [256]: midpoints of neighbouring codewords, last = +inf
    const uint16_t* lut;              // [16384] bucket table over the thresholds (count below | count inside << 8)
    const float* gscale;              // optional device scalar multiplying every gradient
    int* status;                      // device status word (Status enum), may be null
    unsigned long long sr_seed;
    const double* sr_seed_dev;        // optional device counter added to sr_seed (CUDA-graph replays draw
                                      // fresh rounding noise because the counter advances on the device)
    int stochastic;
    long long wait_iters;             // bound of every peer wait
    uint32_t epoch;                   // value the exchange flags must reach in this launch
    int fast;                         // 1: every tensor takes the 8-wide path with one gradient source;
                                      // 2: the same, and that source is an NVLS multicast address (bf16)
                                      // 3: as 1, 2-byte tensors whose rows start on 16-element boundaries:
                                      //    the streamed kernels (shared-memory rings fed by bulk copies)
                                      // 4: as 3 with block periods that are multiples of 16: the streamed
                                      //    kernels with 16 elements per thread; tile_start then holds a
                                      //    second prefix [n_tensors + 1] for their tile geometry
};

// All launchers return the cudaError_t of the launch.
cudaError_t launch_block_update(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t s);
cudaError_t launch_factored_stats(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t s);
cudaError_t launch_factored_ema(const LaunchCommon& c, cudaStream_t s);
cudaError_t launch_factored_apply(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t s);
cudaError_t launch_finalize_magnitude(const LaunchCommon& c, int sm_count, cudaStream_t s);

// out[i] = round(sum_s src[s][i] * scale) and (optionally) partial sums of
// squares of the rounded result, one per CTA, into sumsq_partials[gridDim.x].
cudaError_t launch_reduce_sources(void* out, const void* const* src, int n_src, long long numel,
                                  float scale, float* sumsq_partials, int n_partials, int dtype,
                                  cudaStream_t s);
// coef[0] = min(1, max_norm / (sqrt(sum partials [+ extra]) + 1e-6)), coef[1] = norm
cudaError_t launch_clip_coef(const float* partials, int n, float max_norm, float* coef,
                             cudaStream_t s);

}  // namespace gx
