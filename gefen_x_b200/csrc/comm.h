// Host-visible declarations of the peer-memory communication kernels (comm.cu).
#pragma once
#include <cuda_runtime.h>

namespace gx {

struct GatherSeg {
    long long src_off;   // byte offset inside the source rank's arena
    long long dst_off;   // byte offset inside the local destination buffer
    int src_rank;
    int pad;
};

// One slice of this rank's gradient shard and where every rank's contribution to it lies: in
// the peers' unsharded gradient buffers (summed by peer loads) or in local staging that the copy
// engines filled from them.
struct ReduceSeg {
    void* dst;               // local output (same dtype) or null: only the sum of squares is wanted
    const void* src[8];      // one source per rank, rank order
};

// One parameter shard and the (possibly remote) rows of the update that belong to it.
struct ApplySeg {
    void* p;             // local bf16 parameter shard
    const void* u;       // bf16 update rows (local or in a peer's arena), same length
    float alpha;         // lr * shape ratio
    float wd_factor;     // 1 - lr * weight_decay
};

// p = round(p * wd_factor) - alpha * u over a table of shards (8-element units, bf16).
cudaError_t launch_scatter_apply(const ApplySeg* segs_dev, int n_segs, const long long* unit_prefix_dev,
                                 long long total_units, int ctas, cudaStream_t st);

// flag_ptrs[r]: base of rank r's flag array; writes `value` to element `slot` on every rank.
cudaError_t launch_signal(void* const* flag_ptrs, int world, int slot, unsigned value, cudaStream_t st);
// bounded wait until flags[0..n) >= value
cudaError_t launch_wait(const unsigned* flags, int n, unsigned value, long long max_iters, int* status,
                        cudaStream_t st);
// copy segments (16-byte units) from the ranks' arenas into dst
cudaError_t launch_gather(void* const* src_base, int world, const GatherSeg* segs_dev, int n_segs,
                          void* dst, const long long* unit_prefix_dev, long long total_units, int ctas,
                          cudaStream_t st);
// Reduce-scatter by peer loads, one launch for every slice of a table:
// dst[i] = round(sum_r src[r][i] * scale) in 16-byte units, and (optionally) the sum of squares
// of the rounded result, one partial per CTA, added into partials[blockIdx.x] (partials must
// hold at least `ctas` floats).  dtype: 0 fp32, 1 bf16, 2 fp16.
cudaError_t launch_reduce_segments(int world, const ReduceSeg* segs_dev, int n_segs,
                                   const long long* unit_prefix_dev, long long total_units, float scale,
                                   float* partials, int ctas, int dtype, cudaStream_t st, bool multimem = false);
// multimem = true: src[0] of every segment is the NVLS multicast address of the slice (bf16 only) and
// one multimem.ld_reduce per 16 bytes replaces the per-peer loads.
// out = sum_r value_r ; slot_ptrs[r] / flag_ptrs[r] are rank r's slot and flag array
cudaError_t launch_allreduce_scalar(void* const* slot_ptrs, void* const* flag_ptrs, int world, int rank,
                                    const float* local_val, float* out, unsigned epoch,
                                    long long max_iters, int* status, cudaStream_t st);

// Sparse embedding over a row-sharded table (row r on rank r / rows_per).
// out[t, :] = table[tok[t], :] by peer loads; shard_ptrs[r] = start of rank r's rows; row_bytes % 16 == 0.
cudaError_t launch_gather_rows(void* const* shard_ptrs, int world, long long rows_per, long long rows,
                               int row_bytes, const long long* tok_dev, int n_tok, void* out, cudaStream_t st);
// dst[tok - row0, :] += scale * grad_r[t, :] over every rank's token list (bf16, dst zeroed by the caller);
// tok_ptrs[r] / grad_ptrs[r]: rank r's int64 ids [n_tok] and bf16 rows [n_tok, cols] in its arena.
cudaError_t launch_scatter_add_rows(void* const* tok_ptrs, void* const* grad_ptrs, int world, int n_tok,
                                    long long row0, long long my_rows, int cols, float scale, void* dst,
                                    cudaStream_t st);

}  // namespace gx
