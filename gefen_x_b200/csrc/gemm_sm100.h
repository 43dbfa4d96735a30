// Host-visible declarations of the tcgen05 / TMEM bf16 GEMM (gemm_sm100.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "comm.h"

namespace gx {

struct GemmParams {
    int M, N, K, batch;
    int a_mn_major, b_mn_major;     // 0: operand stored [rows, K]; 1: stored [K, rows]
    float alpha, beta;
    __nv_bfloat16* C;
    const __nv_bfloat16* D;         // optional addend (may be null)
    long long ldc, ldd, batch_stride_c, batch_stride_d;
    int* status;                    // device status word, may be null
    int m_tiles, n_tiles, total_tiles;
    int vec_ok;                     // rows of C / D are 16-byte aligned
};

// All-gather fused into the GEMM: rows of B live as row shards on several ranks; the launch
// pulls them into the local staging matrix while the tensor cores already work on the
// column blocks whose rows have arrived.
struct AgParams {
    int enabled;
    int fetch_ctas;                 // CTAs that copy instead of multiplying
    int n_segs;
    const GatherSeg* segs;          // in arrival order: own rank first, then ring order
    const long long* seg_meta;      // [n_segs][3]: 16-byte units, first staging row, rows
    const int* tile_order;          // [n_tiles]: column blocks sorted by arrival
    char* dst_base;                 // staging matrix base (bytes)
    uint32_t* flags;                // [n_segs], set to `epoch` when a segment has landed
    uint32_t* count;                // [n_segs], monotonic arrival counters
    uint32_t epoch;
    uint32_t count_target;          // value of count[s] that completes segment s in this launch
};

// C = A[M,K] @ Bstage[N,K]^T with Bstage filled from the peers by the launch itself.
cudaError_t launch_gemm_ag_bf16(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* Bstage,
                                long long ldb, GemmParams p, AgParams ag, const void* const* peer_bases,
                                int world, int sm_count, cudaStream_t st);

// C[b] = alpha * op(A[b]) op(B[b]) + beta * D[b], bf16 in/out, fp32 accumulate.
// A: a_mn_major ? [batch, K, M] : [batch, M, K] with leading dimension lda (elements), etc.
// All leading dimensions and batch strides must be multiples of 8 elements and the base
// pointers 16-byte aligned (TMA requirements).  Returns cudaErrorInvalidValue otherwise.
cudaError_t launch_gemm_bf16(const __nv_bfloat16* A, long long lda, long long batch_stride_a,
                             const __nv_bfloat16* B, long long ldb, long long batch_stride_b,
                             GemmParams p, int sm_count, cudaStream_t st);

// ---- CTA-pair GEMM (gemm_pair_sm100.cu): tcgen05.mma.cta_group::2, 256 x BN tile per pair ----
enum PairEpilogue : int {
    kEpiPlain = 0,        // C0 = alpha * A B + beta * D
    kEpiSwigluFwd = 1,    // B = [gate rows | up rows] (2F x K): C0 = gate, C1 = up, C2 = silu(gate) * up
    kEpiSwigluBwd = 2,    // A B = d(act); aux = [gate | up]: C0 = d(gate), C1 = d(up)
    kEpiScaledE4m3 = 3,   // e4m3 operands [rows, K] with one fp32 scale per row: C0 = (A B^T) * sa[row] * sb[col]
};

struct PairParams {
    int M, N, K;                    // N = columns of one output matrix (F for the SwiGLU epilogues)
    int a_mn_major, b_mn_major;     // 0: operand stored [rows, K]; 1: stored [K, rows]
    float alpha, beta;
    const __nv_bfloat16* D;         // optional addend of the plain epilogue (may be null)
    long long ldd;
    int epi;                        // PairEpilogue
    int F;                          // SwiGLU epilogues: width of gate (= N)
    const __nv_bfloat16* aux;       // kEpiSwigluBwd: [M, 2F] gate | up
    long long ldaux;
    const float* row_scale;         // kEpiScaledE4m3: [M] scales of A's rows
    const float* col_scale;         // kEpiScaledE4m3: [N] scales of B's rows (the output's columns)
    int symmetric;                  // plain epilogue, M == N, the result (and D) symmetric: only the tiles on and
                                    // below the diagonal are computed, a second launch mirrors them
    int bn;                         // 0: choose; 128 / 256: force the tile width
    int* status;                    // device status word, may be null
    // plain epilogue, optional: sum of squares of the stored output accumulated into kSumsqSlots fp32
    // slots (the caller sums them; each slot has one writer per launch, so the total is reproducible)
    float* sumsq;
    // K-split of the tail wave (optional): fp32 workspace and zero-initialised arrival counters that
    // the kernel leaves zeroed; launches sharing them must be ordered on one stream
    // dynamic schedule (optional): a zero-initialised counter that every launch leaves at zero; null =
    // static schedule.  Launches sharing the counter must be ordered on one stream.
    uint32_t* sched;
    float* ws;
    long long ws_floats;
    uint32_t* counters;
    int n_counters;
    int m_tiles, n_tiles, total_tiles;
    int full_tiles, rem_tiles, splits;     // set by the launcher
    int group_m;                           // set by the launcher: row tiles per group of the visiting order
    int d_vec_ok;
};
constexpr int kMaxSplits = 8;
constexpr int kSumsqTailBase = 1024;       // slots [0, 1024): per epilogue warp; [1024, 2048): per tail-tile slice
constexpr int kSumsqSlots = 2048;
// workspace that always suffices: half of the pairs' tiles, 256 x 256 fp32 each, and their counters
constexpr long long kPairWsFloats = 74ll * 256 * 256;
constexpr int kPairCounters = 74 * 8 + 8;       // + the schedule counter (last 8 words, 32-byte aligned)

// True when the pair kernel can run the product (otherwise use launch_gemm_bf16).
bool gemm_pair_supported(int M, int N, int K);
// Tile width (128 / 256) that wastes the least of the last wave of pair tiles.
int gemm_pair_pick_bn(int M, int N, int sm_count);

// C0 (and C1, C2 for the SwiGLU epilogues; otherwise null) are row-major with leading dimensions
// ldc*.  Leading dimensions must be multiples of 8 elements and base pointers 16-byte aligned.
cudaError_t launch_gemm_pair_bf16(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* B, long long ldb,
                                  PairParams p, __nv_bfloat16* C0, long long ldc0, __nv_bfloat16* C1,
                                  long long ldc1, __nv_bfloat16* C2, long long ldc2, int sm_count,
                                  cudaStream_t st);
// Row-scaled e4m3 product on the same kernel: C0 = (A B^T) * row_scale[m] * col_scale[n]; A [M, K] and
// B [N, K] hold e4m3 bytes (leading dimensions in bytes, multiples of 16), p carries M, N, K, the two
// scale vectors and the optional K-split / schedule workspaces.
cudaError_t launch_gemm_pair_e4m3(const void* A, long long lda, const void* B, long long ldb, PairParams p,
                                  __nv_bfloat16* C0, long long ldc0, int sm_count, cudaStream_t st);

// Causal attention forward (flash form) on heads-first operands: q [batch, rows, hd] with
// rows = group * seq (the query heads of one KV head stacked along the rows), k / v
// [batch, seq, hd], out [batch, rows, hd], lse [batch * rows].  hd in {64, 128}, seq % 128 == 0.
struct FlashParams {
    int seq, rows, batch;
    float scale;
    __nv_bfloat16* out;
    float* lse;
    int* status;                    // device status word, may be null
};
cudaError_t launch_flash_attention_fwd(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                                       int head_dim, FlashParams p, cudaStream_t st);

}  // namespace gx
