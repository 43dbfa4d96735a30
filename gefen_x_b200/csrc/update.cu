// Multi-tensor Gefen update kernels for sm_100a.
//
// Replaces the reference's per-parameter kernel families (reference
// src/gefen/kernels/automatic_gefen_fused_kernel.cu: block path :474-760 and
// :979-1470, factored path :1596-1990, vmean :40-120 of
// automatic_vmean_kernel.cu) with four persistent, descriptor-driven kernels:
//
//   block_update    one worker (thread / warp / CTA) owns a whole block:
//                   statistics, second-moment EMA, requantisation and the
//                   parameter write in one launch for every tensor of the plan.
//   factored_stats  one pass over grad + indices: per-block |m| maximum, row and
//                   column sums of g^2.
//   factored_ema    one CTA per tensor: v_row / v_col EMAs, the cross-shard sum
//                   of the column statistics (peer loads over NVLink with
//                   bounded waits) and the per-row / per-column step factors.
//   factored_apply  requantise + parameter write with the per-element step
//                   rfac[i] * cfac[j].
//
// The gradient of a tensor may be given as up to eight sources (the slices of
// this rank's shard inside every peer's unsharded bf16 gradient buffer); they
// are summed in fp32 and rounded to the gradient dtype, which is what a
// reduce-scatter would have delivered, so the collective is fused into the
// update.  HBM-bound by design: 16-byte vector loads, 8 elements per thread and
// row, persistent CTAs walking a contiguous range of equally sized work tiles so
// that column partial sums are flushed once per column tile.  Plans whose tensors
// all take the 8-wide single-source path run the "fast" tile loops: one row per
// iteration with the next row's raw chunk prefetched into registers, a loop body
// small enough for the instruction cache, 80 registers and three CTAs per SM.
// Plans of 2-byte tensors whose rows start on 16-element boundaries run the "streamed"
// kernels instead: one CTA per SM holds the tables once and three groups of 256 threads, each
// with a producer warp that feeds a shared-memory ring of row steps with bulk async copies
// (cp.async.bulk, mbarrier transaction counts), so that 150 KB per SM are in flight without
// costing registers and the arithmetic never waits on a global load.
#include "common.cuh"
#include "sm100_ptx.cuh"
#include "update.h"
#include <type_traits>

namespace gx {
namespace {

constexpr int kThreads = 256;

// Dynamic shared memory of a CTA: reduction scratch, lane-replicated codebook and, for
// kernels that requantise, the thresholds and the bucket table.
struct Smem {
    float* cb;         // [256 * 32]
    float* red;        // [16]
    QuantTables q;
};

constexpr int kRepFloats = kCodewords * 32;
constexpr size_t kSmemStats = (size_t)(kRepFloats + 16) * sizeof(float);
constexpr size_t kSmemFull = kSmemStats + kCodewords * sizeof(float) + kLutBuckets * sizeof(uint16_t);

extern __shared__ __align__(16) unsigned char gx_smem_raw[];

__device__ __forceinline__ Smem load_tables(const LaunchCommon& c, bool full) {
    Smem s;
    float* base = reinterpret_cast<float*>(gx_smem_raw);
    s.red = base;
    s.cb = base + 16;
    float* thr = s.cb + kRepFloats;
    uint16_t* lut = reinterpret_cast<uint16_t*>(thr + kCodewords);
    // each thread fetches codewords once and writes their 32 lane copies; the bucket table is
    // copied in 16-byte pieces (few dependent global loads: this prologue is pure latency)
    for (int i = threadIdx.x; i < kCodewords; i += blockDim.x) {
        const float v = c.codebook[i];
        float4* row = reinterpret_cast<float4*>(s.cb + i * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) row[k] = make_float4(v, v, v, v);
    }
    if (full) {
        for (int i = threadIdx.x; i < kCodewords; i += blockDim.x) thr[i] = c.thresholds[i];
        const uint4* src = reinterpret_cast<const uint4*>(c.lut);
        uint4* dst = reinterpret_cast<uint4*>(lut);
        constexpr int kPieces = kLutBuckets * (int)sizeof(uint16_t) / 16;
#pragma unroll 4
        for (int i = threadIdx.x; i < kPieces; i += blockDim.x) dst[i] = src[i];
    }
    s.q.cb = s.cb;
    s.q.thr = full ? thr : nullptr;
    s.q.lut = full ? lut : nullptr;
    __syncthreads();
    return s;
}

__device__ __forceinline__ int find_tensor(const int* __restrict__ start, int n, int tile) {
    int lo = 0, hi = n;  // start[lo] <= tile < start[hi]
    while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (start[mid] <= tile) lo = mid; else hi = mid;
    }
    return lo;
}

// The fields of a descriptor that the tile kernels use, copied into registers when a
// CTA moves to a new tensor (a reference into global memory would be re-read after
// every store or atomic, since the compiler must assume they alias).
struct Hot {
    void* p;
    const void* g0;
    const TensorDesc* full;   // for the rarely used arrays (extra gradient sources)
    uint8_t* idx;
    float* mag;
    float* mag_new;
    float* row_sq;
    float* col_sq;
    const float* rfac;
    const float* cfac;
    const float* scal;
    int rows, cols, period, n_src, blk_mode, tcols, trows, n_col_tiles, rows_per_tile, vec, row_only;
    int small;                // numel < 2^31: 32-bit index arithmetic
    unsigned step_blk, step_rem;   // (trows * cols) / period and % period: block advance of one row step
    float beta1, omb1, eps, src_scale;
};

__device__ __forceinline__ Hot load_hot(const TensorDesc* t) {
    Hot h;
    h.p = t->p; h.g0 = t->g[0]; h.full = t; h.idx = t->idx; h.mag = t->mag; h.mag_new = t->mag_new;
    h.row_sq = t->row_sq; h.col_sq = t->col_sq; h.rfac = t->rfac; h.cfac = t->cfac; h.scal = t->scal;
    h.rows = t->rows; h.cols = t->cols; h.period = t->period; h.n_src = t->n_src;
    h.blk_mode = t->blk_mode; h.tcols = t->tcols; h.trows = t->trows; h.n_col_tiles = t->n_col_tiles;
    h.rows_per_tile = t->rows_per_tile; h.vec = t->vec; h.row_only = t->row_only;
    h.small = t->numel < 2147483647LL ? 1 : 0;
    {
        const unsigned long long step = (unsigned long long)h.trows * (unsigned)h.cols;
        h.step_blk = (unsigned)(step / (unsigned)h.period);
        h.step_rem = (unsigned)(step % (unsigned)h.period);
    }
    h.beta1 = t->beta1; h.omb1 = t->omb1; h.eps = t->eps; h.src_scale = t->src_scale;
    return h;
}

// Gradient chunk of 8 (VEC=8) or 1 element: sum of the sources in fp32, scaled,
// rounded to the storage type when more than one source contributed.
__device__ __forceinline__ const void* grad_src(const TensorDesc& d, int s) { return d.g[s]; }
__device__ __forceinline__ const void* grad_src(const Hot& d, int s) { return s == 0 ? d.g0 : d.full->g[s]; }

template <typename T, int VEC, typename D>
__device__ __forceinline__ void load_grad(const D& d, long long off, float gs, float (&g)[VEC]) {
    if constexpr (VEC == 8) {
        Vec8<T>::load(reinterpret_cast<const T*>(grad_src(d, 0)) + off, g);
        if (d.n_src > 1) {
            for (int s = 1; s < d.n_src; ++s) {
                float t[8];
                Vec8<T>::load(reinterpret_cast<const T*>(grad_src(d, s)) + off, t);
#pragma unroll
                for (int e = 0; e < 8; ++e) g[e] += t[e];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = round_to<T>(__fmul_rn(g[e], d.src_scale));
        }
    } else {
        float a = to_f<T>(reinterpret_cast<const T*>(grad_src(d, 0))[off]);
        if (d.n_src > 1) {
            for (int s = 1; s < d.n_src; ++s) a += to_f<T>(reinterpret_cast<const T*>(grad_src(d, s))[off]);
            a = round_to<T>(__fmul_rn(a, d.src_scale));
        }
        g[0] = a;
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = __fmul_rn(g[e], gs);
}

template <int VEC>
__device__ __forceinline__ void load_index(const uint8_t* p, int (&o)[VEC]) {
    if constexpr (VEC == 8) load_idx8(p, o);
    else o[0] = p[0];
}
template <int VEC>
__device__ __forceinline__ void store_index(uint8_t* p, const int (&v)[VEC]) {
    if constexpr (VEC == 8) store_idx8(p, v);
    else p[0] = (uint8_t)v[0];
}
template <typename T, int VEC>
__device__ __forceinline__ void load_param(const T* p, float (&o)[VEC]) {
    if constexpr (VEC == 8) Vec8<T>::load(p, o);
    else o[0] = to_f<T>(p[0]);
}
template <typename T, int VEC>
__device__ __forceinline__ void store_param(T* p, const float (&v)[VEC]) {
    if constexpr (VEC == 8) Vec8<T>::store(p, v);
    else p[0] = from_f<T>(v[0]);
}

__device__ __forceinline__ float ema_momentum(float cbv, float mag_old, float g, float b1, float omb1) {
    return __fadd_rn(__fmul_rn(__fmul_rn(cbv, mag_old), b1), __fmul_rn(g, omb1));
}

template <typename T>
__device__ __forceinline__ float apply_one(float pf, float q, float step, float lr, float wdf) {
    if (wdf != 1.0f) pf = round_to<T>(__fmul_rn(pf, wdf));
    return __fsub_rn(pf, __fmul_rn(__fmul_rn(q, step), lr));
}

template <bool FAST = false>
__device__ __forceinline__ int quantise(float n, const Smem& s, const LaunchCommon& c, long long elem) {
    if constexpr (FAST) return nearest_index(n, s.q);
    if (c.stochastic) {
        const unsigned long long seed =
            c.sr_seed_dev ? c.sr_seed + (unsigned long long)__ldg(c.sr_seed_dev) : c.sr_seed;
        return stochastic_index(n, s.q, sr_uniform(seed, (uint64_t)elem));
    }
    return nearest_index(n, s.q);
}

// ---------------------------------------------------------------------------
// block path
// ---------------------------------------------------------------------------
// One worker of NL lanes owns block `blk` of tensor d.  MODE 0: NL = 1 thread,
// 1: a warp, 2: the CTA.
template <typename T, int VEC, int MODE>
__device__ void block_worker(const TensorDesc& d, const LaunchCommon& c, const Smem& s, long long blk,
                             bool valid, float gs) {
    const int lane = (MODE == 0) ? 0 : (MODE == 1 ? (threadIdx.x & 31) : threadIdx.x);
    const int nl = (MODE == 0) ? 1 : (MODE == 1 ? 32 : kThreads);
    const int P = d.period;
    const long long base = valid ? blk * (long long)P : 0;
    // state of the block is read before the reduction barrier and written after it
    const float mag_old = valid ? d.mag[blk] : 0.f;
    const float v_old = valid ? d.v0[blk] : 0.f;
    T* p = reinterpret_cast<T*>(d.p);
    float amax = 0.f, ssq = 0.f;
    if (valid) {
        for (int e0 = lane * VEC; e0 < P; e0 += nl * VEC) {
            float g[VEC];
            int ix[VEC];
            load_grad<T, VEC>(d, base + e0, gs, g);
            load_index<VEC>(d.idx + base + e0, ix);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float m = ema_momentum(rep_load(s.cb, ix[e]), mag_old, g[e], d.beta1, d.omb1);
                amax = fmaxf(amax, fabsf(m));
                ssq += g[e] * g[e];
            }
        }
    }
    if (MODE == 1) {
        amax = warp_max(amax);
        ssq = warp_sum(ssq);
    } else if (MODE == 2) {
        amax = warp_max(amax);
        ssq = warp_sum(ssq);
        const int w = threadIdx.x >> 5;
        __syncthreads();
        if ((threadIdx.x & 31) == 0) { s.red[w] = amax; s.red[8 + w] = ssq; }
        __syncthreads();
        amax = s.red[0];
        ssq = s.red[8];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) { amax = fmaxf(amax, s.red[i]); ssq += s.red[8 + i]; }
    }
    if (!valid) return;
    const float lr = d.scal[0], s2 = d.scal[1], inv_bc1 = d.scal[2], wdf = d.scal[3];
    const float ms = __fmul_rn(ssq, 1.0f / (float)P);
    const float v = __fadd_rn(__fmul_rn(v_old, d.beta2), __fmul_rn(ms, d.omb2));
    const float h = __fadd_rn(__fmul_rn(__fsqrt_rn(v), s2), d.eps);
    const float step = __fmul_rn(__frcp_rn(h), inv_bc1);
    const float inv = amax > 0.f ? __frcp_rn(amax) : 0.f;
    if (MODE == 1) __syncwarp();
    if (lane == 0) { d.v0[blk] = v; d.mag[blk] = amax; }
    for (int e0 = lane * VEC; e0 < P; e0 += nl * VEC) {
        float g[VEC], pf[VEC];
        int ix[VEC];
        load_grad<T, VEC>(d, base + e0, gs, g);
        load_index<VEC>(d.idx + base + e0, ix);
        load_param<T, VEC>(p + base + e0, pf);
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            float m = ema_momentum(rep_load(s.cb, ix[e]), mag_old, g[e], d.beta1, d.omb1);
            int k = quantise(__fmul_rn(m, inv), s, c, base + e0 + e);
            ix[e] = k;
            pf[e] = apply_one<T>(pf[e], __fmul_rn(rep_load(s.cb, k), amax), step, lr, wdf);
        }
        store_index<VEC>(d.idx + base + e0, ix);
        store_param<T, VEC>(p + base + e0, pf);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) block_update_kernel(LaunchCommon c) {
    const Smem s = load_tables(c, true);
    const float gs = c.gscale ? *c.gscale : 1.0f;
    for (int tile = blockIdx.x; tile < c.total_tiles; tile += gridDim.x) {
        const int ti = find_tensor(c.tile_start, c.n_tensors, tile);
        const TensorDesc d = c.descs[ti];   // local copy: stores cannot force re-reads of it
        const long long local = tile - c.tile_start[ti];
        if (d.mode == 2) {
            if (d.vec) block_worker<T, 8, 2>(d, c, s, local, local < d.nb, gs);
            else block_worker<T, 1, 2>(d, c, s, local, local < d.nb, gs);
        } else if (d.mode == 1) {
            const long long blk = local * (kThreads / 32) + (threadIdx.x >> 5);
            if (d.vec) block_worker<T, 8, 1>(d, c, s, blk, blk < d.nb, gs);
            else block_worker<T, 1, 1>(d, c, s, blk, blk < d.nb, gs);
        } else {
            const long long blk = local * kThreads + threadIdx.x;
            block_worker<T, 1, 0>(d, c, s, blk, blk < d.nb, gs);
        }
    }
}

// ---------------------------------------------------------------------------
// factored path
// ---------------------------------------------------------------------------
__device__ __forceinline__ long long block_of(const Hot& d, int r, int c0) {
    switch (d.blk_mode) {
        case 0: return r;
        case 1: return (long long)r * (d.cols / d.period) + c0 / d.period;
        case 2: return r / (d.period / d.cols);
        default:
            if (d.small) return (long long)(((unsigned)r * (unsigned)d.cols + (unsigned)c0) / (unsigned)d.period);
            return ((long long)r * d.cols + c0) / d.period;
    }
}

struct TileCursor {
    int ti, ct;          // tensor, column tile
    int r0, r1;          // row range of the tile
};

// Running maximum of |m| for the block a thread (or, when every lane of a warp
// is in the same block, the warp) is currently inside.  It is flushed with one
// atomic when the block changes, so a block that spans many rows or tiles costs
// one atomic per warp instead of one per row.
struct RunMax {
    float* dst;        // mag_new of the tensor the run belongs to
    float* sum_dst;    // row-only tensors: per-block sum of g^2 (null otherwise)
    long long blk;     // -1: empty
    float val;
    float sum;         // per-lane partial of the block's sum of squares (row-only tensors)
    int uniform;
};

__device__ __forceinline__ void runmax_flush(RunMax& r) {
    if (r.uniform) {
        const float m = warp_max(r.val);
        if ((threadIdx.x & 31) == 0 && r.blk >= 0) atomic_max_nonneg(r.dst + r.blk, m);
        if (r.sum_dst) {
            const float t = warp_sum(r.sum);
            if ((threadIdx.x & 31) == 0 && r.blk >= 0) atomicAdd(r.sum_dst + r.blk, t);
        }
    } else if (r.blk >= 0) {
        atomic_max_nonneg(r.dst + r.blk, r.val);
    }
    r.blk = -1;
    r.val = 0.f;
    r.sum = 0.f;
}

// CTA-wide flush at a point every thread of the CTA reaches (end of a tensor or of the CTA's tile
// range): the warps' runs are merged in shared memory first, so that blocks spanning the whole
// range (a few huge blocks per tensor) cost one atomic per CTA instead of one per warp.
__device__ __forceinline__ void runmax_flush_cta(RunMax& r) {
    __shared__ long long sh_blk[kThreads / 32];
    __shared__ float sh_val[kThreads / 32], sh_sum[kThreads / 32];
    if (!r.uniform) {
        runmax_flush(r);
        return;
    }
    const float m = warp_max(r.val);
    const float t = r.sum_dst ? warp_sum(r.sum) : 0.f;
    const int w = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) { sh_blk[w] = r.blk; sh_val[w] = m; sh_sum[w] = t; }
    __syncthreads();
    if (threadIdx.x == 0) {
        long long cur = -1;
        float cv = 0.f, cs = 0.f;
        for (int i = 0; i <= kThreads / 32; ++i) {
            const long long b = i < kThreads / 32 ? sh_blk[i] : -2;
            if (b == cur && b >= 0) {
                cv = fmaxf(cv, sh_val[i]);
                cs += sh_sum[i];
                continue;
            }
            if (cur >= 0) {
                atomic_max_nonneg(r.dst + cur, cv);
                if (r.sum_dst) atomicAdd(r.sum_dst + cur, cs);
            }
            cur = b;
            if (b >= 0) { cv = sh_val[i]; cs = sh_sum[i]; }
        }
    }
    __syncthreads();
    r.blk = -1;
    r.val = 0.f;
    r.sum = 0.f;
}

template <typename T, int VEC, int U, bool FAST = false>
__device__ void stats_tile(const Hot& d, const Smem& s, const TileCursor& t, float gs,
                           float (&csum)[VEC], RunMax& run) {
    const int tx = threadIdx.x % d.tcols, ty = threadIdx.x / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * VEC;
    const bool act = c0 < d.cols;
    const bool uniform = run.uniform != 0;
    const bool multi = FAST ? false : d.n_src > 1;
    const T* g0 = reinterpret_cast<const T*>(d.g0);
    for (int rb = t.r0 + ty; rb < t.r1; rb += d.trows * U) {
        RawVec<T, VEC> rg[U];
        RawIdx<VEC> ri[U];
        if (!multi) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = rb + u * d.trows;
                if (act && r < t.r1) {
                    const long long off = (long long)r * d.cols + c0;
                    rg[u].load(g0 + off);
                    ri[u].load(d.idx + off);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = rb + u * d.trows;
            if (r >= t.r1) break;  // uniform across the warp: a warp shares ty
            float amax = 0.f, rs = 0.f;
            long long blk = -1;
            if (act) {
                float g[VEC];
                int ix[VEC];
                if (multi) {
                    const long long off = (long long)r * d.cols + c0;
                    load_grad<T, VEC>(d, off, gs, g);
                    load_index<VEC>(d.idx + off, ix);
                } else {
                    rg[u].get(g);
                    ri[u].get(ix);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) g[e] = __fmul_rn(g[e], gs);
                }
                blk = block_of(d, r, c0);
                const float mo = d.mag[blk];
#pragma unroll
                for (int e = 0; e < VEC; ++e) {
                    float m = ema_momentum(rep_load(s.cb, ix[e]), mo, g[e], d.beta1, d.omb1);
                    amax = fmaxf(amax, fabsf(m));
                    const float sq = g[e] * g[e];
                    rs += sq;
                    csum[e] += sq;
                }
            }
            if (!run.sum_dst) {
                rs = warp_sum(rs);
                if ((threadIdx.x & 31) == 0 && act) atomicAdd(d.row_sq + r, rs);
            }
            if (uniform) {
                const long long b0 = __shfl_sync(0xffffffffu, blk, 0);   // lane 0 has the lowest column
                if (b0 >= 0) {
                    if (b0 != run.blk) { runmax_flush(run); run.blk = b0; }
                    run.val = fmaxf(run.val, amax);
                    run.sum += rs;
                }
            } else if (act) {
                if (blk != run.blk) { runmax_flush(run); run.blk = blk; }
                run.val = fmaxf(run.val, amax);
                if (run.sum_dst) atomicAdd(run.sum_dst + blk, rs);
            }
        }
    }
}

template <int VEC>
__device__ __forceinline__ void flush_cols(const Hot& d, int ct, float (&csum)[VEC]) {
    const int tx = threadIdx.x % d.tcols;
    const int c0 = (ct * d.tcols + tx) * VEC;
    if (c0 < d.cols) {
        if constexpr (VEC == 8) {
            // col_sq is 16-byte aligned (the plan aligns every scratch array) and c0 % 8 == 0
            float4* dst = reinterpret_cast<float4*>(d.col_sq + c0);
            atomicAdd(dst, make_float4(csum[0], csum[1], csum[2], csum[3]));
            atomicAdd(dst + 1, make_float4(csum[4], csum[5], csum[6], csum[7]));
        } else {
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                if (csum[e] != 0.f) atomicAdd(d.col_sq + c0 + e, csum[e]);
            }
        }
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) csum[e] = 0.f;
}

__device__ __forceinline__ bool warp_uniform_blocks(const Hot& d, int vec) {
    if (d.blk_mode == 0 || d.blk_mode == 2) return true;
    if (d.blk_mode == 1) return (d.period % (32 * vec)) == 0;
    return false;
}

// Walks the contiguous tile range of a CTA.  The descriptor of the current tensor is
// held in a local copy (so that stores and atomics cannot force it to be re-read)
// and the (tensor, column tile, row tile) position advances incrementally; only
// the first tile of the range needs the binary search.
struct TileWalk {
    int ti, ct, rt, n_row_tiles;
};

__device__ __forceinline__ void walk_begin(const LaunchCommon& c, long long tile, TileWalk& w, Hot& d) {
    w.ti = find_tensor(c.tile_start, c.n_tensors, (int)tile);
    d = load_hot(c.descs + w.ti);
    const int local = (int)tile - c.tile_start[w.ti];
    w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
    w.ct = local / w.n_row_tiles;
    w.rt = local - w.ct * w.n_row_tiles;
}

// Cursor over `n` consecutive row tiles of the current column tile (one long row range: the
// pipelined loops then fill and drain once per range instead of once per tile).
__device__ __forceinline__ TileCursor walk_cursor(const TileWalk& w, const Hot& d, int n = 1) {
    TileCursor t;
    t.ti = w.ti;
    t.ct = w.ct;
    t.r0 = w.rt * d.rows_per_tile;
    t.r1 = (int)min((long long)d.rows, (long long)t.r0 + (long long)n * d.rows_per_tile);
    return t;
}


// ---------------------------------------------------------------------------
// fast tile loops (every tensor of the plan: 8-wide chunks, one gradient source, fewer
// than 2^31 elements, nearest rounding)
// ---------------------------------------------------------------------------
// A thread walks the rows of its column chunk with a register ring of raw (unconverted)
// chunks: the loads of the rows ahead are in flight while the current row is computed, and
// the loop body is one chunk of eight elements, small enough to stay in the instruction
// cache.  The block of a chunk advances incrementally (no division per row).
struct BlockIter {
    unsigned off;      // element offset of the chunk the iterator points at
    int blk;           // its block
    unsigned rem;      // off - blk * period
};

__device__ __forceinline__ BlockIter block_iter(const Hot& d, int r, int c0) {
    BlockIter it;
    it.off = (unsigned)r * (unsigned)d.cols + (unsigned)c0;
    it.blk = (int)(it.off / (unsigned)d.period);
    it.rem = it.off - (unsigned)it.blk * (unsigned)d.period;
    return it;
}
__device__ __forceinline__ void block_iter_next(const Hot& d, BlockIter& it) {
    it.off += (unsigned)d.trows * (unsigned)d.cols;
    it.blk += (int)d.step_blk;
    it.rem += d.step_rem;
    if (it.rem >= (unsigned)d.period) { it.rem -= (unsigned)d.period; ++it.blk; }
}

template <typename T> struct StatsChunk {
    RawVec<T, 8> g;
    RawIdx<8> i;
    float mo;          // old magnitude of the chunk's block (fetched with the chunk)
    int blk;
};

constexpr int kFastCtas = 3;     // resident CTAs per SM of the fast kernels
constexpr int kApplyAhead = 1;

// MC: the gradient source is an NVLS multicast address; every chunk is read with one
// multimem.ld_reduce (sum over all ranks inside NVSwitch) and scaled to the mean, as stored
template <typename T, int kStatsAhead, bool MC>
__device__ __forceinline__ void stats_tile_fast(const Hot& d, const Smem& s, const TileCursor& t, float gs,
                                float (&csum)[8], RunMax& run) {
    const int tx = threadIdx.x % d.tcols, ty = threadIdx.x / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * 8;
    const bool act = c0 < d.cols;
    const T* g0 = reinterpret_cast<const T*>(d.g0);
    const int stride = d.trows;
    int r = t.r0 + ty;
    BlockIter it = block_iter(d, r, act ? c0 : 0);
    int rf = r;                                   // row of the next fetch
    StatsChunk<T> q[kStatsAhead + 1];
    auto fetch = [&](StatsChunk<T>& c) {
        if (act && rf < t.r1) {
            if constexpr (MC) c.g.load_mc(g0 + it.off); else c.g.load(g0 + it.off);
            c.i.load(d.idx + it.off);
            c.mo = d.mag[it.blk];
            c.blk = it.blk;
        } else {
            c.blk = -1;
        }
        block_iter_next(d, it);
        rf += stride;
    };
#pragma unroll
    for (int k = 0; k < kStatsAhead; ++k) fetch(q[k]);
#pragma unroll 1
    for (; r < t.r1; r += stride) {
        fetch(q[kStatsAhead]);
        float amax = 0.f, rs = 0.f;
        const int blk = q[0].blk;
        if (act) {
            float g[8];
            int ix[8];
            q[0].g.get(g);
            q[0].i.get(ix);
            const float mo = q[0].mo;
            if constexpr (MC) {
#pragma unroll
                for (int e = 0; e < 8; ++e) g[e] = round_to<T>(__fmul_rn(g[e], d.src_scale));
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float ge = __fmul_rn(g[e], gs);
                const float m = ema_momentum(rep_load(s.cb, ix[e]), mo, ge, d.beta1, d.omb1);
                amax = fmaxf(amax, fabsf(m));
                const float sq = ge * ge;
                rs += sq;
                csum[e] += sq;
            }
        }
        const float rs_lane = rs;
        if (!run.sum_dst) {
            rs = warp_sum(rs);
            if ((threadIdx.x & 31) == 0 && act) atomicAdd(d.row_sq + r, rs);
        }
        // Blocks are contiguous in memory, so the warp's 256 columns of this row lie in one block
        // iff its first and its last active lane do (checked every row: with a period that is not
        // a multiple of the row length only the few rows a block boundary crosses differ).  The
        // warp then shares one running maximum; on a boundary row every lane posts its own value.
        const unsigned live = __ballot_sync(0xffffffffu, act);
        if (live) {
            const int b0 = __shfl_sync(0xffffffffu, blk, 0);               // lane 0 has the lowest column
            const int b1 = __shfl_sync(0xffffffffu, blk, 31 - __clz((int)live));
            if (b0 == b1) {
                if ((long long)b0 != run.blk) { runmax_flush(run); run.blk = b0; }
                run.val = fmaxf(run.val, amax);
                run.sum += rs_lane;   // only read when sum_dst is set
            } else if (act) {
                atomic_max_nonneg(run.dst + blk, amax);
                if (run.sum_dst) atomicAdd(run.sum_dst + blk, rs_lane);
            }
        }
#pragma unroll
        for (int k = 0; k < kStatsAhead; ++k) q[k] = q[k + 1];
    }
}

template <typename T> struct ApplyChunk {
    RawVec<T, 8> g, p;
    RawIdx<8> i;
    int blk;
};

// element e (dynamic) of a raw chunk; only the rare fix-up loop uses it
template <typename T>
__device__ __forceinline__ float raw_elem(const RawVec<T, 8>& v, int e) {
    if constexpr (sizeof(T) == 4) {
        uint32_t w = v.w[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) w = (e == k) ? v.w[k] : w;
        return __uint_as_float(w);
    } else {
        uint32_t w = v.w[0];
#pragma unroll
        for (int k = 1; k < 4; ++k) w = ((e >> 1) == k) ? v.w[k] : w;
        const unsigned short h = (unsigned short)((e & 1) ? (w >> 16) : (w & 0xffffu));
        T x;
        *reinterpret_cast<unsigned short*>(&x) = h;
        return to_f<T>(x);
    }
}

// MODE 0: parameter update; 2: momentum emit; 3: emit with the Nesterov look-ahead
template <typename T, int MODE, bool MC = false>
__device__ __forceinline__ void apply_tile_fast(const Hot& d, const Smem& s, const TileCursor& t, float gs,
                                const float (&cf)[8]) {
    const int tx = threadIdx.x % d.tcols, ty = threadIdx.x / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * 8;
    if (c0 >= d.cols) return;
    constexpr bool emit = MODE >= 2;
    const float lr = emit ? 0.f : d.scal[0], inv_bc1 = emit ? 0.f : d.scal[2], wdf = emit ? 1.f : d.scal[3];
    const float b1 = d.beta1, omb1 = d.omb1, eps = d.eps;
    T* p = reinterpret_cast<T*>(d.p);
    const T* g0 = reinterpret_cast<const T*>(d.g0);
    const int stride = d.trows;
    int r = t.r0 + ty;
    BlockIter it = block_iter(d, r, c0);
    int rfetch = r;
    ApplyChunk<T> q0, q1;
    auto fetch = [&](ApplyChunk<T>& c) {
        if (rfetch < t.r1) {
            if constexpr (MC) c.g.load_mc(g0 + it.off); else c.g.load(g0 + it.off);
            c.i.load(d.idx + it.off);
            if (!emit) c.p.load(p + it.off);
            c.blk = it.blk;
        }
        block_iter_next(d, it);
        rfetch += stride;
    };
    unsigned off = it.off;                         // offset of the chunk being computed
    const unsigned off_step = (unsigned)stride * (unsigned)d.cols;
    static_assert(kApplyAhead == 1, "the register ring below holds one chunk ahead");
    fetch(q0);
#pragma unroll 1
    for (; r < t.r1; r += stride) {
        fetch(q1);
        const ApplyChunk<T> c = q0;
        const float mo = d.mag[c.blk], mn = d.mag_new[c.blk];
        const float rf = emit ? 0.f : d.rfac[d.row_only ? c.blk : r];
        const float inv = mn > 0.f ? __frcp_rn(mn) : 0.f;
        float g[8], pf[8];
        int ix[8];
        c.g.get(g);
        c.i.get(ix);
        if (!emit) c.p.get(pf);
        if constexpr (MC) {
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] = round_to<T>(__fmul_rn(g[e], d.src_scale));
        }
        uint32_t many = 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float ge = __fmul_rn(g[e], gs);
            const float m = ema_momentum(rep_load(s.cb, ix[e]), mo, ge, b1, omb1);
            const float v = __fmul_rn(m, inv);
            const uint32_t en = s.q.lut[lut_bucket(v)];
            const int lo = (int)(en & 0xffu);
            const uint32_t cnt = en >> 8;
            many |= cnt;
            // thr[lo] is the first threshold not in a lower bucket: when this bucket holds none it
            // lies in a higher bucket and cannot be below v (the bucket function is monotonic)
            const int k = lo + ((s.q.thr[lo] < v) ? 1 : 0);
            ix[e] = k;
            const float qv = __fmul_rn(rep_load(s.cb, k), mn);
            if (emit) {
                pf[e] = (MODE == 3) ? __fadd_rn(__fmul_rn(qv, b1), __fmul_rn(ge, omb1)) : qv;
            } else {
                const float h = __fadd_rn(__fmul_rn(rf, cf[e]), eps);
                const float step = __fdividef(inv_bc1, h);
                pf[e] = apply_one<T>(pf[e], qv, step, lr, wdf);
            }
        }
        store_index<8>(d.idx + off, ix);
        store_param<T, 8>(p + off, pf);
        if (many > 1u) {
            // some bucket of this chunk holds more than one threshold: redo those elements with
            // the full search (rare: the buckets are far narrower than the codeword spacing)
#pragma unroll 1
            for (int e = 0; e < 8; ++e) {
                float graw = raw_elem<T>(c.g, e);
                if constexpr (MC) graw = round_to<T>(__fmul_rn(graw, d.src_scale));
                const float ge = __fmul_rn(graw, gs);
                const int i0 = (int)(((e < 4 ? c.i.w[0] : c.i.w[1]) >> (8 * (e & 3))) & 0xffu);
                const float m = ema_momentum(rep_load(s.cb, i0), mo, ge, b1, omb1);
                const float v = __fmul_rn(m, inv);
                if ((s.q.lut[lut_bucket(v)] >> 8) <= 1u) continue;
                const int k = nearest_index(v, s.q);
                const float qv = __fmul_rn(rep_load(s.cb, k), mn);
                float o;
                if (emit) {
                    o = (MODE == 3) ? __fadd_rn(__fmul_rn(qv, b1), __fmul_rn(ge, omb1)) : qv;
                } else {
                    float cfe = cf[0];
#pragma unroll
                    for (int k2 = 1; k2 < 8; ++k2) cfe = (e == k2) ? cf[k2] : cfe;
                    const float h = __fadd_rn(__fmul_rn(rf, cfe), eps);
                    o = apply_one<T>(raw_elem<T>(c.p, e), qv, __fdividef(inv_bc1, h), lr, wdf);
                }
                d.idx[off + e] = (uint8_t)k;
                p[off + e] = from_f<T>(o);
            }
        }
        q0 = q1;
        off += off_step;
    }
}

// FAST: every tensor of the plan takes the 8-wide single-source path (checked on the host),
// so the scalar and multi-source code is not even instantiated: smaller code, fewer registers.
// AHEAD: rows a thread keeps in flight beyond the current one (fast loops only)
template <typename T, bool FAST, int AHEAD = 2, bool MC = false>
__global__ void __launch_bounds__(kThreads, FAST ? kFastCtas : 2) factored_stats_kernel(LaunchCommon c) {
    const Smem s = load_tables(c, false);
    const float gs = c.gscale ? *c.gscale : 1.0f;
    const long long T0 = (long long)c.total_tiles * blockIdx.x / gridDim.x;
    const long long T1 = (long long)c.total_tiles * (blockIdx.x + 1) / gridDim.x;
    if (T0 >= T1) return;
    float csum8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float csum1[1] = {0};
    RunMax run{nullptr, nullptr, -1, 0.f, 0.f, 0};
    Hot d;
    TileWalk w;
    walk_begin(c, T0, w, d);
    run.dst = d.mag_new;
    run.sum_dst = d.row_only ? d.row_sq : nullptr;
    run.uniform = (FAST || warp_uniform_blocks(d, d.vec ? 8 : 1)) ? 1 : 0;
    for (long long tile = T0; tile < T1;) {
        const int n = (int)min(T1 - tile, (long long)(w.n_row_tiles - w.rt));
        const TileCursor t = walk_cursor(w, d, n);
        if constexpr (FAST) {
            stats_tile_fast<T, AHEAD, MC>(d, s, t, gs, csum8, run);
        } else if (d.vec) {
            if (d.n_src > 1) stats_tile<T, 8, 1>(d, s, t, gs, csum8, run);
            else stats_tile<T, 8, 8>(d, s, t, gs, csum8, run);
        } else {
            stats_tile<T, 1, 4>(d, s, t, gs, csum1, run);
        }
        tile += n;
        w.rt += n;
        // advance; flush the column partials when the column tile (or the tensor) changes
        bool col_change = false, tensor_change = false;
        if (w.rt == w.n_row_tiles) {
            w.rt = 0;
            col_change = true;
            if (++w.ct == d.n_col_tiles) { w.ct = 0; tensor_change = true; }
        }
        const bool last = tile == T1;
        if (col_change || last) {
            if (!d.row_only) {
                const int ct_done = col_change ? (tensor_change ? d.n_col_tiles - 1 : w.ct - 1) : w.ct;
                if (d.vec) flush_cols<8>(d, ct_done, csum8); else flush_cols<1>(d, ct_done, csum1);
            }
        }
        if (tensor_change || last) runmax_flush_cta(run);
        if (tensor_change && !last) {
            ++w.ti;
            d = load_hot(c.descs + w.ti);
            w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
            run.dst = d.mag_new;
            run.sum_dst = d.row_only ? d.row_sq : nullptr;
            run.uniform = (FAST || warp_uniform_blocks(d, d.vec ? 8 : 1)) ? 1 : 0;
        }
    }
}

// One CTA (1024 threads) per tensor.
constexpr int kEmaThreads = 1024;

__device__ __forceinline__ float cta_sum_1024(float v, float* red) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kEmaThreads / 32; ++i) t += red[i];
    return t;
}

__global__ void __launch_bounds__(kEmaThreads) factored_ema_kernel(LaunchCommon c) {
    __shared__ float red[kEmaThreads / 32];
    __shared__ int ok_s;
    const int ti = blockIdx.x;
    if (ti >= c.n_tensors) return;
    const TensorDesc& d = c.descs[ti];
    const float inv_cols = 1.0f / (float)d.cols;
    const float inv_rows = 1.0f / (float)d.total_rows;
    const float inv_bc2 = d.scal[1];
    if (d.row_only >= 2) {
        // momentum-emit tensors keep no second moment: only clear the statistics scratch
        for (long long i = threadIdx.x; i < d.nb; i += kEmaThreads) d.row_sq[i] = 0.f;
        return;
    }
    if (d.row_only) {
        // block path seen as a matrix whose rows tile the blocks: one second-moment value per
        // block (the row statistics are accumulated per block), no column factor
        const float inv_period = 1.0f / (float)d.period;
        for (long long i = threadIdx.x; i < d.nb; i += kEmaThreads) {
            const float ms = __fmul_rn(d.row_sq[i], inv_period);
            const float v = __fadd_rn(__fmul_rn(d.v0[i], d.beta2), __fmul_rn(ms, d.omb2));
            d.v0[i] = v;
            d.row_sq[i] = 0.f;
            d.rfac[i] = __fmul_rn(__fsqrt_rn(v), inv_bc2);   // scal[1] is 1/sqrt(bc2) here
        }
        return;
    }
    // rows: EMA and the sum of the new v_row (fixed order: strided per thread, tree per CTA)
    float part = 0.f;
    for (int i = threadIdx.x; i < d.rows; i += kEmaThreads) {
        const float ms = __fmul_rn(d.row_sq[i], inv_cols);
        const float v = __fadd_rn(__fmul_rn(d.v0[i], d.beta2), __fmul_rn(ms, d.omb2));
        d.v0[i] = v;
        d.row_sq[i] = 0.f;
        part += v;
    }
    float sum_v = cta_sum_1024(part, red);
    bool exchanged = false;
    const long long xo = (long long)(c.epoch & 1u) * (d.cols + 1);  // slot parity of this step
    if (d.world > 1) {
        // publish this shard's column partials and sum(v_row), then wait for every peer
        for (int j = threadIdx.x; j < d.cols; j += kEmaThreads) d.xchg_local[xo + j] = d.col_sq[j];
        if (threadIdx.x == 0) d.xchg_local[xo + d.cols] = sum_v;
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x < d.world) st_release_sys(d.flag_peer[threadIdx.x] + d.rank, c.epoch);
        if (threadIdx.x == 0) ok_s = 1;
        __syncthreads();
        if (threadIdx.x < d.world) {
            if (!wait_flag_ge(d.flag_local + threadIdx.x, c.epoch, c.wait_iters)) {
                ok_s = 0;
                if (c.status) atomicExch(c.status, (int)kWaitTimeout);
            }
        }
        __syncthreads();
        exchanged = ok_s != 0;
        if (exchanged) {
            float t = 0.f;
            for (int r = 0; r < d.world; ++r) t += d.xchg_peer[r][xo + d.cols];
            sum_v = t;
        }
    }
    const float mean = fmaxf(__fmul_rn(sum_v, inv_rows), 1.17549435e-38f);
    const float inv_mean = __frcp_rn(mean);
    for (int i = threadIdx.x; i < d.rows; i += kEmaThreads)
        d.rfac[i] = __fsqrt_rn(__fmul_rn(__fmul_rn(d.v0[i], inv_mean), inv_bc2));
    for (int j = threadIdx.x; j < d.cols; j += kEmaThreads) {
        float cs;
        if (exchanged) {
            cs = 0.f;
            for (int r = 0; r < d.world; ++r) cs += d.xchg_peer[r][xo + j];
        } else {
            cs = d.col_sq[j];
        }
        const float ms = __fmul_rn(cs, inv_rows);
        const float v = __fadd_rn(__fmul_rn(d.v1[j], d.beta2), __fmul_rn(ms, d.omb2));
        d.v1[j] = v;
        d.col_sq[j] = 0.f;
        d.cfac[j] = __fsqrt_rn(v);
    }
}

template <typename T, int VEC, int U, bool FAST = false>
__device__ void apply_tile(const Hot& d, const LaunchCommon& c, const Smem& s,
                           const TileCursor& t, float gs, const float (&cf)[VEC]) {
    const int tx = threadIdx.x % d.tcols, ty = threadIdx.x / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * VEC;
    if (c0 >= d.cols) return;
    // emit mode (Muon momentum): no parameter update, d.p receives the dense new momentum
    // (row_only == 3: with the Nesterov look-ahead beta * m + (1 - beta) * g)
    const bool emit = d.row_only >= 2;
    const float lr = emit ? 0.f : d.scal[0], inv_bc1 = emit ? 0.f : d.scal[2], wdf = emit ? 1.f : d.scal[3];
    const bool multi = FAST ? false : d.n_src > 1;
    T* p = reinterpret_cast<T*>(d.p);
    const T* g0 = reinterpret_cast<const T*>(d.g0);
    for (int rb = t.r0 + ty; rb < t.r1; rb += d.trows * U) {
        RawVec<T, VEC> rg[U], rp[U];
        RawIdx<VEC> ri[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = rb + u * d.trows;
            if (r < t.r1) {
                const long long off = (long long)r * d.cols + c0;
                if (!multi) rg[u].load(g0 + off);
                ri[u].load(d.idx + off);
                if (!emit) rp[u].load(p + off);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int r = rb + u * d.trows;
            if (r >= t.r1) break;
            const long long off = (long long)r * d.cols + c0;
            float g[VEC], pf[VEC];
            int ix[VEC];
            if (multi) {
                load_grad<T, VEC>(d, off, gs, g);
            } else {
                rg[u].get(g);
#pragma unroll
                for (int e = 0; e < VEC; ++e) g[e] = __fmul_rn(g[e], gs);
            }
            ri[u].get(ix);
            if (!emit) rp[u].get(pf);
            const long long blk = block_of(d, r, c0);
            const float mo = d.mag[blk], mn = d.mag_new[blk];
            const float inv = mn > 0.f ? __frcp_rn(mn) : 0.f;
            const float rf = emit ? 0.f : d.rfac[d.row_only ? blk : (long long)r];
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                float m = ema_momentum(rep_load(s.cb, ix[e]), mo, g[e], d.beta1, d.omb1);
                int k = quantise<FAST>(__fmul_rn(m, inv), s, c, off + e);
                ix[e] = k;
                const float q = __fmul_rn(rep_load(s.cb, k), mn);
                if (emit) {
                    pf[e] = (d.row_only == 3) ? __fadd_rn(__fmul_rn(q, d.beta1), __fmul_rn(g[e], d.omb1)) : q;
                } else {
                    const float h = __fadd_rn(__fmul_rn(rf, cf[e]), d.eps);
                    const float step = __fdividef(inv_bc1, h);
                    pf[e] = apply_one<T>(pf[e], q, step, lr, wdf);
                }
            }
            store_index<VEC>(d.idx + off, ix);
            store_param<T, VEC>(p + off, pf);
        }
    }
}

template <int VEC>
__device__ __forceinline__ void load_cfac(const Hot& d, int ct, float (&cf)[VEC]) {
    const int tx = threadIdx.x % d.tcols;
    const int c0 = (ct * d.tcols + tx) * VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) cf[e] = d.row_only ? 1.0f : ((c0 + e < d.cols) ? d.cfac[c0 + e] : 0.f);
}

template <typename T, bool FAST, bool MC = false>
__global__ void __launch_bounds__(kThreads, FAST ? kFastCtas : 2) factored_apply_kernel(LaunchCommon c) {
    const Smem s = load_tables(c, true);
    const float gs = c.gscale ? *c.gscale : 1.0f;
    const long long T0 = (long long)c.total_tiles * blockIdx.x / gridDim.x;
    const long long T1 = (long long)c.total_tiles * (blockIdx.x + 1) / gridDim.x;
    if (T0 >= T1) return;
    float cf8[8], cf1[1];
    Hot d;
    TileWalk w;
    walk_begin(c, T0, w, d);
    bool reload = true;
    for (long long tile = T0; tile < T1;) {
        if (reload) {
            if (d.vec) load_cfac<8>(d, w.ct, cf8); else load_cfac<1>(d, w.ct, cf1);
            reload = false;
        }
        const int n = (int)min(T1 - tile, (long long)(w.n_row_tiles - w.rt));
        const TileCursor t = walk_cursor(w, d, n);
        if constexpr (FAST) {
            if (d.row_only < 2) apply_tile_fast<T, 0, MC>(d, s, t, gs, cf8);
            else if (d.row_only == 2) apply_tile_fast<T, 2>(d, s, t, gs, cf8);
            else apply_tile_fast<T, 3>(d, s, t, gs, cf8);
        } else if (d.vec) {
            if (d.n_src > 1) apply_tile<T, 8, 1>(d, c, s, t, gs, cf8);
            else apply_tile<T, 8, 4>(d, c, s, t, gs, cf8);
        } else {
            apply_tile<T, 1, 2>(d, c, s, t, gs, cf1);
        }
        tile += n;
        w.rt += n;
        if (w.rt == w.n_row_tiles) {
            w.rt = 0;
            reload = true;
            if (++w.ct == d.n_col_tiles) {
                w.ct = 0;
                if (tile < T1) {
                    ++w.ti;
                    d = load_hot(c.descs + w.ti);
                    w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// streamed kernels (fast plans of 2-byte tensors with 16-element row alignment)
// ---------------------------------------------------------------------------
// A CTA holds G consumer groups of kThreads threads and one producer warp per group.  A group
// behaves like one CTA of the fast kernels above (contiguous tile range, a thread owns a column
// chunk and walks its rows), but its chunks arrive through a ring of shared-memory stages.  One
// stage is one row step of the group: trows rows of tcols * W elements, stored so that the chunk of
// group thread t lies at element t * W.  The producer warp walks the same tile range and copies one
// row per lane with cp.async.bulk; the copies complete the stage's "full" mbarrier by byte count,
// the eight consumer warps release the stage through its "empty" mbarrier.  Every wait is bounded:
// a wait that runs out raises the CTA's abort flag and the status word, after which no thread waits
// or computes again but all still walk their ranges, so that the group barriers stay matched.
//
// Two widths.  W = 8: three groups per CTA, the tile geometry, thread-to-chunk mapping, arithmetic
// and summation order of the register-pipelined kernels (bit-identical results).  W = 16 (plans whose
// block periods are multiples of 16, so that a 16-element chunk lies in one block): two groups per
// CTA at up to 112 registers, a thread owns 16 contiguous elements of a row, which halves what a row
// step costs besides its elements (stage wait / release, block bookkeeping, magnitude and row-factor
// fetches, the row-sum shuffle tree, the per-row agreement on the block).  Its tile geometry is
// derived on the device from the 8-wide one (same rule as the host's) and its tile prefix follows
// the 8-wide prefix in the plan's tile table.
template <int W> struct StreamCfg {
    static constexpr int kW = W;
    static constexpr int kG = (W == 8) ? 3 : 2;                       // consumer groups per CTA
    static constexpr int kCtaThreads = kG * (kThreads + 32);
    static constexpr int kStatsStages = (W == 8) ? 8 : 5;
    static constexpr int kApplyStages = (W == 8) ? 5 : 3;
    static constexpr int kValBytes = kThreads * W * 2;                // g (or p) of one row step
    static constexpr int kIdxBytes = kThreads * W;
    static constexpr int kStatsStageBytes = kValBytes + kIdxBytes;
    static constexpr int kApplyStageBytes = 2 * kValBytes + kIdxBytes;
};
constexpr int kMaxGroups = 3;
// tables of the streamed kernels: the lane-replicated codebook with one more row of +inf (the
// "next codeword" of the last one), then the thresholds and the bucket table
constexpr int kRepFloatsS = (kCodewords + 1) * 32;
constexpr size_t kTabStats = ((size_t)(16 + kRepFloatsS) * sizeof(float) + 127) / 128 * 128;
constexpr size_t kTabFull = (kTabStats + kCodewords * sizeof(float) + kLutBuckets * sizeof(uint16_t) + 127) / 128 * 128;
template <int W> constexpr size_t smem_stats_stream() {
    return kTabStats + (size_t)StreamCfg<W>::kG * StreamCfg<W>::kStatsStages * StreamCfg<W>::kStatsStageBytes;
}
template <int W> constexpr size_t smem_apply_stream() {
    return kTabFull + (size_t)StreamCfg<W>::kG * StreamCfg<W>::kApplyStages * StreamCfg<W>::kApplyStageBytes;
}
static_assert(smem_apply_stream<8>() <= 232448 && smem_stats_stream<8>() <= 232448 &&
              smem_apply_stream<16>() <= 232448 && smem_stats_stream<16>() <= 232448,
              "shared memory of the streamed kernels");

struct StreamShared {
    uint64_t full[kMaxGroups][8];
    uint64_t empty[kMaxGroups][8];
    long long blk[kMaxGroups][kThreads / 32];
    float val[kMaxGroups][kThreads / 32];
    float sum[kMaxGroups][kThreads / 32];
    int abort_flag;
};

template <int D, int STAGE_BYTES>
struct Ring {
    uint64_t* full;
    uint64_t* empty;
    unsigned char* base;
    volatile int* abort_flag;
    int slot;
    uint32_t phase;
    __device__ __forceinline__ unsigned char* stage() const { return base + slot * STAGE_BYTES; }
    __device__ __forceinline__ void advance() {
        if (++slot == D) { slot = 0; phase ^= 1u; }
    }
};

__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kThreads) : "memory");
}

// runmax_flush_cta for one consumer group (its own named barrier and merge slots)
__device__ __forceinline__ void runmax_flush_group(RunMax& r, StreamShared& sh, int group, int lt) {
    const float m = warp_max(r.val);
    const float t = r.sum_dst ? warp_sum(r.sum) : 0.f;
    const int w = lt >> 5;
    if ((lt & 31) == 0) { sh.blk[group][w] = r.blk; sh.val[group][w] = m; sh.sum[group][w] = t; }
    group_barrier(group);
    if (lt == 0) {
        long long cur = -1;
        float cv = 0.f, cs = 0.f;
        for (int i = 0; i <= kThreads / 32; ++i) {
            const long long b = i < kThreads / 32 ? sh.blk[group][i] : -2;
            if (b == cur && b >= 0) {
                cv = fmaxf(cv, sh.val[group][i]);
                cs += sh.sum[group][i];
                continue;
            }
            if (cur >= 0) {
                atomic_max_nonneg(r.dst + cur, cv);
                if (r.sum_dst) atomicAdd(r.sum_dst + cur, cs);
            }
            cur = b;
            if (b >= 0) { cv = sh.val[group][i]; cs = sh.sum[group][i]; }
        }
    }
    group_barrier(group);
    r.blk = -1;
    r.val = 0.f;
    r.sum = 0.f;
}

__device__ __forceinline__ void bulk_load_row(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(ptx::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(ptx::smem_u32(bar))
                 : "memory");
}

// Tile geometry of the 16-wide kernels, derived from the 8-wide fields of the descriptor with the rule
// the host uses for its tile prefix (ops/update.py: _pick_tcols): the thread columns that waste the
// fewest chunks of the last column tile, the same rows-per-thread factor as the 8-wide tiles.
__device__ __forceinline__ void widen_geometry(Hot& h) {
    const int tile_k = h.rows_per_tile / h.trows;
    const int chunks = h.cols / 16;
    int best = 256, waste = (chunks + 255) / 256 * 256 - chunks;
#pragma unroll
    for (int t = 128; t >= 32; t >>= 1) {
        const int w = (chunks + t - 1) / t * t - chunks;
        if (w < waste) { best = t; waste = w; }
    }
    h.tcols = best;
    h.trows = kThreads / best;
    h.n_col_tiles = (chunks + best - 1) / best;
    h.rows_per_tile = h.trows * tile_k;
    const unsigned long long step = (unsigned long long)h.trows * (unsigned)h.cols;
    h.step_blk = (unsigned)(step / (unsigned)h.period);
    h.step_rem = (unsigned)(step % (unsigned)h.period);
}
template <int W>
__device__ __forceinline__ Hot load_hot_w(const TensorDesc* t) {
    Hot h = load_hot(t);
    if constexpr (W == 16) widen_geometry(h);
    return h;
}
template <int W>
__device__ __forceinline__ const int* tile_prefix(const LaunchCommon& c) {
    return (W == 16) ? c.tile_start + (c.n_tensors + 1) : c.tile_start;
}
template <int W>
__device__ __forceinline__ void walk_begin_w(const LaunchCommon& c, long long tile, TileWalk& w, Hot& d) {
    const int* start = tile_prefix<W>(c);
    w.ti = find_tensor(start, c.n_tensors, (int)tile);
    d = load_hot_w<W>(c.descs + w.ti);
    const int local = (int)tile - start[w.ti];
    w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
    w.ct = local / w.n_row_tiles;
    w.rt = local - w.ct * w.n_row_tiles;
}

// The producer warp of a group: walks tiles [T0, T1) exactly as the consumers do and fills one
// stage per row step.  APPLY also brings the parameter rows.
template <typename T, int W, int D, int STAGE_BYTES, bool APPLY>
__device__ void stream_producer(const LaunchCommon& c, long long T0, long long T1, Ring<D, STAGE_BYTES>& ring) {
    static_assert(sizeof(T) == 2, "the streamed kernels take 2-byte tensors");
    using Cfg = StreamCfg<W>;
    const int lane = threadIdx.x & 31;
    Hot d;
    TileWalk w;
    walk_begin_w<W>(c, T0, w, d);
    for (long long tile = T0; tile < T1;) {
        const int n = (int)min(T1 - tile, (long long)(w.n_row_tiles - w.rt));
        const TileCursor t = walk_cursor(w, d, n);
        const int col0 = t.ct * d.tcols * W;
        const int width = min(d.tcols * W, d.cols - col0);          // elements of a row inside this column tile
        const char* g0 = reinterpret_cast<const char*>(d.g0);
        const char* p0 = reinterpret_cast<const char*>(d.p);
        const char* i0 = reinterpret_cast<const char*>(d.idx);
        for (int rb = t.r0; rb < t.r1; rb += d.trows) {
            const int nrows = min(d.trows, t.r1 - rb);
            if (!ptx::mbar_wait_relaxed(ring.empty + ring.slot, ring.phase ^ 1u, ring.abort_flag, 200u)) {
                if (lane == 0 && c.status) atomicExch(c.status, (int)kWaitTimeout);
                return;
            }
            if (lane == 0) ptx::mbar_expect_tx(ring.full + ring.slot, (uint32_t)(nrows * width * (APPLY ? 5 : 3)));
            __syncwarp();
            if (lane < nrows) {
                const size_t off = (size_t)(rb + lane) * (size_t)d.cols + (size_t)col0;
                unsigned char* st = ring.stage();
                uint64_t* bar = ring.full + ring.slot;
                bulk_load_row(st + lane * d.tcols * (W * 2), g0 + off * 2, (uint32_t)width * 2u, bar);
                if constexpr (APPLY) {
                    bulk_load_row(st + Cfg::kValBytes + lane * d.tcols * (W * 2), p0 + off * 2, (uint32_t)width * 2u, bar);
                    bulk_load_row(st + 2 * Cfg::kValBytes + lane * d.tcols * W, i0 + off, (uint32_t)width, bar);
                } else {
                    bulk_load_row(st + Cfg::kValBytes + lane * d.tcols * W, i0 + off, (uint32_t)width, bar);
                }
            }
            ring.advance();
        }
        tile += n;
        w.rt += n;
        if (w.rt == w.n_row_tiles) {
            w.rt = 0;
            if (++w.ct == d.n_col_tiles) {
                w.ct = 0;
                if (tile < T1) {
                    ++w.ti;
                    d = load_hot_w<W>(c.descs + w.ti);
                    w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
                }
            }
        }
    }
}

// consumer side of one stage: wait for it; release it once this warp has read what it needs
template <int D, int STAGE_BYTES>
__device__ __forceinline__ bool stage_wait(Ring<D, STAGE_BYTES>& ring) {
    return ptx::mbar_wait(ring.full + ring.slot, ring.phase, ring.abort_flag);
}
template <int D, int STAGE_BYTES>
__device__ __forceinline__ void stage_release(Ring<D, STAGE_BYTES>& ring, bool ok, int lt) {
    __syncwarp();
    if (ok && (lt & 31) == 0) ptx::mbar_arrive(ring.empty + ring.slot);
    ring.advance();
}

// Shared-memory addresses of the tables as 32-bit shared-window addresses, so that a lookup is
// one address instruction and one load: `cb_lane` points at this lane's copy of codeword 0 (the
// copies of codeword i lie 128 bytes apart), `lut2` is the bucket table's address minus twice the
// bit pattern of 2^23 (the bucket arrives as the low mantissa bits of 2^23 + bucket).
struct StreamTables {
    uint32_t cb_lane;
    uint32_t lut2;
};

__device__ __forceinline__ StreamTables load_tables_stream(const LaunchCommon& c, bool full) {
    float* base = reinterpret_cast<float*>(gx_smem_raw);
    float* cb = base + 16;
    float* thr = cb + kRepFloatsS;
    uint16_t* lut = reinterpret_cast<uint16_t*>(thr + kCodewords);
    for (int i = threadIdx.x; i <= kCodewords; i += blockDim.x) {
        const float v = i < kCodewords ? c.codebook[i] : __int_as_float(0x7f800000);
        float4* row = reinterpret_cast<float4*>(cb + i * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) row[k] = make_float4(v, v, v, v);
    }
    if (full) {
        const uint4* src = reinterpret_cast<const uint4*>(c.lut);
        uint4* dst = reinterpret_cast<uint4*>(lut);
        constexpr int kPieces = kLutBuckets * (int)sizeof(uint16_t) / 16;
        for (int i = threadIdx.x; i < kPieces; i += blockDim.x) dst[i] = src[i];
    }
    StreamTables t;
    t.cb_lane = ptx::smem_u32(cb) + ((threadIdx.x & 31) << 2);
    t.lut2 = ptx::smem_u32(lut) - 2u * 0x4B000000u;
    __syncthreads();
    return t;
}

// the tables never change after the set-up barrier: plain (non-volatile) loads the compiler may schedule freely
__device__ __forceinline__ float lds_f32(uint32_t a) {
    float v;
    asm("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32_next(uint32_t a) {       // the next codeword's copy
    float v;
    asm("ld.shared.f32 %0, [%1+128];" : "=f"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) {
    uint32_t v;
    asm("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// codeword of byte k of an index word
template <int K>
__device__ __forceinline__ float cb_of_byte(const StreamTables& t, uint32_t w) {
    return lds_f32(t.cb_lane + (__byte_perm(w, 0u, 0x4440u + K) << 7));
}
__device__ __forceinline__ void cb_of_words(const StreamTables& s, uint32_t w0, uint32_t w1, float (&cbv)[8]) {
    cbv[0] = cb_of_byte<0>(s, w0); cbv[1] = cb_of_byte<1>(s, w0);
    cbv[2] = cb_of_byte<2>(s, w0); cbv[3] = cb_of_byte<3>(s, w0);
    cbv[4] = cb_of_byte<0>(s, w1); cbv[5] = cb_of_byte<1>(s, w1);
    cbv[6] = cb_of_byte<2>(s, w1); cbv[7] = cb_of_byte<3>(s, w1);
}
__device__ __forceinline__ float rcp_approx(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

template <typename T, int W, int D>
__device__ __forceinline__ void stats_range_stream(const Hot& d, const StreamTables& s, const TileCursor& t, float gs,
                                                   float (&csum)[W], RunMax& run,
                                                   Ring<D, StreamCfg<W>::kStatsStageBytes>& ring, int lt) {
    using Cfg = StreamCfg<W>;
    constexpr int H = W / 8;
    const int tx = lt % d.tcols, ty = lt / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * W;
    const bool act = c0 < d.cols;
    const int stride = d.trows;
    const int n_steps = (t.r1 - t.r0 + stride - 1) / stride;
    const float b1 = d.beta1, omb1 = d.omb1;
    // rows of one block only (blocks are whole rows or runs of rows): no per-row agreement needed
    const bool row_blocks = d.blk_mode == 0 || d.blk_mode == 2;
    int r = t.r0 + ty;
    BlockIter it = block_iter(d, r, act ? c0 : 0);
    float mo_next = (act && r < t.r1) ? d.mag[it.blk] : 0.f;
#pragma unroll 1
    for (int step = 0; step < n_steps; ++step, r += stride) {
        const bool row_ok = r < t.r1;                 // uniform across the warp: a warp shares ty
        const int blk = (act && row_ok) ? it.blk : -1;
        const float mo = mo_next;
        block_iter_next(d, it);
        mo_next = (act && r + stride < t.r1) ? d.mag[it.blk] : 0.f;
        uint4 gw[H];
        uint2 iw[H];
        const bool ok = stage_wait(ring);
        if (ok && act && row_ok) {
            const unsigned char* st = ring.stage();
#pragma unroll
            for (int h = 0; h < H; ++h) {
                gw[h] = *reinterpret_cast<const uint4*>(st + lt * (W * 2) + h * 16);
                iw[h] = *reinterpret_cast<const uint2*>(st + Cfg::kValBytes + lt * W + h * 8);
            }
        }
        stage_release(ring, ok, lt);
        if (!ok || !row_ok) continue;
        float amax = 0.f, rs = 0.f;
        if (act) {
#pragma unroll
            for (int h = 0; h < H; ++h) {
                float g[8], cbv[8];
                Vec8<T>::unpack(gw[h], g);
                cb_of_words(s, iw[h].x, iw[h].y, cbv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float ge = __fmul_rn(g[e], gs);
                    const float m = ema_momentum(cbv[e], mo, ge, b1, omb1);
                    amax = fmaxf(amax, fabsf(m));
                    rs = __fmaf_rn(ge, ge, rs);
                    csum[h * 8 + e] = __fmaf_rn(ge, ge, csum[h * 8 + e]);
                }
            }
        }
        const float rs_lane = rs;
        if (!run.sum_dst) {
            rs = warp_sum(rs);
            if ((lt & 31) == 0 && act) atomicAdd(d.row_sq + r, rs);
        }
        if (row_blocks) {
            const int b0 = __shfl_sync(0xffffffffu, blk, 0);               // lane 0 has the lowest column
            if (b0 >= 0) {
                if ((long long)b0 != run.blk) { runmax_flush(run); run.blk = b0; }
                run.val = fmaxf(run.val, amax);
                run.sum += rs_lane;
            }
            continue;
        }
        const unsigned live = __ballot_sync(0xffffffffu, act);
        if (live) {
            const int b0 = __shfl_sync(0xffffffffu, blk, 0);
            const int b1l = __shfl_sync(0xffffffffu, blk, 31 - __clz((int)live));
            if (b0 == b1l) {
                if ((long long)b0 != run.blk) { runmax_flush(run); run.blk = b0; }
                run.val = fmaxf(run.val, amax);
                run.sum += rs_lane;
            } else if (act) {
                atomic_max_nonneg(run.dst + blk, amax);
                if (run.sum_dst) atomicAdd(run.sum_dst + blk, rs_lane);
            }
        }
    }
}

__device__ __forceinline__ void stream_init(StreamShared& sh) {
    if (threadIdx.x == 0) {
        for (int g = 0; g < kMaxGroups; ++g) {
            for (int k = 0; k < 8; ++k) {
                ptx::mbar_init(&sh.full[g][k], 1);
                ptx::mbar_init(&sh.empty[g][k], kThreads / 32);
            }
        }
        sh.abort_flag = 0;
        ptx::mbar_init_fence();
    }
    // the __syncthreads of load_tables_stream, which every thread calls next, publishes the barriers
}

// role of a thread inside a streamed CTA and the tile range of its group
struct StreamRole {
    bool producer;
    int group, lt;
    long long T0, T1;
};
template <int W>
__device__ __forceinline__ StreamRole stream_role(const LaunchCommon& c) {
    constexpr int G = StreamCfg<W>::kG;
    StreamRole r;
    r.producer = threadIdx.x >= G * kThreads;
    r.group = r.producer ? (threadIdx.x - G * kThreads) / 32 : threadIdx.x / kThreads;
    r.lt = threadIdx.x - r.group * kThreads;                    // consumers only
    const long long total = (W == 16) ? tile_prefix<16>(c)[c.n_tensors] : c.total_tiles;
    const long long v = (long long)blockIdx.x * G + r.group, nv = (long long)gridDim.x * G;
    r.T0 = total * v / nv;
    r.T1 = total * (v + 1) / nv;
    return r;
}

template <int D, int STAGE_BYTES>
__device__ __forceinline__ Ring<D, STAGE_BYTES> make_ring(StreamShared& sh, int group, size_t tables) {
    Ring<D, STAGE_BYTES> ring;
    ring.full = sh.full[group];
    ring.empty = sh.empty[group];
    ring.base = gx_smem_raw + tables + (size_t)group * D * STAGE_BYTES;
    ring.abort_flag = &sh.abort_flag;
    ring.slot = 0;
    ring.phase = 0;
    return ring;
}

template <int VEC>
__device__ __forceinline__ void flush_cols_w(const Hot& d, int ct, int lt, float (&csum)[VEC]) {
    const int c0 = (ct * d.tcols + lt % d.tcols) * VEC;
    if (c0 < d.cols) {
        // col_sq is 16-byte aligned (the plan aligns every scratch array) and c0 % 8 == 0
        float4* dst = reinterpret_cast<float4*>(d.col_sq + c0);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q)
            atomicAdd(dst + q, make_float4(csum[4 * q], csum[4 * q + 1], csum[4 * q + 2], csum[4 * q + 3]));
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) csum[e] = 0.f;
}

template <typename T, int W>
__global__ void __launch_bounds__(StreamCfg<W>::kCtaThreads, 1) factored_stats_stream_kernel(LaunchCommon c) {
    using Cfg = StreamCfg<W>;
    __shared__ StreamShared sh;
    stream_init(sh);
    const StreamTables s = load_tables_stream(c, false);
    const StreamRole role = stream_role<W>(c);
    const long long T0 = role.T0, T1 = role.T1;
    if (T0 >= T1) return;
    auto ring = make_ring<Cfg::kStatsStages, Cfg::kStatsStageBytes>(sh, role.group, kTabStats);
    if (role.producer) {
        stream_producer<T, W, Cfg::kStatsStages, Cfg::kStatsStageBytes, false>(c, T0, T1, ring);
        return;
    }
    const int group = role.group, lt = role.lt;
    const float gs = c.gscale ? *c.gscale : 1.0f;
    float csum[W];
#pragma unroll
    for (int e = 0; e < W; ++e) csum[e] = 0.f;
    RunMax run{nullptr, nullptr, -1, 0.f, 0.f, 1};
    Hot d;
    TileWalk w;
    walk_begin_w<W>(c, T0, w, d);
    run.dst = d.mag_new;
    run.sum_dst = d.row_only ? d.row_sq : nullptr;
    for (long long tile = T0; tile < T1;) {
        const int n = (int)min(T1 - tile, (long long)(w.n_row_tiles - w.rt));
        const TileCursor t = walk_cursor(w, d, n);
        stats_range_stream<T, W, Cfg::kStatsStages>(d, s, t, gs, csum, run, ring, lt);
        tile += n;
        w.rt += n;
        bool col_change = false, tensor_change = false;
        if (w.rt == w.n_row_tiles) {
            w.rt = 0;
            col_change = true;
            if (++w.ct == d.n_col_tiles) { w.ct = 0; tensor_change = true; }
        }
        const bool last = tile == T1;
        if ((col_change || last) && !d.row_only) {
            const int ct_done = col_change ? (tensor_change ? d.n_col_tiles - 1 : w.ct - 1) : w.ct;
            flush_cols_w<W>(d, ct_done, lt, csum);
        }
        if (tensor_change || last) runmax_flush_group(run, sh, group, lt);
        if (tensor_change && !last) {
            ++w.ti;
            d = load_hot_w<W>(c.descs + w.ti);
            w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
            run.dst = d.mag_new;
            run.sum_dst = d.row_only ? d.row_sq : nullptr;
        }
    }
    if (sh.abort_flag && lt == 0 && c.status) atomicExch(c.status, (int)kWaitTimeout);
}

// One element of the streamed apply: momentum, nearest codeword, parameter.
//   m = (cb[i] * mag_old) * b1 + g * (1 - b1)          (the eager roundings: indices stay bit-exact)
//   v = m / mag_new -> bucket -> lo = thresholds below the bucket; the codewords lo and lo + 1 come
//   from this lane's copies (128 bytes apart); their midpoint is the decision threshold, computed as
//   the host computes it (fp32 sum, halved), so the table of thresholds is not read.  The host sends
//   a plan here only when no bucket holds more than one threshold: one comparison settles it.
//   p = p * wd - (q * mag_new) * (lr / bc1) / (rf * cf + eps)
struct ApplyScalars {
    float gs, mo, mn, inv, rf, b1, omb1, eps, coef, wdf;
};

template <typename T, bool WD>
__device__ __forceinline__ void apply_element(const StreamTables& s, const ApplyScalars& a, float g, float cbv, float cf,
                                              float& pf, uint32_t& knew) {
    const float ge = __fmul_rn(g, a.gs);
    const float m = ema_momentum(cbv, a.mo, ge, a.b1, a.omb1);
    const float v = __fmul_rn(m, a.inv);
    const uint32_t lo = lds_u16(s.lut2 + (lut_bucket_bits(v) << 1)) & 0xffu;
    const uint32_t addr = s.cb_lane + (lo << 7);
    const float clo = lds_f32(addr), chi = lds_f32_next(addr);
    const float thr = __fmul_rn(__fadd_rn(clo, chi), 0.5f);
    const bool up = thr < v;
    knew = lo + (up ? 1u : 0u);
    const float qv = __fmul_rn(up ? chi : clo, a.mn);
    const float h = __fmaf_rn(a.rf, cf, a.eps);
    float pw = pf;
    if constexpr (WD) pw = round_to<T>(__fmul_rn(pf, a.wdf));
    pf = __fmaf_rn(-__fmul_rn(qv, a.coef), rcp_approx(h), pw);
}

template <typename T, bool WD, int W, int D>
__device__ __forceinline__ void apply_range_stream(const Hot& d, const StreamTables& s, const TileCursor& t, float gs,
                                                   const float (&cf)[W],
                                                   Ring<D, StreamCfg<W>::kApplyStageBytes>& ring, int lt) {
    using Cfg = StreamCfg<W>;
    constexpr int H = W / 8;
    const int tx = lt % d.tcols, ty = lt / d.tcols;
    const int c0 = (t.ct * d.tcols + tx) * W;
    const bool act = c0 < d.cols;
    ApplyScalars a;
    a.gs = gs;
    a.b1 = d.beta1; a.omb1 = d.omb1; a.eps = d.eps;
    a.coef = __fmul_rn(d.scal[0], d.scal[2]);      // lr / bias correction 1
    a.wdf = d.scal[3];
    T* p = reinterpret_cast<T*>(d.p);
    const int stride = d.trows;
    const int n_steps = (t.r1 - t.r0 + stride - 1) / stride;
    int r = t.r0 + ty;
    BlockIter it = block_iter(d, r, act ? c0 : 0);
    float mo_n = 0.f, mn_n = 0.f, rf_n = 0.f;
    if (act && r < t.r1) {
        mo_n = d.mag[it.blk];
        mn_n = d.mag_new[it.blk];
        rf_n = d.rfac[d.row_only ? it.blk : r];
    }
#pragma unroll 1
    for (int step = 0; step < n_steps; ++step, r += stride) {
        const bool valid = act && r < t.r1;
        const unsigned off = it.off;
        a.mo = mo_n; a.mn = mn_n; a.rf = rf_n;
        block_iter_next(d, it);
        if (act && r + stride < t.r1) {
            mo_n = d.mag[it.blk];
            mn_n = d.mag_new[it.blk];
            rf_n = d.rfac[d.row_only ? it.blk : r + stride];
        }
        const bool ok = stage_wait(ring);
        if (!ok || !valid) {
            stage_release(ring, ok, lt);
            continue;
        }
        const unsigned char* st = ring.stage();
        a.inv = a.mn > 0.f ? __frcp_rn(a.mn) : 0.f;
#pragma unroll
        for (int h = 0; h < H; ++h) {
            const uint4 gw = *reinterpret_cast<const uint4*>(st + lt * (W * 2) + h * 16);
            const uint4 pwd = *reinterpret_cast<const uint4*>(st + Cfg::kValBytes + lt * (W * 2) + h * 16);
            const uint2 iw = *reinterpret_cast<const uint2*>(st + 2 * Cfg::kValBytes + lt * W + h * 8);
            float g[8], pf[8], cbv[8];
            uint32_t kn[8];
            Vec8<T>::unpack(gw, g);
            Vec8<T>::unpack(pwd, pf);
            cb_of_words(s, iw.x, iw.y, cbv);
#pragma unroll
            for (int e = 0; e < 8; ++e) apply_element<T, WD>(s, a, g[e], cbv[e], cf[h * 8 + e], pf[e], kn[e]);
            uint2 io;
            io.x = __byte_perm(__byte_perm(kn[0], kn[1], 0x0040), __byte_perm(kn[2], kn[3], 0x0040), 0x5410);
            io.y = __byte_perm(__byte_perm(kn[4], kn[5], 0x0040), __byte_perm(kn[6], kn[7], 0x0040), 0x5410);
            *reinterpret_cast<uint2*>(d.idx + off + h * 8) = io;
            store_param<T, 8>(p + off + h * 8, pf);
        }
        stage_release(ring, true, lt);
    }
}

template <typename T, int W>
__global__ void __launch_bounds__(StreamCfg<W>::kCtaThreads, 1) factored_apply_stream_kernel(LaunchCommon c) {
    using Cfg = StreamCfg<W>;
    __shared__ StreamShared sh;
    stream_init(sh);
    const StreamTables s = load_tables_stream(c, true);
    const StreamRole role = stream_role<W>(c);
    const long long T0 = role.T0, T1 = role.T1;
    if (T0 >= T1) return;
    auto ring = make_ring<Cfg::kApplyStages, Cfg::kApplyStageBytes>(sh, role.group, kTabFull);
    if (role.producer) {
        stream_producer<T, W, Cfg::kApplyStages, Cfg::kApplyStageBytes, true>(c, T0, T1, ring);
        return;
    }
    const int lt = role.lt;
    const float gs = c.gscale ? *c.gscale : 1.0f;
    float cf[W];
    Hot d;
    TileWalk w;
    walk_begin_w<W>(c, T0, w, d);
    bool reload = true;
    for (long long tile = T0; tile < T1;) {
        if (reload) {
            const int c0 = (w.ct * d.tcols + lt % d.tcols) * W;
#pragma unroll
            for (int e = 0; e < W; ++e) cf[e] = d.row_only ? 1.0f : ((c0 + e < d.cols) ? d.cfac[c0 + e] : 0.f);
            reload = false;
        }
        const int n = (int)min(T1 - tile, (long long)(w.n_row_tiles - w.rt));
        const TileCursor t = walk_cursor(w, d, n);
        if (d.scal[3] != 1.0f) apply_range_stream<T, true, W, Cfg::kApplyStages>(d, s, t, gs, cf, ring, lt);
        else apply_range_stream<T, false, W, Cfg::kApplyStages>(d, s, t, gs, cf, ring, lt);
        tile += n;
        w.rt += n;
        if (w.rt == w.n_row_tiles) {
            w.rt = 0;
            reload = true;
            if (++w.ct == d.n_col_tiles) {
                w.ct = 0;
                if (tile < T1) {
                    ++w.ti;
                    d = load_hot_w<W>(c.descs + w.ti);
                    w.n_row_tiles = (d.rows + d.rows_per_tile - 1) / d.rows_per_tile;
                }
            }
        }
    }
    if (sh.abort_flag && lt == 0 && c.status) atomicExch(c.status, (int)kWaitTimeout);
}

// mag <- mag_new ; mag_new <- 0, for every tensor of the plan
__global__ void __launch_bounds__(kThreads) finalize_magnitude_kernel(LaunchCommon c) {
    for (int ti = 0; ti < c.n_tensors; ++ti) {
        const TensorDesc& d = c.descs[ti];
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.nb;
             i += (long long)gridDim.x * blockDim.x) {
            d.mag[i] = d.mag_new[i];
            d.mag_new[i] = 0.f;
        }
    }
}

// ---------------------------------------------------------------------------
// gradient reduction (reduce-scatter by peer loads) and clipping coefficient
// ---------------------------------------------------------------------------
struct SrcList { const void* p[kDescMaxSrc]; };

template <typename T>
__global__ void __launch_bounds__(kThreads) reduce_sources_kernel(T* __restrict__ out, SrcList src, int n_src,
                                                                   long long numel, float scale,
                                                                   float* __restrict__ partials) {
    __shared__ float red[kThreads / 32];
    float ssq = 0.f;
    const long long n8 = numel / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
         i += (long long)gridDim.x * blockDim.x) {
        float a[8];
        Vec8<T>::load(reinterpret_cast<const T*>(src.p[0]) + i * 8, a);
        for (int s = 1; s < n_src; ++s) {
            float t[8];
            Vec8<T>::load(reinterpret_cast<const T*>(src.p[s]) + i * 8, t);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] += t[e];
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a[e] = (n_src > 1 || scale != 1.0f) ? round_to<T>(__fmul_rn(a[e], scale)) : a[e];
            ssq += a[e] * a[e];
        }
        if (out) Vec8<T>::store(out + i * 8, a);
    }
    // tail
    for (long long i = n8 * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
         i += (long long)gridDim.x * blockDim.x) {
        float a = to_f<T>(reinterpret_cast<const T*>(src.p[0])[i]);
        for (int s = 1; s < n_src; ++s) a += to_f<T>(reinterpret_cast<const T*>(src.p[s])[i]);
        a = (n_src > 1 || scale != 1.0f) ? round_to<T>(__fmul_rn(a, scale)) : a;
        ssq += a * a;
        if (out) out[i] = from_f<T>(a);
    }
    if (partials) {
        ssq = warp_sum(ssq);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < kThreads / 32; ++i) t += red[i];
            partials[blockIdx.x] += t;
        }
    }
}

__global__ void clip_coef_kernel(const float* __restrict__ partials, int n, float max_norm,
                                 float* __restrict__ coef) {
    __shared__ double red[32];
    double acc = 0.0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) acc += (double)partials[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += red[i];
        const float norm = (float)sqrt(t);
        coef[1] = norm;
        coef[0] = (max_norm > 0.f) ? fminf(1.0f, max_norm / (norm + 1e-6f)) : 1.0f;
    }
}

template <typename F>
cudaError_t dispatch(int dtype, F&& f) {
    switch (dtype) {
        case kF32: return f((float*)nullptr);
        case kBF16: return f((__nv_bfloat16*)nullptr);
        case kF16: return f((__half*)nullptr);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

cudaError_t launch_block_update(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t st) {
    if (c.total_tiles <= 0) return cudaSuccess;
    const int grid = min(c.total_tiles, sm_count * 4);
    return dispatch(dtype, [&](auto* tag) {
        using T = std::remove_pointer_t<decltype(tag)>;
        cudaFuncSetAttribute(block_update_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFull);
        block_update_kernel<T><<<grid, kThreads, kSmemFull, st>>>(c);
        return cudaGetLastError();
    });
}

cudaError_t launch_factored_stats(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t st) {
    if (c.total_tiles <= 0) return cudaSuccess;
    const int grid = min(c.total_tiles, sm_count * (c.fast ? kFastCtas : 4));
    return dispatch(dtype, [&](auto* tag) {
        using T = std::remove_pointer_t<decltype(tag)>;
        // one row of raw chunks in flight beyond the current one (two were measured no faster)
        if (c.fast == 3 || c.fast == 4) {
            if constexpr (sizeof(T) == 2) {
                // persistent: one CTA per SM, groups without tiles return at once
                if (c.fast == 4) {
                    cudaFuncSetAttribute(factored_stats_stream_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_stats_stream<16>());
                    factored_stats_stream_kernel<T, 16><<<sm_count, StreamCfg<16>::kCtaThreads, smem_stats_stream<16>(), st>>>(c);
                } else {
                    cudaFuncSetAttribute(factored_stats_stream_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_stats_stream<8>());
                    factored_stats_stream_kernel<T, 8><<<min(sm_count, (c.total_tiles + 2) / 3), StreamCfg<8>::kCtaThreads,
                                                         smem_stats_stream<8>(), st>>>(c);
                }
            } else {
                return cudaErrorInvalidValue;
            }
        } else if (c.fast == 2) {
            if constexpr (std::is_same_v<T, __nv_bfloat16>)
                factored_stats_kernel<T, true, 1, true><<<grid, kThreads, kSmemStats, st>>>(c);
            else
                return cudaErrorInvalidValue;
        } else if (c.fast) {
            factored_stats_kernel<T, true, 1><<<grid, kThreads, kSmemStats, st>>>(c);
        } else {
            factored_stats_kernel<T, false><<<grid, kThreads, kSmemStats, st>>>(c);
        }
        return cudaGetLastError();
    });
}

cudaError_t launch_factored_ema(const LaunchCommon& c, cudaStream_t st) {
    if (c.n_tensors <= 0) return cudaSuccess;
    factored_ema_kernel<<<c.n_tensors, kEmaThreads, 0, st>>>(c);
    return cudaGetLastError();
}

cudaError_t launch_factored_apply(const LaunchCommon& c, int dtype, int sm_count, cudaStream_t st) {
    if (c.total_tiles <= 0) return cudaSuccess;
    const bool fast = c.fast && !c.stochastic;
    const int grid = min(c.total_tiles, sm_count * (fast ? kFastCtas : 2));
    return dispatch(dtype, [&](auto* tag) {
        using T = std::remove_pointer_t<decltype(tag)>;
        if ((c.fast == 3 || c.fast == 4) && !c.stochastic) {
            if constexpr (sizeof(T) == 2) {
                if (c.fast == 4) {
                    cudaFuncSetAttribute(factored_apply_stream_kernel<T, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_apply_stream<16>());
                    factored_apply_stream_kernel<T, 16><<<sm_count, StreamCfg<16>::kCtaThreads, smem_apply_stream<16>(), st>>>(c);
                } else {
                    cudaFuncSetAttribute(factored_apply_stream_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_apply_stream<8>());
                    factored_apply_stream_kernel<T, 8><<<min(sm_count, (c.total_tiles + 2) / 3), StreamCfg<8>::kCtaThreads,
                                                         smem_apply_stream<8>(), st>>>(c);
                }
            } else {
                return cudaErrorInvalidValue;
            }
        } else if (c.fast == 2) {
            // multicast gradient sources exist only in the fast bf16 kernels (the plan builder makes
            // sure of it): nearest rounding, 8-wide chunks
            if constexpr (std::is_same_v<T, __nv_bfloat16>) {
                if (c.stochastic) return cudaErrorInvalidValue;
                cudaFuncSetAttribute(factored_apply_kernel<T, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFull);
                factored_apply_kernel<T, true, true><<<grid, kThreads, kSmemFull, st>>>(c);
            } else {
                return cudaErrorInvalidValue;
            }
        } else if (fast) {
            cudaFuncSetAttribute(factored_apply_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFull);
            factored_apply_kernel<T, true><<<grid, kThreads, kSmemFull, st>>>(c);
        } else {
            cudaFuncSetAttribute(factored_apply_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemFull);
            factored_apply_kernel<T, false><<<grid, kThreads, kSmemFull, st>>>(c);
        }
        return cudaGetLastError();
    });
}

cudaError_t launch_finalize_magnitude(const LaunchCommon& c, int sm_count, cudaStream_t st) {
    if (c.n_tensors <= 0) return cudaSuccess;
    finalize_magnitude_kernel<<<sm_count, kThreads, 0, st>>>(c);
    return cudaGetLastError();
}

cudaError_t launch_reduce_sources(void* out, const void* const* src, int n_src, long long numel,
                                  float scale, float* partials, int n_partials, int dtype,
                                  cudaStream_t st) {
    if (numel <= 0) return cudaSuccess;
    if (n_src < 1 || n_src > kDescMaxSrc) return cudaErrorInvalidValue;
    SrcList sl;
    for (int i = 0; i < kDescMaxSrc; ++i) sl.p[i] = i < n_src ? src[i] : nullptr;
    long long want = (numel / 8 + kThreads - 1) / kThreads;
    int grid = (int)max(1LL, min(want, (long long)(n_partials > 0 ? n_partials : 1184)));
    return dispatch(dtype, [&](auto* tag) {
        using T = std::remove_pointer_t<decltype(tag)>;
        reduce_sources_kernel<T><<<grid, kThreads, 0, st>>>((T*)out, sl, n_src, numel, scale, partials);
        return cudaGetLastError();
    });
}

cudaError_t launch_clip_coef(const float* partials, int n, float max_norm, float* coef,
                             cudaStream_t st) {
    clip_coef_kernel<<<1, 1024, 0, st>>>(partials, n, max_norm, coef);
    return cudaGetLastError();
}

}  // namespace gx
