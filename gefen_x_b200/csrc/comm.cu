// Peer-memory communication primitives over NVLink / NVSwitch.
//
// Every rank maps every peer's symmetric arena; these kernels move data with
// plain peer loads / stores and synchronise with release/acquire flags that
// live in the arenas.  Every wait is bounded: when the iteration budget runs out
// the kernel writes kWaitTimeout into the status word and returns, so a missing
// peer surfaces as a host-side error instead of a hung GPU.
//
// The reference has no custom collective; it relies on torch FSDP2's NCCL
// all-gather / reduce-scatter (reference collective call sites:
// src/gefen/gefen.py:3496-3499, src/gefen/gefen_muon.py:1849-1896).
#include "comm.h"
#include "common.cuh"

namespace gx {
namespace {

struct PtrList { void* p[kMaxSrc]; };

// Publish `value` into slot `slot` of every peer's flag array (own included).
__global__ void signal_kernel(PtrList flags, int world, int slot, uint32_t value) {
    __threadfence_system();
    if (threadIdx.x < world)
        st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + slot, value);
}

// Wait until flags[0..n) >= value (bounded).
__global__ void wait_kernel(const uint32_t* flags, int n, uint32_t value, long long max_iters, int* status) {
    if (threadIdx.x < n) {
        if (!wait_flag_ge(flags + threadIdx.x, value, max_iters)) {
            if (status) atomicExch(status, (int)kWaitTimeout);
        }
    }
}

// Segment copy: dst[seg.dst_off ...] = src_base[seg.src_rank][seg.src_off ...], 16-byte units.
// All CTAs walk the segments together; within a segment every thread keeps eight
// 16-byte peer loads in flight before it stores them (an NVLink round trip is a few
// microseconds, so the bandwidth a CTA reaches is set by the bytes it has in flight).
constexpr int kGatherUnroll = 8;

__global__ void __launch_bounds__(256) gather_kernel(PtrList src_base, const GatherSeg* __restrict__ segs,
                                                     int n_segs, char* __restrict__ dst,
                                                     const long long* __restrict__ unit_prefix) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    for (int seg = 0; seg < n_segs; ++seg) {
        const GatherSeg s = segs[seg];
        const long long units = unit_prefix[seg + 1] - unit_prefix[seg];
        const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(src_base.p[s.src_rank]) + s.src_off);
        uint4* dp = reinterpret_cast<uint4*>(dst + s.dst_off);
        for (long long u0 = tid; u0 < units; u0 += nthreads * kGatherUnroll) {
            uint4 v[kGatherUnroll];
#pragma unroll
            for (int j = 0; j < kGatherUnroll; ++j) {
                const long long u = u0 + j * nthreads;
                if (u < units) v[j] = sp[u];
            }
#pragma unroll
            for (int j = 0; j < kGatherUnroll; ++j) {
                const long long u = u0 + j * nthreads;
                if (u < units) dp[u] = v[j];
            }
        }
    }
}

// Reduce-scatter of a table of slices: every thread keeps two 16-byte units of every source in
// flight (2 * world peer loads), sums them in fp32 in rank order, scales, rounds to the storage
// type and stores; the CTA adds its sum of squares into partials[blockIdx.x].
constexpr int kReduceUnroll = 2;

template <typename T>
__global__ void __launch_bounds__(256) reduce_segments_kernel(int world,
                                                              const ReduceSeg* __restrict__ segs, int n_segs,
                                                              const long long* __restrict__ unit_prefix,
                                                              float scale, float* __restrict__ partials) {
    constexpr int kPer = 16 / (int)sizeof(T);     // elements per 16-byte unit
    __shared__ float red[8];
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    float ssq = 0.f;
    for (int seg = 0; seg < n_segs; ++seg) {
        const ReduceSeg s = segs[seg];
        const long long units = unit_prefix[seg + 1] - unit_prefix[seg];
        uint4* dp = reinterpret_cast<uint4*>(s.dst);
        for (long long u0 = tid; u0 < units; u0 += nthreads * kReduceUnroll) {
            uint4 v[kReduceUnroll][kMaxSrc];
#pragma unroll
            for (int j = 0; j < kReduceUnroll; ++j) {
                const long long u = u0 + j * nthreads;
#pragma unroll
                for (int r = 0; r < kMaxSrc; ++r) {
                    if (r < world && u < units) v[j][r] = reinterpret_cast<const uint4*>(s.src[r])[u];
                }
            }
#pragma unroll
            for (int j = 0; j < kReduceUnroll; ++j) {
                const long long u = u0 + j * nthreads;
                if (u >= units) continue;
                float acc[kPer];
                const T* e0 = reinterpret_cast<const T*>(&v[j][0]);
#pragma unroll
                for (int e = 0; e < kPer; ++e) acc[e] = to_f<T>(e0[e]);
#pragma unroll
                for (int r = 1; r < kMaxSrc; ++r) {
                    if (r < world) {
                        const T* er = reinterpret_cast<const T*>(&v[j][r]);
#pragma unroll
                        for (int e = 0; e < kPer; ++e) acc[e] += to_f<T>(er[e]);
                    }
                }
                uint4 o;
                T* eo = reinterpret_cast<T*>(&o);
#pragma unroll
                for (int e = 0; e < kPer; ++e) {
                    const float a = (world > 1 || scale != 1.0f) ? round_to<T>(__fmul_rn(acc[e], scale)) : acc[e];
                    ssq += a * a;
                    eo[e] = from_f<T>(a);
                }
                if (dp) dp[u] = o;
            }
        }
    }
    if (partials) {
        ssq = warp_sum(ssq);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) t += red[i];
            partials[blockIdx.x] += t;
        }
    }
}

// The same reduce-scatter through NVSwitch: src[0] of every segment is the multicast address of the
// slice, one multimem.ld_reduce per 16 bytes returns the sum over all ranks (bf16, fp32 accumulation
// in the switch), so a rank receives its shard's bytes once instead of once per peer.
constexpr int kMcUnroll = 4;

__global__ void __launch_bounds__(256) reduce_segments_mc_kernel(const ReduceSeg* __restrict__ segs, int n_segs,
                                                                 const long long* __restrict__ unit_prefix,
                                                                 float scale, float* __restrict__ partials) {
    __shared__ float red[8];
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)gridDim.x * blockDim.x;
    float ssq = 0.f;
    for (int seg = 0; seg < n_segs; ++seg) {
        const ReduceSeg s = segs[seg];
        const long long units = unit_prefix[seg + 1] - unit_prefix[seg];
        uint4* dp = reinterpret_cast<uint4*>(s.dst);
        const uint4* mc = reinterpret_cast<const uint4*>(s.src[0]);
        for (long long u0 = tid; u0 < units; u0 += nthreads * kMcUnroll) {
            uint4 v[kMcUnroll];
#pragma unroll
            for (int j = 0; j < kMcUnroll; ++j) {
                const long long u = u0 + j * nthreads;
                if (u < units) v[j] = multimem_ld_reduce_bf16x8(mc + u);
            }
#pragma unroll
            for (int j = 0; j < kMcUnroll; ++j) {
                const long long u = u0 + j * nthreads;
                if (u >= units) continue;
                float f[8];
                Vec8<__nv_bfloat16>::unpack(v[j], f);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    f[e] = round_to<__nv_bfloat16>(__fmul_rn(f[e], scale));
                    ssq += f[e] * f[e];
                }
                if (dp) Vec8<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(dp + u), f);
            }
        }
    }
    if (partials) {
        ssq = warp_sum(ssq);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
        __syncthreads();
        if (threadIdx.x == 0) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) t += red[i];
            partials[blockIdx.x] += t;
        }
    }
}

// out[0] = sum over ranks of slot[rank][epoch & 1] after everybody has published;
// each rank first stores its own value into its slot (two slots alternate so that a
// fast rank's next reduction cannot overwrite a value a slow rank still has to read).
__global__ void allreduce_scalar_kernel(PtrList slots, PtrList flags, int world, int rank,
                                        const float* __restrict__ local_val, float* __restrict__ out,
                                        uint32_t epoch, long long max_iters, int* status) {
    __shared__ int ok;
    if (threadIdx.x == 0) {
        ok = 1;
        reinterpret_cast<float*>(slots.p[rank])[epoch & 1u] = local_val[0];
        __threadfence_system();
    }
    __syncthreads();
    if (threadIdx.x < world)
        st_release_sys(reinterpret_cast<uint32_t*>(flags.p[threadIdx.x]) + rank, epoch);
    if (threadIdx.x < world) {
        if (!wait_flag_ge(reinterpret_cast<const uint32_t*>(flags.p[rank]) + threadIdx.x, epoch, max_iters)) {
            ok = 0;
            if (status) atomicExch(status, (int)kWaitTimeout);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        if (ok) {
            for (int r = 0; r < world; ++r) t += reinterpret_cast<const volatile float*>(slots.p[r])[epoch & 1u];
        } else {
            t = local_val[0];
        }
        out[0] = t;
    }
}

// p[i] = round(p[i] * wd_factor) - alpha * u[i] for every entry of a table; u may live in a
// peer's arena (the rows of an orthogonalised Muon update that this rank's shard holds).
__global__ void __launch_bounds__(256) scatter_apply_kernel(const ApplySeg* __restrict__ segs, int n_segs,
                                                            const long long* __restrict__ unit_prefix) {
    const long long total = unit_prefix[n_segs];
    for (long long u = (long long)blockIdx.x * blockDim.x + threadIdx.x; u < total;
         u += (long long)gridDim.x * blockDim.x) {
        int lo = 0, hi = n_segs;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (unit_prefix[mid] <= u) lo = mid; else hi = mid;
        }
        const ApplySeg s = segs[lo];
        const long long k = (u - unit_prefix[lo]) * 8;
        float pf[8], uf[8];
        __nv_bfloat16* pp = reinterpret_cast<__nv_bfloat16*>(s.p) + k;
        Vec8<__nv_bfloat16>::load(pp, pf);
        Vec8<__nv_bfloat16>::load(reinterpret_cast<const __nv_bfloat16*>(s.u) + k, uf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            float v = pf[e];
            if (s.wd_factor != 1.0f) v = round_to<__nv_bfloat16>(v * s.wd_factor);
            pf[e] = v - s.alpha * uf[e];
        }
        Vec8<__nv_bfloat16>::store(pp, pf);
    }
}


// ---- sparse embedding: rows of a row-sharded table, fetched from / reduced into their owners ----
// The token embedding is read at a few thousand rows per step; gathering the whole table from the
// peers (and reducing a dense gradient of its size) moves a gigabyte for a few megabytes of use.
// Row r of the table lives on rank r / rows_per, at row r % rows_per of that rank's shard.
struct RowPeers { const char* base[kMaxSrc]; };

// out[t, :] = table[tok[t], :] read from the owner's shard by peer loads (one CTA per token).
__global__ void __launch_bounds__(128) gather_rows_kernel(RowPeers shard, long long rows_per, long long rows,
                                                         int row_units, const long long* __restrict__ tok,
                                                         uint4* __restrict__ out) {
    const long long t = blockIdx.x;
    long long r = tok[t];
    if (r < 0 || r >= rows) r = 0;          // out-of-range ids read row 0 (as a clamped lookup)
    const int owner = (int)(r / rows_per);
    const uint4* src = reinterpret_cast<const uint4*>(shard.base[owner]) + (r - owner * rows_per) * row_units;
    uint4* dst = out + t * row_units;
    uint4 v[4];
    for (int i0 = threadIdx.x; i0 < row_units; i0 += 128 * 4) {
#pragma unroll
        for (int j = 0; j < 4; ++j) if (i0 + j * 128 < row_units) v[j] = src[i0 + j * 128];
#pragma unroll
        for (int j = 0; j < 4; ++j) if (i0 + j * 128 < row_units) dst[i0 + j * 128] = v[j];
    }
}

// dst[row - row0, :] += scale * grad_r[t, :] for every rank r and every token t of rank r whose row
// this rank owns (dst = this rank's bf16 gradient shard, zeroed beforehand).  The token ids and
// gradient rows of rank r are read from its arena.  bf16x2 atomic adds: tokens may repeat.
struct TokPeers { const long long* tok[kMaxSrc]; const __nv_bfloat162* grad[kMaxSrc]; };

__global__ void __launch_bounds__(128) scatter_add_rows_kernel(TokPeers peers, int world, int n_tok,
                                                              long long row0, long long my_rows, int cols2,
                                                              float scale, __nv_bfloat162* __restrict__ dst) {
    const int r = blockIdx.x / n_tok, t = blockIdx.x - r * n_tok;
    if (r >= world) return;
    const long long row = peers.tok[r][t] - row0;
    if (row < 0 || row >= my_rows) return;
    const __nv_bfloat162* src = peers.grad[r] + (long long)t * cols2;
    __nv_bfloat162* out = dst + row * cols2;
    for (int i = threadIdx.x; i < cols2; i += 128) {
        const float2 f = __bfloat1622float2(src[i]);
        atomicAdd(out + i, __floats2bfloat162_rn(f.x * scale, f.y * scale));
    }
}

}  // namespace

cudaError_t launch_scatter_apply(const ApplySeg* segs_dev, int n_segs, const long long* unit_prefix_dev,
                                 long long total_units, int ctas, cudaStream_t st) {
    if (n_segs <= 0 || total_units <= 0) return cudaSuccess;
    long long want = (total_units + 255) / 256;
    int grid = (int)(want < ctas ? want : ctas);
    if (grid < 1) grid = 1;
    scatter_apply_kernel<<<grid, 256, 0, st>>>(segs_dev, n_segs, unit_prefix_dev);
    return cudaGetLastError();
}

cudaError_t launch_signal(void* const* flag_ptrs, int world, int slot, unsigned value, cudaStream_t st) {
    if (world < 1 || world > kMaxSrc) return cudaErrorInvalidValue;
    PtrList l{};
    for (int i = 0; i < world; ++i) l.p[i] = flag_ptrs[i];
    signal_kernel<<<1, 32, 0, st>>>(l, world, slot, value);
    return cudaGetLastError();
}

cudaError_t launch_wait(const unsigned* flags, int n, unsigned value, long long max_iters, int* status,
                        cudaStream_t st) {
    if (n < 1 || n > 32) return cudaErrorInvalidValue;
    wait_kernel<<<1, 32, 0, st>>>(flags, n, value, max_iters, status);
    return cudaGetLastError();
}

cudaError_t launch_gather(void* const* src_base, int world, const GatherSeg* segs_dev, int n_segs,
                          void* dst, const long long* unit_prefix_dev, long long total_units, int ctas,
                          cudaStream_t st) {
    if (world < 1 || world > kMaxSrc) return cudaErrorInvalidValue;
    if (n_segs <= 0 || total_units <= 0) return cudaSuccess;
    PtrList l{};
    for (int i = 0; i < world; ++i) l.p[i] = src_base[i];
    long long want = (total_units + 256 * kGatherUnroll - 1) / (256 * kGatherUnroll);
    int grid = (int)(want < ctas ? want : ctas);
    if (grid < 1) grid = 1;
    gather_kernel<<<grid, 256, 0, st>>>(l, segs_dev, n_segs, reinterpret_cast<char*>(dst), unit_prefix_dev);
    return cudaGetLastError();
}

cudaError_t launch_reduce_segments(int world, const ReduceSeg* segs_dev, int n_segs,
                                   const long long* unit_prefix_dev, long long total_units, float scale,
                                   float* partials, int ctas, int dtype, cudaStream_t st, bool multimem) {
    if (world < 1 || world > kMaxSrc) return cudaErrorInvalidValue;
    if (n_segs <= 0 || total_units <= 0) return cudaSuccess;
    if (multimem) {
        if (dtype != 1) return cudaErrorInvalidValue;           // bf16 only
        long long want_mc = (total_units + 256 * kMcUnroll - 1) / (256 * kMcUnroll);
        int grid_mc = (int)(want_mc < ctas ? want_mc : ctas);
        if (grid_mc < 1) grid_mc = 1;
        reduce_segments_mc_kernel<<<grid_mc, 256, 0, st>>>(segs_dev, n_segs, unit_prefix_dev, scale, partials);
        return cudaGetLastError();
    }
    long long want = (total_units + 256 * kReduceUnroll - 1) / (256 * kReduceUnroll);
    int grid = (int)(want < ctas ? want : ctas);
    if (grid < 1) grid = 1;
    switch (dtype) {
        case 0:
            reduce_segments_kernel<float><<<grid, 256, 0, st>>>(world, segs_dev, n_segs, unit_prefix_dev, scale, partials);
            break;
        case 1:
            reduce_segments_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(world, segs_dev, n_segs, unit_prefix_dev, scale, partials);
            break;
        case 2:
            reduce_segments_kernel<__half><<<grid, 256, 0, st>>>(world, segs_dev, n_segs, unit_prefix_dev, scale, partials);
            break;
        default:
            return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_allreduce_scalar(void* const* slot_ptrs, void* const* flag_ptrs, int world, int rank,
                                    const float* local_val, float* out, unsigned epoch,
                                    long long max_iters, int* status, cudaStream_t st) {
    if (world < 1 || world > kMaxSrc) return cudaErrorInvalidValue;
    PtrList s{}, f{};
    for (int i = 0; i < world; ++i) { s.p[i] = slot_ptrs[i]; f.p[i] = flag_ptrs[i]; }
    allreduce_scalar_kernel<<<1, 32, 0, st>>>(s, f, world, rank, local_val, out, epoch, max_iters, status);
    return cudaGetLastError();
}

cudaError_t launch_gather_rows(void* const* shard_ptrs, int world, long long rows_per, long long rows,
                               int row_bytes, const long long* tok_dev, int n_tok, void* out, cudaStream_t st) {
    if (n_tok <= 0) return cudaSuccess;
    if (world < 1 || world > kMaxSrc || row_bytes % 16 || rows_per <= 0) return cudaErrorInvalidValue;
    RowPeers rp{};
    for (int i = 0; i < world; ++i) rp.base[i] = static_cast<const char*>(shard_ptrs[i]);
    gather_rows_kernel<<<n_tok, 128, 0, st>>>(rp, rows_per, rows, row_bytes / 16, tok_dev,
                                               static_cast<uint4*>(out));
    return cudaGetLastError();
}

cudaError_t launch_scatter_add_rows(void* const* tok_ptrs, void* const* grad_ptrs, int world, int n_tok,
                                    long long row0, long long my_rows, int cols, float scale, void* dst,
                                    cudaStream_t st) {
    if (n_tok <= 0 || my_rows <= 0) return cudaSuccess;
    if (world < 1 || world > kMaxSrc || cols % 2) return cudaErrorInvalidValue;
    TokPeers tp{};
    for (int i = 0; i < world; ++i) {
        tp.tok[i] = static_cast<const long long*>(tok_ptrs[i]);
        tp.grad[i] = static_cast<const __nv_bfloat162*>(grad_ptrs[i]);
    }
    scatter_add_rows_kernel<<<world * n_tok, 128, 0, st>>>(tp, world, n_tok, row0, my_rows, cols / 2, scale,
                                                           static_cast<__nv_bfloat162*>(dst));
    return cudaGetLastError();
}

}  // namespace gx
