// Memory-bound model kernels for the decoder (RMSNorm incl. per-head QK-norm,
// RoPE, SwiGLU, cross-entropy).  The reference ships no model kernels; its
// benchmark model expresses these with torch ops (reference
// benchmarks/training_matrix/tiny_qwen.py:113-138, :180-181, :250-259).
// All of them are HBM-bound: 16-byte vector accesses, fp32 math, one pass over
// HBM per tensor (second passes hit L1/L2).
#include "common.cuh"
#include "model_ops.h"

namespace gx {
namespace {

constexpr int kThreads = 256;

// lanes cooperating on one row: power of two in [8, 256]
__host__ __device__ inline int lanes_for(int d) {
    int chunks = (d + 7) / 8;
    int l = 8;
    while (l < chunks && l < 256) l <<= 1;
    return l;
}

// sum over the `lanes` consecutive threads that share a row (lanes: power of two <= 256)
__device__ __forceinline__ float group_sum(float v, int lanes, float* sh) {
    const int w = min(lanes, 32);
    for (int o = w >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lanes <= 32) return v;
    const int warp = threadIdx.x >> 5, nw = lanes >> 5;
    const int g0 = (warp / nw) * nw;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < nw; ++i) t += sh[g0 + i];
    return t;
}

template <typename T>
__global__ void __launch_bounds__(kThreads) rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                               T* __restrict__ y, float* __restrict__ rstd,
                                                               long long rows, int d, float eps, int lanes) {
    __shared__ float sh[kThreads / 32];
    const int groups = kThreads / lanes;
    const int gi = threadIdx.x / lanes, lane = threadIdx.x % lanes;
    const long long it_rows = (long long)gridDim.x * groups;
    for (long long r0 = (long long)blockIdx.x * groups; r0 < rows; r0 += it_rows) {
        const long long r = r0 + gi;
        const bool ok = r < rows;
        float ss = 0.f;
        if (ok) {
            for (int c = lane * 8; c < d; c += lanes * 8) {
                float v[8];
                Vec8<T>::load(x + r * d + c, v);
#pragma unroll
                for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
            }
        }
        ss = group_sum(ss, lanes, sh);
        if (!ok) continue;
        const float rs = rsqrtf(ss / (float)d + eps);
        if (lane == 0 && rstd) rstd[r] = rs;
        for (int c = lane * 8; c < d; c += lanes * 8) {
            float v[8], ww[8];
            Vec8<T>::load(x + r * d + c, v);
            Vec8<T>::load(w + c, ww);
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = v[e] * rs * ww[e];
            Vec8<T>::store(y + r * d + c, v);
        }
    }
}

// dx = rstd * (g - x * rstd^2 * mean(g * x)) [+ res],  g = dy * w ;  dw += dy * x * rstd
// `res` (optional) is the gradient that bypasses the norm on the residual path: adding it here saves
// the separate elementwise pass over [rows, d].
template <typename T, int CH>
__global__ void __launch_bounds__(kThreads) rmsnorm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                                               const T* __restrict__ w, const float* __restrict__ rstd,
                                                               T* __restrict__ dx, float* __restrict__ dw_partial,
                                                               long long rows, int d, int lanes,
                                                               const T* __restrict__ res) {
    __shared__ float sh[kThreads / 32];
    const int groups = kThreads / lanes;
    const int gi = threadIdx.x / lanes, lane = threadIdx.x % lanes;
    const long long it_rows = (long long)gridDim.x * groups;
    float dw[CH][8];
#pragma unroll
    for (int k = 0; k < CH; ++k)
#pragma unroll
        for (int e = 0; e < 8; ++e) dw[k][e] = 0.f;
    for (long long r0 = (long long)blockIdx.x * groups; r0 < rows; r0 += it_rows) {
        const long long r = r0 + gi;
        const bool ok = r < rows;
        float dot = 0.f;
        const float rs = ok ? rstd[r] : 0.f;
        if (ok) {
#pragma unroll
            for (int k = 0; k < CH; ++k) {
                const int c = (lane + k * lanes) * 8;
                if (c < d) {
                    float a[8], b[8], ww[8];
                    Vec8<T>::load(dy + r * d + c, a);
                    Vec8<T>::load(x + r * d + c, b);
                    Vec8<T>::load(w + c, ww);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        dot += a[e] * ww[e] * b[e];
                        dw[k][e] += a[e] * b[e] * rs;
                    }
                }
            }
        }
        dot = group_sum(dot, lanes, sh);
        if (!ok) continue;
        const float coef = dot * rs * rs / (float)d;
#pragma unroll
        for (int k = 0; k < CH; ++k) {
            const int c = (lane + k * lanes) * 8;
            if (c < d) {
                float a[8], b[8], ww[8];
                Vec8<T>::load(dy + r * d + c, a);
                Vec8<T>::load(x + r * d + c, b);
                Vec8<T>::load(w + c, ww);
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = rs * (a[e] * ww[e] - b[e] * coef);
                if (res) {
                    float rr[8];
                    Vec8<T>::load(res + r * d + c, rr);
#pragma unroll
                    for (int e = 0; e < 8; ++e) a[e] += rr[e];
                }
                Vec8<T>::store(dx + r * d + c, a);
            }
        }
    }
    float* out = dw_partial + ((long long)blockIdx.x * groups + gi) * d;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
        const int c = (lane + k * lanes) * 8;
        if (c < d) {
#pragma unroll
            for (int e = 0; e < 8; ++e) out[c + e] = dw[k][e];
        }
    }
}

// out[c] = sum_r part[r, c]: the per-CTA partial weight gradients of the norm backward.  One CTA per 32
// columns, 8 row groups per CTA (coalesced 128-byte rows), fixed summation order.
__global__ void __launch_bounds__(256) colsum_kernel(const float* __restrict__ part, int n_rows, int d,
                                                     float* __restrict__ out) {
    __shared__ float sh[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    float acc = 0.f;
    if (c < d)
        for (int r = ty; r < n_rows; r += 8) acc += part[(long long)r * d + c];
    sh[ty][tx] = acc;
    __syncthreads();
    if (ty == 0 && c < d) {
        float t = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += sh[i][tx];
        out[c] = t;
    }
}

// Rotary embedding.  src: [tokens, n_heads, head_dim] with `src_stride` elements between tokens
// (a column slice of a fused projection output), dst likewise with `dst_stride` (dst may be src);
// position = token % seq_len; cos/sin: [seq_len, head_dim/2].
// Scalar form (any even head_dim, any alignment):
template <typename T>
__global__ void __launch_bounds__(kThreads) rope_scalar_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                               long long dst_stride, long long src_stride,
                                                               const float* __restrict__ cs,
                                                               const float* __restrict__ sn, long long tokens,
                                                               int seq_len, int n_heads, int head_dim, float sign,
                                                               bool interleaved) {
    const int half = head_dim >> 1;
    const long long pairs = tokens * n_heads * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
         i += (long long)gridDim.x * blockDim.x) {
        const int j = (int)(i % half);
        const long long th = i / half;             // token * n_heads + head
        const long long tok = th / n_heads;
        const int head = (int)(th - tok * n_heads);
        const int pos = (int)(tok % seq_len);
        const float c = cs[(long long)pos * half + j];
        const float s = sn[(long long)pos * half + j] * sign;
        const T* sb = src + tok * src_stride + (long long)head * head_dim;
        T* db = dst + tok * dst_stride + (long long)head * head_dim;
        const int i0 = interleaved ? 2 * j : j;
        const int i1 = interleaved ? 2 * j + 1 : j + half;
        const float a = to_f<T>(sb[i0]), b = to_f<T>(sb[i1]);
        db[i0] = from_f<T>(a * c - b * s);
        db[i1] = from_f<T>(b * c + a * s);
    }
}

// Vector form: a thread rotates eight pairs with 16-byte accesses (head_dim % 16 == 0, strides
// and pointers 16-byte aligned).  Half-rotation layout: elements [j, j + 8) with
// [j + half, j + half + 8); interleaved layout: two neighbouring 8-element vectors.
template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(kThreads) rope_vec_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                                            long long dst_stride, long long src_stride,
                                                            const float* __restrict__ cs,
                                                            const float* __restrict__ sn, long long tokens,
                                                            int seq_len, int n_heads, int head_dim, float sign) {
    const int half = head_dim >> 1;
    const int upr = half >> 3;                       // units (eight pairs) per head
    const long long units = tokens * n_heads * upr;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < units;
         i += (long long)gridDim.x * blockDim.x) {
        const int u = (int)(i % upr);
        const long long th = i / upr;
        const long long tok = th / n_heads;
        const int head = (int)(th - tok * n_heads);
        const int pos = (int)(tok % seq_len);
        const int j = u * 8;                         // first pair of the unit
        float c[8], s[8];
        {
            const float4* cp = reinterpret_cast<const float4*>(cs + (long long)pos * half + j);
            const float4* sp = reinterpret_cast<const float4*>(sn + (long long)pos * half + j);
            const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
            c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
            s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
        }
        const T* sb = src + tok * src_stride + (long long)head * head_dim;
        T* db = dst + tok * dst_stride + (long long)head * head_dim;
        const int o0 = INTERLEAVED ? 2 * j : j;
        const int o1 = INTERLEAVED ? 2 * j + 8 : j + half;
        float a[8], b[8];
        Vec8<T>::load(sb + o0, a);
        Vec8<T>::load(sb + o1, b);
        if constexpr (INTERLEAVED) {
            // pairs (a0,a1) (a2,a3) ... (b6,b7): pair p of the unit uses c[p]
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const float x0 = a[2 * p], x1 = a[2 * p + 1];
                a[2 * p] = x0 * c[p] - x1 * s[p] * sign;
                a[2 * p + 1] = x1 * c[p] + x0 * s[p] * sign;
                const float y0 = b[2 * p], y1 = b[2 * p + 1];
                b[2 * p] = y0 * c[4 + p] - y1 * s[4 + p] * sign;
                b[2 * p + 1] = y1 * c[4 + p] + y0 * s[4 + p] * sign;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float x0 = a[e], x1 = b[e];
                a[e] = x0 * c[e] - x1 * s[e] * sign;
                b[e] = x1 * c[e] + x0 * s[e] * sign;
            }
        }
        Vec8<T>::store(db + o0, a);
        Vec8<T>::store(db + o1, b);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out,
                                                              long long rows, int f) {
    const long long chunks = rows * (f / 8);
    const int cpr = f / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const int c = (int)(i % cpr) * 8;
        float g[8], u[8];
        Vec8<T>::load(gu + r * 2 * f + c, g);
        Vec8<T>::load(gu + r * 2 * f + f + c, u);
#pragma unroll
        for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
        Vec8<T>::store(out + r * f + c, g);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) swiglu_bwd_kernel(const T* __restrict__ gu, const T* __restrict__ dout,
                                                              T* __restrict__ dgu, long long rows, int f) {
    const long long chunks = rows * (f / 8);
    const int cpr = f / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < chunks;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cpr;
        const int c = (int)(i % cpr) * 8;
        float g[8], u[8], dz[8], dg[8], du[8];
        Vec8<T>::load(gu + r * 2 * f + c, g);
        Vec8<T>::load(gu + r * 2 * f + f + c, u);
        Vec8<T>::load(dout + r * f + c, dz);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float sg = 1.f / (1.f + __expf(-g[e]));
            const float silu = g[e] * sg;
            dg[e] = dz[e] * u[e] * sg * (1.f + g[e] * (1.f - sg));
            du[e] = dz[e] * silu;
        }
        Vec8<T>::store(dgu + r * 2 * f + c, dg);
        Vec8<T>::store(dgu + r * 2 * f + f + c, du);
    }
}

// One CTA per row of logits: online (max, sum-exp), loss = lse - logit[target],
// then the row is overwritten with (softmax - onehot) * grad_scale.
template <typename T>
__global__ void __launch_bounds__(1024) xent_kernel(T* __restrict__ logits, const long long* __restrict__ targets,
                                                    float* __restrict__ loss_rows, long long rows, int v,
                                                    float grad_scale, long long ignore_index) {
    __shared__ float sm[32], ss[32];
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
        T* row = logits + r * v;
        const long long tgt = targets[r];
        float mx = -INFINITY, sum = 0.f;
        const int v8 = (v % 8 == 0) ? v / 8 : 0;  // rows are 16-byte aligned only then
        for (int i = threadIdx.x; i < v8; i += blockDim.x) {
            float a[8];
            Vec8<T>::load(row + i * 8, a);
            float lm = a[0];
#pragma unroll
            for (int e = 1; e < 8; ++e) lm = fmaxf(lm, a[e]);
            if (lm > mx) { sum *= __expf(mx - lm); mx = lm; }
#pragma unroll
            for (int e = 0; e < 8; ++e) sum += __expf(a[e] - mx);
        }
        for (int i = v8 * 8 + threadIdx.x; i < v; i += blockDim.x) {
            const float a = to_f<T>(row[i]);
            if (a > mx) { sum *= __expf(mx - a); mx = a; }
            sum += __expf(a - mx);
        }
        // combine (max, sum) pairs
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, mx, o);
            const float os = __shfl_xor_sync(0xffffffffu, sum, o);
            const float nm = fmaxf(mx, om);
            sum = (mx == -INFINITY ? 0.f : sum * __expf(mx - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
            mx = nm;
        }
        __syncthreads();
        if ((threadIdx.x & 31) == 0) { sm[threadIdx.x >> 5] = mx; ss[threadIdx.x >> 5] = sum; }
        __syncthreads();
        float gm = -INFINITY, gs = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) {
            const float om = sm[i], os = ss[i];
            const float nm = fmaxf(gm, om);
            gs = (gm == -INFINITY ? 0.f : gs * __expf(gm - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
            gm = nm;
        }
        const float lse = gm + logf(gs);
        const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= v;
        if (threadIdx.x == 0) loss_rows[r] = ignored ? 0.f : (lse - to_f<T>(row[tgt]));
        __syncthreads();  // the target logit is read before the row is overwritten
        const float sc = ignored ? 0.f : grad_scale;
        for (int i = threadIdx.x; i < v8; i += blockDim.x) {
            float a[8];
            Vec8<T>::load(row + i * 8, a);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float p = __expf(a[e] - lse);
                a[e] = (p - ((long long)(i * 8 + e) == tgt ? 1.f : 0.f)) * sc;
            }
            Vec8<T>::store(row + i * 8, a);
        }
        for (int i = v8 * 8 + threadIdx.x; i < v; i += blockDim.x) {
            const float p = __expf(to_f<T>(row[i]) - lse);
            row[i] = from_f<T>((p - ((long long)i == tgt ? 1.f : 0.f)) * sc);
        }
    }
}

inline int grid_for(long long work_items, int per_cta, int cap) {
    long long g = (work_items + per_cta - 1) / per_cta;
    return (int)max(1LL, min(g, (long long)cap));
}

#define GX_DISPATCH(dtype, ...)                                        \
    switch (dtype) {                                                   \
        case 0: { using T = float; __VA_ARGS__; break; }               \
        case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; }       \
        case 2: { using T = __half; __VA_ARGS__; break; }              \
        default: return cudaErrorInvalidValue;                         \
    }

}  // namespace

int rmsnorm_bwd_partials(long long rows, int d) {
    const int lanes = lanes_for(d);
    const int groups = kThreads / lanes;
    const int grid = grid_for(rows, groups * 4, 148 * 4);
    return grid * groups;
}

cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int d,
                               float eps, int dtype, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (d % 8) return cudaErrorInvalidValue;
    const int lanes = lanes_for(d);
    const int groups = kThreads / lanes;
    const int grid = grid_for(rows, groups, 148 * 8);
    GX_DISPATCH(dtype, rmsnorm_fwd_kernel<T><<<grid, kThreads, 0, st>>>((const T*)x, (const T*)w, (T*)y, rstd, rows, d, eps, lanes));
    return cudaGetLastError();
}

cudaError_t launch_colsum(const float* part, int n_rows, int d, float* out, cudaStream_t st) {
    if (d <= 0) return cudaSuccess;
    colsum_kernel<<<(d + 31) / 32, 256, 0, st>>>(part, n_rows, d, out);
    return cudaGetLastError();
}

cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* dw_partial, int n_partial, long long rows, int d, int dtype,
                               cudaStream_t st, const void* res) {
    if (rows <= 0) return cudaSuccess;
    if (d % 8) return cudaErrorInvalidValue;
    const int lanes = lanes_for(d);
    const int groups = kThreads / lanes;
    if (n_partial % groups) return cudaErrorInvalidValue;
    const int grid = n_partial / groups;
    const int ch = ((d + 7) / 8 + lanes - 1) / lanes;
    if (ch > 8) return cudaErrorInvalidValue;
    GX_DISPATCH(dtype,
        if (ch <= 1) rmsnorm_bwd_kernel<T, 1><<<grid, kThreads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, d, lanes, (const T*)res);
        else if (ch <= 2) rmsnorm_bwd_kernel<T, 2><<<grid, kThreads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, d, lanes, (const T*)res);
        else if (ch <= 4) rmsnorm_bwd_kernel<T, 4><<<grid, kThreads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, d, lanes, (const T*)res);
        else rmsnorm_bwd_kernel<T, 8><<<grid, kThreads, 0, st>>>((const T*)dy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, d, lanes, (const T*)res));
    return cudaGetLastError();
}

cudaError_t launch_rope(void* dst, const void* src, long long dst_stride, long long src_stride,
                        const float* cs, const float* sn, long long tokens, int seq_len,
                        int n_heads, int head_dim, bool inverse, bool interleaved, int dtype,
                        cudaStream_t st) {
    if (tokens <= 0) return cudaSuccess;
    if (head_dim % 2) return cudaErrorInvalidValue;
    const float sign = inverse ? -1.f : 1.f;
    const int esz = dtype == 0 ? 4 : 2;
    const bool vec = head_dim % 16 == 0 && (dst_stride * esz) % 16 == 0 && (src_stride * esz) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(dst) % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(cs) % 16 == 0 && reinterpret_cast<uintptr_t>(sn) % 16 == 0;
    if (vec) {
        const long long units = tokens * n_heads * (head_dim / 16);
        const int grid = grid_for(units, kThreads, 148 * 16);
        if (interleaved) {
            GX_DISPATCH(dtype, (rope_vec_kernel<T, true><<<grid, kThreads, 0, st>>>((T*)dst, (const T*)src, dst_stride, src_stride, cs, sn, tokens, seq_len, n_heads, head_dim, sign)));
        } else {
            GX_DISPATCH(dtype, (rope_vec_kernel<T, false><<<grid, kThreads, 0, st>>>((T*)dst, (const T*)src, dst_stride, src_stride, cs, sn, tokens, seq_len, n_heads, head_dim, sign)));
        }
        return cudaGetLastError();
    }
    const long long pairs = tokens * n_heads * (head_dim / 2);
    const int grid = grid_for(pairs, kThreads * 4, 148 * 16);
    GX_DISPATCH(dtype, rope_scalar_kernel<T><<<grid, kThreads, 0, st>>>((T*)dst, (const T*)src, dst_stride, src_stride, cs, sn, tokens, seq_len, n_heads, head_dim, sign, interleaved));
    return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const void* gu, void* out, long long rows, int f, int dtype, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (f % 8) return cudaErrorInvalidValue;
    const int grid = grid_for(rows * (f / 8), kThreads * 2, 148 * 16);
    GX_DISPATCH(dtype, swiglu_fwd_kernel<T><<<grid, kThreads, 0, st>>>((const T*)gu, (T*)out, rows, f));
    return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* gu, const void* dout, void* dgu, long long rows, int f, int dtype,
                              cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    if (f % 8) return cudaErrorInvalidValue;
    const int grid = grid_for(rows * (f / 8), kThreads * 2, 148 * 16);
    GX_DISPATCH(dtype, swiglu_bwd_kernel<T><<<grid, kThreads, 0, st>>>((const T*)gu, (const T*)dout, (T*)dgu, rows, f));
    return cudaGetLastError();
}

cudaError_t launch_xent_fwd_bwd(void* logits, const long long* targets, float* loss_rows, long long rows,
                                int v, float grad_scale, long long ignore_index, int dtype, cudaStream_t st) {
    if (rows <= 0) return cudaSuccess;
    const int grid = (int)min(rows, (long long)148 * 8);
    GX_DISPATCH(dtype, xent_kernel<T><<<grid, 1024, 0, st>>>((T*)logits, targets, loss_rows, rows, v, grad_scale, ignore_index));
    return cudaGetLastError();
}

}  // namespace gx
