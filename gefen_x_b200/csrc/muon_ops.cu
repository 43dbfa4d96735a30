// Muon epilogue kernels for sm_100a: NorMuon row normalisation, cautious mask and parameter update
// (reference src/gefen/gefen_muon.py:1192-1300: `_normuon_normalize`, the cautious branch and
// `_apply_muon_update`, a chain of eight to ten elementwise / reduction torch ops per matrix).
//
//   NorMuon:  row_sq[r] = sum_c u[r,c]^2;  v[r] = beta2 v[r] + (1 - beta2) row_sq[r] / cols;
//             denom[r] = sqrt(v[r] / bc) + eps;  frob = sqrt(sum_r row_sq[r]) / ||sqrt(row_sq) / denom||;
//             u[r,:] *= frob / denom[r]                      (the update keeps its Frobenius norm)
//   cautious: mask = (u * g > 0);  u *= mask * (numel / max(sum(mask), 1))
//   apply:    p = p * (1 - lr * wd) - (lr * ratio) * u
//
// Every product is rounded where the torch chain rounds it (the row factor and the cautious rescale
// are cast to the update's dtype before they multiply it; the decayed parameter is stored before the
// update is subtracted), so that the kernels reproduce the torch statement to the last bit of a bf16
// update except for the order of the fp32 sums.  All three kernels are memory-bound: 16-byte vector
// accesses, one CTA per row in the two passes over the matrix.
#include "common.cuh"
#include "muon_ops.h"

namespace gx {
namespace {

constexpr int kThreads = 256;

template <typename T> struct Pack8 {
    static __device__ __forceinline__ void load(const T* p, float (&o)[8]) { Vec8<T>::load(p, o); }
    static __device__ __forceinline__ void store(T* p, const float (&v)[8]) { Vec8<T>::store(p, v); }
};

__device__ __forceinline__ float cta_sum_f(float v, float* sh) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sh[i];
    return t;
}

// pass 1: per-row sum of squares and sign agreement with the gradient
template <typename T>
__global__ void __launch_bounds__(kThreads) muon_row_stats_kernel(MuonEpilogue e) {
    __shared__ float sh[kThreads / 32];
    const T* u = reinterpret_cast<const T*>(e.update);
    const T* g = reinterpret_cast<const T*>(e.grad);
    const bool vec = (e.cols % 8) == 0;
    for (long long r = blockIdx.x; r < e.rows; r += gridDim.x) {
        const T* ur = u + r * e.cols;
        const T* gr = g ? g + r * e.cols : nullptr;
        float sq = 0.f, ag = 0.f;
        if (vec) {
            for (int c = threadIdx.x * 8; c < e.cols; c += kThreads * 8) {
                float a[8];
                Pack8<T>::load(ur + c, a);
#pragma unroll
                for (int k = 0; k < 8; ++k) sq = __fmaf_rn(a[k], a[k], sq);
                if (gr) {
                    float b[8];
                    Pack8<T>::load(gr + c, b);
#pragma unroll
                    for (int k = 0; k < 8; ++k) ag += (a[k] * b[k] > 0.f) ? 1.f : 0.f;
                }
            }
        } else {
            for (int c = threadIdx.x; c < e.cols; c += kThreads) {
                const float a = to_f<T>(ur[c]);
                sq = __fmaf_rn(a, a, sq);
                if (gr) ag += (a * to_f<T>(gr[c]) > 0.f) ? 1.f : 0.f;
            }
        }
        sq = cta_sum_f(sq, sh);
        if (e.cautious) ag = cta_sum_f(ag, sh);
        if (threadIdx.x == 0) {
            e.row_sq[r] = sq;
            if (e.cautious) e.agree[r] = (int)ag;        // exact: a row has fewer than 2^24 elements
        }
    }
}

// pass 2: one CTA, fixed-order sums: NorMuon moments and row factors, the cautious rescale
template <typename T>
__global__ void __launch_bounds__(1024) muon_row_factors_kernel(MuonEpilogue e) {
    __shared__ float sh[32];
    const float bc = e.scal[0];
    float s_sq = 0.f, s_scaled = 0.f, s_agree = 0.f;
    for (long long r = threadIdx.x; r < e.rows; r += blockDim.x) {
        const float sq = e.row_sq[r];
        if (e.normuon) {
            const float v = __fmaf_rn(e.v[r], e.beta2, sq * ((1.0f - e.beta2) / (float)e.cols));
            e.v[r] = v;
            const float denom = sqrtf(v / bc) + e.eps;
            e.row_scale[r] = denom;                       // the factor needs the global norms first
            s_sq += sq;
            s_scaled += sq / (denom * denom);
        }
        if (e.cautious) s_agree += (float)e.agree[r];     // exact below 2^24 per thread; summed as doubles below
    }
    s_sq = cta_sum_f(s_sq, sh);
    s_scaled = cta_sum_f(s_scaled, sh);
    s_agree = cta_sum_f(s_agree, sh);
    if (e.normuon) {
        const float frob = sqrtf(s_sq) / fmaxf(sqrtf(s_scaled), 1.17549435e-38f);
        for (long long r = threadIdx.x; r < e.rows; r += blockDim.x)
            e.row_scale[r] = round_to<T>(frob / e.row_scale[r]);      // cast to the update's dtype, as the torch chain does
    }
    if (threadIdx.x == 0) {
        const float total = (float)e.rows * (float)e.cols;
        e.glob[0] = e.cautious ? round_to<T>(total / fmaxf(s_agree, 1.0f)) : 1.0f;
    }
}

// pass 3: write the final update, and the parameter when one is given
template <typename T>
__global__ void __launch_bounds__(kThreads) muon_finish_kernel(MuonEpilogue e) {
    T* u = reinterpret_cast<T*>(e.update);
    const T* g = reinterpret_cast<const T*>(e.grad);
    T* p = reinterpret_cast<T*>(e.param);
    const bool vec = (e.cols % 8) == 0;
    const float cscale = e.glob[0];
    const float lr_ratio = e.scal[1], wdf = e.scal[2];
    for (long long r = blockIdx.x; r < e.rows; r += gridDim.x) {
        const float rs = e.normuon ? e.row_scale[r] : 1.0f;
        T* ur = u + r * e.cols;
        const T* gr = (e.cautious && g) ? g + r * e.cols : nullptr;
        T* pr = p ? p + r * e.cols : nullptr;
        auto one = [&](float a, float b, float pv, float& out_u, float& out_p) {
            if (e.normuon) a = round_to<T>(a * rs);
            if (gr) {
                const float m = (a * b > 0.f) ? 1.0f : 0.0f;
                a = round_to<T>(round_to<T>(a * m) * cscale);
            }
            out_u = a;
            if (pr) {
                if (wdf != 1.0f) pv = round_to<T>(pv * wdf);
                out_p = __fmaf_rn(-lr_ratio, a, pv);
            }
        };
        if (vec) {
            for (int c = threadIdx.x * 8; c < e.cols; c += kThreads * 8) {
                float a[8], b[8], pv[8], ou[8], op[8];
                Pack8<T>::load(ur + c, a);
                if (gr) Pack8<T>::load(gr + c, b);
                if (pr) Pack8<T>::load(pr + c, pv);
#pragma unroll
                for (int k = 0; k < 8; ++k) one(a[k], gr ? b[k] : 0.f, pr ? pv[k] : 0.f, ou[k], op[k]);
                Pack8<T>::store(ur + c, ou);
                if (pr) Pack8<T>::store(pr + c, op);
            }
        } else {
            for (int c = threadIdx.x; c < e.cols; c += kThreads) {
                float ou, op = 0.f;
                one(to_f<T>(ur[c]), gr ? to_f<T>(gr[c]) : 0.f, pr ? to_f<T>(pr[c]) : 0.f, ou, op);
                ur[c] = from_f<T>(ou);
                if (pr) pr[c] = from_f<T>(op);
            }
        }
    }
}

template <typename T>
cudaError_t run(const MuonEpilogue& e, int sm_count, cudaStream_t st) {
    const int grid = (int)min((long long)sm_count * 8, e.rows);
    if (e.normuon || e.cautious) {
        muon_row_stats_kernel<T><<<grid, kThreads, 0, st>>>(e);
        muon_row_factors_kernel<T><<<1, 1024, 0, st>>>(e);
    }
    muon_finish_kernel<T><<<grid, kThreads, 0, st>>>(e);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_muon_epilogue(const MuonEpilogue& e, int dtype, int sm_count, cudaStream_t st) {
    if (e.rows <= 0 || e.cols <= 0) return cudaSuccess;
    if (!e.update || !e.scal || !e.glob || ((e.normuon || e.cautious) && (!e.row_sq || !e.row_scale)) ||
        (e.normuon && !e.v) || (e.cautious && (!e.grad || !e.agree)))
        return cudaErrorInvalidValue;
    // the 8-wide accesses need 16-byte aligned rows
    const bool aligned = (reinterpret_cast<uintptr_t>(e.update) % 16 == 0) &&
                         (!e.grad || reinterpret_cast<uintptr_t>(e.grad) % 16 == 0) &&
                         (!e.param || reinterpret_cast<uintptr_t>(e.param) % 16 == 0);
    if (!aligned && e.cols % 8 == 0) return cudaErrorInvalidValue;
    switch (dtype) {
        case 0: return run<float>(e, sm_count, st);
        case 1: return run<__nv_bfloat16>(e, sm_count, st);
        case 2: return run<__half>(e, sm_count, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gx
