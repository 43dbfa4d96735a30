// First-step analysis kernels: block-normalised histogram and the period search.
//
//   histogram       per block: absmax, x = g / absmax, bin x over [-1, 1] into
//                   4096 bins (shared-memory int32 counters per CTA, flushed
//                   once with 64-bit global atomics).  Integer counts, so the
//                   result does not depend on scheduling.
//                   Reference: exact_histogram_fused_kernel.cu:19-140.
//   period_errors   for EVERY proper divisor P of numel in ONE launch
//                   (blockIdx.y = divisor): sum over blocks of the within-block
//                   population variance of g^2, accumulated in fp64 with a fixed
//                   assignment of blocks to CTAs, one partial per CTA; the host
//                   sums the partials in index order.  The reference launches
//                   one kernel per divisor, finishes it with a float atomicAdd
//                   and synchronises the host after each
//                   (period_variance_kernel.cu:15-80, partitioning.py:190-234).
#include "common.cuh"
#include "quant.h"

namespace gx {
namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kThreads) histogram_kernel(const T* __restrict__ x, long long nb,
                                                             int period, int bins,
                                                             unsigned long long* __restrict__ counts) {
    extern __shared__ int sh_counts[];
    __shared__ float red[kThreads / 32];
    for (int i = threadIdx.x; i < bins; i += blockDim.x) sh_counts[i] = 0;
    __syncthreads();
    const float scale = (float)bins * 0.5f;
    auto bin_of = [&](float v, float amax) {
        float n = amax > 0.f ? __fdiv_rn(v, amax) : 0.f;
        float t = __fmul_rn(__fadd_rn(n, 1.0f), scale);
        int b = (t >= 0.f) ? (int)floorf(t) : 0;
        return min(b, bins - 1);
    };
    if (period <= 32) {
        // a thread owns whole blocks
        for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nb;
             b += (long long)gridDim.x * blockDim.x) {
            const T* p = x + b * period;
            float amax = 0.f;
            for (int e = 0; e < period; ++e) amax = fmaxf(amax, fabsf(to_f<T>(p[e])));
            for (int e = 0; e < period; ++e) atomicAdd(&sh_counts[bin_of(to_f<T>(p[e]), amax)], 1);
        }
    } else if (period <= 2048) {
        // a warp owns a block
        const int lane = threadIdx.x & 31;
        const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
        for (long long b = wid; b < nb; b += nw) {
            const T* p = x + b * period;
            float amax = 0.f;
            for (int e = lane; e < period; e += 32) amax = fmaxf(amax, fabsf(to_f<T>(p[e])));
            amax = warp_max(amax);
            for (int e = lane; e < period; e += 32) atomicAdd(&sh_counts[bin_of(to_f<T>(p[e]), amax)], 1);
        }
    } else {
        // the CTA owns a block
        for (long long b = blockIdx.x; b < nb; b += gridDim.x) {
            const T* p = x + b * period;
            float amax = 0.f;
            for (int e = threadIdx.x; e < period; e += blockDim.x) amax = fmaxf(amax, fabsf(to_f<T>(p[e])));
            amax = warp_max(amax);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
            __syncthreads();
            amax = red[0];
#pragma unroll
            for (int i = 1; i < kThreads / 32; ++i) amax = fmaxf(amax, red[i]);
            for (int e = threadIdx.x; e < period; e += blockDim.x)
                atomicAdd(&sh_counts[bin_of(to_f<T>(p[e]), amax)], 1);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < bins; i += blockDim.x) {
        const int c = sh_counts[i];
        if (c) atomicAdd(counts + i, (unsigned long long)c);
    }
}

template <typename T>
__device__ __forceinline__ double sq_or_id(const T* p, long long i, bool squared) {
    const float v = to_f<T>(p[i]);
    return squared ? (double)v : (double)__fmul_rn(v, v);
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// partials[d * gridDim.x + blockIdx.x] = sum over this CTA's blocks of var_b
template <typename T>
__global__ void __launch_bounds__(kThreads) period_errors_kernel(const T* __restrict__ x, long long numel,
                                                                 const long long* __restrict__ divisors,
                                                                 bool squared, double* __restrict__ partials) {
    __shared__ double red[kThreads / 32];
    __shared__ double bc;
    const long long P = divisors[blockIdx.y];
    const long long nb = numel / P;
    const double invP = 1.0 / (double)P;
    double acc = 0.0;  // meaningful in thread 0 of a worker
    if (P <= 32) {
        for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < nb;
             b += (long long)gridDim.x * blockDim.x) {
            const long long o = b * P;
            double s = 0.0;
            for (int e = 0; e < (int)P; ++e) s += sq_or_id(x, o + e, squared);
            const double mean = s * invP;
            double v = 0.0;
            for (int e = 0; e < (int)P; ++e) { const double dlt = sq_or_id(x, o + e, squared) - mean; v += dlt * dlt; }
            acc += v * invP;
        }
    } else if (P <= 8192) {
        const int lane = threadIdx.x & 31;
        const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
        const long long nw = ((long long)gridDim.x * blockDim.x) >> 5;
        for (long long b = wid; b < nb; b += nw) {
            const long long o = b * P;
            double s = 0.0;
            for (long long e = lane; e < P; e += 32) s += sq_or_id(x, o + e, squared);
            const double mean = warp_sum_d(s) * invP;
            double v = 0.0;
            for (long long e = lane; e < P; e += 32) { const double dlt = sq_or_id(x, o + e, squared) - mean; v += dlt * dlt; }
            v = warp_sum_d(v);
            if (lane == 0) acc += v * invP;
        }
    } else {
        for (long long b = blockIdx.x; b < nb; b += gridDim.x) {
            const long long o = b * P;
            double s = 0.0;
            for (long long e = threadIdx.x; e < P; e += blockDim.x) s += sq_or_id(x, o + e, squared);
            s = warp_sum_d(s);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
            __syncthreads();
            if (threadIdx.x == 0) {
                double t = 0.0;
                for (int i = 0; i < kThreads / 32; ++i) t += red[i];
                bc = t * invP;
            }
            __syncthreads();
            const double mean = bc;
            double v = 0.0;
            for (long long e = threadIdx.x; e < P; e += blockDim.x) { const double dlt = sq_or_id(x, o + e, squared) - mean; v += dlt * dlt; }
            v = warp_sum_d(v);
            __syncthreads();
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
            __syncthreads();
            if (threadIdx.x == 0) {
                double t = 0.0;
                for (int i = 0; i < kThreads / 32; ++i) t += red[i];
                acc += t * invP;
            }
        }
    }
    // CTA total in a fixed order
    acc = warp_sum_d(acc);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int i = 0; i < kThreads / 32; ++i) t += red[i];
        partials[(long long)blockIdx.y * gridDim.x + blockIdx.x] = t;
    }
}

// idx[i] <- map[idx[i]] in place: moves stored momentum indices onto a re-learned codebook
// (map[c] = nearest new codeword of old codeword c).  16 indices per access.
__global__ void __launch_bounds__(kThreads) remap_indices_kernel(uint8_t* __restrict__ idx,
                                                                 const uint8_t* __restrict__ map,
                                                                 long long numel) {
    __shared__ uint8_t m[256];
    if (threadIdx.x < 256) m[threadIdx.x] = map[threadIdx.x];
    __syncthreads();
    const long long n16 = numel / 16;
    uint4* v = reinterpret_cast<uint4*>(idx);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n16;
         i += (long long)gridDim.x * blockDim.x) {
        uint4 r = v[i];
        uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            w[k] = (uint32_t)m[w[k] & 0xff] | ((uint32_t)m[(w[k] >> 8) & 0xff] << 8) |
                   ((uint32_t)m[(w[k] >> 16) & 0xff] << 16) | ((uint32_t)m[w[k] >> 24] << 24);
        }
        v[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (long long i = n16 * 16 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
         i += (long long)gridDim.x * blockDim.x)
        idx[i] = m[idx[i]];
}

// out[i] = codebook[idx[i]] * mag[i / period]: the dense momentum of a tensor (checkpoint
// export, resharding).  Eight elements per thread when period % 8 == 0.
template <typename T>
__global__ void __launch_bounds__(kThreads) dequantize_kernel(const uint8_t* __restrict__ idx,
                                                              const float* __restrict__ mag,
                                                              const float* __restrict__ codebook,
                                                              long long numel, long long period,
                                                              T* __restrict__ out, int vec) {
    __shared__ float cb[256];
    if (threadIdx.x < 256) cb[threadIdx.x] = codebook[threadIdx.x];
    __syncthreads();
    if (vec) {
        const long long n8 = numel / 8;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8;
             i += (long long)gridDim.x * blockDim.x) {
            int ix[8];
            load_idx8(idx + i * 8, ix);
            const float m = mag[(i * 8) / period];
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = cb[ix[e]] * m;
            Vec8<T>::store(out + i * 8, v);
        }
        return;
    }
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
         i += (long long)gridDim.x * blockDim.x)
        out[i] = from_f<T>(cb[idx[i]] * mag[i / period]);
}

}  // namespace

cudaError_t launch_histogram(const void* x, int dtype, long long numel, int period, int bins,
                             unsigned long long* counts, int sm_count, cudaStream_t st) {
    if (numel <= 0) return cudaSuccess;
    const long long nb = numel / period;
    long long want;
    if (period <= 32) want = (nb + kThreads - 1) / kThreads;
    else if (period <= 2048) want = (nb + 7) / 8;
    else want = nb;
    const int grid = (int)max(1LL, min(want, (long long)sm_count * 8));
    const size_t sh = (size_t)bins * sizeof(int);
    switch (dtype) {
        case 0: histogram_kernel<float><<<grid, kThreads, sh, st>>>((const float*)x, nb, period, bins, counts); break;
        case 1: histogram_kernel<__nv_bfloat16><<<grid, kThreads, sh, st>>>((const __nv_bfloat16*)x, nb, period, bins, counts); break;
        case 2: histogram_kernel<__half><<<grid, kThreads, sh, st>>>((const __half*)x, nb, period, bins, counts); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_period_errors(const void* x, int dtype, long long numel, const long long* divisors_dev,
                                 int n_div, bool squared, double* partials, int ctas_per_div,
                                 cudaStream_t st) {
    if (numel <= 0 || n_div <= 0) return cudaSuccess;
    dim3 grid(ctas_per_div, n_div);
    switch (dtype) {
        case 0: period_errors_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, numel, divisors_dev, squared, partials); break;
        case 1: period_errors_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, numel, divisors_dev, squared, partials); break;
        case 2: period_errors_kernel<__half><<<grid, kThreads, 0, st>>>((const __half*)x, numel, divisors_dev, squared, partials); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_remap_indices(uint8_t* idx, const uint8_t* map, long long numel, int sm_count,
                                 cudaStream_t st) {
    if (numel <= 0) return cudaSuccess;
    if (reinterpret_cast<uintptr_t>(idx) % 16) return cudaErrorInvalidValue;
    const long long want = (numel / 16 + kThreads - 1) / kThreads;
    const int grid = (int)max(1LL, min(want, (long long)sm_count * 8));
    remap_indices_kernel<<<grid, kThreads, 0, st>>>(idx, map, numel);
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const uint8_t* idx, const float* mag, const float* codebook, long long numel,
                              long long period, void* out, int dtype, int sm_count, cudaStream_t st) {
    if (numel <= 0) return cudaSuccess;
    if (period <= 0) return cudaErrorInvalidValue;
    const int esz = dtype == 0 ? 4 : 2;
    const int vec = (period % 8 == 0 && numel % 8 == 0 && reinterpret_cast<uintptr_t>(idx) % 8 == 0 &&
                     reinterpret_cast<uintptr_t>(out) % (8 * esz) == 0) ? 1 : 0;
    const long long want = ((vec ? numel / 8 : numel) + kThreads - 1) / kThreads;
    const int grid = (int)max(1LL, min(want, (long long)sm_count * 8));
    switch (dtype) {
        case 0: dequantize_kernel<float><<<grid, kThreads, 0, st>>>(idx, mag, codebook, numel, period, (float*)out, vec); break;
        case 1: dequantize_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>(idx, mag, codebook, numel, period, (__nv_bfloat16*)out, vec); break;
        case 2: dequantize_kernel<__half><<<grid, kThreads, 0, st>>>(idx, mag, codebook, numel, period, (__half*)out, vec); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace gx
