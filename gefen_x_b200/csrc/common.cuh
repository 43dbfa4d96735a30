// Shared device helpers for the sm_100a kernels: typed vector loads/stores,
// rounding-pinned arithmetic, the codebook search and bounded waits.
//
// Rounding is pinned (__fmul_rn/__fadd_rn, no fused multiply-add) wherever a
// value feeds the quantised momentum, so that the kernels reproduce the torch
// statement of the math (optim/functional.py) bit for bit.  The reference pins
// its rounding for the same reason (reference
// src/gefen/kernels/automatic_gefen_fused_kernel.cu:410-418, :598-603).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gx {

constexpr int kMaxSrc = 8;          // gradient sources (peer slices) summed in-kernel
constexpr int kCodewords = 256;
constexpr int kLutBuckets = 16384;

// ---- status word: kernels never trap; they record why they gave up --------
enum Status : int {
    kOk = 0,
    kWaitTimeout = 1,   // a bounded wait on a peer flag / mbarrier ran out
    kBadArgument = 2,
};

// ---- scalar conversions ----------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// round-trip through the storage type (what writing and re-reading would give)
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

// ---- 8-element vector access -----------------------------------------------
template <typename T> struct Vec8 {
    // 16-bit types: one 16-byte transaction
    static __device__ __forceinline__ void unpack(const uint4& r, float (&o)[8]) {
        const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = to_f<T>(e[i]);
    }
    static __device__ __forceinline__ void load(const T* p, float (&o)[8]) {
        unpack(*reinterpret_cast<const uint4*>(p), o);
    }
    static __device__ __forceinline__ void store(T* p, const float (&v)[8]) {
        uint4 r;
        T* e = reinterpret_cast<T*>(&r);
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = from_f<T>(v[i]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};
// bf16: packed conversions (two elements per instruction)
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void unpack(const uint4& r, float (&o)[8]) {
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&o)[8]) {
        unpack(*reinterpret_cast<const uint4*>(p), o);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&o)[8]) {
        float4 a = *reinterpret_cast<const float4*>(p);
        float4 b = *reinterpret_cast<const float4*>(p + 4);
        o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
        o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};

__device__ __forceinline__ void unpack_idx8(const uint2& r, int (&o)[8]) {
    o[0] = r.x & 0xff; o[1] = (r.x >> 8) & 0xff; o[2] = (r.x >> 16) & 0xff; o[3] = r.x >> 24;
    o[4] = r.y & 0xff; o[5] = (r.y >> 8) & 0xff; o[6] = (r.y >> 16) & 0xff; o[7] = r.y >> 24;
}
__device__ __forceinline__ void load_idx8(const uint8_t* p, int (&o)[8]) {
    uint2 r = *reinterpret_cast<const uint2*>(p);
    o[0] = r.x & 0xff; o[1] = (r.x >> 8) & 0xff; o[2] = (r.x >> 16) & 0xff; o[3] = r.x >> 24;
    o[4] = r.y & 0xff; o[5] = (r.y >> 8) & 0xff; o[6] = (r.y >> 16) & 0xff; o[7] = r.y >> 24;
}
__device__ __forceinline__ void store_idx8(uint8_t* p, const int (&v)[8]) {
    uint2 r;
    r.x = (uint32_t)v[0] | ((uint32_t)v[1] << 8) | ((uint32_t)v[2] << 16) | ((uint32_t)v[3] << 24);
    r.y = (uint32_t)v[4] | ((uint32_t)v[5] << 8) | ((uint32_t)v[6] << 16) | ((uint32_t)v[7] << 24);
    *reinterpret_cast<uint2*>(p) = r;
}

// Sum over all ranks of eight bf16 at a multicast address, reduced inside NVSwitch (NVLS): one load
// brings this rank's share of a reduce-scatter instead of one load per peer.  `mc` is the multicast
// mapping of a symmetric buffer (16-byte aligned); the sum is accumulated in fp32 in the switch and
// returned rounded to bf16.  This is a multimem instruction on peer memory, not a TMA load.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(mc)
                 : "memory");
    return r;
}

// Raw (unconverted) chunk of VEC elements: loaded early to keep many requests in
// flight at a low register cost, converted to fp32 only when consumed.
template <typename T, int VEC> struct RawVec {
    static constexpr int kWords = (VEC == 8) ? (int)(sizeof(T) * 2) : 1;
    uint32_t w[kWords];
    __device__ __forceinline__ void load(const T* p) {
        if constexpr (VEC == 8) {
            const uint4* q = reinterpret_cast<const uint4*>(p);
#pragma unroll
            for (int i = 0; i < kWords / 4; ++i) {
                const uint4 r = q[i];
                w[4 * i] = r.x; w[4 * i + 1] = r.y; w[4 * i + 2] = r.z; w[4 * i + 3] = r.w;
            }
        } else {
            w[0] = __float_as_uint(to_f<T>(p[0]));
        }
    }
    // eight bf16 summed over all ranks through the NVLS multicast address `p` (bf16, VEC == 8 only)
    __device__ __forceinline__ void load_mc(const T* p) {
        if constexpr (VEC == 8 && sizeof(T) == 2) {
            const uint4 r = multimem_ld_reduce_bf16x8(p);
            w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
        } else {
            load(p);
        }
    }
    __device__ __forceinline__ void get(float (&o)[VEC]) const {
        if constexpr (VEC == 8) {
            if constexpr (sizeof(T) == 4) {
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(w[i]);
            } else {
                const T* e = reinterpret_cast<const T*>(w);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = to_f<T>(e[i]);
            }
        } else {
            o[0] = __uint_as_float(w[0]);
        }
    }
};
template <int VEC> struct RawIdx {
    uint32_t w[(VEC == 8) ? 2 : 1];
    __device__ __forceinline__ void load(const uint8_t* p) {
        if constexpr (VEC == 8) {
            const uint2 r = *reinterpret_cast<const uint2*>(p);
            w[0] = r.x; w[1] = r.y;
        } else {
            w[0] = p[0];
        }
    }
    __device__ __forceinline__ void get(int (&o)[VEC]) const {
        if constexpr (VEC == 8) unpack_idx8(make_uint2(w[0], w[1]), o);
        else o[0] = (int)w[0];
    }
};

// ---- codebook search --------------------------------------------------------
// The nearest codeword of v is found with the 255 decision thresholds
// thr[i] = fp32((cb[i] + cb[i + 1]) / 2):  index = #{ i : thr[i] < v }, so a value on
// a threshold goes to the lower codeword.  A 16384-bucket table resolves almost
// every value with one load: lut[b] = (thresholds in lower buckets) | (thresholds
// inside bucket b) << 8, with bucket(x) = rint(sat(fma(x, 0.5, 0.5)) * 16383) in
// [0, 16383]; only values whose bucket holds a threshold compare against it.
// NaN maps to index 0.
//
// The codebook itself is replicated per lane in shared memory (entry i of lane l at
// [i * 32 + l]) so that the two data-dependent codeword loads per element never
// collide on a bank.
struct QuantTables {
    const float* cb;          // [256 * 32] lane-replicated codebook
    const float* thr;         // [256] thresholds (entry 255 = +inf)
    const uint16_t* lut;      // [16384]
};

__device__ __forceinline__ float rep_load(const float* t, int i) {
    return t[(i << 5) | (threadIdx.x & 31)];
}

// bucket(x) = round-to-nearest-even(sat(fma(x, 0.5, 0.5)) * 16383): a saturating fma maps [-1, 1]
// to [0, 1] (NaN to 0), a second fma adds 2^23 so that the rounded product lands in the low mantissa
// bits; no clamp and no float-to-int conversion.  Monotonic, and the table is built with the same
// function on the host.
__device__ __forceinline__ uint32_t lut_bucket_bits(float v) {
    const float t = __saturatef(__fmaf_rn(v, 0.5f, 0.5f));
    return __float_as_uint(__fmaf_rn(t, (float)(kLutBuckets - 1), 8388608.0f));
}
__device__ __forceinline__ int lut_bucket(float v) {
    return (int)(lut_bucket_bits(v) & (uint32_t)(kLutBuckets - 1));
}

__device__ __forceinline__ int nearest_index(float v, const QuantTables& q) {
    const uint32_t e = q.lut[lut_bucket(v)];
    int i = (int)(e & 0xffu);
    const int cnt = (int)(e >> 8);
    // first probe without a branch: thr[i] is the first threshold not in a lower bucket, so with no
    // threshold inside this bucket it lies in a higher one and is not below v (the bucket function
    // is monotonic; thr[255] = +inf); buckets with more than one threshold are rare and finish in
    // the loop
    i += (q.thr[i] < v) ? 1 : 0;
    if (cnt > 1) {
        const int hi = (int)(e & 0xffu) + cnt;
        while (i < hi && i > (int)(e & 0xffu) && q.thr[i] < v) ++i;
    }
    return i;
}

// SplitMix64 finaliser of (seed, element index) -> 24 uniform bits in [0, 1).
__device__ __forceinline__ float sr_uniform(uint64_t seed, uint64_t elem) {
    uint64_t z = seed * 0x9E3779B97F4A7C15ull + elem + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(uint32_t)(z >> 40) * (1.0f / 16777216.0f);
}

// Stochastic variant: between the two neighbouring codewords lo <= v <= hi pick
// hi with probability (v - lo) / (hi - lo).
__device__ __forceinline__ int stochastic_index(float v, const QuantTables& q, float u) {
    const int n = nearest_index(v, q);
    const float c = rep_load(q.cb, n);
    int l, r;
    if (v >= c) { l = n; r = min(n + 1, kCodewords - 1); }
    else { l = max(n - 1, 0); r = n; }
    const float lo_v = rep_load(q.cb, l), hi_v = rep_load(q.cb, r);
    if (!(hi_v > lo_v) || v <= lo_v) return (v >= hi_v) ? r : l;
    if (v >= hi_v) return r;
    const float pr = (v - lo_v) / (hi_v - lo_v);
    return (u < pr) ? r : l;
}

// ---- block reductions -------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// float atomic max for non-negative values (their int bit patterns order alike)
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
    atomicMax(reinterpret_cast<int*>(addr), __float_as_int(v));
}

// ---- bounded waits on flags written by another GPU --------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Spin until *flag >= want or the iteration budget runs out.  Returns false on
// timeout; the caller records kWaitTimeout and leaves without touching peers.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t want,
                                             long long max_iters) {
    for (long long it = 0; it < max_iters; ++it) {
        if ((int32_t)(ld_acquire_sys(flag) - want) >= 0) return true;
        __nanosleep(64);
    }
    return false;
}

}  // namespace gx
