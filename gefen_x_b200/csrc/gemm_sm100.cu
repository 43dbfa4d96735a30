// bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), TMA-fed.
//
//   C[b] = alpha * op(A[b]) * op(B[b]) + beta * D[b]        (fp32 accumulate, bf16 out)
//
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: per-CTA cp.async.bulk.tensor loads into a 4-stage ring of
//               128B-swizzled shared-memory tiles, completion on mbarriers
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma (cta_group::1,
//               kind::f16, M=128, N=BN, K=16) reading shared-memory descriptors and
//               accumulating into one of two TMEM buffers; tcgen05.commit frees the
//               stage / publishes the accumulator
//   warps 2-5   epilogue: tcgen05.ld (32x32b.x32) the finished accumulator, scale, add
//               beta * D, convert and store, while the MMA warp already works on the
//               next tile in the other TMEM buffer
//
// Operands may be K-major (row-major [rows, K]) or MN-major (row-major [K, rows]),
// which gives the NT / NN / TN products used by the Newton-Schulz chain
// (reference src/gefen/gefen_muon.py:278-287 calls cuBLAS through torch.addmm for
// these) and by the all-gather-fused projection.  Every mbarrier wait is bounded:
// on time-out the kernel raises an abort flag, records kWaitTimeout in the status
// word, drains, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "gemm_sm100.h"

namespace gx {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kGemmThreads = 192;      // 6 warps
constexpr uint32_t kTmemCols = 512;
constexpr long long kSpinLimit = 1ll << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the budget ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (long long it = 0; it < kSpinLimit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// ---- TMA ----------------------------------------------------------------------
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- tcgen05 ----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2, descriptor version 1).
//   K-major tile : rows of 128 B (64 bf16 along K), 8-row groups 1024 B apart (SBO).
//   MN-major tile: rows of 128 B (64 bf16 along M/N) indexed by K, 8-row groups 1024 B
//                  apart (SBO); the next 64 elements along M/N start LBO bytes further.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;          // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;          // SWIZZLE_128B
    return d;
}

struct SharedStorage {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct PeerBases { const void* p[kMaxSrc]; };

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// The first `fetch_ctas` CTAs of an all-gather-fused launch: they pull the peers' row
// shards of B into the local staging matrix segment by segment (own rows first, then the
// peers in ring order) and publish one flag per segment once every fetch CTA has
// finished its part of it.
__device__ void ag_fetch_role(const AgParams& ag, PeerBases bases) {
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long nthreads = (long long)ag.fetch_ctas * blockDim.x;
    constexpr int U = 8;
    for (int s = 0; s < ag.n_segs; ++s) {
        const GatherSeg seg = ag.segs[s];
        const long long units = ag.seg_meta[3 * s];
        const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(bases.p[seg.src_rank]) + seg.src_off);
        uint4* dp = reinterpret_cast<uint4*>(ag.dst_base + seg.dst_off);
        for (long long u0 = tid; u0 < units; u0 += nthreads * U) {
            uint4 v[U];
#pragma unroll
            for (int j = 0; j < U; ++j) { const long long u = u0 + j * nthreads; if (u < units) v[j] = sp[u]; }
#pragma unroll
            for (int j = 0; j < U; ++j) { const long long u = u0 + j * nthreads; if (u < units) dp[u] = v[j]; }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t prev = atomicAdd(ag.count + s, 1u);
            if (prev + 1u == ag.count_target) st_release_gpu(ag.flags + s, ag.epoch);
        }
    }
}

// Producer side: before the first B tile of column block n0 is loaded, every segment that
// overlaps rows [n0, n0 + BN) of the staging matrix must have landed (bounded wait).
__device__ bool ag_wait_rows(const AgParams& ag, int n0, int bn, volatile int* abort_flag) {
    for (int s = 0; s < ag.n_segs; ++s) {
        const long long r0 = ag.seg_meta[3 * s + 1], nr = ag.seg_meta[3 * s + 2];
        if (r0 < n0 + bn && r0 + nr > n0) {
            bool ok = false;
            for (long long it = 0; it < kSpinLimit; ++it) {
                if ((int32_t)(ld_acquire_gpu(ag.flags + s) - ag.epoch) >= 0) { ok = true; break; }
                if ((it & 255) == 255 && *abort_flag) return false;
                __nanosleep(100);
            }
            if (!ok) { *abort_flag = 1; return false; }
        }
    }
    asm volatile("fence.proxy.async;" ::: "memory");   // peer data written through the generic proxy -> TMA reads
    return true;
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 GemmParams p, AgParams ag, PeerBases bases) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // carve: [stages x A tile][stages x B tile][barriers]
    constexpr uint32_t kABytes = BM * BK * 2;
    constexpr uint32_t kBBytes = BN * BK * 2;
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* smA = base;
    unsigned char* smB = base + kStages * kABytes;
    SharedStorage* ss = reinterpret_cast<SharedStorage*>(smB + kStages * kBBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &ss->abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kStages; ++i) { mbar_init(&ss->full[i], 1); mbar_init(&ss->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&ss->tmem_full[i], 1); mbar_init(&ss->tmem_empty[i], 4); }
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) tmem_alloc(&ss->tmem_base, kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;

    const int k_blocks = (p.K + BK - 1) / BK;
    const int tiles_per_batch = p.m_tiles * p.n_tiles;
    // all-gather-fused launches reserve the first CTAs for fetching; the others share the tiles
    const int first_worker = ag.enabled ? ag.fetch_ctas : 0;
    const int worker = (int)blockIdx.x - first_worker;
    const int n_workers = (int)gridDim.x - first_worker;
    const bool is_fetch = ag.enabled && (int)blockIdx.x < ag.fetch_ctas;
    // tile -> (batch, m0, n0); fused launches visit the column blocks in arrival order
    auto coords = [&](int tile, int& b, int& m0, int& n0) {
        b = tile / tiles_per_batch;
        const int t = tile - b * tiles_per_batch;
        m0 = (t % p.m_tiles) * BM;
        int nt = t / p.m_tiles;
        if (ag.enabled) nt = ag.tile_order[nt];
        n0 = nt * BN;
    };

    if (is_fetch) {
        ag_fetch_role(ag, bases);
    } else if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int waited_n0 = -1;
            for (int tile = worker; tile < p.total_tiles && ok; tile += n_workers) {
                int b, m0, n0;
                coords(tile, b, m0, n0);
                if (ag.enabled && n0 != waited_n0) {
                    if (!ag_wait_rows(ag, n0, BN, abort_flag)) { ok = false; break; }
                    waited_n0 = n0;
                }
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&ss->empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(&ss->full[stage], kABytes + kBBytes);
                    unsigned char* a_dst = smA + stage * kABytes;
                    unsigned char* b_dst = smB + stage * kBBytes;
                    const int k0 = kb * BK;
                    if (!p.a_mn_major) {
                        tma_load_3d(a_dst, &tmA, &ss->full[stage], k0, m0, b);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j)
                            tma_load_3d(a_dst + j * (BK * 128), &tmA, &ss->full[stage], m0 + 64 * j, k0, b);
                    }
                    if (!p.b_mn_major) {
                        tma_load_3d(b_dst, &tmB, &ss->full[stage], k0, n0, b);
                    } else {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j)
                            tma_load_3d(b_dst + j * (BK * 128), &tmB, &ss->full[stage], n0 + 64 * j, k0, b);
                    }
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------- MMA issuer --------------------------------
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)(p.a_mn_major ? 1 : 0) << 15) |
                                   ((uint32_t)(p.b_mn_major ? 1 : 0) << 16) |
                                   ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = worker; tile < p.total_tiles && ok; tile += n_workers) {
                if (!mbar_wait(&ss->tmem_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&ss->full[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smA + stage * kABytes);
                    const uint32_t b_addr = smem_u32(smB + stage * kBBytes);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = p.a_mn_major
                            ? make_desc(a_addr + k * (UMMA_K * 128), BK * 128, 1024)
                            : make_desc(a_addr + k * (UMMA_K * 2), 16, 1024);
                        const uint64_t bd = p.b_mn_major
                            ? make_desc(b_addr + k * (UMMA_K * 128), BK * 128, 1024)
                            : make_desc(b_addr + k * (UMMA_K * 2), 16, 1024);
                        umma_bf16(d_tmem, ad, bd, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&ss->empty[stage]);            // stage reusable once these MMAs retire
                    if (++stage == kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&ss->tmem_full[acc]);              // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // --------------------------------- epilogue ----------------------------------
        const int q = warp & 3;                                // TMEM lane quadrant of this warp
        int acc = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        for (int tile = worker; tile < p.total_tiles && ok; tile += n_workers) {
            int b, m0, n0;
            coords(tile, b, m0, n0);
            if (!mbar_wait(&ss->tmem_full[acc], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const int row = m0 + q * 32 + lane;
            __nv_bfloat16* crow = p.C + (long long)b * p.batch_stride_c + (long long)row * p.ldc;
            const __nv_bfloat16* drow =
                p.D ? p.D + (long long)b * p.batch_stride_d + (long long)row * p.ldd : nullptr;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + c), r);
                tmem_ld_wait();
                const int col0 = n0 + c;
                if (row < p.M && col0 < p.N) {
#pragma unroll
                    for (int v8 = 0; v8 < 4; ++v8) {
                        const int col = col0 + v8 * 8;
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v8 * 8 + e]) * p.alpha;
                        if (col + 8 <= p.N && p.vec_ok) {
                            if (drow) {
                                float dd[8];
                                Vec8<__nv_bfloat16>::load(drow + col, dd);
#pragma unroll
                                for (int e = 0; e < 8; ++e) f[e] += p.beta * dd[e];
                            }
                            Vec8<__nv_bfloat16>::store(crow + col, f);
                        } else {
                            for (int e = 0; e < 8; ++e) {
                                if (col + e < p.N) {
                                    float v = f[e];
                                    if (drow) v += p.beta * __bfloat162float(drow[col + e]);
                                    crow[col + e] = __float2bfloat16_rn(v);
                                }
                            }
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&ss->tmem_empty[acc]);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    }

    // teardown: everybody meets, the allocating warp frees TMEM
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && ss->abort_flag && p.status) atomicExch(p.status, (int)kWaitTimeout);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Causal attention forward on the same building blocks (flash form: the score tile lives in
// TMEM, the probabilities go through shared memory straight into the second product, nothing
// of size S x S touches HBM).
//
//   one CTA (128 threads) per 128 query rows of one (sequence, KV head); the group's query heads
//   are stacked along the rows, so row r belongs to head r / seq and query position r % seq;
//   per 128-key tile:  TMA K, V  ->  S = Q K^T (tcgen05, TMEM cols 0..127)
//                      thread t owns row t: running maximum, p = exp2((s - m) * scale * log2e),
//                      P (bf16) written in the 128-byte-swizzled K-major layout the MMA reads
//                      PV (tcgen05, TMEM cols 128..) -> o = o * alpha + PV in registers
//   epilogue: o / l -> bf16, log-sum-exp per row.
// Every mbarrier wait is bounded; a time-out is voted CTA-wide and ends the kernel cleanly.
struct FlashShared {
    uint64_t bar_q, bar_kv[2], bar_s, bar_o;
    uint32_t tmem_base;
    int abort_flag;
};

template <int HD>
__global__ void __launch_bounds__(128, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, FlashParams p) {
    constexpr int KB = HD / 64;                       // 64-wide head-dimension blocks
    constexpr uint32_t kBlk = 128 * 128;              // one [128 rows x 128 B] operand block
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = base;                         // [KB][128 x 128 B]   K-major A
    constexpr uint32_t kKV = KB * kBlk;               // bytes of one K (or V) tile
    unsigned char* sK = sQ + KB * kBlk;               // [2 buffers][KB][128 x 128 B]   K-major B
    unsigned char* sV = sK + 2 * kKV;                 // [2 buffers][2][KB][64 keys x 128 B]  MN-major B
    unsigned char* sP = sV + 2 * kKV;                 // [2][128 x 128 B]   K-major A (keys along K)
    FlashShared* ss = reinterpret_cast<FlashShared*>(sP + 2 * kBlk);

    const int tid = threadIdx.x, warp = tid >> 5;
    volatile int* abort_flag = &ss->abort_flag;
    const int n_row_tiles = p.rows / 128;
    const int rt = n_row_tiles - 1 - (int)blockIdx.x;          // long rows first
    const int b = blockIdx.y;
    const int r0 = rt * 128;
    const int s0 = r0 % p.seq;                                 // query position of the tile's first row
    const int n_kv = s0 / 128 + 1;

    if (tid == 0) {
        mbar_init(&ss->bar_q, 1);
        mbar_init(&ss->bar_kv[0], 1);
        mbar_init(&ss->bar_kv[1], 1);
        mbar_init(&ss->bar_s, 1);
        mbar_init(&ss->bar_o, 1);
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_tmap(&tmQ);
        prefetch_tmap(&tmK);
        prefetch_tmap(&tmV);
    }
    if (warp == 0) tmem_alloc(&ss->tmem_base, 256);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);

    if (tid == 0) {
        mbar_expect_tx(&ss->bar_q, KB * kBlk);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) tma_load_3d(sQ + kb * kBlk, &tmQ, &ss->bar_q, 64 * kb, r0, b);
    }
    const uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(128 >> 3) << 17) |
                             ((uint32_t)(128 >> 4) << 24);
    const uint32_t idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(HD >> 3) << 17) |
                             ((uint32_t)(128 >> 4) << 24);
    const float sl = p.scale * 1.4426950408889634f;
    float o[HD];
#pragma unroll
    for (int e = 0; e < HD; ++e) o[e] = 0.f;
    float m = -INFINITY, l = 0.f;
    uint32_t ph_s = 0, ph_o = 0;
    // K / V tiles are double-buffered: tile j + 1 is fetched while tile j is being processed
    auto fetch_kv = [&](int j) {
        const int bf = j & 1;
        mbar_expect_tx(&ss->bar_kv[bf], 2 * kKV);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
            tma_load_3d(sK + bf * kKV + kb * kBlk, &tmK, &ss->bar_kv[bf], 64 * kb, 128 * j, b);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int jn = 0; jn < KB; ++jn)
                tma_load_3d(sV + bf * kKV + (h * KB + jn) * 8192, &tmV, &ss->bar_kv[bf], 64 * jn,
                            128 * j + 64 * h, b);
    };
    int issued[2] = {0, 0}, landed[2] = {0, 0};     // per buffer: loads started / seen complete
    if (tid == 0) { fetch_kv(0); issued[0] = 1; }
    bool ok = mbar_wait(&ss->bar_q, 0, abort_flag);
    ok = __syncthreads_and(ok);

    for (int j = 0; j < n_kv && ok; ++j) {
        const int bf = j & 1;
        // buffer (j + 1) & 1 held tile j - 1, whose products have retired (bar_o of that tile)
        if (tid == 0 && j + 1 < n_kv) { fetch_kv(j + 1); ++issued[bf ^ 1]; }
        ok = mbar_wait(&ss->bar_kv[bf], (uint32_t)((j >> 1) & 1), abort_flag);
        if (ok) ++landed[bf];
        ok = __syncthreads_and(ok);
        if (!ok) break;
        const unsigned char* cK = sK + bf * kKV;
        const unsigned char* cV = sV + bf * kKV;
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem_base, make_desc(smem_u32(sQ + kb * kBlk) + k * 32, 16, 1024),
                              make_desc(smem_u32(cK + kb * kBlk) + k * 32, 16, 1024), idesc_s,
                              (kb > 0 || k > 0) ? 1u : 0u);
            umma_commit(&ss->bar_s);
        }
        ok = mbar_wait(&ss->bar_s, ph_s, abort_flag);
        ph_s ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after();

        // ---- softmax of this thread's row --------------------------------------------------
        const bool diag = (j == n_kv - 1);
        const int qpos = s0 + tid;
        float mx = m;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + (uint32_t)(c * 32), r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int col = 128 * j + c * 32 + e;
                const float v = (diag && col > qpos) ? -INFINITY : __uint_as_float(r[e]);
                mx = fmaxf(mx, v);
            }
        }
        const float alpha = exp2f((m - mx) * sl);          // 0 on the first tile (m = -inf)
        float rs = 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + (uint32_t)(c * 32), r);
            tmem_ld_wait();
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const int col = 128 * j + c * 32 + e;
                float p0 = exp2f((__uint_as_float(r[e]) - mx) * sl);
                float p1 = exp2f((__uint_as_float(r[e + 1]) - mx) * sl);
                if (diag && col > qpos) p0 = 0.f;
                if (diag && col + 1 > qpos) p1 = 0.f;
                const __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                // the row sum uses the rounded probabilities, like the product that consumes them
                rs += __low2float(h) + __high2float(h);
                w[e >> 1] = *reinterpret_cast<const uint32_t*>(&h);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int cc = c * 4 + q4;                 // 16-byte chunk of the 128-key row
                const int kb = cc >> 3, ci = cc & 7;
                uint4* dst = reinterpret_cast<uint4*>(sP + kb * kBlk + tid * 128 + ((ci ^ (tid & 7)) << 4));
                *dst = make_uint4(w[4 * q4], w[4 * q4 + 1], w[4 * q4 + 2], w[4 * q4 + 3]);
            }
        }
        l = l * alpha + rs;
        m = mx;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P: generic writes -> MMA reads
        tc_fence_before();
        __syncthreads();

        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem_base + 128, make_desc(smem_u32(sP + h * kBlk) + k * 32, 16, 1024),
                              make_desc(smem_u32(cV + h * KB * 8192) + k * 2048, 8192, 1024), idesc_o,
                              (h > 0 || k > 0) ? 1u : 0u);
            umma_commit(&ss->bar_o);
        }
        ok = mbar_wait(&ss->bar_o, ph_o, abort_flag);
        ph_o ^= 1;
        ok = __syncthreads_and(ok);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(lane_base + (uint32_t)(128 + c * 32), r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[c * 32 + e] = o[c * 32 + e] * alpha + __uint_as_float(r[e]);
        }
        tc_fence_before();
        __syncthreads();          // K, V, P and both TMEM regions are free for the next tile
    }

    if (ok) {
        const float inv = 1.0f / l;
        const long long row = (long long)b * p.rows + r0 + tid;
        __nv_bfloat16* orow = p.out + row * HD;
#pragma unroll
        for (int v8 = 0; v8 < HD / 8; ++v8) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = o[v8 * 8 + e] * inv;
            Vec8<__nv_bfloat16>::store(orow + v8 * 8, f);
        }
        p.lse[row] = m * p.scale + logf(l);
    }
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && ss->abort_flag) {
        // a load may still be in flight: give it one more bounded chance to land before the
        // shared memory it targets is released
        volatile int no_abort = 0;
        for (int bf = 0; bf < 2; ++bf)
            if (issued[bf] > landed[bf]) mbar_wait(&ss->bar_kv[bf], (uint32_t)(landed[bf] & 1), &no_abort);
        if (p.status) atomicExch(p.status, (int)kWaitTimeout);
    }
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 256);
    }
}

}  // namespace

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// Operand stored row-major [batch, outer, inner] with leading dimension ld (elements).
bool make_map(CUtensorMap* map, const __nv_bfloat16* base, long long inner, long long outer, long long batch,
              long long ld, long long batch_stride, int box_inner, int box_outer) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    if (batch_stride <= 0) batch_stride = outer * ld;
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)batch_stride * 2};
    cuuint32_t box[3] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<__nv_bfloat16*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int BN>
cudaError_t launch_bn(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, int sm_count,
                      cudaStream_t st) {
    constexpr size_t smem = (size_t)kStages * (BM * BK * 2 + BN * BK * 2) + sizeof(SharedStorage) + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    p.m_tiles = (p.M + BM - 1) / BM;
    p.n_tiles = (p.N + BN - 1) / BN;
    p.total_tiles = p.m_tiles * p.n_tiles * p.batch;
    const int grid = p.total_tiles < sm_count ? p.total_tiles : sm_count;
    AgParams ag{};
    PeerBases pb{};
    gemm_bf16_kernel<BN><<<grid, kGemmThreads, smem, st>>>(ta, tb, p, ag, pb);
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_ag_bf16(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* Bstage, long long ldb,
                                GemmParams p, AgParams ag, const void* const* peer_bases, int world,
                                int sm_count, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0) return cudaSuccess;
    if ((lda % 8) || (ldb % 8) || world < 1 || world > kMaxSrc) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(Bstage) % 16)) return cudaErrorInvalidValue;
    if (ag.fetch_ctas < 1 || ag.fetch_ctas >= sm_count) return cudaErrorInvalidValue;
    constexpr int BN = 256;
    p.batch = 1;
    p.a_mn_major = 0;
    p.b_mn_major = 0;
    CUtensorMap ta, tb;
    if (!make_map(&ta, A, p.K, p.M, 1, lda, 0, BK, BM) || !make_map(&tb, Bstage, p.K, p.N, 1, ldb, 0, BK, BN))
        return cudaErrorInvalidValue;
    p.vec_ok = (p.ldc % 8 == 0) && (reinterpret_cast<uintptr_t>(p.C) % 16 == 0);
    p.D = nullptr;
    constexpr size_t smem = (size_t)kStages * (BM * BK * 2 + BN * BK * 2) + sizeof(SharedStorage) + 1024;
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return e;
    p.m_tiles = (p.M + BM - 1) / BM;
    p.n_tiles = (p.N + BN - 1) / BN;
    p.total_tiles = p.m_tiles * p.n_tiles;
    ag.enabled = 1;
    PeerBases pb{};
    for (int i = 0; i < world; ++i) pb.p[i] = peer_bases[i];
    // every CTA must be resident at once: the GEMM CTAs wait on flags the fetch CTAs set
    gemm_bf16_kernel<BN><<<sm_count, kGemmThreads, smem, st>>>(ta, tb, p, ag, pb);
    return cudaGetLastError();
}

cudaError_t launch_gemm_bf16(const __nv_bfloat16* A, long long lda, long long batch_stride_a,
                             const __nv_bfloat16* B, long long ldb, long long batch_stride_b,
                             GemmParams p, int sm_count, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0 || p.batch <= 0) return cudaSuccess;
    if ((lda % 8) || (ldb % 8) || (batch_stride_a % 8) || (batch_stride_b % 8)) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(A) % 16) || (reinterpret_cast<uintptr_t>(B) % 16)) return cudaErrorInvalidValue;
    const long long tiles256 = (long long)((p.M + BM - 1) / BM) * ((p.N + 255) / 256) * p.batch;
    const bool use128 = p.N <= 128 || tiles256 < sm_count;
    const int bn = use128 ? 128 : 256;
    CUtensorMap ta, tb;
    bool ok = p.a_mn_major ? make_map(&ta, A, p.M, p.K, p.batch, lda, batch_stride_a, 64, BK)
                           : make_map(&ta, A, p.K, p.M, p.batch, lda, batch_stride_a, BK, BM);
    ok = ok && (p.b_mn_major ? make_map(&tb, B, p.N, p.K, p.batch, ldb, batch_stride_b, 64, BK)
                             : make_map(&tb, B, p.K, p.N, p.batch, ldb, batch_stride_b, BK, bn));
    if (!ok) return cudaErrorInvalidValue;
    p.vec_ok = (p.ldc % 8 == 0) && (reinterpret_cast<uintptr_t>(p.C) % 16 == 0) && (p.batch_stride_c % 8 == 0) &&
               (!p.D || ((p.ldd % 8 == 0) && (reinterpret_cast<uintptr_t>(p.D) % 16 == 0) &&
                         (p.batch_stride_d % 8 == 0)));
    return use128 ? launch_bn<128>(ta, tb, p, sm_count, st) : launch_bn<256>(ta, tb, p, sm_count, st);
}

cudaError_t launch_flash_attention_fwd(const __nv_bfloat16* q, const __nv_bfloat16* k, const __nv_bfloat16* v,
                                       int head_dim, FlashParams p, cudaStream_t st) {
    if (p.batch <= 0 || p.rows <= 0) return cudaSuccess;
    if ((head_dim != 64 && head_dim != 128) || p.seq % 128 || p.rows % p.seq) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(q) % 16) || (reinterpret_cast<uintptr_t>(k) % 16) ||
        (reinterpret_cast<uintptr_t>(v) % 16) || (reinterpret_cast<uintptr_t>(p.out) % 16))
        return cudaErrorInvalidValue;
    CUtensorMap tq, tk, tv;
    if (!make_map(&tq, q, head_dim, p.rows, p.batch, head_dim, (long long)p.rows * head_dim, 64, 128) ||
        !make_map(&tk, k, head_dim, p.seq, p.batch, head_dim, (long long)p.seq * head_dim, 64, 128) ||
        !make_map(&tv, v, head_dim, p.seq, p.batch, head_dim, (long long)p.seq * head_dim, 64, 64))
        return cudaErrorInvalidValue;
    const int kb = head_dim / 64;
    const size_t smem = (size_t)(kb * 16384 + 4 * kb * 16384 + 2 * 16384) + sizeof(FlashShared) + 1024;
    dim3 grid(p.rows / 128, p.batch);
    cudaError_t e;
    if (head_dim == 128) {
        e = cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        flash_fwd_kernel<128><<<grid, 128, smem, st>>>(tq, tk, tv, p);
    } else {
        e = cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        flash_fwd_kernel<64><<<grid, 128, smem, st>>>(tq, tk, tv, p);
    }
    return cudaGetLastError();
}

}  // namespace gx
