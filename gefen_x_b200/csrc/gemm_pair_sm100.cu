// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 with a 256 x BN accumulator tile per pair.
//
//   C = alpha * op(A) * op(B) + beta * D           (fp32 accumulate in TMEM, bf16 out)
//
// Two CTAs on neighbouring SMs (a cluster of two) work on one 256 x BN output tile.  Each
// CTA fetches its own 128 rows of A and its own half of B (BN / 2 rows) with plain per-CTA
// TMA tile loads -- no load is shared or multicast -- and holds the 128 x BN half of the
// accumulator that belongs to its rows in its own tensor memory.  The MMA reads the A tile
// of each CTA once and both halves of B, so the shared-memory traffic per FLOP is two
// thirds of the single-CTA kernel's (gemm_sm100.cu), which is what that kernel is bound by.
//
// Roles per CTA (192 threads, persistent over the tiles of its pair):
//   warp 0      TMA producer.  Ring of kStages [A 128x64 | B (BN/2)x64] tiles, 128-byte
//               swizzle.  The "full" barrier of a stage lives in the leader CTA (rank 0)
//               and counts the bytes of both CTAs' loads (cp.async.bulk.tensor with
//               .cta_group::2 lets the peer's loads signal it).
//   warp 1      leader only: one thread issues tcgen05.mma.cta_group::2 (M 256, N BN,
//               K 16) and commits to the "empty" / "accumulator full" barriers of both
//               CTAs at once (tcgen05.commit ... multicast::cluster).  In both CTAs this
//               warp owns the TMEM allocation.
//   warps 2-5   epilogue.  tcgen05.ld the finished accumulator (two TMEM buffers, so the
//               next tile's MMAs run meanwhile), apply the epilogue, pack bf16 rows into a
//               swizzled shared-memory tile and hand it to a TMA store (clipped at the
//               matrix edge).  Then arrive on the leader's "accumulator empty" barrier.
//
// Epilogues: plain (alpha, beta * D: the residual add of the o_proj / down_proj outputs),
// SwiGLU forward fused into the gate/up projection (the pair's B halves are the gate rows
// and the up rows of the same columns; writes [gate | up] and silu(gate) * up), and the
// SwiGLU derivative fused into the down_proj input-gradient product.
//
// Tail wave: with T tiles on P pairs the last T mod P tiles would leave most pairs idle, and a
// narrower tile does not help (256 x 128 tiles need 1.5x the operand bytes per FLOP and run into
// the L2 -> SM bandwidth).  Instead the tiles of the tail are split along K over the idle pairs;
// each split parks its fp32 partial in a workspace, and the split that arrives last (an atomic
// counter per 32-row slice, nobody waits) sums the partials in split order and runs the epilogue.
//
// Schedule: static (pair p takes units p, p + P, ...: reproducible placement) or, when the launch
// is given a counter, dynamic: the leader's producer thread draws the next unit with an atomic add
// one unit ahead, publishes it to the other roles of both CTAs through a small ring in shared
// memory (mbarriers; a plain store into the peer's shared memory for the peer's copy), and every
// pair simply takes the next unit when it is free.  A pair that shares its SMs with another stream's
// kernels (reduce-scatter, copies) then falls behind without holding the whole product back.
//
// The reference multiplies through cuBLAS (src/gefen/gefen_muon.py:278-287 and its
// benchmark model benchmarks/training_matrix/tiny_qwen.py:168-181).  Every mbarrier wait
// is bounded; on time-out the roles drain, TMEM is freed and kWaitTimeout is recorded.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"
#include "gemm_sm100.h"
#include "sm100_ptx.cuh"

namespace gx {
namespace {

using namespace ptx;

constexpr int kBM = 128;              // accumulator rows held by one CTA (pair tile: 256)
constexpr int kBK = 64;               // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUK = 16;
constexpr int kPairThreads = 192;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kEpiTile = 32 * 128;          // one warp's staging tile: 32 rows x 64 bf16
constexpr int kEpiBufs = 4;                      // staging tiles per epilogue warp (TMA stores in flight)

constexpr int kRing = 4;                         // work units published ahead of their consumers

struct PairShared {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint64_t ring_full[kRing];       // dynamic schedule: unit published (one arrival, from the leader's producer)
    uint64_t ring_empty[kRing];      // leader only: every consumer of both CTAs has read the unit (10 arrivals)
    int ring_unit[kRing];
    uint32_t tmem_base;
    int abort_flag;
};

template <int BN> struct PairTile {
    // 5 x 32 KB (or 6 x 24 KB) of operand stages + 64 KB of epilogue staging + barriers <= 227 KB
    static constexpr int kHalfN = BN / 2;
    static constexpr uint32_t kABytes = kBM * kBK * 2;
    static constexpr uint32_t kBBytes = kHalfN * kBK * 2;
    static constexpr int kStages = (BN == 256) ? 5 : 6;
    static constexpr uint32_t kEpiBytes = 4 * kEpiBufs * kEpiTile;
    static constexpr size_t kSmem = (size_t)kStages * (kABytes + kBBytes) + kEpiBytes + sizeof(PairShared) + 1024;
    static_assert(kSmem <= 232448, "shared memory of the pair kernel exceeds 227 KB");
};

struct PairMaps {
    CUtensorMap a, b, c0, c1, c2;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// 64 bf16 of one row (32 packed words) -> row `lane` of a swizzled [32 x 128 B] tile
__device__ __forceinline__ void write_row_swizzled(unsigned char* tile, int lane, const uint32_t (&w)[32]) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint4* dst = reinterpret_cast<uint4*>(tile + lane * 128 + ((j ^ (lane & 7)) << 4));
        *dst = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
    }
}

// 64 bf16 of row `row` starting at column `col` of a row-major matrix (zero outside it)
__device__ __forceinline__ void load_row64(const __nv_bfloat16* base, long long ld, int row, int col, int rows,
                                           int cols, bool vec_ok, uint32_t (&w)[32]) {
    if (row < rows && col + 64 <= cols && vec_ok) {
        const uint4* src = reinterpret_cast<const uint4*>(base + (long long)row * ld + col);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint4 v = src[j];
            w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            float a = 0.f, b = 0.f;
            if (row < rows && col + 2 * j < cols) a = __bfloat162float(base[(long long)row * ld + col + 2 * j]);
            if (row < rows && col + 2 * j + 1 < cols) b = __bfloat162float(base[(long long)row * ld + col + 2 * j + 1]);
            w[j] = pack2(a, b);
        }
    }
}

__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// the `bytes` of row `row` starting at column `col` that an epilogue thread will read later
__device__ __forceinline__ void prefetch_row(const __nv_bfloat16* base, long long ld, int row, int col, int rows,
                                             int cols, int n) {
    if (row >= rows) return;
    const char* ptr = reinterpret_cast<const char*>(base + (long long)row * ld + col);
    for (int b = 0; b < n * 2; b += 128)
        if (col + b / 2 < cols) prefetch_l2(ptr + b);
}

// Tile index -> (row tile, column tile).  Tiles are visited in groups of `group_m` row tiles,
// column-major inside a group, so that the ~74 tiles in flight at any time form a near-square
// block of the output: they share the fewest distinct operand panels, and the panels of a group
// are fetched from HBM once while the other operand streams past.
__device__ __forceinline__ void tile_coords(const PairParams& p, int tile, int& mt, int& nt) {
    if (p.symmetric) {
        // tiles on and below the diagonal, row by row: tile = mt (mt + 1) / 2 + nt, nt <= mt
        mt = (int)((sqrtf(8.0f * (float)tile + 1.0f) - 1.0f) * 0.5f);
        while ((mt + 1) * (mt + 2) / 2 <= tile) ++mt;        // the float root can be one off either way
        while (mt * (mt + 1) / 2 > tile) --mt;
        nt = tile - mt * (mt + 1) / 2;
        return;
    }
    const int per_group = p.group_m * p.n_tiles;
    const int g = tile / per_group;
    const int first_m = g * p.group_m;
    const int gsize = min(p.group_m, p.m_tiles - first_m);
    const int r = tile - g * per_group;
    mt = first_m + r % gsize;
    nt = r / gsize;
}

// One unit of work of a pair: a whole tile, or one K-range of a tile of the tail wave.
struct Work {
    int tile, kb0, kb1, split, n_split;
};
__device__ __forceinline__ bool get_work(const PairParams& p, int it, int pair, int n_pairs, int k_blocks, Work& w) {
    const int full_iters = p.full_tiles / n_pairs;
    if (it < full_iters) {
        w.tile = pair + it * n_pairs;
        w.kb0 = 0; w.kb1 = k_blocks; w.split = 0; w.n_split = 1;
        return true;
    }
    if (it == full_iters && pair < p.rem_tiles * p.splits) {
        w.tile = p.full_tiles + pair / p.splits;
        w.split = pair % p.splits;
        w.n_split = p.splits;
        w.kb0 = (int)((long long)w.split * k_blocks / p.splits);
        w.kb1 = (int)((long long)(w.split + 1) * k_blocks / p.splits);
        return true;
    }
    return false;
}

__device__ __forceinline__ void decode_unit(const PairParams& p, int unit, int k_blocks, Work& w) {
    if (unit < p.full_tiles) {
        w.tile = unit;
        w.kb0 = 0; w.kb1 = k_blocks; w.split = 0; w.n_split = 1;
    } else {
        const int v = unit - p.full_tiles;
        w.tile = p.full_tiles + v / p.splits;
        w.split = v % p.splits;
        w.n_split = p.splits;
        w.kb0 = (int)((long long)w.split * k_blocks / p.splits);
        w.kb1 = (int)((long long)(w.split + 1) * k_blocks / p.splits);
    }
}

// The sequence of work units of one role.  Static schedule: computed.  Dynamic schedule: the
// leader's producer thread is the fetcher (atomic counter, one unit ahead, publishes into the ring
// of both CTAs); every other role reads the ring and acknowledges on the leader's ring_empty.
struct UnitStream {
    const PairParams& p;
    PairShared* ss;
    volatile int* abort_flag;
    int pair, n_pairs, k_blocks;
    uint32_t rank;
    bool fetcher;        // leader CTA, producer thread
    bool warp_role;      // called by all 32 lanes of a warp (epilogue): lane 0 acknowledges
    int it;
    int pending;         // fetcher: the unit fetched ahead (-2: nothing fetched yet)

    __device__ UnitStream(const PairParams& p_, PairShared* ss_, volatile int* ab, int pair_, int n_pairs_, int kb,
                          uint32_t rank_, bool fetcher_, bool warp_role_)
        : p(p_), ss(ss_), abort_flag(ab), pair(pair_), n_pairs(n_pairs_), k_blocks(kb), rank(rank_),
          fetcher(fetcher_), warp_role(warp_role_), it(0), pending(-2) {}

    __device__ int fetch_and_publish() {
        const int slot = it % kRing;
        const uint32_t ph = (uint32_t)((it / kRing) & 1);
        ++it;
        if (!mbar_wait_cluster(&ss->ring_empty[slot], ph ^ 1, abort_flag)) return -1;
        const unsigned n_units = (unsigned)(p.full_tiles + p.rem_tiles * p.splits);
        const unsigned u = atomicAdd(p.sched, 1u);
        const int unit = u < n_units ? (int)u : -1;
        // every pair draws exactly one value past the end; the very last of them rewinds the counter
        if (unit < 0 && u == n_units + (unsigned)n_pairs - 1u) atomicExch(p.sched, 0u);
        ss->ring_unit[slot] = unit;
        st_shared_cluster_u32(mapa(smem_u32(&ss->ring_unit[slot]), 1), (uint32_t)unit);
        mbar_arrive(&ss->ring_full[slot]);
        mbar_arrive_cluster(mapa(smem_u32(&ss->ring_full[slot]), 1));
        return unit;
    }

    __device__ bool next(Work& w) {
        if (p.sched == nullptr) return get_work(p, it++, pair, n_pairs, k_blocks, w);
        int unit;
        if (fetcher) {
            if (pending == -2) pending = fetch_and_publish();
            unit = pending;
            if (unit >= 0) pending = fetch_and_publish();
        } else {
            const int slot = it % kRing;
            const uint32_t ph = (uint32_t)((it / kRing) & 1);
            ++it;
            if (!mbar_wait_cluster(&ss->ring_full[slot], ph, abort_flag)) return false;
            unit = *reinterpret_cast<volatile int*>(&ss->ring_unit[slot]);
            if (warp_role) __syncwarp();
            if (!warp_role || (threadIdx.x & 31) == 0)
                mbar_arrive_cluster(mapa(smem_u32(&ss->ring_empty[slot]), 0));
        }
        if (unit < 0) return false;
        decode_unit(p, unit, k_blocks, w);
        return true;
    }
};

template <int BN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ PairMaps maps, PairParams p) {
    using TL = PairTile<BN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* smA = base;
    unsigned char* smB = smA + TL::kStages * TL::kABytes;
    unsigned char* smE = smB + TL::kStages * TL::kBBytes;
    PairShared* ss = reinterpret_cast<PairShared*>(smE + TL::kEpiBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    volatile int* abort_flag = &ss->abort_flag;

    if (threadIdx.x == 0) {
        for (int i = 0; i < TL::kStages; ++i) { mbar_init(&ss->full[i], 1); mbar_init(&ss->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&ss->tmem_full[i], 1); mbar_init(&ss->tmem_empty[i], 8); }
        for (int i = 0; i < kRing; ++i) { mbar_init(&ss->ring_full[i], 1); mbar_init(&ss->ring_empty[i], 10); }
        ss->abort_flag = 0;
        mbar_init_fence();
        prefetch_tmap(&maps.a);
        prefetch_tmap(&maps.b);
        prefetch_tmap(&maps.c0);
    }
    if (warp == 1) tmem_alloc<2>(&ss->tmem_base, kTmemCols);
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;

    // a k-block is one 128-byte row of each operand tile: 64 bf16 or 128 e4m3 elements of K
    constexpr bool kF8 = EPI == kEpiScaledE4m3;
    constexpr int kKElems = kF8 ? 2 * kBK : kBK;
    const int k_blocks = (p.K + kKElems - 1) / kKElems;
    const int pair = (int)(blockIdx.x >> 1);
    const int n_pairs = (int)(gridDim.x >> 1);

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            Work wk;
            UnitStream units(p, ss, abort_flag, pair, n_pairs, k_blocks, rank, rank == 0, false);
            while (units.next(wk)) {
                int mt, nt;
                tile_coords(p, wk.tile, mt, nt);
                const int m0 = mt * 256 + (int)rank * kBM;
                // plain: this CTA's half of the BN columns.  SwiGLU forward: rank 0 fetches the
                // gate rows, rank 1 the up rows of the same BN / 2 columns.
                const int nb0 = (EPI == kEpiSwigluFwd) ? (int)rank * p.F + nt * TL::kHalfN
                                                       : nt * BN + (int)rank * TL::kHalfN;
                bool ok = true;
                for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
                    if (!mbar_wait(&ss->empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) mbar_expect_tx(&ss->full[stage], 2 * (TL::kABytes + TL::kBBytes));
                    const uint32_t bar = mapa(smem_u32(&ss->full[stage]), 0);
                    unsigned char* a_dst = smA + stage * TL::kABytes;
                    unsigned char* b_dst = smB + stage * TL::kBBytes;
                    const int k0 = kb * kKElems;
                    if (!p.a_mn_major) {
                        tma_load_2d_pair(a_dst, &maps.a, bar, k0, m0);
                    } else {
#pragma unroll
                        for (int j = 0; j < kBM / 64; ++j)
                            tma_load_2d_pair(a_dst + j * (kBK * 128), &maps.a, bar, m0 + 64 * j, k0);
                    }
                    if (!p.b_mn_major) {
                        tma_load_2d_pair(b_dst, &maps.b, bar, k0, nb0);
                    } else {
#pragma unroll
                        for (int j = 0; j < TL::kHalfN / 64; ++j)
                            tma_load_2d_pair(b_dst + j * (kBK * 128), &maps.b, bar, nb0 + 64 * j, k0);
                    }
                    if (++stage == TL::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
            }
        }
    } else if (warp == 1) {
        // --------------------------- MMA issuer (leader CTA) ---------------------------
        if (rank == 0 && lane == 0) {
            const uint32_t idesc = kF8 ? make_idesc_e4m3(256, BN)
                                       : make_idesc(256, BN, p.a_mn_major != 0, p.b_mn_major != 0);
            // descriptors differ from stage to stage and from k-step to k-step only in the start address
            // (low word, in 16-byte units): keep the constant part and add
            const uint64_t a_desc0 = p.a_mn_major ? make_desc(smem_u32(smA), kBK * 128, 1024) : make_desc(smem_u32(smA), 16, 1024);
            const uint64_t b_desc0 = p.b_mn_major ? make_desc(smem_u32(smB), kBK * 128, 1024) : make_desc(smem_u32(smB), 16, 1024);
            const uint32_t a_kstep = (p.a_mn_major ? kUK * 128 : kUK * 2) >> 4;
            const uint32_t b_kstep = (p.b_mn_major ? kUK * 128 : kUK * 2) >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            Work wk;
            UnitStream units(p, ss, abort_flag, pair, n_pairs, k_blocks, rank, false, false);
            while (ok && units.next(wk)) {
                if (!mbar_wait(&ss->tmem_empty[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
                for (int kb = wk.kb0; kb < wk.kb1; ++kb) {
                    if (!mbar_wait(&ss->full[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t ad = a_desc0 + (uint64_t)((uint32_t)stage * (TL::kABytes >> 4));
                    const uint64_t bd = b_desc0 + (uint64_t)((uint32_t)stage * (TL::kBBytes >> 4));
#pragma unroll
                    for (int k = 0; k < kBK / kUK; ++k) {
                        // every instruction consumes 32 bytes of K per row: 16 bf16 or 32 e4m3
                        if constexpr (kF8)
                            umma_f8_pair(d_tmem, ad + (uint64_t)(k * a_kstep), bd + (uint64_t)(k * b_kstep), idesc,
                                         (kb > wk.kb0 || k > 0) ? 1u : 0u);
                        else
                            umma_bf16<2>(d_tmem, ad + (uint64_t)(k * a_kstep), bd + (uint64_t)(k * b_kstep), idesc,
                                         (kb > wk.kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(&ss->empty[stage], 3);        // both CTAs may refill the stage
                    if (++stage == TL::kStages) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&ss->tmem_full[acc], 3);          // accumulator complete in both CTAs
                if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
        }
    } else {
        // --------------------------------- epilogue ----------------------------------
        const int q = warp & 3;                                    // TMEM lane quadrant of this warp
        unsigned char* my_stage = smE + (warp - 2) * kEpiBufs * kEpiTile;
        const uint32_t leader_empty0 = mapa(smem_u32(&ss->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = mapa(smem_u32(&ss->tmem_empty[1]), 0);
        int acc = 0;
        uint32_t acc_phase = 0;
        uint32_t unit = 0;                                         // staging tiles handed to TMA so far
        // pack 64 fp32 values to bf16, stage them and store the [32 x 64] tile at (col, row0)
        auto emit = [&](const CUtensorMap* map, const uint32_t (&w)[32], int col, int row0) {
            unsigned char* tile = my_stage + (unit & (kEpiBufs - 1)) * kEpiTile;
            if (lane == 0) bulk_wait_read<kEpiBufs - 1>();         // the store that last read this buffer is done
            __syncwarp();
            write_row_swizzled(tile, lane, w);
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
                tma_store_2d(map, tile, col, row0);
                bulk_commit();
            }
            ++unit;
        };
        Work wk;
        UnitStream units(p, ss, abort_flag, pair, n_pairs, k_blocks, rank, false, true);
        while (units.next(wk)) {
            int mt, nt;
            tile_coords(p, wk.tile, mt, nt);
            const int row0 = mt * 256 + (int)rank * kBM + q * 32;
            const int row = row0 + lane;
            // what the epilogue will read from global memory: start it towards L2 while the MMAs run
            if constexpr (EPI == kEpiPlain) {
                if (p.D) prefetch_row(p.D, p.ldd, row, nt * BN, p.M, p.N, BN);
            } else if constexpr (EPI == kEpiSwigluBwd) {
                prefetch_row(p.aux, p.ldaux, row, nt * BN, p.M, p.F, BN);
                prefetch_row(p.aux + p.F, p.ldaux, row, nt * BN, p.M, p.F, BN);
            }
            if (!mbar_wait(&ss->tmem_full[acc], acc_phase, abort_flag)) break;
            tc_fence_after();
            const uint32_t t_acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
            float sq = 0.f;                                        // this thread's share of sum(C^2) of the tile
            // one slot per epilogue warp of the launch (static schedule: one writer per slot, reproducible
            // sums), per tile under the dynamic schedule (placement varies: atomic adds) ...
            int sq_slot = p.sched ? ((wk.tile * 8 + (int)rank * 4 + q) & (kSumsqTailBase - 1)) : (int)blockIdx.x * 4 + q;
            // ---- K-split tile: park the partial; only the slice's last arriver goes on ----
            const float* ws_tile = nullptr;                        // set: sum the parked partials
            if (wk.n_split > 1) {
                const int slice = ((wk.tile - p.full_tiles) * 2 + (int)rank) * 4 + q;
                float* ws_slice = p.ws + (size_t)slice * wk.n_split * (BN * 32);
                float* mine = ws_slice + (size_t)wk.split * (BN * 32) + lane;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(t_acc + (uint32_t)c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int e = 0; e < 32; ++e) __stcg(mine + (c + e) * 32, __uint_as_float(r[e]));
                }
                __threadfence();
                __syncwarp();
                uint32_t arrived = 0;
                if (lane == 0) arrived = atomicAdd(p.counters + slice, 1u);
                arrived = __shfl_sync(0xffffffffu, arrived, 0);
                if (arrived + 1u == (uint32_t)wk.n_split) {
                    __threadfence();
                    if (lane == 0) p.counters[slice] = 0;          // ready for the next launch
                    ws_tile = ws_slice + lane;
                    sq_slot = kSumsqTailBase + slice;              // ... or per slice of a tail tile: whichever
                                                                   // split arrives last, the same slot gets the sum
                } else {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                    continue;
                }
            }
            // 64 accumulator columns starting at `c`: from tensor memory, or the partials in split order
            auto load_acc64 = [&](int c, uint32_t (&r)[64]) {
                if (ws_tile == nullptr) {
                    tmem_ld_32x32b_x32(t_acc + (uint32_t)c, r);
                    tmem_ld_32x32b_x32(t_acc + (uint32_t)(c + 32), r + 32);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int e = 0; e < 64; ++e) r[e] = __float_as_uint(__ldcg(ws_tile + (c + e) * 32));
                    for (int sp = 1; sp < wk.n_split; ++sp) {
                        const float* part = ws_tile + (size_t)sp * (BN * 32);
#pragma unroll
                        for (int e = 0; e < 64; ++e)
                            r[e] = __float_as_uint(__uint_as_float(r[e]) + __ldcg(part + (c + e) * 32));
                    }
                }
            };
            if constexpr (EPI == kEpiSwigluFwd) {
                // accumulator columns [0, BN/2) = gate, [BN/2, BN) = up of output columns nt * BN/2 + ...
#pragma unroll 1
                for (int c = 0; c < TL::kHalfN; c += 64) {
                    uint32_t r[64], g[32], u[32];
                    load_acc64(c, r);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        g[j] = pack2(__uint_as_float(r[2 * j]) * p.alpha, __uint_as_float(r[2 * j + 1]) * p.alpha);
                    load_acc64(TL::kHalfN + c, r);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        u[j] = pack2(__uint_as_float(r[2 * j]) * p.alpha, __uint_as_float(r[2 * j + 1]) * p.alpha);
                    const int col = nt * TL::kHalfN + c;
                    emit(&maps.c0, g, col, row0);
                    emit(&maps.c1, u, col, row0);
                    // silu(gate) * up from the rounded values, as the unfused kernel reads them back
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float g0 = lo_f(g[j]), g1 = hi_f(g[j]);
                        const float a0 = g0 / (1.f + __expf(-g0)) * lo_f(u[j]);
                        const float a1 = g1 / (1.f + __expf(-g1)) * hi_f(u[j]);
                        g[j] = pack2(a0, a1);
                    }
                    emit(&maps.c2, g, col, row0);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 64) {
                    uint32_t r[64], w[32];
                    load_acc64(c, r);
                    const int col = nt * BN + c;
                    if constexpr (EPI == kEpiScaledE4m3) {
                        // dequantise: one scale per output row (A's row) and one per column (B's row);
                        // the column scales are the same addresses for every lane (broadcast loads)
                        const float sa = row < p.M ? __ldg(p.row_scale + row) : 0.f;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int c0 = col + 2 * j;
                            const float s0 = c0 < p.N ? __ldg(p.col_scale + c0) : 0.f;
                            const float s1 = c0 + 1 < p.N ? __ldg(p.col_scale + c0 + 1) : 0.f;
                            w[j] = pack2(__uint_as_float(r[2 * j]) * sa * s0, __uint_as_float(r[2 * j + 1]) * sa * s1);
                        }
                        emit(&maps.c0, w, col, row0);
                    } else if constexpr (EPI == kEpiPlain) {
                        if (p.D) {
                            uint32_t d[32];
                            load_row64(p.D, p.ldd, row, col, p.M, p.N, p.d_vec_ok != 0, d);
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                w[j] = pack2(__uint_as_float(r[2 * j]) * p.alpha + p.beta * lo_f(d[j]),
                                             __uint_as_float(r[2 * j + 1]) * p.alpha + p.beta * hi_f(d[j]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                w[j] = pack2(__uint_as_float(r[2 * j]) * p.alpha, __uint_as_float(r[2 * j + 1]) * p.alpha);
                        }
                        if (p.sumsq != nullptr && row < p.M) {
                            // sum of squares of the values as stored (bf16), for the gradient norm
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                const float a = lo_f(w[j]), b = hi_f(w[j]);
                                if (col + 2 * j < p.N) sq = __fmaf_rn(a, a, sq);
                                if (col + 2 * j + 1 < p.N) sq = __fmaf_rn(b, b, sq);
                            }
                        }
                        emit(&maps.c0, w, col, row0);
                    } else {
                        // SwiGLU derivative: the accumulator is d(act); aux = [gate | up] of the forward pass
                        uint32_t g[32], u[32];
                        load_row64(p.aux, p.ldaux, row, col, p.M, p.F, p.d_vec_ok != 0, g);
                        load_row64(p.aux + p.F, p.ldaux, row, col, p.M, p.F, p.d_vec_ok != 0, u);
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            // d(act) rounded to bf16 first, as the unfused path stores it
                            const uint32_t dzp = pack2(__uint_as_float(r[2 * j]) * p.alpha,
                                                       __uint_as_float(r[2 * j + 1]) * p.alpha);
                            float dg[2], du[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const float gv = h ? hi_f(g[j]) : lo_f(g[j]);
                                const float uv = h ? hi_f(u[j]) : lo_f(u[j]);
                                const float dz = h ? hi_f(dzp) : lo_f(dzp);
                                const float sg = 1.f / (1.f + __expf(-gv));
                                dg[h] = dz * uv * sg * (1.f + gv * (1.f - sg));
                                du[h] = dz * (gv * sg);
                            }
                            w[j] = pack2(dg[0], dg[1]);
                            u[j] = pack2(du[0], du[1]);
                        }
                        emit(&maps.c0, w, col, row0);
                        emit(&maps.c1, u, col, row0);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
            if constexpr (EPI == kEpiPlain) {
                if (p.sumsq != nullptr) {
                    // fixed order: lanes by shuffle tree, tiles of this warp in visiting order, one writer per slot
                    sq = warp_sum(sq);
                    if (lane == 0) {
                        if (p.sched) atomicAdd(p.sumsq + sq_slot, sq); else p.sumsq[sq_slot] += sq;
                    }
                }
            }
        }
        if (lane == 0) bulk_wait<0>();                             // all stores of this warp have landed
    }

    // teardown: both CTAs meet (nobody may leave while the peer can still signal its barriers or
    // read its operand tiles), then the allocating warps free the tensor memory
    tc_fence_before();
    cluster_sync_all();
    if (threadIdx.x == 0 && ss->abort_flag && p.status) atomicExch(p.status, (int)kWaitTimeout);
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn pair_encode_fn() {
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

// row-major [outer, inner] bf16 matrix with leading dimension ld (elements)
bool map2d(CUtensorMap* map, const __nv_bfloat16* base, long long inner, long long outer, long long ld,
           int box_inner, int box_outer) {
    EncodeTiledFn fn = pair_encode_fn();
    if (!fn || inner <= 0 || outer <= 0) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// row-major [outer, inner] matrix of 1-byte elements with leading dimension ld (bytes)
bool map2d_u8(CUtensorMap* map, const void* base, long long inner, long long outer, long long ld,
              int box_inner, int box_outer) {
    EncodeTiledFn fn = pair_encode_fn();
    if (!fn || inner <= 0 || outer <= 0) return false;
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld};
    cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

template <int BN, int EPI>
cudaError_t launch_pair(const PairMaps& maps, PairParams p, int sm_count, cudaStream_t st) {
    constexpr size_t smem = PairTile<BN>::kSmem;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int n_cols = (EPI == kEpiSwigluFwd) ? PairTile<BN>::kHalfN : BN;   // output columns per tile
    p.m_tiles = (p.M + 255) / 256;
    p.n_tiles = (p.N + n_cols - 1) / n_cols;
    p.total_tiles = p.symmetric ? p.m_tiles * (p.m_tiles + 1) / 2 : p.m_tiles * p.n_tiles;
    // row-tile group of the visiting order: all rows when A is small enough to stay in L2 (then B
    // streams through once), otherwise 8 (near-square waves)
    p.group_m = ((long long)p.M * p.K * (EPI == kEpiScaledE4m3 ? 1 : 2) <= (48ll << 20) || p.m_tiles <= 8) ? p.m_tiles : 8;
    const int max_pairs = sm_count / 2 > 0 ? sm_count / 2 : 1;
    constexpr int k_elems = (EPI == kEpiScaledE4m3) ? 2 * kBK : kBK;     // elements of K per 128-byte row
    const int k_blocks = (p.K + k_elems - 1) / k_elems;
    int pairs = max_pairs;
    p.full_tiles = (p.total_tiles / max_pairs) * max_pairs;
    p.rem_tiles = p.total_tiles - p.full_tiles;
    p.splits = 1;
    if (p.rem_tiles > 0 && p.ws != nullptr && p.counters != nullptr) {
        int sp = max_pairs / p.rem_tiles;                    // idle pairs per tail tile
        if (sp > kMaxSplits) sp = kMaxSplits;
        if (sp > k_blocks / 4) sp = k_blocks / 4;            // at least four k-blocks per split
        if (sp > 1 && (long long)p.rem_tiles * sp * 2 * 4 * BN * 32 <= p.ws_floats &&
            p.rem_tiles * 2 * 4 <= p.n_counters)
            p.splits = sp;
    }
    if (p.full_tiles == 0) pairs = p.rem_tiles * p.splits;   // fewer tiles than pairs: one unit each
    if (pairs < 1) pairs = 1;
    gemm_pair_kernel<BN, EPI><<<2 * pairs, kPairThreads, smem, st>>>(maps, p);
    return cudaGetLastError();
}

// C[j, i] = C[i, j] for every element of the 256 x 256 tiles strictly below the diagonal: completes a
// symmetric product of which only those tiles and the diagonal ones were computed.  32 x 32 blocks
// through shared memory, coalesced on both sides.
__global__ void __launch_bounds__(256) mirror_lower_kernel(__nv_bfloat16* __restrict__ C, long long ldc, int M) {
    __shared__ __nv_bfloat16 t[32][33];
    const int bi = blockIdx.y, bj = blockIdx.x;              // 32-row / 32-column block of the source
    if ((bi >> 3) <= (bj >> 3)) return;                      // its 256-tile lies on or above the diagonal
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = bi * 32 + ty + 8 * k, c = bj * 32 + tx;
        if (r < M && c < M) t[ty + 8 * k][tx] = C[(long long)r * ldc + c];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = bj * 32 + ty + 8 * k, c = bi * 32 + tx; // destination row / column
        if (r < M && c < M) C[(long long)r * ldc + c] = t[tx][ty + 8 * k];
    }
}

}  // namespace

bool gemm_pair_supported(int M, int N, int K) { return M >= 129 && N >= 64 && K >= 64; }

int gemm_pair_pick_bn(int M, int N, int sm_count) {
    // 256 x 128 tiles fetch 1.5x the operand bytes per FLOP of 256 x 256 tiles and are bound by the
    // L2 -> SM bandwidth (measured: 0.85 against 1.5 PFLOP/s on 4096^3), so the narrow tile only
    // serves narrow outputs; the tail wave is balanced by the K-split instead
    (void)M; (void)sm_count;
    return N <= 128 ? 128 : 256;
}

cudaError_t launch_gemm_pair_bf16(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* B, long long ldb,
                                  PairParams p, __nv_bfloat16* C0, long long ldc0, __nv_bfloat16* C1,
                                  long long ldc1, __nv_bfloat16* C2, long long ldc2, int sm_count,
                                  cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0) return cudaSuccess;
    if ((lda % 8) || (ldb % 8) || (ldc0 % 8) || !aligned16(A) || !aligned16(B) || !aligned16(C0))
        return cudaErrorInvalidValue;
    if (p.epi < kEpiPlain || p.epi > kEpiSwigluBwd) return cudaErrorInvalidValue;
    const int bn = p.epi == kEpiSwigluFwd ? 256 : (p.bn ? p.bn : gemm_pair_pick_bn(p.M, p.N, sm_count));
    if (bn != 128 && bn != 256) return cudaErrorInvalidValue;
    PairMaps maps;
    bool ok = p.a_mn_major ? map2d(&maps.a, A, p.M, p.K, lda, 64, kBK) : map2d(&maps.a, A, p.K, p.M, lda, kBK, kBM);
    const long long b_rows = p.epi == kEpiSwigluFwd ? 2ll * p.F : p.N;
    ok = ok && (p.b_mn_major ? map2d(&maps.b, B, b_rows, p.K, ldb, 64, kBK)
                             : map2d(&maps.b, B, p.K, b_rows, ldb, kBK, bn / 2));
    // outputs: every map spans exactly the columns its tiles may touch, so the store clips there
    ok = ok && map2d(&maps.c0, C0, p.N, p.M, ldc0, 64, 32);
    maps.c1 = maps.c0;
    maps.c2 = maps.c0;
    if (p.epi != kEpiPlain) {
        if (!C1 || (ldc1 % 8) || !aligned16(C1)) return cudaErrorInvalidValue;
        ok = ok && map2d(&maps.c1, C1, p.N, p.M, ldc1, 64, 32);
    }
    if (p.epi == kEpiSwigluFwd) {
        if (!C2 || (ldc2 % 8) || !aligned16(C2) || p.b_mn_major || p.F != p.N) return cudaErrorInvalidValue;
        ok = ok && map2d(&maps.c2, C2, p.N, p.M, ldc2, 64, 32);
    }
    if (p.epi == kEpiSwigluBwd) {
        if (!p.aux || p.F != p.N) return cudaErrorInvalidValue;
        p.d_vec_ok = (p.ldaux % 8 == 0) && aligned16(p.aux) && (p.F % 8 == 0);
    } else {
        p.d_vec_ok = !p.D || ((p.ldd % 8 == 0) && aligned16(p.D));
    }
    if (!ok) return cudaErrorInvalidValue;
    if (p.epi == kEpiSwigluFwd) return launch_pair<256, kEpiSwigluFwd>(maps, p, sm_count, st);
    if (p.epi == kEpiSwigluBwd)
        return bn == 256 ? launch_pair<256, kEpiSwigluBwd>(maps, p, sm_count, st)
                         : launch_pair<128, kEpiSwigluBwd>(maps, p, sm_count, st);
    if (p.symmetric) {
        if (p.M != p.N || bn != 256 || p.sumsq != nullptr) return cudaErrorInvalidValue;
        cudaError_t e = launch_pair<256, kEpiPlain>(maps, p, sm_count, st);
        if (e != cudaSuccess) return e;
        const int blocks = (p.M + 31) / 32;
        if (blocks > 8) mirror_lower_kernel<<<dim3(blocks, blocks), 256, 0, st>>>(C0, ldc0, p.M);
        return cudaGetLastError();
    }
    return bn == 256 ? launch_pair<256, kEpiPlain>(maps, p, sm_count, st)
                     : launch_pair<128, kEpiPlain>(maps, p, sm_count, st);
}

// C0[M, N] (bf16) = (A[M, K] B[N, K]^T) * row_scale[m] * col_scale[n], A and B e4m3 bytes, fp32 accumulation on
// the tensor cores (kind::f8f6f4): the row-scaled product of the fp8 Newton-Schulz iteration.
cudaError_t launch_gemm_pair_e4m3(const void* A, long long lda, const void* B, long long ldb, PairParams p,
                                  __nv_bfloat16* C0, long long ldc0, int sm_count, cudaStream_t st) {
    if (p.M <= 0 || p.N <= 0 || p.K <= 0) return cudaSuccess;
    if ((lda % 16) || (ldb % 16) || (ldc0 % 8) || !aligned16(A) || !aligned16(B) || !aligned16(C0) ||
        !p.row_scale || !p.col_scale)
        return cudaErrorInvalidValue;
    p.epi = kEpiScaledE4m3;
    p.a_mn_major = p.b_mn_major = 0;
    p.D = nullptr;
    p.sumsq = nullptr;
    p.d_vec_ok = 1;
    PairMaps maps;
    bool ok = map2d_u8(&maps.a, A, p.K, p.M, lda, 2 * kBK, kBM);
    ok = ok && map2d_u8(&maps.b, B, p.K, p.N, ldb, 2 * kBK, 128);
    ok = ok && map2d(&maps.c0, C0, p.N, p.M, ldc0, 64, 32);
    if (!ok) return cudaErrorInvalidValue;
    maps.c1 = maps.c0;
    maps.c2 = maps.c0;
    return launch_pair<256, kEpiScaledE4m3>(maps, p, sm_count, st);
}

}  // namespace gx
