// torch operator registrations (namespace gefenx) for the sm_100a kernels.
//
// The kernel files carry no torch headers; this file only unwraps tensors into
// raw pointers, checks devices / dtypes / contiguity, picks the current stream
// and calls the launchers.  Every launcher returns its cudaError_t, which is
// turned into a C++ exception here (the reference validates on the host before
// each raw-pointer launch as well, reference
// src/gefen/kernels/automatic_gefen_fused_kernel.cu:2102-2231).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <map>
#include <mutex>
#include <utility>

#include "attention.h"
#include "comm.h"
#include "fp8_quant.h"
#include "gemm_sm100.h"
#include "model_ops.h"
#include "muon_ops.h"
#include "quant.h"
#include "update.h"

namespace {

using at::Tensor;

inline void check(cudaError_t e, const char* what) {
    TORCH_CHECK(e == cudaSuccess, "gefenx::", what, " failed: ", cudaGetErrorString(e));
}

inline int dtype_code(at::ScalarType t) {
    switch (t) {
        case at::kFloat: return gx::kF32;
        case at::kBFloat16: return gx::kBF16;
        case at::kHalf: return gx::kF16;
        default: TORCH_CHECK(false, "gefenx: unsupported dtype ", t); return -1;
    }
}

inline int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

inline cudaStream_t stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

int64_t desc_size() { return (int64_t)sizeof(gx::TensorDesc); }

gx::LaunchCommon make_common(const Tensor& descs, const Tensor& tile_start, int64_t n_tensors,
                             int64_t total_tiles, const Tensor& codebook, const Tensor& thr,
                             const Tensor& lut, const c10::optional<Tensor>& gscale, const c10::optional<Tensor>& status,
                             int64_t sr_seed, bool stochastic, int64_t wait_iters,
                             const c10::optional<Tensor>& sr_seed_dev = c10::nullopt) {
    TORCH_CHECK(descs.is_cuda() && descs.scalar_type() == at::kByte && descs.is_contiguous(),
                "descs must be a contiguous CUDA uint8 tensor");
    TORCH_CHECK(descs.numel() >= n_tensors * (int64_t)sizeof(gx::TensorDesc), "descs too small");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(descs.data_ptr()) % 16 == 0, "descs must be 16-byte aligned");
    TORCH_CHECK(tile_start.is_cuda() && tile_start.scalar_type() == at::kInt &&
                    tile_start.numel() >= n_tensors + 1,
                "tile_start must be CUDA int32 [n_tensors + 1]");
    TORCH_CHECK(codebook.is_cuda() && codebook.scalar_type() == at::kFloat && codebook.numel() == 256 &&
                    codebook.is_contiguous(),
                "codebook must be CUDA fp32 [256]");
    TORCH_CHECK(lut.is_cuda() && lut.scalar_type() == at::kShort && lut.numel() == 16384 && lut.is_contiguous(),
                "lut must be CUDA int16 [16384]");
    gx::LaunchCommon c{};
    c.descs = reinterpret_cast<const gx::TensorDesc*>(descs.data_ptr());
    c.tile_start = tile_start.data_ptr<int>();
    c.n_tensors = (int)n_tensors;
    c.total_tiles = (int)total_tiles;
    TORCH_CHECK(thr.is_cuda() && thr.scalar_type() == at::kFloat && thr.numel() == 256 && thr.is_contiguous(),
                "thresholds must be CUDA fp32 [256]");
    c.codebook = codebook.data_ptr<float>();
    c.thresholds = thr.data_ptr<float>();
    c.lut = reinterpret_cast<const uint16_t*>(lut.data_ptr<int16_t>());
    c.gscale = nullptr;
    if (gscale.has_value() && gscale->defined()) {
        TORCH_CHECK(gscale->is_cuda() && gscale->scalar_type() == at::kFloat, "gscale must be CUDA fp32");
        c.gscale = gscale->data_ptr<float>();
    }
    c.status = nullptr;
    if (status.has_value() && status->defined()) {
        TORCH_CHECK(status->is_cuda() && status->scalar_type() == at::kInt, "status must be CUDA int32");
        c.status = status->data_ptr<int>();
    }
    c.sr_seed = (unsigned long long)sr_seed;
    c.sr_seed_dev = nullptr;
    if (sr_seed_dev.has_value() && sr_seed_dev->defined()) {
        TORCH_CHECK(sr_seed_dev->is_cuda() && sr_seed_dev->scalar_type() == at::kDouble && sr_seed_dev->numel() == 1,
                    "sr_seed_dev must be a CUDA float64 scalar");
        c.sr_seed_dev = sr_seed_dev->data_ptr<double>();
    }
    c.stochastic = stochastic ? 1 : 0;
    c.wait_iters = wait_iters;
    return c;
}

void block_update(const Tensor& descs, const Tensor& tile_start, int64_t n_tensors, int64_t total_tiles,
                  const Tensor& codebook, const Tensor& thr, const Tensor& lut,
                  const c10::optional<Tensor>& gscale, const c10::optional<Tensor>& status,
                  int64_t dtype, int64_t sr_seed, bool stochastic, const c10::optional<Tensor>& sr_seed_dev) {
    c10::cuda::CUDAGuard guard(descs.device());
    auto c = make_common(descs, tile_start, n_tensors, total_tiles, codebook, thr, lut, gscale, status,
                         sr_seed, stochastic, 0, sr_seed_dev);
    check(gx::launch_block_update(c, (int)dtype, sm_count(), stream()), "block_update");
}

void factored_update(const Tensor& descs, const Tensor& tile_start, int64_t n_tensors,
                     int64_t total_tiles, const Tensor& codebook, const Tensor& thr, const Tensor& lut,
                     const c10::optional<Tensor>& gscale, const c10::optional<Tensor>& status,
                     int64_t dtype, int64_t sr_seed, bool stochastic, int64_t wait_iters,
                     int64_t phases, int64_t epoch, int64_t fast, const c10::optional<Tensor>& sr_seed_dev) {
    // phases bit 0: statistics, bit 1: EMA (+ exchange), bit 2: apply + finalize
    c10::cuda::CUDAGuard guard(descs.device());
    auto c = make_common(descs, tile_start, n_tensors, total_tiles, codebook, thr, lut, gscale, status,
                         sr_seed, stochastic, wait_iters, sr_seed_dev);
    c.epoch = (uint32_t)epoch;
    c.fast = (int)fast;
    // the 16-wide streamed kernels read their own tile prefix behind the 8-wide one
    TORCH_CHECK(fast != 4 || tile_start.numel() >= 2 * (n_tensors + 1),
                "factored_update: the 16-wide kernels need both tile prefixes in tile_start");
    const int sms = sm_count();
    auto st = stream();
    if (phases & 1) check(gx::launch_factored_stats(c, (int)dtype, sms, st), "factored_stats");
    if (phases & 2) check(gx::launch_factored_ema(c, st), "factored_ema");
    if (phases & 4) {
        check(gx::launch_factored_apply(c, (int)dtype, sms, st), "factored_apply");
        check(gx::launch_finalize_magnitude(c, sms, st), "finalize_magnitude");
    }
}

void reduce_sources(const c10::optional<Tensor>& out, at::IntArrayRef src_ptrs, int64_t numel,
                    double scale, const c10::optional<Tensor>& partials, int64_t dtype,
                    int64_t device_index) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_index);
    TORCH_CHECK(src_ptrs.size() >= 1 && src_ptrs.size() <= (size_t)gx::kDescMaxSrc, "1..8 sources");
    const void* src[gx::kDescMaxSrc];
    for (size_t i = 0; i < src_ptrs.size(); ++i) src[i] = reinterpret_cast<const void*>(src_ptrs[i]);
    void* o = nullptr;
    if (out.has_value() && out->defined()) {
        TORCH_CHECK(out->is_cuda() && out->is_contiguous() && out->numel() >= numel, "bad out");
        o = out->data_ptr();
    }
    float* part = nullptr;
    int n_part = 0;
    if (partials.has_value() && partials->defined()) {
        TORCH_CHECK(partials->is_cuda() && partials->scalar_type() == at::kFloat, "partials fp32");
        part = partials->data_ptr<float>();
        n_part = (int)partials->numel();
    }
    check(gx::launch_reduce_sources(o, src, (int)src_ptrs.size(), numel, (float)scale, part, n_part,
                                    (int)dtype, stream()),
          "reduce_sources");
}

void clip_coef(const Tensor& partials, double max_norm, Tensor coef) {
    c10::cuda::CUDAGuard guard(partials.device());
    TORCH_CHECK(partials.is_cuda() && partials.scalar_type() == at::kFloat && partials.is_contiguous());
    TORCH_CHECK(coef.is_cuda() && coef.scalar_type() == at::kFloat && coef.numel() >= 2);
    check(gx::launch_clip_coef(partials.data_ptr<float>(), (int)partials.numel(), (float)max_norm,
                               coef.data_ptr<float>(), stream()),
          "clip_coef");
}

void remap_indices(Tensor idx, const Tensor& map) {
    c10::cuda::CUDAGuard guard(idx.device());
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kByte && idx.is_contiguous());
    TORCH_CHECK(map.is_cuda() && map.scalar_type() == at::kByte && map.is_contiguous() && map.numel() == 256);
    check(gx::launch_remap_indices(idx.data_ptr<uint8_t>(), map.data_ptr<uint8_t>(), idx.numel(), sm_count(),
                                   stream()),
          "remap_indices");
}

void quantize_rows_e4m3(const Tensor& x, const c10::optional<Tensor>& x2, double alpha, double beta, Tensor q,
                        Tensor scale, const c10::optional<Tensor>& y_out) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1,
                "x must be a 2-D bf16 CUDA tensor with unit column stride");
    const int64_t rows = x.size(0), cols = x.size(1);
    const void* x2p = nullptr;
    int64_t ld2 = 0;
    if (x2.has_value()) {
        TORCH_CHECK(x2->is_cuda() && x2->scalar_type() == at::kBFloat16 && x2->sizes() == x.sizes() &&
                    x2->stride(1) == 1 && x2->device() == x.device());
        x2p = x2->data_ptr();
        ld2 = x2->stride(0);
    }
    TORCH_CHECK(q.is_cuda() && q.scalar_type() == at::kFloat8_e4m3fn && q.is_contiguous() && q.sizes() == x.sizes());
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.is_contiguous() && scale.numel() == rows);
    void* yp = nullptr;
    if (y_out.has_value()) {
        TORCH_CHECK(y_out->is_cuda() && y_out->scalar_type() == at::kBFloat16 && y_out->is_contiguous() &&
                    y_out->sizes() == x.sizes());
        TORCH_CHECK(y_out->data_ptr() != x.data_ptr() && y_out->data_ptr() != x2p, "y_out must not alias an input");
        yp = y_out->data_ptr();
    }
    check(gx::launch_quantize_rows_e4m3(x.data_ptr(), x.stride(0), x2p, ld2, (float)alpha, (float)beta, rows, cols,
                                        static_cast<uint8_t*>(q.data_ptr()), scale.data_ptr<float>(), yp, sm_count(),
                                        stream()),
          "quantize_rows_e4m3");
}

void quantize_cols_e4m3_t(const Tensor& x, Tensor colmax, Tensor q_t, Tensor scale_t) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == at::kBFloat16 && x.stride(1) == 1,
                "x must be a 2-D bf16 CUDA tensor with unit column stride");
    const int64_t rows = x.size(0), cols = x.size(1);
    TORCH_CHECK(colmax.is_cuda() && colmax.scalar_type() == at::kInt && colmax.is_contiguous() && colmax.numel() == cols);
    TORCH_CHECK(q_t.is_cuda() && q_t.scalar_type() == at::kFloat8_e4m3fn && q_t.is_contiguous() && q_t.dim() == 2 &&
                q_t.size(0) == cols && q_t.size(1) == rows);
    TORCH_CHECK(scale_t.is_cuda() && scale_t.scalar_type() == at::kFloat && scale_t.is_contiguous() &&
                scale_t.numel() == cols);
    check(gx::launch_quantize_cols_e4m3_t(x.data_ptr(), x.stride(0), rows, cols,
                                          reinterpret_cast<unsigned int*>(colmax.data_ptr<int>()),
                                          static_cast<uint8_t*>(q_t.data_ptr()), scale_t.data_ptr<float>(), stream()),
          "quantize_cols_e4m3_t");
}

void dequantize(const Tensor& idx, const Tensor& mag, const Tensor& codebook, int64_t period, Tensor out) {
    c10::cuda::CUDAGuard guard(idx.device());
    TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kByte && idx.is_contiguous());
    TORCH_CHECK(mag.is_cuda() && mag.scalar_type() == at::kFloat && mag.is_contiguous());
    TORCH_CHECK(codebook.is_cuda() && codebook.scalar_type() == at::kFloat && codebook.numel() == 256);
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.numel() == idx.numel());
    TORCH_CHECK(period > 0 && idx.numel() % period == 0 && mag.numel() * period == idx.numel());
    check(gx::launch_dequantize(idx.data_ptr<uint8_t>(), mag.data_ptr<float>(), codebook.data_ptr<float>(),
                                idx.numel(), period, out.data_ptr(), dtype_code(out.scalar_type()), sm_count(),
                                stream()),
          "dequantize");
}

void histogram(const Tensor& flat, int64_t period, Tensor counts) {
    c10::cuda::CUDAGuard guard(flat.device());
    TORCH_CHECK(flat.is_cuda() && flat.is_contiguous(), "flat must be contiguous CUDA");
    TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kLong && counts.is_contiguous());
    TORCH_CHECK(period > 0 && flat.numel() % period == 0, "period must divide numel");
    TORCH_CHECK(counts.numel() * sizeof(int) <= 48 * 1024, "too many bins for shared memory");
    check(gx::launch_histogram(flat.data_ptr(), dtype_code(flat.scalar_type()), flat.numel(),
                               (int)period, (int)counts.numel(),
                               reinterpret_cast<unsigned long long*>(counts.data_ptr<int64_t>()),
                               sm_count(), stream()),
          "histogram");
}

Tensor period_errors(const Tensor& flat, const Tensor& divisors_dev, bool input_is_squared) {
    c10::cuda::CUDAGuard guard(flat.device());
    TORCH_CHECK(flat.is_cuda() && flat.is_contiguous(), "flat must be contiguous CUDA");
    TORCH_CHECK(divisors_dev.is_cuda() && divisors_dev.scalar_type() == at::kLong);
    const int n_div = (int)divisors_dev.numel();
    const int ctas = sm_count() * 2;
    auto partials = at::zeros({n_div, ctas}, flat.options().dtype(at::kDouble));
    check(gx::launch_period_errors(flat.data_ptr(), dtype_code(flat.scalar_type()), flat.numel(),
                                   reinterpret_cast<const long long*>(divisors_dev.data_ptr<int64_t>()),
                                   n_div, input_is_squared, partials.data_ptr<double>(), ctas, stream()),
          "period_errors");
    return partials;
}

// ---------------------------------------------------------------------------
// tcgen05 GEMM (gemm_sm100.cu)
// ---------------------------------------------------------------------------
// c[b] = alpha * op(a[b]) op(b[b]) + beta * d[b]; a is [B, M, K] (or [B, K, M] when a_t),
// b is [B, N, K] (or [B, K, N] when b_t); 2-D tensors are a batch of one.
void gemm_bf16(const Tensor& a, const Tensor& b, Tensor c, const c10::optional<Tensor>& d, bool a_t,
               bool b_t, double alpha, double beta, const c10::optional<Tensor>& status) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && c.is_cuda(), "gemm_bf16: CUDA tensors required");
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                    c.scalar_type() == at::kBFloat16,
                "gemm_bf16: bf16 tensors required");
    TORCH_CHECK(a.dim() == b.dim() && a.dim() == c.dim() && (a.dim() == 2 || a.dim() == 3));
    const bool batched = a.dim() == 3;
    auto dimof = [&](const Tensor& t, int i) { return t.size(batched ? i + 1 : i); };
    auto ldof = [&](const Tensor& t) { return t.stride(batched ? 1 : 0); };
    auto bsof = [&](const Tensor& t) { return batched ? t.stride(0) : (int64_t)0; };
    TORCH_CHECK(a.stride(-1) == 1 && b.stride(-1) == 1 && c.stride(-1) == 1, "innermost stride must be 1");
    gx::GemmParams p{};
    p.batch = batched ? (int)a.size(0) : 1;
    p.M = (int)(a_t ? dimof(a, 1) : dimof(a, 0));
    p.K = (int)(a_t ? dimof(a, 0) : dimof(a, 1));
    p.N = (int)(b_t ? dimof(b, 1) : dimof(b, 0));
    TORCH_CHECK((b_t ? dimof(b, 0) : dimof(b, 1)) == p.K, "gemm_bf16: inner dimensions differ");
    TORCH_CHECK(dimof(c, 0) == p.M && dimof(c, 1) == p.N, "gemm_bf16: bad output shape");
    TORCH_CHECK(!batched || (b.size(0) == p.batch && c.size(0) == p.batch));
    p.a_mn_major = a_t ? 1 : 0;
    p.b_mn_major = b_t ? 1 : 0;
    p.alpha = (float)alpha;
    p.beta = (float)beta;
    p.C = reinterpret_cast<__nv_bfloat16*>(c.data_ptr());
    p.ldc = ldof(c);
    p.batch_stride_c = bsof(c);
    p.D = nullptr;
    if (d.has_value() && d->defined()) {
        TORCH_CHECK(d->scalar_type() == at::kBFloat16 && d->sizes() == c.sizes() && d->stride(-1) == 1);
        p.D = reinterpret_cast<const __nv_bfloat16*>(d->data_ptr());
        p.ldd = ldof(*d);
        p.batch_stride_d = bsof(*d);
    }
    p.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    check(gx::launch_gemm_bf16(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), ldof(a), bsof(a),
                               reinterpret_cast<const __nv_bfloat16*>(b.data_ptr()), ldof(b), bsof(b), p,
                               sm_count(), stream()),
          "gemm_bf16");
}

// CTA-pair GEMM (gemm_pair_sm100.cu).  2-D bf16 operands: a [M, K] (or [K, M] when a_t), b [N, K]
// (or [K, N] when b_t).  epi 0: c0 [M, N] = alpha a b + beta d.  epi 1 (SwiGLU forward): b is the
// stacked [gate | up] weight (2F rows), c0 = the [M, 2F] gate|up buffer, c1 = act [M, F].
// epi 2 (SwiGLU derivative): a b = d(act) [M, F]; aux = gate|up [M, 2F]; c0 = d(gate|up) [M, 2F].
// workspace of the pair kernel's K-split tail wave and its schedule counter: one per (device, stream),
// since launches that share it must be ordered; counters start at zero and every launch leaves them zeroed
static void pair_workspace(const Tensor& like, gx::PairParams& p, bool dynamic) {
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, std::pair<Tensor, Tensor>> pool;
    std::lock_guard<std::mutex> lock(mu);
    auto key = std::make_pair((int)like.get_device(), stream());
    auto it = pool.find(key);
    if (it == pool.end()) {
        auto ws = at::empty({gx::kPairWsFloats}, like.options().dtype(at::kFloat));
        auto cnt = at::zeros({gx::kPairCounters}, like.options().dtype(at::kInt));
        it = pool.emplace(key, std::make_pair(ws, cnt)).first;
    }
    p.ws = it->second.first.data_ptr<float>();
    p.ws_floats = gx::kPairWsFloats;
    p.counters = reinterpret_cast<uint32_t*>(it->second.second.data_ptr<int>());
    p.n_counters = gx::kPairCounters - 8;
    p.sched = dynamic ? p.counters + (gx::kPairCounters - 8) : nullptr;
}

void gemm_pair_bf16(const Tensor& a, const Tensor& b, Tensor c0, const c10::optional<Tensor>& c1,
                    const c10::optional<Tensor>& d, const c10::optional<Tensor>& aux, bool a_t, bool b_t,
                    double alpha, double beta, int64_t epi, int64_t bn, const c10::optional<Tensor>& status,
                    const c10::optional<Tensor>& sumsq, bool dynamic, bool symmetric) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && c0.is_cuda(), "gemm_pair_bf16: CUDA tensors required");
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                    c0.scalar_type() == at::kBFloat16, "gemm_pair_bf16: bf16 tensors required");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c0.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                    c0.stride(1) == 1, "gemm_pair_bf16: 2-D operands with unit inner stride required");
    gx::PairParams p{};
    p.M = (int)(a_t ? a.size(1) : a.size(0));
    p.K = (int)(a_t ? a.size(0) : a.size(1));
    const int64_t b_rows = b_t ? b.size(1) : b.size(0);
    TORCH_CHECK((b_t ? b.size(0) : b.size(1)) == p.K, "gemm_pair_bf16: inner dimensions differ");
    p.a_mn_major = a_t ? 1 : 0;
    p.b_mn_major = b_t ? 1 : 0;
    p.alpha = (float)alpha;
    p.beta = (float)beta;
    p.epi = (int)epi;
    p.bn = (int)bn;
    p.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    p.sumsq = nullptr;
    p.symmetric = symmetric ? 1 : 0;
    TORCH_CHECK(!symmetric || epi == gx::kEpiPlain, "gemm_pair_bf16: the symmetric mode takes the plain epilogue");
    if (sumsq.has_value() && sumsq->defined()) {
        TORCH_CHECK(epi == gx::kEpiPlain, "gemm_pair_bf16: sumsq is available with the plain epilogue only");
        TORCH_CHECK(sumsq->is_cuda() && sumsq->scalar_type() == at::kFloat && sumsq->is_contiguous() &&
                        sumsq->numel() >= gx::kSumsqSlots,
                    "gemm_pair_bf16: sumsq must be a contiguous CUDA fp32 tensor of at least 2048 slots");
        p.sumsq = sumsq->data_ptr<float>();
    }
    auto bf = [](const Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); };
    __nv_bfloat16 *C0 = bf(c0), *C1 = nullptr, *C2 = nullptr;
    long long ld0 = c0.stride(0), ld1 = 0, ld2 = 0;
    if (epi == gx::kEpiPlain) {
        p.N = (int)b_rows;
        TORCH_CHECK(c0.size(0) == p.M && c0.size(1) == p.N, "gemm_pair_bf16: bad output shape");
        if (d.has_value() && d->defined() && beta != 0.0) {
            TORCH_CHECK(d->scalar_type() == at::kBFloat16 && d->sizes() == c0.sizes() && d->stride(1) == 1);
            p.D = bf(*d);
            p.ldd = d->stride(0);
        }
    } else if (epi == gx::kEpiSwigluFwd) {
        TORCH_CHECK(b_rows % 2 == 0 && c1.has_value() && c1->defined(), "gemm_pair_bf16: SwiGLU needs c1");
        p.N = p.F = (int)(b_rows / 2);
        TORCH_CHECK(c0.size(0) == p.M && c0.size(1) == 2 * p.F && c1->size(0) == p.M && c1->size(1) == p.F &&
                    c1->stride(1) == 1 && c1->scalar_type() == at::kBFloat16 && p.F % 8 == 0);
        C1 = C0 + p.F;
        ld1 = ld0;
        C2 = bf(*c1);
        ld2 = c1->stride(0);
    } else {
        TORCH_CHECK(epi == gx::kEpiSwigluBwd && aux.has_value() && aux->defined(), "gemm_pair_bf16: bad epilogue");
        p.N = p.F = (int)b_rows;
        TORCH_CHECK(c0.size(0) == p.M && c0.size(1) == 2 * p.F && aux->sizes() == c0.sizes() &&
                    aux->stride(1) == 1 && aux->scalar_type() == at::kBFloat16 && p.F % 8 == 0);
        C1 = C0 + p.F;
        ld1 = ld0;
        p.aux = bf(*aux);
        p.ldaux = aux->stride(0);
    }
    TORCH_CHECK(gx::gemm_pair_supported(p.M, p.N, p.K), "gemm_pair_bf16: shape too small for the pair kernel");
    pair_workspace(a, p, dynamic);
    check(gx::launch_gemm_pair_bf16(bf(a), a.stride(0), bf(b), b.stride(0), p, C0, ld0, C1, ld1, C2, ld2,
                                    sm_count(), stream()),
          "gemm_pair_bf16");
}


// out [M, N] (bf16) = (a [M, K] @ b [N, K]^T) * sa[m] * sb[n] with e4m3 operands on the pair kernel
void gemm_pair_e4m3(const Tensor& a, const Tensor& b, const Tensor& sa, const Tensor& sb, Tensor out,
                    const c10::optional<Tensor>& status, bool dynamic) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda() && sa.is_cuda() && sb.is_cuda(),
                "gemm_pair_e4m3: CUDA tensors required");
    TORCH_CHECK(a.element_size() == 1 && b.element_size() == 1 && out.scalar_type() == at::kBFloat16 &&
                    sa.scalar_type() == at::kFloat && sb.scalar_type() == at::kFloat,
                "gemm_pair_e4m3: e4m3 operands, fp32 scales and a bf16 output required");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 &&
                    out.stride(1) == 1 && sa.is_contiguous() && sb.is_contiguous(),
                "gemm_pair_e4m3: 2-D operands with unit inner stride required");
    gx::PairParams p{};
    p.M = (int)a.size(0);
    p.K = (int)a.size(1);
    p.N = (int)b.size(0);
    TORCH_CHECK(b.size(1) == p.K && out.size(0) == p.M && out.size(1) == p.N && sa.numel() == p.M && sb.numel() == p.N,
                "gemm_pair_e4m3: shapes do not fit");
    TORCH_CHECK(gx::gemm_pair_supported(p.M, p.N, p.K) && p.K >= 128, "gemm_pair_e4m3: shape too small for the pair kernel");
    p.alpha = 1.f;
    p.row_scale = sa.data_ptr<float>();
    p.col_scale = sb.data_ptr<float>();
    p.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    pair_workspace(a, p, dynamic);
    check(gx::launch_gemm_pair_e4m3(a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), p,
                                    reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), out.stride(0), sm_count(), stream()),
          "gemm_pair_e4m3");
}


// NorMuon row normalisation, cautious mask and (optionally) the parameter update on an orthogonalised
// Muon update, in place.  scal: device fp32 {1 - beta2^t, lr * ratio, 1 - lr * weight_decay}.
void muon_epilogue(Tensor update, const c10::optional<Tensor>& grad, const c10::optional<Tensor>& normuon_v,
                   const c10::optional<Tensor>& param, const Tensor& scal, bool normuon, bool cautious,
                   double beta2, double eps) {
    c10::cuda::CUDAGuard guard(update.device());
    TORCH_CHECK(update.is_cuda() && update.dim() == 2 && update.is_contiguous(), "muon_epilogue: contiguous 2-D CUDA update");
    TORCH_CHECK(scal.is_cuda() && scal.scalar_type() == at::kFloat && scal.numel() >= 3 && scal.is_contiguous(),
                "muon_epilogue: scal must be a CUDA fp32 tensor of 3 values");
    gx::MuonEpilogue e{};
    e.update = update.data_ptr();
    e.rows = update.size(0);
    e.cols = (int)update.size(1);
    e.normuon = normuon ? 1 : 0;
    e.cautious = cautious ? 1 : 0;
    e.beta2 = (float)beta2;
    e.eps = (float)eps;
    e.scal = scal.data_ptr<float>();
    if (cautious) {
        TORCH_CHECK(grad.has_value() && grad->defined() && grad->is_cuda() && grad->is_contiguous() &&
                        grad->sizes() == update.sizes() && grad->scalar_type() == update.scalar_type(),
                    "muon_epilogue: the cautious mask needs a gradient of the update's shape and dtype");
        e.grad = grad->data_ptr();
    }
    if (normuon) {
        TORCH_CHECK(normuon_v.has_value() && normuon_v->defined() && normuon_v->is_cuda() &&
                        normuon_v->scalar_type() == at::kFloat && normuon_v->is_contiguous() &&
                        normuon_v->numel() == e.rows,
                    "muon_epilogue: normuon_v must hold one fp32 value per row");
        e.v = normuon_v->data_ptr<float>();
    }
    if (param.has_value() && param->defined()) {
        TORCH_CHECK(param->is_cuda() && param->is_contiguous() && param->sizes() == update.sizes() &&
                        param->scalar_type() == update.scalar_type(),
                    "muon_epilogue: the parameter must have the update's shape and dtype");
        e.param = param->data_ptr();
    }
    auto fopt = update.options().dtype(at::kFloat);
    Tensor row_sq = at::empty({e.rows}, fopt), row_scale = at::empty({e.rows}, fopt), glob = at::empty({2}, fopt);
    Tensor agree = at::empty({e.rows}, update.options().dtype(at::kInt));
    e.row_sq = row_sq.data_ptr<float>();
    e.row_scale = row_scale.data_ptr<float>();
    e.glob = glob.data_ptr<float>();
    e.agree = agree.data_ptr<int>();
    check(gx::launch_muon_epilogue(e, dtype_code(update.scalar_type()), sm_count(), stream()), "muon_epilogue");
}

inline void to_ptrs(at::IntArrayRef v, void** out);

// c = a [M, K] @ bstage [N, K]^T where bstage is filled inside the launch from the peers'
// row shards (segments in arrival order); see gemm_sm100.h.
void gemm_ag_bf16(const Tensor& a, Tensor bstage, Tensor c, at::IntArrayRef peer_bases, const Tensor& segs,
                  const Tensor& seg_meta, const Tensor& tile_order, Tensor flags, Tensor count,
                  int64_t epoch, int64_t count_target, int64_t fetch_ctas,
                  const c10::optional<Tensor>& status) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && bstage.scalar_type() == at::kBFloat16 &&
                c.scalar_type() == at::kBFloat16, "gemm_ag_bf16: bf16 tensors required");
    TORCH_CHECK(a.dim() == 2 && bstage.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 &&
                bstage.stride(1) == 1 && c.stride(1) == 1);
    TORCH_CHECK(a.size(1) == bstage.size(1) && c.size(0) == a.size(0) && c.size(1) == bstage.size(0));
    const int64_t n_segs = seg_meta.size(0);
    TORCH_CHECK(segs.scalar_type() == at::kByte && segs.numel() >= n_segs * (int64_t)sizeof(gx::GatherSeg));
    TORCH_CHECK(seg_meta.scalar_type() == at::kLong && seg_meta.is_contiguous() && seg_meta.size(1) == 3);
    TORCH_CHECK(tile_order.scalar_type() == at::kInt && tile_order.numel() >= (bstage.size(0) + 255) / 256);
    TORCH_CHECK(flags.scalar_type() == at::kInt && flags.numel() >= n_segs && count.scalar_type() == at::kInt &&
                count.numel() >= n_segs);
    gx::GemmParams p{};
    p.M = (int)a.size(0);
    p.K = (int)a.size(1);
    p.N = (int)bstage.size(0);
    p.alpha = 1.0f;
    p.beta = 0.0f;
    p.C = reinterpret_cast<__nv_bfloat16*>(c.data_ptr());
    p.ldc = c.stride(0);
    p.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    gx::AgParams ag{};
    ag.fetch_ctas = (int)fetch_ctas;
    ag.n_segs = (int)n_segs;
    ag.segs = reinterpret_cast<const gx::GatherSeg*>(segs.data_ptr());
    ag.seg_meta = reinterpret_cast<const long long*>(seg_meta.data_ptr<int64_t>());
    ag.tile_order = tile_order.data_ptr<int>();
    ag.dst_base = reinterpret_cast<char*>(bstage.data_ptr());
    ag.flags = reinterpret_cast<uint32_t*>(flags.data_ptr<int>());
    ag.count = reinterpret_cast<uint32_t*>(count.data_ptr<int>());
    ag.epoch = (uint32_t)epoch;
    ag.count_target = (uint32_t)count_target;
    void* bases[8];
    to_ptrs(peer_bases, bases);
    check(gx::launch_gemm_ag_bf16(reinterpret_cast<const __nv_bfloat16*>(a.data_ptr()), a.stride(0),
                                  reinterpret_cast<const __nv_bfloat16*>(bstage.data_ptr()), bstage.stride(0),
                                  p, ag, bases, (int)peer_bases.size(), sm_count(), stream()),
          "gemm_ag_bf16");
}

// ---------------------------------------------------------------------------
// peer-memory communication (comm.cu)
// ---------------------------------------------------------------------------
inline void to_ptrs(at::IntArrayRef v, void** out) {
    TORCH_CHECK(v.size() >= 1 && v.size() <= 8, "1..8 ranks");
    for (size_t i = 0; i < v.size(); ++i) out[i] = reinterpret_cast<void*>(v[i]);
}

void comm_signal(at::IntArrayRef flag_ptrs, int64_t slot, int64_t value, int64_t device_index) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_index);
    void* p[8];
    to_ptrs(flag_ptrs, p);
    check(gx::launch_signal(p, (int)flag_ptrs.size(), (int)slot, (unsigned)value, stream()), "signal");
}

void comm_wait(const Tensor& flags, int64_t n, int64_t value, int64_t max_iters,
               const c10::optional<Tensor>& status) {
    c10::cuda::CUDAGuard guard(flags.device());
    TORCH_CHECK(flags.is_cuda() && flags.scalar_type() == at::kInt && flags.numel() >= n);
    int* st = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    check(gx::launch_wait(reinterpret_cast<const unsigned*>(flags.data_ptr<int>()), (int)n, (unsigned)value,
                          max_iters, st, stream()),
          "wait");
}

void comm_gather(at::IntArrayRef src_base, const Tensor& segs, int64_t n_segs, Tensor dst,
                 const Tensor& unit_prefix, int64_t total_units, int64_t ctas) {
    c10::cuda::CUDAGuard guard(dst.device());
    TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kByte && segs.is_contiguous());
    TORCH_CHECK(segs.numel() >= n_segs * (int64_t)sizeof(gx::GatherSeg));
    TORCH_CHECK(unit_prefix.is_cuda() && unit_prefix.scalar_type() == at::kLong &&
                unit_prefix.numel() >= n_segs + 1);
    TORCH_CHECK(reinterpret_cast<uintptr_t>(dst.data_ptr()) % 16 == 0);
    void* p[8];
    to_ptrs(src_base, p);
    check(gx::launch_gather(p, (int)src_base.size(), reinterpret_cast<const gx::GatherSeg*>(segs.data_ptr()),
                            (int)n_segs, dst.data_ptr(),
                            reinterpret_cast<const long long*>(unit_prefix.data_ptr<int64_t>()),
                            total_units, (int)ctas, stream()),
          "gather");
}

void comm_reduce_segments(int64_t world, const Tensor& segs, int64_t n_segs,
                          const Tensor& unit_prefix, int64_t total_units, double scale,
                          const c10::optional<Tensor>& partials, int64_t ctas, int64_t dtype, bool multimem) {
    c10::cuda::CUDAGuard guard(segs.device());
    TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kByte && segs.is_contiguous());
    TORCH_CHECK(segs.numel() >= n_segs * (int64_t)sizeof(gx::ReduceSeg));
    TORCH_CHECK(unit_prefix.is_cuda() && unit_prefix.scalar_type() == at::kLong &&
                unit_prefix.numel() >= n_segs + 1);
    float* part = nullptr;
    if (partials.has_value() && partials->defined()) {
        TORCH_CHECK(partials->is_cuda() && partials->scalar_type() == at::kFloat &&
                    partials->numel() >= ctas, "partials: fp32, at least `ctas` entries");
        part = partials->data_ptr<float>();
    }
    check(gx::launch_reduce_segments((int)world,
                                     reinterpret_cast<const gx::ReduceSeg*>(segs.data_ptr()), (int)n_segs,
                                     reinterpret_cast<const long long*>(unit_prefix.data_ptr<int64_t>()),
                                     total_units, (float)scale, part, (int)ctas, (int)dtype, stream(), multimem),
          "reduce_segments");
}

// One asynchronous device-to-device copy per row of a host table [n, 3] = (dst, src, bytes): the
// copies run on the copy engines, so a parameter all-gather from the peers' arenas takes no SM away
// from the GEMMs it overlaps with.  With `lanes` > 1 the copies are spread round-robin over that many
// auxiliary streams that fork from the current stream and join it again (events), so that several
// copy engines work at once; the call keeps the current stream's ordering either way.
void comm_copy_list(const Tensor& table, int64_t device_index, int64_t lanes) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_index);
    TORCH_CHECK(!table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() &&
                table.dim() == 2 && table.size(1) == 3, "table: CPU int64 [n, 3]");
    const int64_t* t = table.data_ptr<int64_t>();
    cudaStream_t st = stream();
    const int64_t n = table.size(0);
    constexpr int kMaxLanes = 8;
    const int k = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(lanes, kMaxLanes), n));
    if (k == 1) {
        for (int64_t i = 0; i < n; ++i) {
            if (t[3 * i + 2] <= 0) continue;
            check(cudaMemcpyAsync(reinterpret_cast<void*>(t[3 * i]), reinterpret_cast<const void*>(t[3 * i + 1]),
                                  (size_t)t[3 * i + 2], cudaMemcpyDeviceToDevice, st),
                  "copy_list");
        }
        return;
    }
    struct Lanes {
        cudaStream_t s[kMaxLanes];
        cudaEvent_t done[kMaxLanes];
        cudaEvent_t start;
    };
    static std::mutex mu;
    static std::map<int, Lanes> pool;
    Lanes* L;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = pool.find((int)device_index);
        if (it == pool.end()) {
            Lanes fresh{};
            for (int i = 0; i < kMaxLanes; ++i) {
                check(cudaStreamCreateWithFlags(&fresh.s[i], cudaStreamNonBlocking), "copy_list stream");
                check(cudaEventCreateWithFlags(&fresh.done[i], cudaEventDisableTiming), "copy_list event");
            }
            check(cudaEventCreateWithFlags(&fresh.start, cudaEventDisableTiming), "copy_list event");
            it = pool.emplace((int)device_index, fresh).first;
        }
        L = &it->second;
    }
    check(cudaEventRecord(L->start, st), "copy_list fork");
    for (int i = 0; i < k; ++i) check(cudaStreamWaitEvent(L->s[i], L->start, 0), "copy_list fork");
    for (int64_t i = 0; i < n; ++i) {
        if (t[3 * i + 2] <= 0) continue;
        check(cudaMemcpyAsync(reinterpret_cast<void*>(t[3 * i]), reinterpret_cast<const void*>(t[3 * i + 1]),
                              (size_t)t[3 * i + 2], cudaMemcpyDeviceToDevice, L->s[i % k]),
              "copy_list");
    }
    for (int i = 0; i < k; ++i) {
        check(cudaEventRecord(L->done[i], L->s[i]), "copy_list join");
        check(cudaStreamWaitEvent(st, L->done[i], 0), "copy_list join");
    }
}

void comm_scatter_apply(const Tensor& segs, int64_t n_segs, const Tensor& unit_prefix, int64_t total_units,
                        int64_t ctas) {
    c10::cuda::CUDAGuard guard(segs.device());
    TORCH_CHECK(segs.is_cuda() && segs.scalar_type() == at::kByte &&
                segs.numel() >= n_segs * (int64_t)sizeof(gx::ApplySeg));
    TORCH_CHECK(unit_prefix.is_cuda() && unit_prefix.scalar_type() == at::kLong &&
                unit_prefix.numel() >= n_segs + 1);
    check(gx::launch_scatter_apply(reinterpret_cast<const gx::ApplySeg*>(segs.data_ptr()), (int)n_segs,
                                   reinterpret_cast<const long long*>(unit_prefix.data_ptr<int64_t>()),
                                   total_units, (int)ctas, stream()),
          "scatter_apply");
}

void comm_allreduce_scalar(at::IntArrayRef slot_ptrs, at::IntArrayRef flag_ptrs, int64_t rank,
                           const Tensor& local_val, Tensor out, int64_t epoch, int64_t max_iters,
                           const c10::optional<Tensor>& status) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(local_val.is_cuda() && local_val.scalar_type() == at::kFloat);
    TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kFloat);
    void* s[8];
    void* f[8];
    to_ptrs(slot_ptrs, s);
    to_ptrs(flag_ptrs, f);
    int* st = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    check(gx::launch_allreduce_scalar(s, f, (int)slot_ptrs.size(), (int)rank, local_val.data_ptr<float>(),
                                      out.data_ptr<float>(), (unsigned)epoch, max_iters, st, stream()),
          "allreduce_scalar");
}

// out [n_tok, cols] = rows tok[] of a row-sharded table, read from the owners' shards
void comm_gather_rows(at::IntArrayRef shard_ptrs, int64_t rows_per, int64_t rows, const Tensor& tok, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(tok.is_cuda() && tok.scalar_type() == at::kLong && tok.is_contiguous());
    TORCH_CHECK(out.is_cuda() && out.is_contiguous() && out.dim() == 2 && out.size(0) == tok.numel());
    const int64_t row_bytes = out.size(1) * out.element_size();
    TORCH_CHECK(row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0);
    void* p[8];
    to_ptrs(shard_ptrs, p);
    check(gx::launch_gather_rows(p, (int)shard_ptrs.size(), rows_per, rows, (int)row_bytes,
                                 reinterpret_cast<const long long*>(tok.data_ptr<int64_t>()), (int)tok.numel(),
                                 out.data_ptr(), stream()),
          "gather_rows");
}

// dst [my_rows, cols] (bf16, zeroed) += scale * every rank's gradient rows of the tokens this rank owns
void comm_scatter_add_rows(at::IntArrayRef tok_ptrs, at::IntArrayRef grad_ptrs, int64_t n_tok, int64_t row0,
                           double scale, Tensor dst) {
    c10::cuda::CUDAGuard guard(dst.device());
    TORCH_CHECK(dst.is_cuda() && dst.scalar_type() == at::kBFloat16 && dst.is_contiguous() && dst.dim() == 2);
    TORCH_CHECK(tok_ptrs.size() == grad_ptrs.size());
    void *t[8], *g[8];
    to_ptrs(tok_ptrs, t);
    to_ptrs(grad_ptrs, g);
    check(gx::launch_scatter_add_rows(t, g, (int)tok_ptrs.size(), (int)n_tok, row0, dst.size(0), (int)dst.size(1),
                                      (float)scale, dst.data_ptr(), stream()),
          "scatter_add_rows");
}

// ---------------------------------------------------------------------------
// model operators (model_ops.cu)
// ---------------------------------------------------------------------------
void rmsnorm_fwd(const Tensor& x, const Tensor& w, Tensor y, Tensor rstd, double eps) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && y.is_contiguous() && w.is_contiguous());
    const int64_t d = x.size(-1);
    check(gx::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(),
                                 x.numel() / d, (int)d, (float)eps, dtype_code(x.scalar_type()), stream()),
          "rmsnorm_fwd");
}

// dx = norm backward (+ res), dw = column sums of the per-CTA partials (both kernels of this file)
void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor dx,
                 Tensor dw_partial, const c10::optional<Tensor>& res, const c10::optional<Tensor>& dw) {
    c10::cuda::CUDAGuard guard(x.device());
    TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous());
    const int64_t d = x.size(-1);
    const void* r = nullptr;
    if (res.has_value() && res->defined()) {
        TORCH_CHECK(res->is_contiguous() && res->scalar_type() == x.scalar_type() && res->numel() == x.numel(),
                    "rmsnorm_bwd: res must match x");
        r = res->data_ptr();
    }
    check(gx::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                                 dx.data_ptr(), dw_partial.data_ptr<float>(), (int)dw_partial.size(0),
                                 x.numel() / d, (int)d, dtype_code(x.scalar_type()), stream(), r),
          "rmsnorm_bwd");
    if (dw.has_value() && dw->defined()) {
        TORCH_CHECK(dw->scalar_type() == at::kFloat && dw->is_contiguous() && dw->numel() == d &&
                    dw_partial.is_contiguous() && dw_partial.size(1) == d);
        check(gx::launch_colsum(dw_partial.data_ptr<float>(), (int)dw_partial.size(0), (int)d,
                                dw->data_ptr<float>(), stream()),
              "rmsnorm_bwd colsum");
    }
}

int64_t rmsnorm_bwd_partials(int64_t rows, int64_t d) { return gx::rmsnorm_bwd_partials(rows, (int)d); }

// dst, src: 2-D views [tokens, n_heads * head_dim] whose rows may be strided (column slices of a
// fused projection buffer); dst may be src.
void rope(Tensor dst, const Tensor& src, const Tensor& cos, const Tensor& sin, int64_t seq_len,
          int64_t n_heads, int64_t head_dim, bool inverse, bool interleaved) {
    c10::cuda::CUDAGuard guard(dst.device());
    TORCH_CHECK(dst.is_cuda() && src.is_cuda() && cos.scalar_type() == at::kFloat && cos.is_contiguous() &&
                sin.is_contiguous());
    TORCH_CHECK(dst.dim() == 2 && src.dim() == 2 && dst.size(0) == src.size(0) &&
                dst.size(1) == n_heads * head_dim && src.size(1) == n_heads * head_dim &&
                dst.stride(1) == 1 && src.stride(1) == 1 && dst.scalar_type() == src.scalar_type(),
                "rope: [tokens, n_heads * head_dim] views with unit inner stride");
    check(gx::launch_rope(dst.data_ptr(), src.data_ptr(), dst.stride(0), src.stride(0),
                          cos.data_ptr<float>(), sin.data_ptr<float>(), dst.size(0), (int)seq_len,
                          (int)n_heads, (int)head_dim, inverse, interleaved,
                          dtype_code(dst.scalar_type()), stream()),
          "rope");
}

void flash_attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor out, Tensor lse,
                         int64_t seq, double scale, const c10::optional<Tensor>& status) {
    c10::cuda::CUDAGuard guard(q.device());
    TORCH_CHECK(q.is_cuda() && q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.is_contiguous() &&
                k.is_contiguous() && v.is_contiguous() && out.is_contiguous() && lse.is_contiguous());
    TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                v.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 &&
                lse.scalar_type() == at::kFloat);
    TORCH_CHECK(k.sizes() == v.sizes() && k.size(0) == q.size(0) && k.size(1) == seq && k.size(2) == q.size(2) &&
                out.sizes() == q.sizes() && lse.numel() == q.size(0) * q.size(1));
    gx::FlashParams p{};
    p.seq = (int)seq;
    p.rows = (int)q.size(1);
    p.batch = (int)q.size(0);
    p.scale = (float)scale;
    p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
    p.lse = lse.data_ptr<float>();
    p.status = (status.has_value() && status->defined()) ? status->data_ptr<int>() : nullptr;
    check(gx::launch_flash_attention_fwd(reinterpret_cast<const __nv_bfloat16*>(q.data_ptr()),
                                         reinterpret_cast<const __nv_bfloat16*>(k.data_ptr()),
                                         reinterpret_cast<const __nv_bfloat16*>(v.data_ptr()), (int)q.size(2), p,
                                         stream()),
          "flash_attention_fwd");
}

void attn_softmax(Tensor scores, Tensor lse, int64_t seq_q, double scale) {
    c10::cuda::CUDAGuard guard(scores.device());
    TORCH_CHECK(scores.is_cuda() && scores.is_contiguous() && scores.scalar_type() == at::kBFloat16);
    TORCH_CHECK(lse.is_cuda() && lse.scalar_type() == at::kFloat && lse.is_contiguous());
    const int64_t n_keys = scores.size(-1), rows = scores.numel() / n_keys;
    TORCH_CHECK(lse.numel() == rows && rows % seq_q == 0);
    check(gx::launch_causal_softmax(scores.data_ptr(), lse.data_ptr<float>(), rows, (int)n_keys, (int)seq_q,
                                    (float)scale, stream()),
          "attn_softmax");
}

void attn_row_dot(const Tensor& a, const Tensor& b, Tensor out) {
    c10::cuda::CUDAGuard guard(a.device());
    TORCH_CHECK(a.is_cuda() && a.is_contiguous() && b.is_contiguous() && a.sizes() == b.sizes() &&
                a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16);
    const int64_t d = a.size(-1), rows = a.numel() / d;
    TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == rows);
    check(gx::launch_row_dot(a.data_ptr(), b.data_ptr(), out.data_ptr<float>(), rows, (int)d, stream()),
          "attn_row_dot");
}

void attn_bwd_rows(Tensor scores, Tensor dprob, const Tensor& lse, const Tensor& delta, int64_t seq_q,
                   double scale) {
    c10::cuda::CUDAGuard guard(scores.device());
    TORCH_CHECK(scores.is_contiguous() && dprob.is_contiguous() && scores.sizes() == dprob.sizes() &&
                scores.scalar_type() == at::kBFloat16 && dprob.scalar_type() == at::kBFloat16);
    const int64_t n_keys = scores.size(-1), rows = scores.numel() / n_keys;
    TORCH_CHECK(lse.scalar_type() == at::kFloat && delta.scalar_type() == at::kFloat && lse.numel() == rows &&
                delta.numel() == rows && lse.is_contiguous() && delta.is_contiguous());
    check(gx::launch_attn_bwd_rows(scores.data_ptr(), dprob.data_ptr(), lse.data_ptr<float>(),
                                   delta.data_ptr<float>(), rows, (int)n_keys, (int)seq_q, (float)scale, stream()),
          "attn_bwd_rows");
}

void swiglu_fwd(const Tensor& gate_up, Tensor out) {
    c10::cuda::CUDAGuard guard(out.device());
    TORCH_CHECK(gate_up.is_contiguous() && out.is_contiguous());
    const int64_t f = out.size(-1);
    check(gx::launch_swiglu_fwd(gate_up.data_ptr(), out.data_ptr(), out.numel() / f, (int)f,
                                dtype_code(out.scalar_type()), stream()),
          "swiglu_fwd");
}

void swiglu_bwd(const Tensor& gate_up, const Tensor& dout, Tensor dgate_up) {
    c10::cuda::CUDAGuard guard(dout.device());
    TORCH_CHECK(gate_up.is_contiguous() && dout.is_contiguous() && dgate_up.is_contiguous());
    const int64_t f = dout.size(-1);
    check(gx::launch_swiglu_bwd(gate_up.data_ptr(), dout.data_ptr(), dgate_up.data_ptr(),
                                dout.numel() / f, (int)f, dtype_code(dout.scalar_type()), stream()),
          "swiglu_bwd");
}

void xent_fwd_bwd(Tensor logits, const Tensor& targets, Tensor loss_rows, double grad_scale,
                  int64_t ignore_index) {
    c10::cuda::CUDAGuard guard(logits.device());
    TORCH_CHECK(logits.is_contiguous() && targets.scalar_type() == at::kLong);
    const int64_t v = logits.size(-1);
    check(gx::launch_xent_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                                  loss_rows.data_ptr<float>(), logits.numel() / v, (int)v,
                                  (float)grad_scale, ignore_index, dtype_code(logits.scalar_type()),
                                  stream()),
          "xent_fwd_bwd");
}

}  // namespace

TORCH_LIBRARY(gefenx, m) {
    m.def("desc_size() -> int", &desc_size);
    m.def("rmsnorm_bwd_partials(int rows, int d) -> int", &rmsnorm_bwd_partials);
    m.def("block_update(Tensor descs, Tensor tile_start, int n_tensors, int total_tiles, Tensor codebook, "
          "Tensor thr, Tensor lut, Tensor? gscale, Tensor? status, int dtype, int sr_seed, bool stochastic, "
          "Tensor? sr_seed_dev) -> ()");
    m.def("factored_update(Tensor descs, Tensor tile_start, int n_tensors, int total_tiles, Tensor codebook, "
          "Tensor thr, Tensor lut, Tensor? gscale, Tensor? status, int dtype, int sr_seed, bool stochastic, "
          "int wait_iters, int phases, int epoch, int fast, Tensor? sr_seed_dev) -> ()");
    m.def("reduce_sources(Tensor? out, int[] src_ptrs, int numel, float scale, Tensor? partials, "
          "int dtype, int device_index) -> ()", &reduce_sources);
    m.def("clip_coef(Tensor partials, float max_norm, Tensor(a!) coef) -> ()");
    m.def("histogram(Tensor flat, int period, Tensor(a!) counts) -> ()");
    m.def("remap_indices(Tensor(a!) idx, Tensor map) -> ()");
    m.def("quantize_rows_e4m3(Tensor x, Tensor? x2, float alpha, float beta, Tensor(a!) q, Tensor(b!) scale, "
          "Tensor(c!)? y_out) -> ()");
    m.def("quantize_cols_e4m3_t(Tensor x, Tensor(a!) colmax, Tensor(b!) q_t, Tensor(c!) scale_t) -> ()");
    m.def("dequantize(Tensor idx, Tensor mag, Tensor codebook, int period, Tensor(a!) out) -> ()");
    m.def("period_errors(Tensor flat, Tensor divisors, bool input_is_squared) -> Tensor");
    m.def("gemm_bf16(Tensor a, Tensor b, Tensor(a!) c, Tensor? d, bool a_t, bool b_t, float alpha, "
          "float beta, Tensor? status) -> ()");
    m.def("gemm_pair_bf16(Tensor a, Tensor b, Tensor(a!) c0, Tensor(b!)? c1, Tensor? d, Tensor? aux, bool a_t, "
          "bool b_t, float alpha, float beta, int epi, int bn, Tensor? status, Tensor(c!)? sumsq, bool dynamic, "
          "bool symmetric) -> ()");
    m.def("muon_epilogue(Tensor(a!) update, Tensor? grad, Tensor(b!)? normuon_v, Tensor(c!)? param, Tensor scal, "
          "bool normuon, bool cautious, float beta2, float eps) -> ()");
    m.def("gemm_pair_e4m3(Tensor a, Tensor b, Tensor sa, Tensor sb, Tensor(a!) out, Tensor? status, bool dynamic) -> ()");
    m.def("gemm_ag_bf16(Tensor a, Tensor(a!) bstage, Tensor(b!) c, int[] peer_bases, Tensor segs, "
          "Tensor seg_meta, Tensor tile_order, Tensor(c!) flags, Tensor(d!) count, int epoch, "
          "int count_target, int fetch_ctas, Tensor? status) -> ()");
    m.def("comm_signal(int[] flag_ptrs, int slot, int value, int device_index) -> ()", &comm_signal);
    m.def("comm_wait(Tensor flags, int n, int value, int max_iters, Tensor? status) -> ()");
    m.def("comm_gather(int[] src_base, Tensor segs, int n_segs, Tensor(a!) dst, Tensor unit_prefix, "
          "int total_units, int ctas) -> ()");
    m.def("comm_scatter_apply(Tensor segs, int n_segs, Tensor unit_prefix, int total_units, int ctas) -> ()");
    m.def("comm_reduce_segments(int world, Tensor segs, int n_segs, Tensor unit_prefix, int total_units, "
          "float scale, Tensor? partials, int ctas, int dtype, bool multimem) -> ()");
    m.def("comm_copy_list(Tensor table, int device_index, int lanes) -> ()", &comm_copy_list);
    m.def("comm_gather_rows(int[] shard_ptrs, int rows_per, int rows, Tensor tok, Tensor(a!) out) -> ()");
    m.def("comm_scatter_add_rows(int[] tok_ptrs, int[] grad_ptrs, int n_tok, int row0, float scale, "
          "Tensor(a!) dst) -> ()");
    m.def("comm_allreduce_scalar(int[] slot_ptrs, int[] flag_ptrs, int rank, Tensor local_val, "
          "Tensor(a!) out, int epoch, int max_iters, Tensor? status) -> ()");
    m.def("rmsnorm_fwd(Tensor x, Tensor w, Tensor(a!) y, Tensor(b!) rstd, float eps) -> ()");
    m.def("rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, Tensor(a!) dx, Tensor(b!) dw_partial, "
          "Tensor? res, Tensor(c!)? dw) -> ()");
    m.def("rope(Tensor(a!) dst, Tensor src, Tensor cos, Tensor sin, int seq_len, int n_heads, int head_dim, "
          "bool inverse, bool interleaved) -> ()");
    m.def("flash_attention_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) out, Tensor(b!) lse, int seq, "
          "float scale, Tensor? status) -> ()");
    m.def("attn_softmax(Tensor(a!) scores, Tensor(b!) lse, int seq_q, float scale) -> ()");
    m.def("attn_row_dot(Tensor a, Tensor b, Tensor(a!) out) -> ()");
    m.def("attn_bwd_rows(Tensor(a!) scores, Tensor(b!) dprob, Tensor lse, Tensor delta, int seq_q, float scale) -> ()");
    m.def("swiglu_fwd(Tensor gate_up, Tensor(a!) out) -> ()");
    m.def("swiglu_bwd(Tensor gate_up, Tensor dout, Tensor(a!) dgate_up) -> ()");
    m.def("xent_fwd_bwd(Tensor(a!) logits, Tensor targets, Tensor(b!) loss_rows, float grad_scale, "
          "int ignore_index) -> ()");
}

TORCH_LIBRARY_IMPL(gefenx, CUDA, m) {
    m.impl("block_update", &block_update);
    m.impl("factored_update", &factored_update);
    m.impl("clip_coef", &clip_coef);
    m.impl("histogram", &histogram);
    m.impl("remap_indices", &remap_indices);
    m.impl("dequantize", &dequantize);
    m.impl("quantize_cols_e4m3_t", &quantize_cols_e4m3_t);
    m.impl("quantize_rows_e4m3", &quantize_rows_e4m3);
    m.impl("period_errors", &period_errors);
    m.impl("gemm_bf16", &gemm_bf16);
    m.impl("gemm_pair_bf16", &gemm_pair_bf16);
    m.impl("gemm_pair_e4m3", &gemm_pair_e4m3);
    m.impl("muon_epilogue", &muon_epilogue);
    m.impl("gemm_ag_bf16", &gemm_ag_bf16);
    m.impl("comm_wait", &comm_wait);
    m.impl("comm_gather", &comm_gather);
    m.impl("comm_gather_rows", &comm_gather_rows);
    m.impl("comm_scatter_add_rows", &comm_scatter_add_rows);
    m.impl("comm_scatter_apply", &comm_scatter_apply);
    m.impl("comm_reduce_segments", &comm_reduce_segments);
    m.impl("comm_allreduce_scalar", &comm_allreduce_scalar);
    m.impl("rmsnorm_fwd", &rmsnorm_fwd);
    m.impl("rmsnorm_bwd", &rmsnorm_bwd);
    m.impl("rope", &rope);
    m.impl("flash_attention_fwd", &flash_attention_fwd);
    m.impl("attn_softmax", &attn_softmax);
    m.impl("attn_row_dot", &attn_row_dot);
    m.impl("attn_bwd_rows", &attn_bwd_rows);
    m.impl("swiglu_fwd", &swiglu_fwd);
    m.impl("swiglu_bwd", &swiglu_bwd);
    m.impl("xent_fwd_bwd", &xent_fwd_bwd);
}
