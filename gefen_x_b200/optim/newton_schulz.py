"""Newton–Schulz orthogonalisation (the Muon inner loop) on the tcgen05 GEMM.

One quintic iteration on ``X`` (oriented rows <= cols, bf16, pre-divided by its
Frobenius norm)::

    G = X X^T            U = b G + c G G            X <- a X + U X

Three GEMMs per iteration, all through ``ops.tcgemm`` on CUDA (``G G`` uses the
symmetry of ``G``: ``G G = G G^T`` is a K-major x K-major product; ``U X`` reads
``X`` in its stored row-major form as the MN-major operand, so no transpose is
ever materialised).  Same-shape matrices are stacked and run as batched GEMMs.
CPU tensors and dtypes the kernel does not cover use ``torch.matmul``.

Schedules and coefficients follow the reference (``src/gefen/gefen_muon.py:19-72``
constants, ``:236-291`` single matrix, ``:353-393`` batched); the reference runs
these products through cuBLAS (``torch.addmm`` / ``baddbmm``).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch

EPS = 1e-7
DEFAULT_A, DEFAULT_B, DEFAULT_C = 3.4445, -4.7750, 2.0315
DEFAULT_NS_STEPS = 5

NS_SCHEDULE_3STEP = [
    (5.0067, -14.4125, 10.6001),
    (3.7534, -6.8083, 3.3840),
    (3.2080, -4.3501, 2.0330),
]
NS_SCHEDULE_4STEP = [
    (5.4261, -15.5285, 11.2657),
    (3.0766, -4.9701, 2.1297),
    (3.0008, -6.4486, 4.3696),
    (2.8386, -4.1421, 2.5758),
]
NS_SCHEDULES = {"standard": None, "tuned3": NS_SCHEDULE_3STEP, "tuned4": NS_SCHEDULE_4STEP}

Coeffs = Tuple[float, float, float]


def normalize_schedule(ns_coefficients, ns_steps: int) -> List[Coeffs]:
    """A single (a, b, c) repeated ``ns_steps`` times (``1 <= ns_steps < 100``), or an explicit
    per-iteration list of fewer than 100 entries, whose length is the iteration count
    (``ns_steps`` is then ignored).  Same checks as the reference (``gefen_muon.py:189-233``)."""
    if ns_coefficients is None:
        ns_coefficients = (DEFAULT_A, DEFAULT_B, DEFAULT_C)
    seq = list(ns_coefficients)
    if len(seq) == 0:
        raise ValueError("ns_coefficients must be non-empty")
    if isinstance(seq[0], (int, float)):
        if not 1 <= ns_steps < 100:
            raise ValueError(
                "ns_steps must be in [1, 100) but is: {}. 0 or a negative value would produce an empty "
                "Newton-Schulz schedule (Muon degrades to normalized momentum SGD); 100+ is rejected for "
                "computational efficiency".format(ns_steps))
        if len(seq) != 3:
            raise ValueError("A single coefficient set must be a tuple of exactly 3 values")
        return [tuple(float(x) for x in seq)] * int(ns_steps)
    out = []
    for item in seq:
        if len(item) != 3:
            raise ValueError("Each Newton-Schulz schedule entry must have exactly 3 values")
        out.append(tuple(float(x) for x in item))
    if len(out) >= 100:
        raise ValueError("Newton-Schulz schedule length must be less than 100 for computational efficiency")
    return out


def resolve_schedule(ns_schedule: Optional[str], ns_coefficients, ns_steps: int) -> List[Coeffs]:
    if ns_schedule is None or ns_schedule == "standard":
        return normalize_schedule(ns_coefficients, ns_steps)
    if ns_schedule not in NS_SCHEDULES:
        raise ValueError("unknown ns_schedule {!r}; choose from {}".format(
            ns_schedule, sorted(NS_SCHEDULES)))
    return list(NS_SCHEDULES[ns_schedule])


def _use_kernel(x: torch.Tensor) -> bool:
    if not x.is_cuda or x.dtype != torch.bfloat16:
        return False
    from ..ops import tcgemm
    from ..ops._ext import available

    return available(required=True) and tcgemm.supports(x, x)


def _iterate(x: torch.Tensor, schedule: Sequence[Coeffs]) -> torch.Tensor:
    """The quintic iterations on an oriented, normalised bf16 ``[..., m, n]`` (m <= n)."""
    if _use_kernel(x):
        from ..ops import tcgemm

        x = x.contiguous()
        g = torch.empty(*x.shape[:-1], x.shape[-2], dtype=x.dtype, device=x.device)
        u = torch.empty_like(g)
        nxt = torch.empty_like(x)
        for a, b, c in schedule:
            # G and U are symmetric: only the tiles on and below the diagonal are computed
            tcgemm.gemm(x, x, out=g, symmetric=True)                                   # G = X X^T
            tcgemm.gemm(g, g, alpha=c, beta=b, d=g, out=u, symmetric=True)             # U = c G G^T + b G
            tcgemm.gemm(u, x, b_t=True, alpha=1.0, beta=a, d=x, out=nxt)  # X' = U X + a X
            x, nxt = nxt, x
        return x
    # same roundings as the kernel path's alpha/beta epilogue (one rounding per product) and as the
    # reference's addmm / baddbmm chain
    fused = torch.addmm if x.dim() == 2 else torch.baddbmm
    for a, b, c in schedule:
        g = x @ x.transpose(-1, -2)
        u = fused(g, g, g, beta=b, alpha=c)
        x = fused(x, u, x, beta=a)
    return x


FP8_DTYPE = torch.float8_e4m3fn
FP8_MAX = 448.0                      # largest finite e4m3 magnitude
FP8_MIN_SCALE = 1e-12
FP8_MIN_DIM = 1536                   # below this the fp8 products lose to bf16 (reference gefen_muon.py:83-89)


_FP8_GEMM = "tcgen05"


def set_fp8_gemm(backend: str) -> None:
    """``"tcgen05"`` (own kernel, default) or ``"library"`` for the products of the fp8 iteration."""
    global _FP8_GEMM
    if backend not in ("tcgen05", "library"):
        raise ValueError("fp8 GEMM backend must be 'tcgen05' or 'library'")
    _FP8_GEMM = backend


def fp8_supported(device=None) -> bool:
    """fp8 tensor-core GEMMs need compute capability 8.9 or later; the CPU statement always runs."""
    if device is not None and torch.device(device).type != "cuda":
        return True
    if not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(device) >= (8, 9)


def fp8_applies(shape, use_fp8: bool) -> bool:
    """Size gate of the fp8 path: both dimensions large enough and multiples of 16 (the
    library's fp8 GEMM wants 16-byte rows)."""
    return bool(use_fp8) and min(shape) >= FP8_MIN_DIM and all(int(d) % 16 == 0 for d in shape)


def quantize_rowwise_fp8(x: torch.Tensor):
    """``x[r, :] ~= q[r, :] * scale[r]`` with ``q`` in e4m3 and each row's absmax mapped to 448."""
    scale = (x.abs().amax(dim=-1, keepdim=True).float() / FP8_MAX).clamp_(min=FP8_MIN_SCALE)
    q = (x.float() / scale).clamp_(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q, scale


def _mm_fp8(aq, sa, bq_rows, sb_rows) -> torch.Tensor:
    """``(aq * sa) @ (bq_rows * sb_rows)^T`` in bf16.  ``bq_rows`` holds the second operand's
    COLUMNS as rows (so its transpose view is the column-major operand the fp8 GEMM reads and
    ``sb_rows`` its per-column scales).  CUDA: the e4m3 variant of the own CTA-pair kernel (default;
    ``set_fp8_gemm("library")`` selects ``torch._scaled_mm`` with row-wise scales, which also takes the
    shapes the pair kernel does not); CPU: the same quantised values multiplied in fp32."""
    if aq.is_cuda:
        if _FP8_GEMM == "tcgen05":
            from ..ops import tcgemm

            if tcgemm.e4m3_eligible(aq.shape[0], bq_rows.shape[0], aq.shape[1]) and aq.stride(1) == 1 \
                    and bq_rows.stride(1) == 1 and aq.stride(0) % 16 == 0 and bq_rows.stride(0) % 16 == 0:
                return tcgemm.gemm_e4m3(aq, sa, bq_rows, sb_rows)
        return torch._scaled_mm(aq, bq_rows.t(), scale_a=sa, scale_b=sb_rows.t(), out_dtype=torch.bfloat16)
    return ((aq.float() * sa) @ (bq_rows.float() * sb_rows).t()).bfloat16()


def _iterate_fp8(x: torch.Tensor, schedule: Sequence[Coeffs]) -> torch.Tensor:
    """The quintic iterations with the three products in e4m3 and bf16 results (reference
    ``src/gefen/gefen_muon.py:134-171``).  ``X X^T`` and ``G G`` quantise their operand once (the
    second operand is the same matrix, by symmetry for ``G``); ``U X`` needs ``X`` quantised along
    its columns as well.  On CUDA every quantisation is one kernel that also does the
    elementwise combine before it (``b G + c G G``; ``a X + U X`` of the previous iteration)."""
    if x.is_cuda and _use_kernel(x):
        return _iterate_fp8_kernels(x, schedule)
    for a, b, c in schedule:
        xq, sx = quantize_rowwise_fp8(x)
        g = _mm_fp8(xq, sx, xq, sx)
        gq, sg = quantize_rowwise_fp8(g)
        gg = _mm_fp8(gq, sg, gq, sg)
        u = b * g + c * gg
        uq, su = quantize_rowwise_fp8(u)
        xtq, sxt = quantize_rowwise_fp8(x.t().contiguous())
        x = _mm_fp8(uq, su, xtq, sxt).add_(x, alpha=a)
    return x


def _iterate_fp8_kernels(x: torch.Tensor, schedule: Sequence[Coeffs]) -> torch.Tensor:
    from ..ops.quant import quantize_cols_e4m3_t as quant_t, quantize_rows_e4m3 as quant

    ux, a_prev = None, 0.0                       # U X of the previous iteration, not yet added to a X
    for a, b, c in schedule:
        if ux is None:
            xq, sx, _ = quant(x)
        else:                                    # X <- a X + U X and its quantisation, one pass
            xq, sx, x = quant(x, ux, a_prev, 1.0, want_y=True)
        g = _mm_fp8(xq, sx, xq, sx)
        gq, sg, _ = quant(g)
        gg = _mm_fp8(gq, sg, gq, sg)
        uq, su, _ = quant(g, gg, b, c)           # U = b G + c G G
        xtq, sxt = quant_t(x)
        ux, a_prev = _mm_fp8(uq, su, xtq, sxt), a
    return ux.add_(x, alpha=a_prev)


def zeropower_via_newtonschulz(grad: torch.Tensor, ns_coefficients=None,
                               ns_steps: int = DEFAULT_NS_STEPS, eps: float = EPS,
                               use_fp8: bool = False, compile_fp8: bool = True) -> torch.Tensor:
    """Approximate ``U V^T`` of ``grad = U S V^T`` (2-D).  ``use_fp8`` runs the products in e4m3
    for matrices that pass ``fp8_applies`` on a device that has fp8 GEMMs, bf16 otherwise (the
    reference's gates, ``src/gefen/gefen_muon.py:258-275``).  ``compile_fp8`` is accepted and
    unused: nothing here goes through a tracing compiler."""
    if grad.dim() != 2:
        raise ValueError("Input tensor gradient must be a 2D matrix")
    schedule = normalize_schedule(ns_coefficients, ns_steps)
    x = grad.bfloat16() if grad.dtype != torch.float64 else grad
    transposed = grad.size(0) > grad.size(1)
    if transposed:
        x = x.t()
    x = x / x.norm().clamp(min=eps)
    if x.dtype == torch.bfloat16 and fp8_applies(x.shape, use_fp8) and fp8_supported(x.device):
        x = _iterate_fp8(x.contiguous(), schedule)
    else:
        x = _iterate(x.contiguous(), schedule)
    return x.t() if transposed else x


def zeropower_batched(mats: Sequence[torch.Tensor], ns_coefficients=None,
                      ns_steps: int = DEFAULT_NS_STEPS, eps: float = EPS,
                      use_fp8: bool = False) -> List[torch.Tensor]:
    """Newton–Schulz on many same-shape matrices at once (one batched GEMM per product).  With
    ``use_fp8`` and a shape that passes the gates, each matrix goes through the fp8 path on its
    own (the library's fp8 GEMM is not batched)."""
    if not mats:
        return []
    shape = mats[0].shape
    if any(m.shape != shape for m in mats):
        raise ValueError("zeropower_batched needs matrices of one shape")
    if fp8_applies(shape, use_fp8) and fp8_supported(mats[0].device):
        return [zeropower_via_newtonschulz(m, ns_coefficients, ns_steps, eps, use_fp8=True) for m in mats]
    schedule = normalize_schedule(ns_coefficients, ns_steps)
    x = torch.stack([m.bfloat16() for m in mats])
    transposed = shape[0] > shape[1]
    if transposed:
        x = x.transpose(1, 2)
    norms = torch.linalg.vector_norm(x.float(), dim=(1, 2), keepdim=True).clamp(min=eps)
    x = (x / norms.to(x.dtype)).contiguous()
    x = _iterate(x, schedule)
    if transposed:
        x = x.transpose(1, 2)
    return [x[i] for i in range(x.shape[0])]
