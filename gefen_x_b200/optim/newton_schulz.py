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
    """A single (a, b, c) repeated ``ns_steps`` times, or an explicit per-iteration list."""
    if ns_coefficients is None:
        ns_coefficients = (DEFAULT_A, DEFAULT_B, DEFAULT_C)
    seq = list(ns_coefficients)
    if len(seq) == 3 and all(isinstance(x, (int, float)) for x in seq):
        return [tuple(float(x) for x in seq)] * int(ns_steps)
    out = []
    for item in seq:
        item = tuple(float(x) for x in item)
        if len(item) != 3:
            raise ValueError("every Newton-Schulz coefficient entry must be (a, b, c)")
        out.append(item)
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
            tcgemm.gemm(x, x, out=g)                                   # G = X X^T
            tcgemm.gemm(g, g, alpha=c, beta=b, d=g, out=u)             # U = c G G^T + b G
            tcgemm.gemm(u, x, b_t=True, alpha=1.0, beta=a, d=x, out=nxt)  # X' = U X + a X
            x, nxt = nxt, x
        return x
    for a, b, c in schedule:
        g = x @ x.transpose(-1, -2)
        u = b * g + c * (g @ g)
        x = a * x + u @ x
    return x


def zeropower_via_newtonschulz(grad: torch.Tensor, ns_coefficients=None,
                               ns_steps: int = DEFAULT_NS_STEPS, eps: float = EPS,
                               use_fp8: bool = False, compile_fp8: bool = True) -> torch.Tensor:
    """Approximate ``U V^T`` of ``grad = U S V^T`` (2-D).  ``use_fp8`` is accepted and
    ignored: the products stay bf16 (the reference documents fp8 as an optional
    accelerator with a bf16 fallback, ``README.md:597``)."""
    if grad.dim() != 2:
        raise ValueError("Input tensor gradient must be a 2D matrix")
    schedule = normalize_schedule(ns_coefficients, ns_steps)
    x = grad.bfloat16() if grad.dtype != torch.float64 else grad
    transposed = grad.size(0) > grad.size(1)
    if transposed:
        x = x.t()
    x = x / x.norm().clamp(min=eps)
    x = _iterate(x.contiguous(), schedule)
    return x.t() if transposed else x


def zeropower_batched(mats: Sequence[torch.Tensor], ns_coefficients=None,
                      ns_steps: int = DEFAULT_NS_STEPS, eps: float = EPS) -> List[torch.Tensor]:
    """Newton–Schulz on many same-shape matrices at once (one batched GEMM per product)."""
    if not mats:
        return []
    shape = mats[0].shape
    if any(m.shape != shape for m in mats):
        raise ValueError("zeropower_batched needs matrices of one shape")
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
