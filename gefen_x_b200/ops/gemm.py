"""Matrix products used by the decoder and by Newton–Schulz.

Plain layer GEMMs go to the vendor library through ``torch.matmul``; the fused
paths (all-gather -> GEMM, the Newton–Schulz chain) use the tcgen05 kernel of
``csrc/gemm_sm100.cu`` through :func:`tc_gemm_nt`, which can also serve the
plain products (``set_backend("tcgen05")``).
"""
from __future__ import annotations

from typing import Optional

import torch

_BACKEND = "library"


def set_backend(name: str) -> None:
    """``"library"`` (cuBLAS via torch) or ``"tcgen05"`` (own kernel where shapes allow)."""
    global _BACKEND
    if name not in ("library", "tcgen05"):
        raise ValueError("unknown GEMM backend {!r}".format(name))
    _BACKEND = name


def backend() -> str:
    return _BACKEND


def _tc_ok(a: torch.Tensor, b: torch.Tensor) -> bool:
    if _BACKEND != "tcgen05" or not a.is_cuda or a.dtype != torch.bfloat16:
        return False
    from . import tcgemm

    return tcgemm.supports_nt(a, b)


def mm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T``."""
    if _tc_ok(a, b):
        from . import tcgemm

        return tcgemm.gemm_nt(a, b, out=out)
    if out is None:
        return a @ b.t()
    return torch.matmul(a, b.t(), out=out)


def mm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [K, N]``."""
    if out is None:
        return a @ b
    return torch.matmul(a, b, out=out)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [K, M]^T @ b [K, N]``."""
    if out is None:
        return a.t() @ b
    return torch.matmul(a.t(), b, out=out)
