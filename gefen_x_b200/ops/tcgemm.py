"""tcgen05 / TMEM bf16 GEMM (``csrc/gemm_sm100.cu``).

``gemm(a, b, ...)`` computes ``alpha * op(a) @ op(b)^T-or-not + beta * d`` on the
5th-generation tensor cores with TMA-fed operands.  Layout convention: with
``a_t=False`` the first operand is ``[M, K]`` (K contiguous), with ``a_t=True`` it
is stored ``[K, M]``; with ``b_t=False`` the second operand is ``[N, K]`` (so the
product is ``a @ b.T``), with ``b_t=True`` it is stored ``[K, N]`` (``a @ b``).
3-D inputs are batches.  The reference uses cuBLAS through torch for the same
products (reference ``src/gefen/gefen_muon.py:278-287``, ``:353-393``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ._ext import available, ops

_status = {}


def status_word(device: torch.device) -> torch.Tensor:
    t = _status.get(device)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _status[device] = t
    return t


def _ok_operand(t: torch.Tensor) -> bool:
    if t.dtype != torch.bfloat16 or not t.is_cuda or t.stride(-1) != 1:
        return False
    if t.data_ptr() % 16:
        return False
    return all(s % 8 == 0 for s in t.stride()[:-1])


def supports(a: torch.Tensor, b: torch.Tensor) -> bool:
    return _ok_operand(a) and _ok_operand(b) and a.dim() == b.dim() and a.dim() in (2, 3)


def supports_nt(a: torch.Tensor, b: torch.Tensor) -> bool:
    return supports(a, b) and a.shape[-1] == b.shape[-1]


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         alpha: float = 1.0, beta: float = 0.0, d: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """See the module docstring for the layout convention."""
    m = a.shape[-1] if a_t else a.shape[-2]
    n = b.shape[-1] if b_t else b.shape[-2]
    if out is None:
        out = torch.empty(*a.shape[:-2], m, n, dtype=torch.bfloat16, device=a.device)
    ops().gemm_bf16(a, b, out, d if beta != 0.0 else None, bool(a_t), bool(b_t), float(alpha),
                    float(beta), status_word(a.device))
    return out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T``."""
    return gemm(a, b, out=out)
