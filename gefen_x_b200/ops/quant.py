"""First-step analysis on the GPU: histogram and the all-divisor period search.

Kernels: ``csrc/quant.cu``.  Parity targets: reference
``src/gefen/kernels/exact_histogram_fused.py:23-79`` and
``src/gefen/kernels/period_variance.py:62-84``.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import torch

from ._ext import available, ops  # noqa: F401  (re-exported)


def histogram(flat: torch.Tensor, period: int, bins: int = 4096) -> torch.Tensor:
    """int64 counts of the block-normalised values of a contiguous CUDA tensor."""
    flat = flat.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    if flat.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        flat = flat.float()
    counts = torch.zeros(bins, dtype=torch.int64, device=flat.device)
    ops().histogram(flat, int(period), counts)
    return counts


def period_errors(flat: torch.Tensor, divisors: Sequence[int], input_is_squared: bool = False) -> List[float]:
    """``sqrt(mean_b var_b)`` of ``g^2`` for every divisor, one launch, no host sync in between."""
    flat = flat.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    if flat.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        flat = flat.float()
    n = flat.numel()
    divs = torch.tensor(list(divisors), dtype=torch.int64, device=flat.device)
    partials = ops().period_errors(flat, divs, bool(input_is_squared))
    sums = partials.sum(dim=1).cpu().tolist()
    return [math.sqrt(max(s, 0.0) / (n // p)) for s, p in zip(sums, divisors)]
