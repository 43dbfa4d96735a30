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


def remap_indices_(idx: torch.Tensor, index_map: torch.Tensor) -> torch.Tensor:
    """``idx[i] = index_map[idx[i]]`` in place on a contiguous uint8 CUDA tensor (no temporaries).

    Moves stored momentum indices onto a re-learned codebook: ``index_map[c]`` is the nearest new
    codeword of old codeword ``c`` (reference ``src/gefen/gefen.py:3020-3061`` dequantises and
    re-searches every element instead)."""
    ops().remap_indices(idx, index_map.to(device=idx.device, dtype=torch.uint8).contiguous())
    return idx


def dequantize(idx: torch.Tensor, mag: torch.Tensor, codebook: torch.Tensor, period: int,
               dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Dense momentum ``codebook[idx] * mag[block]`` of a contiguous uint8 CUDA index tensor
    (reference ``src/gefen/dcp.py:54-81``); ``mag`` holds one value per block of ``period``."""
    out = torch.empty(idx.shape, dtype=dtype, device=idx.device)
    ops().dequantize(idx, mag.reshape(-1).contiguous(), codebook.to(idx.device, torch.float32).contiguous(),
                     int(period), out)
    return out


def quantize_rows_e4m3(x: torch.Tensor, x2: torch.Tensor = None, alpha: float = 1.0, beta: float = 0.0,
                       want_y: bool = False):
    """Row-wise e4m3 quantisation of ``y = alpha * x + beta * x2`` (``y = x`` without ``x2``), one
    kernel: returns ``(q, scale, y)`` with ``q`` in ``torch.float8_e4m3fn``, ``scale`` fp32
    ``[rows, 1]`` such that ``q * scale ~= y`` (each row's absmax maps to 448) and ``y`` in bf16
    when ``want_y`` (else ``None``).  ``x`` / ``x2``: 2-D bf16 CUDA with unit column stride and a
    column count that is a multiple of 8 (kernel: ``csrc/fp8_quant.cu``)."""
    q = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    scale = torch.empty(x.shape[0], 1, dtype=torch.float32, device=x.device)
    y = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device) if want_y else None
    ops().quantize_rows_e4m3(x, x2, float(alpha), float(beta), q, scale, y)
    return q, scale, y


def quantize_cols_e4m3_t(x: torch.Tensor):
    """``quantize_rows_e4m3(x.t().contiguous())`` without the transposed copy: returns
    ``(q_t, scale_t)`` with ``q_t`` ``[cols, rows]`` in e4m3 and ``scale_t`` fp32 ``[cols, 1]``
    (each column's absmax maps to 448).  ``x``: 2-D bf16 CUDA, unit column stride, rows a multiple
    of 4 and columns a multiple of 8."""
    rows, cols = x.shape
    colmax = torch.zeros(cols, dtype=torch.int32, device=x.device)
    q_t = torch.empty(cols, rows, dtype=torch.float8_e4m3fn, device=x.device)
    scale_t = torch.empty(cols, 1, dtype=torch.float32, device=x.device)
    ops().quantize_cols_e4m3_t(x, colmax, q_t, scale_t)
    return q_t, scale_t
