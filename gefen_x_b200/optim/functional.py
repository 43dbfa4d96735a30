"""Decomposed (pure torch) statement of the update math.

These functions are the numerical definition of the optimizer: the CUDA kernels
in ``csrc/update.cu`` evaluate exactly the same fp32 expression trees (products
and sums rounded separately, no fused multiply-add), so the quantised momentum
indices and magnitudes they produce are bit-identical to what is computed here,
and parameters / second moments agree up to the order of the sum-of-squares
reductions.  They also serve CPU tensors, fp64 tensors and CPU-offloaded shards.

Math of one block ``b`` of ``P`` contiguous elements (reference
``src/gefen/gefen.py:3329-3436``, ``:2959-3018`` and the kernel comments at
``src/gefen/kernels/automatic_gefen_fused_kernel.cu:1756-1956``)::

    m_old = codebook[idx] * mag_old[b]
    m     = m_old * beta1 + g * (1 - beta1)
    mag[b]= max |m|                      inv = 1 / mag[b]  (0 when mag[b] == 0)
    idx'  = nearest(codebook, m * inv)   (ties -> lower index)
    q     = codebook[idx'] * mag[b]
    p     = round(p * (1 - lr * wd)) - (q * step) * lr

``step`` is per block on the block path and per element on the factored path.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from ..quant.codebook import dequantize_indices, nearest_codebook_indices

_TINY = torch.finfo(torch.float32).tiny
# Rows of a [blocks, period] view handled at once by the streamed update.
UPDATE_CHUNK_ELEMS = 1 << 23


def partition_view(flat: torch.Tensor, period: int) -> torch.Tensor:
    if flat.dim() != 1:
        raise ValueError("Automatic partition view expects a 1D tensor, got dim={}".format(flat.dim()))
    if period <= 0 or flat.numel() % period:
        raise ValueError(
            "Automatic partition period {} does not divide numel {}".format(period, flat.numel()))
    return flat.view(-1, period)


def _scaled(g: torch.Tensor, grad_scale) -> torch.Tensor:
    g = g.float()
    if grad_scale is None:
        return g
    return g * grad_scale


def momentum_requantize_(
    codebook: torch.Tensor,
    m_codebook: torch.Tensor,
    m_magnitude: torch.Tensor,
    grad_view: torch.Tensor,
    beta1: float,
    grad_scale=None,
) -> torch.Tensor:
    """Advance the quantised EMA of ``grad_view`` in place; return ``q`` (fp32).

    ``m_codebook`` uint8 ``[blocks, P]`` and ``m_magnitude`` fp32 ``[blocks, 1]``
    are overwritten with the new indices / magnitudes.
    """
    m_old = dequantize_indices(codebook, m_codebook, torch.float32) * m_magnitude
    m = m_old * beta1 + _scaled(grad_view, grad_scale) * (1.0 - beta1)
    mag = m.abs().amax(dim=1, keepdim=True)
    inv = torch.where(mag > 0, 1.0 / mag, torch.zeros_like(mag))
    idx = nearest_codebook_indices(codebook, m * inv)
    m_codebook.copy_(idx)
    m_magnitude.copy_(mag)
    return dequantize_indices(codebook, idx, torch.float32) * mag


def block_second_moment_(vmean: torch.Tensor, grad_view: torch.Tensor, beta2: float,
                         grad_scale=None) -> None:
    """``vmean = vmean*beta2 + mean_b(g^2)*(1-beta2)`` with the square taken in fp32."""
    g = _scaled(grad_view, grad_scale)
    ms = (g * g).sum(dim=1, keepdim=True) * (1.0 / grad_view.shape[1])
    vmean.mul_(beta2).add_(ms * (1.0 - beta2))


def block_stepsize(vmean: torch.Tensor, eps: float, bc1, bc2) -> torch.Tensor:
    """``(1 / (sqrt(vmean) * (1/sqrt(bc2)) + eps)) * (1/bc1)``; bc may be device scalars."""
    if torch.is_tensor(bc2):
        inv_sqrt_bc2 = 1.0 / bc2.sqrt()
    else:
        inv_sqrt_bc2 = 1.0 / math.sqrt(bc2)
    inv_bc1 = 1.0 / bc1
    h = vmean.sqrt() * inv_sqrt_bc2 + eps
    return h.reciprocal() * inv_bc1


def factored_second_moment_(
    v_row: torch.Tensor,
    v_col: torch.Tensor,
    grad2d: torch.Tensor,
    beta2: float,
    grad_scale=None,
    *,
    total_rows: Optional[int] = None,
    reduce_cols=None,
) -> None:
    """Row / column EMAs of ``g^2`` for a (row shard of a) matrix.

    ``total_rows`` is the row count of the whole matrix when ``grad2d`` is a
    ``Shard(0)`` slice of it; ``reduce_cols`` then sums the column partials over
    the shards (an all-reduce) so that ``v_col`` stays replicated.
    """
    rows, cols = grad2d.shape
    total_rows = rows if total_rows is None else total_rows
    row_sq = torch.empty(rows, dtype=torch.float32, device=grad2d.device)
    col_sq = torch.zeros(cols, dtype=torch.float32, device=grad2d.device)
    step_rows = max(1, (1 << 20) // max(1, cols))
    for r0 in range(0, rows, step_rows):
        g = _scaled(grad2d[r0:r0 + step_rows], grad_scale)
        sq = g * g
        row_sq[r0:r0 + step_rows] = sq.sum(dim=1)
        col_sq += sq.sum(dim=0)
    if reduce_cols is not None:
        col_sq = reduce_cols(col_sq)
    v_row.mul_(beta2).add_(row_sq * (1.0 / cols) * (1.0 - beta2))
    v_col.mul_(beta2).add_(col_sq * (1.0 / total_rows) * (1.0 - beta2))


def factored_factors(
    v_row: torch.Tensor, v_col: torch.Tensor, bc2, *, total_rows: Optional[int] = None,
    reduce_scalar=None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-row and per-column factors whose product is ``sqrt(v_hat / bc2)``.

    ``v_hat[i, j] = v_row[i] * v_col[j] / max(mean(v_row), tiny)``; the row
    factor carries ``1 / mean`` and ``1 / bc2``.
    """
    total_rows = v_row.numel() if total_rows is None else total_rows
    s = v_row.sum()
    if reduce_scalar is not None:
        s = reduce_scalar(s)
    mean = (s * (1.0 / total_rows)).clamp(min=_TINY)
    inv_mean = 1.0 / mean
    inv_bc2 = 1.0 / bc2
    rfac = (v_row * inv_mean * inv_bc2).sqrt()
    cfac = v_col.sqrt()
    return rfac, cfac


def factored_stepsize(rfac: torch.Tensor, cfac: torch.Tensor, eps: float, bc1) -> torch.Tensor:
    h = torch.outer(rfac, cfac) + eps
    return h.reciprocal() * (1.0 / bc1)


def apply_update_(p: torch.Tensor, q: torch.Tensor, stepsize: torch.Tensor, lr,
                  weight_decay_factor) -> None:
    """``p = round(p * wdf) - (q * step) * lr`` (the product is rounded to p's dtype first)."""
    if torch.is_tensor(weight_decay_factor) or weight_decay_factor != 1.0:
        p.mul_(weight_decay_factor)
    upd = (q * stepsize).mul_(lr)
    if p.dtype == torch.float32:
        p.sub_(upd.view(p.shape))
    else:
        p.copy_((p.float() - upd.view(p.shape)).to(p.dtype))


def block_update_(
    p: torch.Tensor,
    grad_view: torch.Tensor,
    codebook: torch.Tensor,
    m_codebook: torch.Tensor,
    m_magnitude: torch.Tensor,
    vmean: torch.Tensor,
    *,
    beta1: float,
    beta2: float,
    eps: float,
    lr,
    weight_decay_factor,
    bc1,
    bc2,
    grad_scale=None,
) -> None:
    """Full block-path step of one (contiguous) parameter, streamed over row chunks."""
    period = grad_view.shape[1]
    block_second_moment_(vmean, grad_view, beta2, grad_scale)
    stepsize = block_stepsize(vmean, eps, bc1, bc2)
    contiguous = p.is_contiguous()
    work = p if contiguous else p.contiguous()
    flat = work.view(-1)
    if torch.is_tensor(weight_decay_factor) or weight_decay_factor != 1.0:
        flat.mul_(weight_decay_factor)
    rows = max(1, UPDATE_CHUNK_ELEMS // period)
    for r0 in range(0, grad_view.shape[0], rows):
        r1 = min(r0 + rows, grad_view.shape[0])
        q = momentum_requantize_(codebook, m_codebook[r0:r1], m_magnitude[r0:r1],
                                 grad_view[r0:r1], beta1, grad_scale)
        upd = (q * stepsize[r0:r1]).mul_(lr).reshape(-1)
        seg = flat[r0 * period:r1 * period]
        if seg.dtype == torch.float32:
            seg.sub_(upd)
        else:
            seg.copy_((seg.float() - upd).to(seg.dtype))
    if not contiguous:
        p.copy_(work)


def factored_update_(
    p: torch.Tensor,
    grad2d: torch.Tensor,
    period: int,
    codebook: torch.Tensor,
    m_codebook: torch.Tensor,
    m_magnitude: torch.Tensor,
    v_row: torch.Tensor,
    v_col: torch.Tensor,
    *,
    beta1: float,
    beta2: float,
    eps: float,
    lr,
    weight_decay_factor,
    bc1,
    bc2,
    grad_scale=None,
    total_rows: Optional[int] = None,
    reduce_cols=None,
    reduce_scalar=None,
) -> None:
    """Full factored-path step of one 2-D parameter (or ``Shard(0)`` slice of one)."""
    factored_second_moment_(v_row, v_col, grad2d, beta2, grad_scale,
                            total_rows=total_rows, reduce_cols=reduce_cols)
    rfac, cfac = factored_factors(v_row, v_col, bc2, total_rows=total_rows,
                                  reduce_scalar=reduce_scalar)
    stepsize = factored_stepsize(rfac, cfac, eps, bc1)
    gv = partition_view(grad2d.reshape(-1), period)
    q = momentum_requantize_(codebook, m_codebook, m_magnitude, gv, beta1, grad_scale)
    contiguous = p.is_contiguous()
    work = p if contiguous else p.contiguous()
    apply_update_(work, q.view(work.shape), stepsize, lr, weight_decay_factor)
    if not contiguous:
        p.copy_(work)
