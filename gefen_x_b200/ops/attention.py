"""Causal GQA attention on own kernels (no library attention).

Forward, fused ("flash") form, when the sequence length is a multiple of 128 and the head size is
64 or 128: ``flash_fwd_kernel`` (``csrc/gemm_sm100.cu``) keeps the score tile in TMEM and feeds the
probabilities through shared memory into the second tcgen05 product; only O and the row
log-sum-exp reach HBM.  Otherwise the forward is composed like the backward:

Forward (composed):  S = Q K^T (batched tcgen05 GEMM, one batch entry per (sequence, KV head) with the
group's query heads stacked along the rows), P = causal softmax(S / sqrt(d)) in place
(``attention.cu``), O = P V (GEMM).  Only O and the row log-sum-exp are kept.
Backward: S and P are recomputed, dP = dO V^T, dS = P * (dP - rowsum(dO * O)) / sqrt(d) in place,
dV = P^T dO, dK = dS^T Q, dQ = dS K; the products over the group's heads fall out of the stacked
rows, so no extra reduction over query heads is needed.

The score matrix is materialised (``B * n_q * S * S`` bf16 values), so this path is for moderate
sequence lengths; the default attention of the model remains the fused library kernel
(``ops.model.attention_fwd``).  The reference calls ``F.scaled_dot_product_attention``
(reference ``benchmarks/training_matrix/tiny_qwen.py:168``).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch

from . import tcgemm
from ._ext import ops


def supported(q: torch.Tensor, k: torch.Tensor) -> bool:
    B, S, nq, hd = q.shape
    return (q.is_cuda and q.dtype == torch.bfloat16 and hd % 8 == 0 and S % 8 == 0 and k.shape[1] == S
            and nq % k.shape[2] == 0)


def _heads_first(x: torch.Tensor, nkv: int) -> torch.Tensor:
    """[B, S, n, hd] -> [B * nkv, (n / nkv) * S, hd] (the group's heads stacked along the rows)."""
    B, S, n, hd = x.shape
    return x.permute(0, 2, 1, 3).contiguous().view(B * nkv, (n // nkv) * S, hd)


def _heads_last(x: torch.Tensor, B: int, S: int, n: int) -> torch.Tensor:
    """Inverse of :func:`_heads_first`: -> [B, S, n, hd] contiguous."""
    hd = x.shape[-1]
    return x.view(B, n, S, hd).permute(0, 2, 1, 3).contiguous()


def flash_supported(S: int, hd: int) -> bool:
    return S % 128 == 0 and hd in (64, 128)


def attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, flash: bool = True) -> Tuple[torch.Tensor, tuple]:
    """q: [B, S, nq, hd], k / v: [B, S, nkv, hd] (bf16).  Returns (out [B, S, nq, hd], ctx)."""
    B, S, nq, hd = q.shape
    nkv = k.shape[2]
    scale = 1.0 / math.sqrt(hd)
    qh, kh, vh = _heads_first(q, nkv), _heads_first(k, nkv), _heads_first(v, nkv)
    if flash and flash_supported(S, hd):
        oh = torch.empty_like(qh)
        lse = torch.empty(qh.shape[0] * qh.shape[1], dtype=torch.float32, device=q.device)
        ops().flash_attention_fwd(qh, kh, vh, oh, lse, S, scale, tcgemm.status_word(q.device))
        return _heads_last(oh, B, S, nq), (qh, kh, vh, oh, lse, (B, S, nq, nkv, hd, scale))
    scores = tcgemm.gemm(qh, kh)                                   # [B*nkv, G*S, S]
    lse = torch.empty(scores.shape[0] * scores.shape[1], dtype=torch.float32, device=q.device)
    ops().attn_softmax(scores, lse, S, scale)
    oh = tcgemm.gemm(scores, vh, b_t=True)                         # [B*nkv, G*S, hd]
    del scores
    out = _heads_last(oh, B, S, nq)
    return out, (qh, kh, vh, oh, lse, (B, S, nq, nkv, hd, scale))


def attention_bwd(ctx, dout: torch.Tensor):
    qh, kh, vh, oh, lse, (B, S, nq, nkv, hd, scale) = ctx
    doh = _heads_first(dout, nkv)                                  # [B*nkv, G*S, hd]
    delta = torch.empty_like(lse)
    ops().attn_row_dot(doh, oh, delta)
    scores = tcgemm.gemm(qh, kh)                                   # recomputed
    dprob = tcgemm.gemm(doh, vh)                                   # dO V^T
    ops().attn_bwd_rows(scores, dprob, lse, delta, S, scale)       # -> P, dS in place
    dv = tcgemm.gemm(scores, doh, a_t=True, b_t=True)              # P^T dO   [B*nkv, S, hd]
    dk = tcgemm.gemm(dprob, qh, a_t=True, b_t=True)                # dS^T Q
    dq = tcgemm.gemm(dprob, kh, b_t=True)                          # dS K     [B*nkv, G*S, hd]
    return (_heads_last(dq, B, S, nq), _heads_last(dk, B, S, nkv), _heads_last(dv, B, S, nkv))
