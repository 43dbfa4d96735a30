"""tcgen05 / TMEM bf16 GEMMs (``csrc/gemm_pair_sm100.cu``, ``csrc/gemm_sm100.cu``).

``gemm(a, b, ...)`` computes ``alpha * op(a) @ op(b)^T-or-not + beta * d`` on the
5th-generation tensor cores with TMA-fed operands.  Layout convention: with
``a_t=False`` the first operand is ``[M, K]`` (K contiguous), with ``a_t=True`` it
is stored ``[K, M]``; with ``b_t=False`` the second operand is ``[N, K]`` (so the
product is ``a @ b.T``), with ``b_t=True`` it is stored ``[K, N]`` (``a @ b``).
3-D inputs are batches.

Two kernels serve it.  Large 2-D products run on CTA pairs
(``tcgen05.mma.cta_group::2``, a 256 x 256 or 256 x 128 tile per pair, TMA-store
epilogue); batches and small products run on the single-CTA kernel.  The pair
kernel also carries the fused epilogues of the decoder's MLP:
:func:`gemm_swiglu_fwd` (gate/up projection + ``silu(gate) * up``) and
:func:`gemm_swiglu_bwd` (input gradient of ``down_proj`` + the SwiGLU derivative).

The reference uses cuBLAS through torch for the same products (reference
``src/gefen/gefen_muon.py:278-287``, ``:353-393``;
``benchmarks/training_matrix/tiny_qwen.py:168-181``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from ._ext import available, ops

_status = {}
_PAIR = True            # route eligible 2-D products to the CTA-pair kernel
_FORCE_BN = 0           # 0: choose per shape; 128 / 256: force the pair tile width (benchmarks)
_DYNAMIC = False        # pair kernel: draw tiles from a counter instead of the fixed assignment


def set_pair_kernel(enabled: bool, bn: int = 0) -> None:
    """Switch the CTA-pair kernel on or off (off: every product uses the single-CTA kernel)."""
    global _PAIR, _FORCE_BN
    if bn not in (0, 128, 256):
        raise ValueError("bn must be 0, 128 or 256")
    _PAIR, _FORCE_BN = bool(enabled), int(bn)


def set_dynamic_schedule(enabled: bool) -> None:
    """Dynamic tile schedule of the pair kernel: pairs draw the next tile from a device counter when
    they are free, so a pair slowed down by kernels of other streams on its SMs (gradient
    reduce-scatter, copies: the sharded runtime) does not hold a product back.  The static schedule
    (default) places every tile on a fixed pair, which makes the fused gradient-norm sums
    reproducible bit for bit."""
    global _DYNAMIC
    _DYNAMIC = bool(enabled)


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


def pair_eligible(m: int, n: int, k: int) -> bool:
    """Shapes the CTA-pair kernel takes (the rest goes to the single-CTA kernel)."""
    return _PAIR and m >= 129 and n >= 128 and k >= 64 and n % 8 == 0


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_t: bool = False, b_t: bool = False,
         alpha: float = 1.0, beta: float = 0.0, d: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None, sumsq: Optional[torch.Tensor] = None,
         symmetric: bool = False) -> torch.Tensor:
    """See the module docstring for the layout convention.

    ``symmetric``: the caller states that the result is a symmetric matrix (``X X^T``, or ``c G G + b G``
    with ``G`` symmetric).  The CTA-pair kernel then computes only the 256 x 256 tiles on and below the
    diagonal (T (T + 1) / 2 of T^2) and a small second launch copies them across it; matrices of
    fewer than 2048 rows and the other kernels ignore the hint.

    ``sumsq`` (fp32, at least 2048 slots) receives, added slot-wise, the sum of squares of the stored
    output -- the gradient-norm contribution of a weight-gradient product, computed in its epilogue.
    Only the CTA-pair kernel provides it: check :func:`pair_eligible` (``gemm`` raises otherwise)."""
    m = a.shape[-1] if a_t else a.shape[-2]
    n = b.shape[-1] if b_t else b.shape[-2]
    k = a.shape[-2] if a_t else a.shape[-1]
    if out is None:
        out = torch.empty(*a.shape[:-2], m, n, dtype=torch.bfloat16, device=a.device)
    dd = d if beta != 0.0 else None
    if a.dim() == 2 and pair_eligible(m, n, k) and _ok_operand(out) and (dd is None or _ok_operand(dd)):
        # from eight tile rows on (36 of 64 tiles): below that the second launch costs what the tiles save
        sym = bool(symmetric) and m == n and m >= 2048 and sumsq is None and _FORCE_BN in (0, 256)
        ops().gemm_pair_bf16(a, b, out, None, dd, None, bool(a_t), bool(b_t), float(alpha), float(beta), 0,
                             _FORCE_BN, status_word(a.device), sumsq, _DYNAMIC, sym)
        return out
    if sumsq is not None:
        raise ValueError("sumsq needs the CTA-pair kernel; this product does not qualify")
    ops().gemm_bf16(a, b, out, dd, bool(a_t), bool(b_t), float(alpha), float(beta), status_word(a.device))
    return out


def gemm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T``."""
    return gemm(a, b, out=out)


def e4m3_eligible(m: int, n: int, k: int) -> bool:
    """Shapes the e4m3 variant of the CTA-pair kernel takes: 16-byte rows for the tensor maps."""
    return _PAIR and m >= 129 and n >= 128 and k >= 128 and k % 16 == 0 and n % 8 == 0


def gemm_e4m3(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``out[m, n] = sum_k aq[m, k] * bq[n, k] * sa[m] * sb[n]`` in bf16: the row-scaled e4m3 product on
    the tensor cores (``tcgen05.mma`` of kind f8f6f4 in the CTA-pair kernel, fp32 accumulation, the two
    scale vectors applied in the epilogue).  ``aq`` [M, K] and ``bq`` [N, K] are ``float8_e4m3fn`` with
    unit inner stride and rows that start on 16-byte boundaries; ``sa`` / ``sb`` hold M / N fp32 scales."""
    m, k = aq.shape
    n = bq.shape[0]
    if not (aq.is_cuda and e4m3_eligible(m, n, k)):
        raise ValueError("gemm_e4m3: shape {}x{}x{} is not eligible for the pair kernel".format(m, n, k))
    if out is None:
        out = torch.empty(m, n, dtype=torch.bfloat16, device=aq.device)
    ops().gemm_pair_e4m3(aq, bq, sa.reshape(-1).contiguous(), sb.reshape(-1).contiguous(), out,
                         status_word(aq.device), _DYNAMIC)
    return out


def swiglu_eligible(m: int, f: int, k: int) -> bool:
    return _PAIR and m >= 129 and f >= 128 and f % 8 == 0 and k >= 64


def gemm_swiglu_fwd(x: torch.Tensor, w_gate_up: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gu = x @ w_gate_up^T`` and ``act = silu(gu[:, :F]) * gu[:, F:]`` in one launch.

    ``w_gate_up`` is the stacked ``[2F, K]`` weight (gate rows first).  Returns ``(gu [M, 2F],
    act [M, F])``; ``act`` is computed from the bf16-rounded ``gu``, exactly as the separate
    activation kernel would.
    """
    m, f = x.shape[0], w_gate_up.shape[0] // 2
    gu = torch.empty(m, 2 * f, dtype=torch.bfloat16, device=x.device)
    act = torch.empty(m, f, dtype=torch.bfloat16, device=x.device)
    ops().gemm_pair_bf16(x, w_gate_up, gu, act, None, None, False, False, 1.0, 0.0, 1, 0, status_word(x.device),
                         None, _DYNAMIC, False)
    return gu, act


def gemm_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """``d(gate|up)`` from ``d(act) = dy @ w_down`` without storing ``d(act)``.

    ``w_down`` is ``[H, F]`` (the ``down_proj`` weight), ``gate_up`` the forward's ``[M, 2F]``.
    """
    dgu = torch.empty_like(gate_up)
    ops().gemm_pair_bf16(dy, w_down, dgu, None, None, gate_up, False, True, 1.0, 0.0, 2, _FORCE_BN,
                         status_word(dy.device), None, _DYNAMIC, False)
    return dgu
