"""Matrix products used by the decoder and by Newton–Schulz.

``set_backend("tcgen05")`` (the default on CUDA bf16 operands) sends every layer product
-- forward ``x W^T``, input gradient ``dy W`` and weight gradient ``dy^T x`` -- to the
hand-written tcgen05 kernels of ``csrc/gemm_pair_sm100.cu`` / ``csrc/gemm_sm100.cu``
through :mod:`gefen_x_b200.ops.tcgemm`, including the fused forms of the decoder layer:
residual add in the epilogue (:func:`mm_nt_add`), SwiGLU inside the gate/up projection
(:func:`mlp_gate_up`) and its derivative inside the ``down_proj`` input gradient
(:func:`mlp_down_dgrad`).  ``set_backend("library")`` keeps the same call sites on the
vendor library (``torch.matmul``) with the unfused elementwise kernels, as the comparison
path; CPU tensors and other dtypes always take it.  The reference's model multiplies
through torch (reference ``benchmarks/training_matrix/tiny_qwen.py:168-181``, ``:250-259``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

_BACKEND = "tcgen05"


def set_backend(name: str) -> None:
    """``"tcgen05"`` (own kernels where shapes allow) or ``"library"`` (cuBLAS via torch)."""
    global _BACKEND
    if name not in ("library", "tcgen05"):
        raise ValueError("unknown GEMM backend {!r}".format(name))
    _BACKEND = name


def backend() -> str:
    return _BACKEND


def _tc(*ts: torch.Tensor) -> bool:
    if _BACKEND != "tcgen05":
        return False
    from . import tcgemm

    return all(t is None or tcgemm._ok_operand(t) for t in ts) and ts[0].dim() == 2


def mm_nt(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T``."""
    if _tc(a, b, out):
        from . import tcgemm

        return tcgemm.gemm(a, b, out=out)
    if out is None:
        return a @ b.t()
    return torch.matmul(a, b.t(), out=out)


def mm_nt_add(a: torch.Tensor, b: torch.Tensor, res: torch.Tensor) -> torch.Tensor:
    """``res + a [M, K] @ b [N, K]^T`` (the residual add runs in the product's epilogue)."""
    if _tc(a, b, res):
        from . import tcgemm

        return tcgemm.gemm(a, b, beta=1.0, d=res)
    return res + a @ b.t()


def mm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [K, N]``."""
    if _tc(a, b, out):
        from . import tcgemm

        return tcgemm.gemm(a, b, b_t=True, out=out)
    if out is None:
        return a @ b
    return torch.matmul(a, b, out=out)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [K, M]^T @ b [K, N]``."""
    if _tc(a, b, out):
        from . import tcgemm

        return tcgemm.gemm(a, b, a_t=True, b_t=True, out=out)
    if out is None:
        return a.t() @ b
    return torch.matmul(a.t(), b, out=out)


_GRAD_SUMSQ: Optional[torch.Tensor] = None


def set_grad_sumsq(partials: Optional[torch.Tensor]) -> None:
    """While set (an fp32 tensor of at least 2048 slots), :func:`mm_tn_wgrad` adds the sum of squares
    of every weight gradient it writes into ``partials`` -- the global gradient norm then needs no
    extra pass over the gradients (single-GPU runs; with several ranks the norm is that of the
    reduced gradient and is taken after the reduction)."""
    global _GRAD_SUMSQ
    _GRAD_SUMSQ = partials


def grad_sumsq() -> Optional[torch.Tensor]:
    return _GRAD_SUMSQ


def mm_tn_wgrad(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Weight gradient ``out = a [T, M]^T @ b [T, N]``, contributing to the gradient norm when
    :func:`set_grad_sumsq` is active (in the product's epilogue where the kernel allows, by one pass
    over ``out`` otherwise)."""
    sq = _GRAD_SUMSQ
    if sq is None:
        return mm_tn(a, b, out=out)
    if _tc(a, b, out):
        from . import tcgemm

        if tcgemm.pair_eligible(a.shape[1], b.shape[1], a.shape[0]):
            return tcgemm.gemm(a, b, a_t=True, b_t=True, out=out, sumsq=sq)
    mm_tn(a, b, out=out)
    add_sumsq(out, sq)
    return out


def add_sumsq(t: torch.Tensor, partials: torch.Tensor) -> None:
    """``partials += slot-wise partial sums of t^2`` (one pass over a contiguous tensor)."""
    from . import update as U

    if t.is_cuda and t.is_contiguous() and t.dtype in U.DTYPE_CODE:
        U.reduce_sources(None, [t.data_ptr()], t.numel(), 1.0, partials, t.dtype, t.device)
    else:
        partials[0] += t.float().square().sum()


def mlp_gate_up(h: torch.Tensor, w_gate_up: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(gu, act)`` with ``gu = h @ w_gate_up^T`` (``[M, 2F]``) and ``act = silu(gate) * up``."""
    from . import model as M

    if _tc(h, w_gate_up):
        from . import tcgemm

        if tcgemm.swiglu_eligible(h.shape[0], w_gate_up.shape[0] // 2, h.shape[1]):
            return tcgemm.gemm_swiglu_fwd(h, w_gate_up)
    gu = mm_nt(h, w_gate_up)
    return gu, M.swiglu_fwd(gu)


def mlp_down_dgrad(dy: torch.Tensor, w_down: torch.Tensor, gate_up: torch.Tensor) -> torch.Tensor:
    """``d(gate|up)`` given ``dy`` (gradient of the ``down_proj`` output), ``w_down [H, F]`` and the
    forward's ``gate_up``: the SwiGLU derivative is applied in the epilogue of ``dy @ w_down``."""
    from . import model as M

    if _tc(dy, w_down, gate_up):
        from . import tcgemm

        if tcgemm.swiglu_eligible(dy.shape[0], w_down.shape[1], dy.shape[1]):
            return tcgemm.gemm_swiglu_bwd(dy, w_down, gate_up)
    return M.swiglu_bwd(gate_up, mm_nn(dy, w_down))
