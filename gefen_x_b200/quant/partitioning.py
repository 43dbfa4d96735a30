"""Block-period search for the shared second moment / momentum magnitude.

A parameter's flattened gradient is cut into ``numel / P`` blocks of ``P``
contiguous elements; every block shares one momentum magnitude and (on the
block path) one second-moment value.  ``P`` is chosen once, at the first step,
as the proper divisor of ``numel`` whose score
``err[P] - err[previous divisor]`` is smallest, where
``err[P] = sqrt(mean_over_blocks(var_within_block(g^2)))``.

Behavioural parity: reference ``src/gefen/partitioning.py`` (divisor
enumeration ``:50-59``, scoring and the ``< 8 -> 1`` rule ``:237-271``, the
memory-safe fallback ``:31-47``, dispatcher ``:274-313``).  The evaluation
itself is organised differently here: all divisors are scored from one
vectorised pass (CPU, float64) or from one CUDA launch (``ops.quant``) instead
of one host-synchronised launch per divisor.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

# When the search finds no block structure (period 1) the state would cost ~9
# bytes per parameter.  With the fallback on, such tensors get a coarse
# shape-aligned block instead (the input-feature row of a matrix, or the largest
# divisor up to FALLBACK_PERIOD_CAP), keeping state near 1 byte per parameter.
MEMORY_SAFE_FALLBACK = True
FALLBACK_PERIOD_CAP = 2048


def _largest_divisor_at_most(n: int, cap: int) -> int:
    best = 1
    for i in range(1, math.isqrt(n) + 1):
        if n % i:
            continue
        j = n // i
        if best < i <= cap:
            best = i
        if best < j <= cap:
            best = j
    return best


def memory_safe_fallback_period(n: int, parameter_shape) -> int:
    """Coarse block used instead of period 1 (reference ``partitioning.py:31-47``)."""
    if n < 8:
        return 1
    picks = []
    if parameter_shape is not None and len(parameter_shape) >= 2:
        in_features = int(parameter_shape[-1])
        if in_features >= 8 and n % in_features == 0:
            picks.append(in_features)
    capped = _largest_divisor_at_most(n, FALLBACK_PERIOD_CAP)
    if capped >= 8:
        picks.append(capped)
    return max(picks) if picks else 1


def divisors(n: int) -> List[int]:
    """Proper divisors of ``n`` (``n`` itself excluded), ascending."""
    lo, hi = [], []
    for i in range(1, math.isqrt(n) + 1):
        if n % i:
            continue
        if i != n:
            lo.append(i)
        j = n // i
        if j != i and j != n:
            hi.append(j)
    return lo + hi[::-1]


def average_within_block_variance_torch(values: torch.Tensor, period: int, parameter_name=None,
                                        parameter_shape=None) -> float:
    """``sqrt(mean_b var_b)`` for one candidate period (population variance)."""
    v = values.detach().reshape(-1)
    if v.numel() % period:
        raise ValueError(
            "Expected length {} to be divisible by period {}.".format(v.numel(), period)
        )
    dt = torch.float64 if v.device.type == "cpu" else torch.float32
    blocks = v.to(dt).view(-1, period)
    return float(torch.sqrt(blocks.var(dim=1, correction=0).mean()).item())


def average_within_block_variance_cpu(list_of_values, period_to_check, parameter_name=None,
                                      parameter_shape=None) -> float:
    """Float64 CPU scorer, accepts anything ``torch.as_tensor`` accepts."""
    t = torch.as_tensor(list_of_values, dtype=torch.float64, device="cpu")
    return average_within_block_variance_torch(t, int(period_to_check))


def block_variance_errors(values: torch.Tensor, divs: Sequence[int]) -> List[float]:
    """``err[p]`` for every candidate in ``divs`` with fixed-order reductions.

    On CUDA tensors this stays on torch reductions (deterministic order); the
    single-launch kernel lives in ``ops.quant.period_errors``.
    """
    v = values.detach().reshape(-1)
    dt = torch.float64 if v.device.type == "cpu" else torch.float32
    v = v.to(dt)
    out = []
    for p in divs:
        out.append(
            float(torch.sqrt(v.view(-1, p).var(dim=1, correction=0).mean()).item())
        )
    return out


def select_period(
    candidates: Sequence[Tuple[int, float]], print_results: bool = False
) -> int:
    """Pick the period from ``(p, err)`` pairs listed in ascending ``p``.

    Score of the first candidate is ``1e-12``, of every later one
    ``err - previous err``; the smallest score wins, ties go to the smaller
    period, and a winner below 8 collapses to 1.
    """
    if len(candidates) == 0:
        raise ValueError("Expected at least one valid period candidate.")
    scored = []
    prev = None
    for p, err in candidates:
        score = 1e-12 if prev is None else err - prev
        prev = err
        scored.append((score, p, err))
    best_score, best_period, _ = min(scored)
    if print_results:
        for score, p, err in scored:
            mark = " <-" if score == best_score else ""
            print("p={} | err={:.15f} | score={:.15f}{}".format(p, err, score, mark))
    return 1 if best_period < 8 else best_period


# Name kept for callers that know the reference's helper.
_finalize_period_results = select_period


def find_period_by_block_variance(
    squared_grad_flattened_values,
    print_results: bool = True,
    parameter_name: Optional[str] = None,
    parameter_shape=None,
    backend: str = "cpu",
    input_is_squared: bool = True,
) -> int:
    """Search the block period of one tensor.

    ``backend``: ``"cpu"`` (float64 torch on the host), ``"gpu"`` (fixed-order
    torch reductions on the tensor's CUDA device) or ``"cuda_kernel"`` (one
    launch scoring every divisor, fixed-order partial sums).  With
    ``input_is_squared=False`` the values are raw gradients and are squared in
    fp32 first.
    """
    vals = squared_grad_flattened_values
    if backend == "cpu":
        t = torch.as_tensor(vals).detach().reshape(-1).to("cpu", torch.float64)
        if not input_is_squared:
            t = t.square()
    elif backend in ("gpu", "cuda_kernel"):
        if not isinstance(vals, torch.Tensor):
            raise TypeError(
                "Expected torch.Tensor for {} backend, got {}".format(
                    backend, type(vals).__name__
                )
            )
        if vals.device.type != "cuda":
            raise ValueError(
                "Expected a CUDA tensor for {} backend, got device {}".format(
                    backend, vals.device
                )
            )
        t = vals.detach().reshape(-1)
    else:
        raise ValueError("Unexpected backend: {}".format(backend))

    n = int(t.numel())
    divs = divisors(n)
    if not divs:
        raise ValueError(
            "Could not find any valid period candidates. parameter_name={} "
            "parameter_shape={}".format(parameter_name, parameter_shape)
        )
    if backend == "cuda_kernel":
        from ..ops import quant as _q

        errs = _q.period_errors(t, divs, input_is_squared=input_is_squared)
    else:
        if backend == "gpu" and not input_is_squared:
            t = t.float().square()
        errs = block_variance_errors(t, divs)
    period = select_period(list(zip(divs, errs)), print_results)
    if MEMORY_SAFE_FALLBACK and period == 1:
        return memory_safe_fallback_period(n, parameter_shape)
    return period
