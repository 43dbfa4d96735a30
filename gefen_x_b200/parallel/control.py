"""Tiny host-synchronous agreement collectives used before any mutation.

A step that is about to enter a collective (or to mutate sharded state) first
agrees with its peers on "did anybody fail?" and on the AMP controls, so that a
failure on one rank raises on every rank and nobody is left waiting inside a
collective.  These stay on ``torch.distributed`` (NCCL or Gloo): they are a few
bytes, latency-bound and correctness-critical.

Parity: reference ``src/gefen/gefen.py:534-556`` (device choice), ``:559-583``
(failure flag, all-reduce MAX of one int32) and ``:586-615`` (bounds agreement,
all-reduce MIN over ``(min, -max)`` packed as fp64).
"""
from __future__ import annotations

from typing import Iterable, Optional, Sequence, Tuple

import torch


def _dist():
    import torch.distributed as dist

    return dist


def distributed_ready() -> bool:
    return torch.distributed.is_available() and torch.distributed.is_initialized()


def control_device(process_group=None, *, collective_device=None) -> torch.device:
    """Device on which a control flag must live for ``process_group``'s backend."""
    if collective_device is not None:
        return torch.device(collective_device)
    dist = _dist()
    group = process_group if process_group is not None else dist.group.WORLD
    bound = getattr(group, "bound_device_id", None)
    if bound is not None:
        return torch.device(bound)
    backend = str(dist.get_backend(process_group)).lower()
    if "nccl" in backend and "gloo" not in backend:
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


@torch.no_grad()
def synchronize_step_failure(local_failed, process_group=None, *, collective_device=None) -> bool:
    """True on every rank iff any rank of the group reports a failure."""
    failed = bool(local_failed)
    if not distributed_ready():
        return failed
    dist = _dist()
    if dist.get_world_size(process_group) < 2:
        return failed
    flag = torch.tensor(int(failed), dtype=torch.int32,
                        device=control_device(process_group, collective_device=collective_device))
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=process_group)
    return bool(flag.item())


@torch.no_grad()
def synchronize_step_control_range(
    local_minimum: Sequence[float], local_maximum: Sequence[float], process_group=None, *,
    collective_device=None,
) -> Tuple[Tuple[float, ...], Tuple[float, ...]]:
    """Element-wise (min over ranks, max over ranks) of two equally long tuples."""
    lo = tuple(float(x) for x in local_minimum)
    hi = tuple(float(x) for x in local_maximum)
    if len(lo) != len(hi):
        raise ValueError("step-control bounds must have equal lengths")
    if not distributed_ready():
        return lo, hi
    dist = _dist()
    if dist.get_world_size(process_group) < 2:
        return lo, hi
    packed = torch.tensor(lo + tuple(-x for x in hi), dtype=torch.float64,
                          device=control_device(process_group, collective_device=collective_device))
    dist.all_reduce(packed, op=dist.ReduceOp.MIN, group=process_group)
    vals = packed.cpu().tolist()
    n = len(lo)
    return tuple(vals[:n]), tuple(-x for x in vals[n:])


def raise_if_any_rank_failed(local_exc: Optional[BaseException], process_groups: Iterable = (None,),
                             what: str = "optimizer step") -> None:
    """Fan a local exception out: every rank of every group raises before mutating.

    The failing rank re-raises its own exception; the others raise a
    ``RuntimeError`` naming the peer failure.
    """
    any_failed = local_exc is not None
    for pg in process_groups:
        any_failed = synchronize_step_failure(any_failed, pg) or any_failed
    if local_exc is not None:
        raise local_exc
    if any_failed:
        raise RuntimeError(
            "gefen_x_b200: another rank failed during the {}; this rank aborts before "
            "mutating any state".format(what))
