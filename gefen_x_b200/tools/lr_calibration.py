"""Non-destructive learning-rate probes for the Gefen optimizers.

Every probe snapshots parameters and optimizer state, runs a short dry run and
restores both, so it can be pointed at a live training setup.

* :func:`measure_update_rms` – per-group RMS of the applied update ``|dp| / lr``;
* :func:`calibrate_relative` – per-group lr multipliers that equalise the update RMS
  to a reference group;
* :func:`calibrate_vs_adamw` – per-parameter ratio between the optimizer's update and
  the update a shadow AdamW would have made on the same gradients;
* :func:`lr_range_test` – exponential lr ramp with a smoothed-loss suggestion.

Public names and result fields follow the reference (``src/gefen/tools/lr_calibration.py``:
``measure_update_rms`` ``:214``, ``calibrate_relative`` ``:388``, ``calibrate_vs_adamw``
``:502``, ``lr_range_test`` ``:652``).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

import torch


def _local(t: torch.Tensor) -> torch.Tensor:
    return t.to_local() if hasattr(t, "to_local") else t


def _rms(t: torch.Tensor) -> float:
    t = _local(t)
    if t.numel() == 0:
        return 0.0
    return float(t.detach().float().square().mean().sqrt().item())


def _is_muon_group(group: dict) -> bool:
    return "ns_steps" in group or "momentum" in group and "beta2" not in group


def _group_label(idx: int, group: dict) -> str:
    name = group.get("name")
    kind = "muon" if _is_muon_group(group) else "adam"
    return "{}:{}:{}".format(idx, kind, name) if name else "{}:{}".format(idx, kind)


def _snapshot(optimizer):
    params = [p for g in optimizer.param_groups for p in g["params"]]
    return {
        "params": [_local(p).detach().clone() for p in params],
        "state": copy.deepcopy(optimizer.local_state_dict() if hasattr(optimizer, "local_state_dict")
                               else optimizer.state_dict()),
        "hypers": [{k: v for k, v in g.items() if k != "params"} for g in optimizer.param_groups],
    }


def _restore(optimizer, snap) -> None:
    params = [p for g in optimizer.param_groups for p in g["params"]]
    with torch.no_grad():
        for p, saved in zip(params, snap["params"]):
            _local(p).copy_(saved)
    optimizer.load_state_dict(snap["state"])
    for g, h in zip(optimizer.param_groups, snap["hypers"]):
        for k in ("lr", "weight_decay"):
            if k in h:
                g[k] = h[k]


@dataclass
class GroupUpdateStats:
    index: int
    label: str
    lr: float
    num_params: int
    update_rms: float            # RMS of dp per step
    unit_update_rms: float       # update_rms / lr
    param_rms: float
    relative_update: float       # update_rms / param_rms
    per_step: List[float] = field(default_factory=list)


def measure_update_rms(optimizer, closure: Callable[[], torch.Tensor], *, num_steps: int = 20,
                       warmup: int = 3, zero_weight_decay: bool = True) -> List[GroupUpdateStats]:
    """Per-group RMS of the applied update over a dry run; state and weights are restored."""
    if num_steps <= warmup:
        raise ValueError("num_steps must exceed warmup")
    snap = _snapshot(optimizer)
    sums = [[] for _ in optimizer.param_groups]
    try:
        if zero_weight_decay:
            for g in optimizer.param_groups:
                if "weight_decay" in g:
                    g["weight_decay"] = 0.0
        for step in range(num_steps):
            optimizer.zero_grad()
            closure()
            before = [[_local(p).detach().float().clone() for p in g["params"]]
                      for g in optimizer.param_groups]
            optimizer.step()
            if step < warmup:
                continue
            for gi, g in enumerate(optimizer.param_groups):
                sq, n = 0.0, 0
                for p, b in zip(g["params"], before[gi]):
                    d = _local(p).detach().float() - b
                    sq += float(d.square().sum().item())
                    n += d.numel()
                sums[gi].append(math.sqrt(sq / max(1, n)))
        out = []
        for gi, g in enumerate(optimizer.param_groups):
            lr = float(g["lr"])
            upd = sum(sums[gi]) / max(1, len(sums[gi]))
            prm_sq = sum(float(_local(p).detach().float().square().sum().item()) for p in g["params"])
            n = sum(_local(p).numel() for p in g["params"])
            prm = math.sqrt(prm_sq / max(1, n))
            out.append(GroupUpdateStats(gi, _group_label(gi, g), lr, len(g["params"]), upd,
                                        upd / lr if lr > 0 else float("nan"), prm,
                                        upd / prm if prm > 0 else float("nan"), list(sums[gi])))
        return out
    finally:
        _restore(optimizer, snap)


@dataclass
class RelativeCalibration:
    reference_label: str
    target_unit_rms: float
    multipliers: Dict[str, float]
    suggested_lrs: Dict[str, float]
    stats: List[GroupUpdateStats]


def _pick_reference(stats: List[GroupUpdateStats], reference: str) -> GroupUpdateStats:
    if reference == "median":
        ordered = sorted(stats, key=lambda s: s.unit_update_rms)
        return ordered[len(ordered) // 2]
    for s in stats:
        if s.label == reference or str(s.index) == str(reference) or reference in s.label:
            return s
    raise ValueError("no group matches reference {!r}".format(reference))


def calibrate_relative(optimizer, closure, *, reference: str = "median", num_steps: int = 20,
                       warmup: int = 3) -> RelativeCalibration:
    """lr multipliers per group that bring every group's unit update RMS to the reference's."""
    stats = measure_update_rms(optimizer, closure, num_steps=num_steps, warmup=warmup)
    ref = _pick_reference(stats, reference)
    mult, lrs = {}, {}
    for s in stats:
        m = ref.unit_update_rms / s.unit_update_rms if s.unit_update_rms > 0 else 1.0
        mult[s.label] = m
        lrs[s.label] = s.lr * m
    return RelativeCalibration(ref.label, ref.unit_update_rms, mult, lrs, stats)


def _shadow_adamw_unit_update(m, v, grad, t, beta1, beta2, eps):
    m.mul_(beta1).add_(grad, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(grad, grad, value=1 - beta2)
    mhat = m / (1 - beta1 ** t)
    vhat = v / (1 - beta2 ** t)
    return mhat / (vhat.sqrt() + eps)


@dataclass
class ParamVsAdamw:
    name: str
    shape: tuple
    optimizer_unit_rms: float
    adamw_unit_rms: float
    ratio: float


def calibrate_vs_adamw(optimizer, closure, *, num_steps: int = 20, warmup: int = 3, beta1: float = 0.9,
                       beta2: float = 0.999, eps: float = 1e-8) -> List[ParamVsAdamw]:
    """Unit update RMS of every parameter against a shadow AdamW fed the same gradients."""
    snap = _snapshot(optimizer)
    params = [(g, p) for g in optimizer.param_groups for p in g["params"]]
    shadow = [(torch.zeros_like(_local(p), dtype=torch.float32), torch.zeros_like(_local(p), dtype=torch.float32))
              for _, p in params]
    ours = [[] for _ in params]
    ref = [[] for _ in params]
    names = []
    for g in optimizer.param_groups:
        gn = g.get("param_names") or [None] * len(g["params"])
        names.extend(gn)
    try:
        for g in optimizer.param_groups:
            if "weight_decay" in g:
                g["weight_decay"] = 0.0
        for step in range(1, num_steps + 1):
            optimizer.zero_grad()
            closure()
            before = [_local(p).detach().float().clone() for _, p in params]
            grads = [None if p.grad is None else _local(p.grad).detach().float().clone() for _, p in params]
            optimizer.step()
            for i, ((g, p), b, gr) in enumerate(zip(params, before, grads)):
                if gr is None:
                    continue
                unit = _shadow_adamw_unit_update(shadow[i][0], shadow[i][1], gr, step, beta1, beta2, eps)
                if step > warmup:
                    lr = float(g["lr"])
                    ours[i].append(_rms(_local(p).detach().float() - b) / lr if lr > 0 else float("nan"))
                    ref[i].append(_rms(unit))
        out = []
        for i, (g, p) in enumerate(params):
            if not ours[i]:
                continue
            a = sum(ours[i]) / len(ours[i])
            b = sum(ref[i]) / len(ref[i])
            out.append(ParamVsAdamw(str(names[i]) if i < len(names) and names[i] else "param_{}".format(i),
                                    tuple(p.shape), a, b, a / b if b > 0 else float("nan")))
        return out
    finally:
        _restore(optimizer, snap)


@dataclass
class LRRangeResult:
    lrs: List[float]
    losses: List[float]
    smoothed: List[float]
    suggested_lr: float
    min_loss_lr: float
    diverged_at: Optional[float]


def _suggest_from_curve(lrs: Sequence[float], smoothed: Sequence[float]) -> float:
    """lr at the steepest descent of the smoothed loss in log-lr, backed off from the minimum."""
    if len(lrs) < 3:
        return lrs[0]
    best_i, best_slope = 1, 0.0
    i_min = min(range(len(smoothed)), key=lambda i: smoothed[i])
    for i in range(1, max(2, i_min)):
        slope = (smoothed[i] - smoothed[i - 1]) / (math.log(lrs[i]) - math.log(lrs[i - 1]))
        if slope < best_slope:
            best_slope, best_i = slope, i
    return min(lrs[best_i], lrs[i_min] / 3.0) if best_slope < 0 else lrs[i_min] / 10.0


def lr_range_test(optimizer, closure, *, start_lr: float = 1e-6, end_lr: float = 1e-1, num_iter: int = 100,
                  smooth_beta: float = 0.9, diverge_factor: float = 5.0,
                  restore: bool = True) -> LRRangeResult:
    """Exponential lr ramp over ``num_iter`` steps; stops when the smoothed loss diverges."""
    if not (0 < start_lr < end_lr):
        raise ValueError("need 0 < start_lr < end_lr")
    snap = _snapshot(optimizer) if restore else None
    base = [float(g["lr"]) for g in optimizer.param_groups]
    ref = base[0] if base[0] > 0 else 1.0
    lrs, losses, smoothed = [], [], []
    avg, best, diverged = 0.0, float("inf"), None
    try:
        for it in range(num_iter):
            lr = start_lr * (end_lr / start_lr) ** (it / max(1, num_iter - 1))
            for g, b in zip(optimizer.param_groups, base):
                g["lr"] = lr * (b / ref)
            optimizer.zero_grad()
            loss = float(closure())
            optimizer.step()
            avg = smooth_beta * avg + (1 - smooth_beta) * loss
            sm = avg / (1 - smooth_beta ** (it + 1))
            lrs.append(lr)
            losses.append(loss)
            smoothed.append(sm)
            if not math.isfinite(loss) or sm > diverge_factor * best:
                diverged = lr
                break
            best = min(best, sm)
        i_min = min(range(len(smoothed)), key=lambda i: smoothed[i])
        return LRRangeResult(lrs, losses, smoothed, _suggest_from_curve(lrs, smoothed), lrs[i_min], diverged)
    finally:
        if snap is not None:
            _restore(optimizer, snap)
        else:
            for g, b in zip(optimizer.param_groups, base):
                g["lr"] = b
