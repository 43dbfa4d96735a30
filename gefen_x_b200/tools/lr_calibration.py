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

    def summary(self) -> str:
        lines = ["relative lr calibration", "  reference: {}".format(self.reference_label)]
        for s in self.stats:
            lines.append("  {:<28} lr={:.3e} unit_rms={:.4e} multiplier={:.4f} suggested_lr={:.3e}".format(
                s.label, s.lr, s.unit_update_rms, self.multipliers[s.label], self.suggested_lrs[s.label]))
        return "\n".join(lines)


def _pick_reference(stats: List[GroupUpdateStats], reference: str) -> GroupUpdateStats:
    if reference == "median":
        ordered = sorted(stats, key=lambda s: s.unit_update_rms)
        return ordered[len(ordered) // 2]
    if reference in ("gefen", "muon"):              # first usable group of that kind (reference tool's names)
        want = "muon" if reference == "muon" else "adam"
        for s in stats:
            if ":{}".format(want) in s.label and math.isfinite(s.update_rms) and s.update_rms > 0:
                return s
        raise ValueError("no usable {} group found for reference".format(reference))
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
    """One parameter's applied update RMS against a shadow AdamW fed the same gradients (fields of
    the reference's record, ``tools/lr_calibration.py:486-499``)."""
    name: str
    is_muon: bool
    rows: int
    cols: int
    gefen_rms: float
    adamw_rms: float
    ratio: float                 # LR multiplier that makes this parameter's update RMS match AdamW's
    active_ratio: float          # the adjust_lr_fn ratio in effect (Muon), else 1.0
    sqrt_max: Optional[float]    # sqrt(max(rows, cols)) for Muon, else None

    @property
    def shape(self) -> tuple:
        return (self.rows, self.cols)


def _analytic_ratios(group: dict, p=None) -> Dict[str, Optional[float]]:
    """The ``adjust_lr_fn`` ratios of a Muon group for ``p`` (or the group's largest matrix)."""
    none = {"original": None, "match_rms_adamw": None, "active": 1.0}
    if not _is_muon_group(group):
        return none
    mats = [q for q in ([p] if p is not None else group["params"]) if q.ndim >= 2]
    if not mats:
        return none
    big = max(mats, key=lambda q: q.shape[0] * q.shape[1])
    rows, cols = big.shape[:2]
    original = math.sqrt(max(1, rows / cols))
    match = 0.2 * math.sqrt(max(rows, cols))
    return {"original": original, "match_rms_adamw": match,
            "active": match if group.get("adjust_lr_fn") == "match_rms_adamw" else original}


def _median(xs: Sequence[float]) -> float:
    ys = sorted(x for x in xs if math.isfinite(x))
    if not ys:
        return float("nan")
    n = len(ys)
    return ys[n // 2] if n % 2 else 0.5 * (ys[n // 2 - 1] + ys[n // 2])


def calibrate_vs_adamw(optimizer, closure, *, betas=(0.9, 0.999), eps: float = 1e-8, num_steps: int = 40,
                       warmup: int = 5) -> List[ParamVsAdamw]:
    """Per parameter: the optimizer's applied update RMS against the update a shadow AdamW would
    have applied at the same lr on the same gradients (the shadow is never applied).  Weight decay
    is off during the probe; parameters and optimizer state are restored afterwards
    (reference ``tools/lr_calibration.py:502-625``)."""
    beta1, beta2 = betas
    snap = _snapshot(optimizer)
    metas = []
    for g in optimizer.param_groups:
        names = g.get("param_names") or []
        lr = g["lr"]
        lr = float(lr.item() if torch.is_tensor(lr) else lr)
        base = g.get("name", "?")
        for i, p in enumerate(g["params"]):
            name = names[i] if i < len(names) and names[i] else (base if len(g["params"]) == 1
                                                                 else "{}.{}".format(base, i))
            metas.append((p, g, lr, str(name)))
    m, v, ours, ref = {}, {}, {}, {}
    try:
        for g in optimizer.param_groups:
            if "weight_decay" in g:
                g["weight_decay"] = 0.0
        for step in range(num_steps):
            optimizer.zero_grad(set_to_none=True)
            loss = closure()
            if loss is None or not bool(torch.isfinite(torch.as_tensor(loss)).all()):
                raise RuntimeError("non-finite loss at step {}: {}".format(step, loss))
            before = {}
            for p, g, lr, _ in metas:
                if p.grad is None:
                    continue
                grad = _local(p.grad).detach().float()
                k = id(p)
                if k not in m:
                    m[k], v[k] = torch.zeros_like(grad), torch.zeros_like(grad)
                unit = _shadow_adamw_unit_update(m[k], v[k], grad, step + 1, beta1, beta2, eps)
                before[k] = _local(p).detach().clone()
                if step >= warmup:
                    ref.setdefault(k, []).append(_rms(unit * lr))
            optimizer.step()
            if step < warmup:
                continue
            for p, g, lr, _ in metas:
                k = id(p)
                if k in before:
                    ours.setdefault(k, []).append(_rms((_local(p).detach() - before[k]).float()))
        out = []
        for p, g, lr, name in metas:
            k = id(p)
            if k not in ours or k not in ref:
                continue
            a, b = _median(ours[k]), _median(ref[k])
            ar = _analytic_ratios(g, p)
            out.append(ParamVsAdamw(name=name, is_muon=_is_muon_group(g),
                                    rows=p.shape[0] if p.ndim >= 1 else 1, cols=p.shape[1] if p.ndim >= 2 else 1,
                                    gefen_rms=a, adamw_rms=b, ratio=(b / a) if a > 0 else float("nan"),
                                    active_ratio=ar["active"],
                                    sqrt_max=(ar["match_rms_adamw"] / 0.2) if ar["match_rms_adamw"] else None))
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

    def summary(self) -> str:
        return "lr range test: suggested lr {:.3e}, lowest loss at {:.3e}, {}".format(
            self.suggested_lr, self.min_loss_lr,
            "no divergence" if self.diverged_at is None else "diverged at {:.3e}".format(self.diverged_at))


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
