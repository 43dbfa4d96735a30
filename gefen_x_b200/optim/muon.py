"""``GefenMuon``: Muon (orthogonalised momentum) with Gefen's quantised momentum state.

For every 2-D hidden matrix: advance the codebook-quantised momentum EMA
(``beta = momentum``), take the dense momentum (plus the Nesterov look-ahead),
orthogonalise it with Newton–Schulz, optionally apply NorMuon row normalisation
and the cautious mask, and apply it with the shape-dependent lr ratio.  There is
no second moment, so the state is ~1 byte per parameter.

Sharded parameters (DTensor ``Shard(0)``):

* ``sharded_mode="exact"`` – every rank gathers the full gradient, runs the full
  Newton–Schulz redundantly and keeps its rows of the result;
* ``"distributed"`` – matrix ``i`` is owned by rank ``i mod world``: owners
  compute, the bf16 update is broadcast, every rank keeps its rows;
* ``"approx"`` – Newton–Schulz on the local row shard, no collectives.

Parity: reference ``src/gefen/gefen_muon.py`` (constructor ``:546-573``, momentum
``:1064-1190``, NorMuon ``:1192-1230``, apply ``:1234-1300``, modes ``:1821-2050``,
step ``:2944-3030``).  The Newton–Schulz products run on the tcgen05 GEMM
(``optim/newton_schulz.py``) instead of cuBLAS.
"""
from __future__ import annotations

import math
import warnings
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..parallel.control import raise_if_any_rank_failed, synchronize_step_failure
from ..quant import codebook as _cbk
from . import functional as F_
from . import newton_schulz as NS
from .newton_schulz import (DEFAULT_A, DEFAULT_B, DEFAULT_C, DEFAULT_NS_STEPS, FP8_MIN_DIM,  # noqa: F401
                            NS_SCHEDULE_3STEP, NS_SCHEDULE_4STEP, NS_SCHEDULES)
from .gefen import Gefen, _local, _assert_gradients_structurally_valid, _amp_prepare_optimizer_step

EPS = NS.EPS
BATCHED_NS_MIN_BATCH = 8
BATCHED_NS_MAX_MIN_DIM = 512
BATCHED_NS_MAX_NUMEL = 1 << 20
BATCHED_NS_DEFAULT_WORKSPACE_BYTES = 256 << 20
_SHARDED_MODES = ("exact", "distributed", "approx")


def stable_distributed_owner(stable_index: int, world: int) -> int:
    """Owner rank of the ``stable_index``-th Muon matrix (``index mod world``)."""
    if world <= 0:
        raise ValueError("world must be positive, got {}".format(world))
    if stable_index < 0:
        raise ValueError("stable_index must be non-negative, got {}".format(stable_index))
    return stable_index % world


def adjust_lr_ratio(adjust_lr_fn: Optional[str], shape) -> float:
    rows, cols = shape[:2]
    if adjust_lr_fn is None or adjust_lr_fn == "original":
        return math.sqrt(max(1, rows / cols))
    if adjust_lr_fn == "match_rms_adamw":
        return 0.2 * math.sqrt(max(rows, cols))
    return 1.0


def cautious_mask_(update: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
    """Zero the coordinates whose sign disagrees with the gradient; rescale by 1/mean(mask)."""
    mask = (update * grad) > 0
    agree = mask.sum()
    scale = mask.numel() / agree.clamp(min=1).to(torch.float32)
    return update.mul_(mask.to(update.dtype)).mul_(scale.to(update.dtype))


def batched_ns_shape_eligible(rows: int, cols: int) -> bool:
    return rows > 0 and cols > 0 and min(rows, cols) <= BATCHED_NS_MAX_MIN_DIM \
        and rows * cols <= BATCHED_NS_MAX_NUMEL


class GefenMuon(Gefen):
    """Muon on 2-D matrices with codebook-quantised momentum (see module docstring)."""

    def __init__(self, params, lr=1e-3, weight_decay: float = 0.1, momentum: float = 0.95,
                 nesterov: bool = True, ns_coefficients=(NS.DEFAULT_A, NS.DEFAULT_B, NS.DEFAULT_C),
                 eps: float = EPS, ns_steps: int = NS.DEFAULT_NS_STEPS, ns_schedule: Optional[str] = None,
                 adjust_lr_fn: Optional[str] = None, *, fused: bool = True,
                 sharded_mode: str = "exact", fp8_ns: bool = False, fp8_ns_compile: bool = True,
                 batched_ns: bool = False,
                 batched_ns_workspace_bytes: int = BATCHED_NS_DEFAULT_WORKSPACE_BYTES,
                 stochastic_round: bool = False, deterministic: bool = False, normuon: bool = False,
                 normuon_beta2: float = 0.95, normuon_eps: float = 1e-8, cautious: bool = False,
                 capturable: bool = False, verbose: bool = False):
        if sharded_mode not in _SHARDED_MODES:
            raise ValueError("sharded_mode must be one of {}, got {!r}".format(_SHARDED_MODES, sharded_mode))
        if not 0.0 <= momentum < 1.0:
            raise ValueError("Invalid momentum value: {}".format(momentum))
        if adjust_lr_fn not in (None, "original", "match_rms_adamw"):
            raise ValueError("Unknown adjust_lr_fn {!r}".format(adjust_lr_fn))
        if not math.isfinite(eps) or eps <= 0.0:
            raise ValueError("eps must be finite and > 0 but is: {}".format(eps))
        if not 0.0 <= normuon_beta2 < 1.0:
            raise ValueError("normuon_beta2 must be in [0, 1) but is: {}".format(normuon_beta2))
        if not math.isfinite(normuon_eps) or normuon_eps <= 0.0:
            raise ValueError("normuon_eps must be finite and > 0 but is: {}".format(normuon_eps))
        # A schedule (a name or an explicit list of (a, b, c)) overrides ns_coefficients / ns_steps
        # and is stored resolved, so a parameter group carries the reference's keys only
        # (reference src/gefen/gefen_muon.py:605-626, group keys :716-735).
        if ns_schedule is not None:
            if isinstance(ns_schedule, str):
                if ns_schedule not in NS.NS_SCHEDULES:
                    raise ValueError("Unknown ns_schedule {!r}; choose from {}".format(
                        ns_schedule, sorted(NS.NS_SCHEDULES)))
                resolved = NS.NS_SCHEDULES[ns_schedule]
            else:
                resolved = ns_schedule
            if resolved is not None:           # "standard" defers to ns_coefficients / ns_steps
                sched = NS.normalize_schedule(resolved, ns_steps)
                ns_coefficients, ns_steps = [tuple(c) for c in sched], len(sched)
        NS.normalize_schedule(ns_coefficients, ns_steps)                  # validates
        if fp8_ns and torch.cuda.is_available() and not NS.fp8_supported():
            warnings.warn("fp8_ns=True but this GPU has no fp8 GEMM (compute capability below 8.9); "
                          "the Newton-Schulz products run in bf16.", RuntimeWarning, stacklevel=2)
        coeffs = (tuple(ns_coefficients) if isinstance(ns_coefficients[0], (int, float))
                  else [tuple(c) for c in ns_coefficients])
        self._muon_defaults = dict(momentum=momentum, nesterov=nesterov, ns_coefficients=coeffs,
                                   ns_steps=ns_steps, adjust_lr_fn=adjust_lr_fn, sharded_mode=sharded_mode,
                                   fp8_ns=fp8_ns, fp8_ns_compile=fp8_ns_compile, batched_ns=batched_ns,
                                   batched_ns_workspace_bytes=int(batched_ns_workspace_bytes),
                                   normuon=normuon, normuon_beta2=normuon_beta2,
                                   normuon_eps=normuon_eps, cautious=cautious)
        self.sharded_mode = sharded_mode
        self.fp8_ns, self.fp8_ns_compile = fp8_ns, fp8_ns_compile
        self.batched_ns = self._batched_ns = batched_ns
        self.batched_ns_workspace_bytes = self._batched_ns_workspace_bytes = int(batched_ns_workspace_bytes)
        # the group's `eps` is the Newton-Schulz normalisation epsilon and beta2 is unused (0), as in
        # the reference's groups
        super().__init__(params, lr=lr, betas=(momentum, 0.0), eps=eps, weight_decay=weight_decay,
                         fused=fused, factored_v_2d=False, stochastic_round=stochastic_round,
                         deterministic=deterministic, capturable=capturable, verbose=verbose)

    # ------------------------------------------------------------------
    def add_param_group(self, param_group):
        """Register a group with every Muon option resolved and validated before anything is
        mutated: group values override the constructor's, a named or explicit ``ns_schedule`` is
        stored as ``ns_coefficients`` / ``ns_steps``, ``beta1`` mirrors ``momentum`` and ``beta2``
        is 0 (reference ``gefen_muon.py:790-880``)."""
        if not isinstance(param_group, dict):
            raise TypeError("param_group must be a dict")
        merged = dict(param_group)
        for k, v in getattr(self, "_muon_defaults", {}).items():
            merged.setdefault(k, v)
        if merged["sharded_mode"] not in _SHARDED_MODES:
            raise ValueError("sharded_mode must be one of {}, got {!r}".format(_SHARDED_MODES, merged["sharded_mode"]))
        if merged["adjust_lr_fn"] not in (None, "original", "match_rms_adamw"):
            raise ValueError("Unknown adjust_lr_fn {!r}".format(merged["adjust_lr_fn"]))
        if not 0.0 <= merged["momentum"] < 1.0:
            raise ValueError("Invalid momentum value: {}".format(merged["momentum"]))
        if not 0.0 <= merged["normuon_beta2"] < 1.0:
            raise ValueError("normuon_beta2 must be in [0, 1) but is: {}".format(merged["normuon_beta2"]))
        if not math.isfinite(merged["normuon_eps"]) or merged["normuon_eps"] <= 0.0:
            raise ValueError("normuon_eps must be finite and > 0 but is: {}".format(merged["normuon_eps"]))
        schedule = merged.pop("ns_schedule", None)
        if schedule is not None:
            if isinstance(schedule, str):
                if schedule not in NS.NS_SCHEDULES:
                    raise ValueError("Unknown ns_schedule {!r}; choose from {}".format(schedule, sorted(NS.NS_SCHEDULES)))
                schedule = NS.NS_SCHEDULES[schedule]
            if schedule is not None:
                resolved = NS.normalize_schedule(schedule, merged["ns_steps"])
                merged["ns_coefficients"], merged["ns_steps"] = [tuple(c) for c in resolved], len(resolved)
        NS.normalize_schedule(merged["ns_coefficients"], merged["ns_steps"])
        merged.pop("betas", None)
        merged["beta1"], merged["beta2"] = merged["momentum"], 0.0
        params = merged.get("params")
        if params is not None:
            for _, p in self._iter_params_with_names(params):
                if p.ndim != 2:
                    raise ValueError(
                        "GefenMuon only supports 2D matrices; got a {}-D parameter of shape {}. "
                        "Route embeddings, heads, norms and biases to a backup optimizer "
                        "(GefenMuonHybrid does this).".format(p.ndim, tuple(p.shape)))
        super().add_param_group(merged)

    def _is_factored(self, p) -> bool:
        return False

    def _state_shape_for(self, p):
        # exact / distributed modes keep the momentum of the FULL matrix of a sharded parameter
        if hasattr(p, "to_local") and self.sharded_mode != "approx":
            return tuple(p.shape)
        return tuple(_local(p).shape)

    # ------------------------------------------------------------------
    # momentum
    # ------------------------------------------------------------------
    def _muon_state(self, name: str, p: torch.Tensor, grad: torch.Tensor) -> Dict[str, Any]:
        """State sized to ``grad`` (the full matrix in exact/distributed mode, the shard in approx)."""
        state = self.state[p]
        numel = grad.numel()
        if "step" not in state:
            if "automatic_period" in state:
                period = state["automatic_period"]
            elif numel == 1:
                period = 1
            else:
                period = self._resolve_automatic_period(name, p, grad)
            if numel % period:
                raise ValueError(
                    "Automatic partition period {} does not divide parameter {} with numel {}".format(
                        period, name, numel))
            state["automatic_period"] = period
            state["step"] = self._new_step_counter(grad.device)
            state["m_codebook"] = torch.zeros(numel // period, period, dtype=torch.uint8, device=grad.device)
            state["m_magnitude"] = torch.zeros(numel // period, 1, dtype=torch.float32, device=grad.device)
        self._colocate_param_state_(state, grad.device)
        return state

    def _prepare_muon_momentum(self, group, name: str, p: torch.Tensor, grad: torch.Tensor,
                               private: bool = False) -> torch.Tensor:
        """Advance the quantised momentum with ``grad``; return the dense Newton–Schulz input.

        The dense momentum is scratch: it is written into one buffer per (shape, dtype, device) that the
        next matrix of that shape overwrites once Newton–Schulz has consumed it, so the launch plan of
        a matrix keeps the same addresses from step to step (no rebuild, and nothing to allocate or
        upload while a CUDA graph is being captured).  ``private=True`` (batched Newton–Schulz, which
        holds many of them at once) returns a tensor of its own."""
        state = self._muon_state(name, p, grad)
        state["step"] += 1
        beta = group["momentum"]
        cb = self._gefen_codebook_on(grad.device)
        if cb is None:
            raise ValueError("Expected Gefen codebook to be initialized before the Muon momentum update.")
        if self._fused_for(grad) and grad.dtype in (torch.bfloat16, torch.float16, torch.float32):
            # one multi-pass-free kernel sequence: block maxima, then requantise + dense emit
            from ..ops import update as _u

            dev = grad.device
            if private:
                out = torch.empty(grad.shape, dtype=grad.dtype, device=dev)
            else:
                scratch = self.__dict__.setdefault("_emit_scratch", {})
                key = (tuple(grad.shape), grad.dtype, dev)
                out = scratch.get(key)
                if out is None:
                    out = scratch[key] = torch.empty(grad.shape, dtype=grad.dtype, device=dev)
            _u.momentum_emit(grad.contiguous(), state, out, cb, self._gefen_thresholds_on(dev),
                             self._gefen_codebook_lut_on(dev), beta=beta, nesterov=bool(group["nesterov"]),
                             gscale=self._grad_scale_tensor(dev))
            return out if out.dtype == torch.bfloat16 else out.to(torch.bfloat16)
        gv = F_.partition_view(grad.reshape(-1), state["automatic_period"])
        q = F_.momentum_requantize_(cb, state["m_codebook"], state["m_magnitude"], gv, beta,
                                    self._pending_grad_scale)
        m = q.view(grad.shape)
        if group["nesterov"]:
            g = grad.float()
            if self._pending_grad_scale is not None:
                g = g * self._pending_grad_scale
            m = m * beta + g * (1.0 - beta)
        return m.to(torch.bfloat16 if grad.dtype != torch.float64 else grad.dtype)

    def _iter_gefen_grad_periods(self, reuse_existing_periods: bool = False):
        """Codebook learning sees what the momentum will see: full matrices unless ``approx``."""
        for group in self.param_groups:
            for name, p in self._iter_group_params_with_names(group):
                if p.grad is None:
                    continue
                grad = self._momentum_grad(p)
                flat = grad.reshape(-1)
                if flat.numel() == 0:
                    continue
                state = self.state[p]
                if reuse_existing_periods:
                    if "automatic_period" not in state:
                        raise ValueError(
                            "Expected automatic_period to exist for {} before refreshing Gefen "
                            "codebook at optimizer step {}".format(name, self._gefen_global_step))
                    period = state["automatic_period"]
                elif flat.numel() == 1:
                    period = 1
                else:
                    period = self._resolve_automatic_period(name, p, grad)
                state["automatic_period"] = period
                yield name, flat, period, grad

    def _momentum_grad(self, p: torch.Tensor) -> torch.Tensor:
        g = p.grad
        if hasattr(g, "full_tensor") and self.sharded_mode != "approx":
            return g.full_tensor().detach()
        return _local(g).detach()

    # ------------------------------------------------------------------
    # update pieces
    # ------------------------------------------------------------------
    def _normuon_normalize(self, state, ortho: torch.Tensor, beta2: float, eps: float) -> torch.Tensor:
        v = state.get("normuon_v")
        if v is None or v.shape[0] != ortho.shape[0]:
            v = torch.zeros(ortho.shape[0], 1, dtype=torch.float32, device=ortho.device)
            state["normuon_v"] = v
            state["normuon_step"] = self._new_step_counter(ortho.device)
        row_norm = torch.linalg.vector_norm(ortho, dim=1, keepdim=True, dtype=torch.float32)
        row_sq = row_norm.square()
        v.mul_(beta2).add_(row_sq, alpha=(1 - beta2) / ortho.shape[1])
        state["normuon_step"] += 1
        bc = 1 - beta2 ** state["normuon_step"]
        denom = (v / bc).sqrt_().add_(eps)
        frob = row_sq.sum().sqrt_() / torch.linalg.vector_norm(row_norm / denom).clamp(
            min=torch.finfo(torch.float32).tiny)
        return ortho.mul_((frob / denom).to(ortho.dtype))

    def _orthogonalize(self, group, m: torch.Tensor) -> torch.Tensor:
        sched = NS.resolve_schedule(group.get("ns_schedule"), group["ns_coefficients"], group["ns_steps"])
        return NS.zeropower_via_newtonschulz(m, sched, len(sched), group["eps"],
                                             use_fp8=group.get("fp8_ns", self.fp8_ns))

    def _compute_muon_update(self, group, name, p, grad) -> torch.Tensor:
        m = self._prepare_muon_momentum(group, name, p, grad)
        update = self._orthogonalize(group, m)
        if not update.is_contiguous():
            update = update.contiguous()
        state = self.state[p]
        if (group["normuon"] or group["cautious"]) and self._epilogue_kernels_apply(update, grad):
            return self._muon_epilogue_kernels(state, group, update, grad)
        if group["normuon"]:
            update = self._normuon_normalize(state, update, group["normuon_beta2"], group["normuon_eps"])
        if group["cautious"]:
            update = cautious_mask_(update, grad.to(update.dtype))
        return update

    @staticmethod
    def _epilogue_kernels_apply(update: torch.Tensor, grad: torch.Tensor) -> bool:
        """CUDA matrices in a kernel dtype: NorMuon and the cautious mask run as three launches over the
        update (row statistics, row factors, finish) instead of the chain of torch ops."""
        if not (update.is_cuda and update.dim() == 2 and update.is_contiguous()
                and update.dtype in (torch.float32, torch.bfloat16, torch.float16)
                and tuple(grad.shape) == tuple(update.shape) and update.numel() > 0):
            return False
        from ..ops import _ext

        return _ext.available()

    def _muon_epilogue_kernels(self, state, group, update: torch.Tensor, grad: torch.Tensor) -> torch.Tensor:
        """Same values as ``_normuon_normalize`` followed by ``cautious_mask_`` (every product rounded
        where those round it), computed by ``csrc/muon_ops.cu``; the update is rewritten in place."""
        from ..ops._ext import ops

        dev = update.device
        v = None
        bc = 1.0
        if group["normuon"]:
            beta2 = group["normuon_beta2"]
            v = state.get("normuon_v")
            if v is None or v.shape[0] != update.shape[0]:
                v = torch.zeros(update.shape[0], 1, dtype=torch.float32, device=dev)
                state["normuon_v"] = v
                state["normuon_step"] = self._new_step_counter(dev)
            state["normuon_step"] += 1
            bc = 1 - beta2 ** state["normuon_step"]
        if torch.is_tensor(bc) and bc.is_cuda:        # device-resident step counter (capturable)
            scal = torch.stack([bc.to(device=dev, dtype=torch.float32).reshape(()),
                                torch.zeros((), dtype=torch.float32, device=dev),
                                torch.ones((), dtype=torch.float32, device=dev)])
        else:
            scal = torch.tensor([float(bc), 0.0, 1.0], dtype=torch.float32).to(dev, non_blocking=True)
        g = grad.to(update.dtype).contiguous() if group["cautious"] else None
        ops().muon_epilogue(update, g, v, None, scal, bool(group["normuon"]), bool(group["cautious"]),
                            float(group["normuon_beta2"]), float(group["normuon_eps"]))
        return update

    @staticmethod
    def _shard_like(full_update: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
        """Rows of ``full_update`` that this rank's ``Shard(0)`` local tensor holds."""
        local = p.to_local()
        mesh = p.device_mesh
        world = mesh.size(0)
        rank = mesh.get_local_rank(0)
        rows = full_update.shape[0]
        per = (rows + world - 1) // world
        r0 = min(rows, rank * per)
        return full_update[r0:r0 + local.shape[0]]

    def _apply_muon_update(self, group, p: torch.Tensor, update: torch.Tensor, sharded: bool,
                           approx: bool) -> None:
        """``p <- p * (1 - lr * wd) - lr * ratio * update`` on this rank's rows.

        A tensor learning rate is never read back to the host: under ``capturable=True`` (and always
        while a CUDA graph is being captured) the scalars stay on the device, so a captured step
        follows in-place changes of the lr tensor on replay (reference ``gefen_muon.py:1243-1300``)."""
        ratio = adjust_lr_ratio(group["adjust_lr_fn"], p.shape)
        target = p.to_local() if sharded else p
        lr = group["lr"]
        on_device = torch.is_tensor(lr) and (self.capturable or (
            lr.is_cuda and torch.cuda.is_current_stream_capturing()))
        if on_device:
            lr_t = lr.to(device=target.device, dtype=torch.float32).reshape(())
            if group["weight_decay"] > 0.0:
                target.mul_((1.0 - lr_t * group["weight_decay"]).to(target.dtype))
            if target.numel() == 0:
                return
            local_update = update if (approx or not sharded) else self._shard_like(update, p)
            target.sub_((local_update.float() * (lr_t * ratio)).to(target.dtype))
            return
        lr = self._lr_scalar(group)
        if group["weight_decay"] > 0.0:
            target.mul_(1 - lr * group["weight_decay"])
        if target.numel() == 0:
            return
        local_update = update if (approx or not sharded) else self._shard_like(update, p)
        target.add_(local_update.to(target.dtype), alpha=-(lr * ratio))

    # ------------------------------------------------------------------
    # the step
    # ------------------------------------------------------------------
    def _process_group_of(self, p):
        mesh = getattr(p, "device_mesh", None)
        if mesh is None:
            return None, 1, 0
        if mesh.ndim != 1:
            return None, 0, 0           # multi-dim mesh: fall back to exact
        return mesh.get_group(0), mesh.size(0), mesh.get_local_rank(0)

    def _assert_sharded_grad_presence_consistent(self, items) -> None:
        """Every rank must step the same sharded matrices before any collective (reference
        ``tests/test_muon_grad_presence.py``).  The agreement runs over every sharded parameter of the
        optimizer, with or without a gradient on this rank, so that a rank whose gradients are all
        missing still takes part in it (and learns, like the others, that the step is refused)."""
        import torch.distributed as dist

        with_grad = {id(p) for _g, _n, p in items}
        everyone = [q for g in self.param_groups for q in g["params"]]
        by_pg: Dict[int, Tuple[Any, List[int]]] = {}
        for idx, q in enumerate(everyone):
            pg, world, _ = self._process_group_of(q)
            if pg is None or world < 2:
                continue
            by_pg.setdefault(id(pg), (pg, []))[1].append(idx)
        for pg, idxs in by_pg.values():
            mask = torch.zeros(len(everyone) + 1, dtype=torch.int32)
            for i in idxs:
                if id(everyone[i]) in with_grad:
                    mask[i] = 1
            mask[-1] = int(mask.sum())
            from ..parallel.control import control_device

            dev = control_device(pg)
            lo = mask.to(dev).clone()
            hi = mask.to(dev).clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=pg)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=pg)
            if not torch.equal(lo.cpu(), hi.cpu()):
                raise RuntimeError(
                    "GefenMuon: ranks disagree on which sharded parameters have gradients this "
                    "step; refusing to enter the gather collectives")

    @torch.compiler.disable
    @torch.no_grad()
    def step(self, closure=None):
        self._assert_capturable_if_capturing()
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        local_exc = None
        try:
            _assert_gradients_structurally_valid(self)
            for g in self.param_groups:
                for p in g["params"]:
                    if p.ndim != 2:
                        raise ValueError(
                            "GefenMuon found a {}-D parameter (shape {}) in its param groups at step time: an "
                            "optimizer wrapper replaced param_groups[*]['params'] with flat 1-D fp32 partitions "
                            "(DeepSpeed ZeRO does this). Muon's 2-D Newton-Schulz step cannot be applied to a "
                            "flat partition. Use plain Gefen with DeepSpeed ZeRO.".format(p.ndim, tuple(p.shape)))
        except Exception as exc:           # noqa: BLE001 - fanned out below
            local_exc = exc
        pgs = []
        seen = set()
        for g in self.param_groups:
            for p in g["params"]:
                pg, world, _ = self._process_group_of(p)
                if pg is not None and world > 1 and id(pg) not in seen:
                    seen.add(id(pg))
                    pgs.append(pg)
        if pgs and not getattr(self, "_gefen_hybrid_precollective_preflight", False):
            raise_if_any_rank_failed(local_exc, pgs, "GefenMuon step")
        elif local_exc is not None:
            raise local_exc
        self._pending_grad_scale = None
        if (hasattr(self, "found_inf") or hasattr(self, "grad_scale")) and \
                not _amp_prepare_optimizer_step(self):
            return loss

        items = [(g, n, p) for g in self.param_groups
                 for n, p in self._iter_group_params_with_names(g) if p.grad is not None]
        if pgs:
            self._assert_sharded_grad_presence_consistent(items)
        try:
            self._maybe_refresh_gefen_codebook()
            regular, distributed = [], []
            stable = {p: i for i, p in enumerate(q for g in self.param_groups for q in g["params"])}
            for g, n, p in items:
                pg, world, _ = self._process_group_of(p)
                if self.sharded_mode == "distributed" and pg is not None and world > 1:
                    distributed.append((g, n, p))
                else:
                    regular.append((g, n, p))
            self._step_regular(regular)
            if distributed:
                self._step_distributed(distributed, stable)
        finally:
            self._pending_grad_scale = None
        self._advance_gefen_global_step()
        return loss

    def _step_regular(self, items) -> None:
        batches: Dict[Any, list] = {}
        for g, n, p in items:
            sharded = hasattr(p, "to_local")
            approx = sharded and self.sharded_mode == "approx"
            grad = self._momentum_grad(p)
            if grad.numel() == 0:
                continue
            if (self.batched_ns and not sharded and not g["normuon"] and not g["cautious"]
                    and batched_ns_shape_eligible(*grad.shape)):
                key = (tuple(grad.shape), grad.device, id(g))
                batches.setdefault(key, []).append((g, n, p, grad))
                continue
            update = self._compute_muon_update(g, n, p, grad)
            self._apply_muon_update(g, p, update, sharded, approx)
        for (_shape, _dev, _gid), members in batches.items():
            g = members[0][0]
            if len(members) < BATCHED_NS_MIN_BATCH:
                for g_, n, p, grad in members:
                    self._apply_muon_update(g_, p, self._compute_muon_update(g_, n, p, grad), False, False)
                continue
            moms = [self._prepare_muon_momentum(g_, n, p, grad, private=True) for g_, n, p, grad in members]
            sched = NS.resolve_schedule(g.get("ns_schedule"), g["ns_coefficients"], g["ns_steps"])
            per = max(1, self.batched_ns_workspace_bytes // max(1, 16 * moms[0].numel()))
            for s in range(0, len(moms), per):
                outs = NS.zeropower_batched(moms[s:s + per], sched, len(sched), g["eps"],
                                            use_fp8=g.get("fp8_ns", self.fp8_ns))
                for (g_, n, p, grad), upd in zip(members[s:s + per], outs):
                    self._apply_muon_update(g_, p, upd.contiguous(), False, False)

    def _step_distributed(self, items, stable) -> None:
        """Parallel-Muon in buckets of ``world`` matrices (reference ``gefen_muon.py:1821-1900``):

        1. every rank joins the all-gather of every gradient of the bucket and keeps only the
           matrices it owns (owner = stable parameter index mod world, so a matrix's momentum never
           moves when unrelated gradients come and go);
        2. the owners orthogonalise *their* matrices at the same time -- no collective in this
           phase, which is where the mode gets its parallelism;
        3. every update is broadcast from its owner (bf16) and each rank keeps its rows.
        """
        import torch.distributed as dist

        by_pg: Dict[int, Tuple[Any, list]] = {}
        for g, n, p in items:
            pg, _world, _rank = self._process_group_of(p)
            by_pg.setdefault(id(pg), (pg, []))[1].append((g, n, p))
        for pg, pg_items in by_pg.values():
            world = dist.get_world_size(pg)
            rank = dist.get_rank(pg)
            for b in range(0, len(pg_items), world):
                bucket = pg_items[b:b + world]
                owners = [stable_distributed_owner(stable[p], world) for _g, _n, p in bucket]
                owned = []
                for k, (g, n, p) in enumerate(bucket):                 # phase 1: matched gathers only
                    full_grad = p.grad.full_tensor().detach()
                    if owners[k] == rank:
                        owned.append((k, g, n, p, full_grad))
                    del full_grad
                updates: Dict[int, torch.Tensor] = {}
                for k, g, n, p, full_grad in owned:                    # phase 2: owners work concurrently
                    updates[k] = self._compute_muon_update(g, n, p, full_grad)
                owned = None
                for k, (g, n, p) in enumerate(bucket):                 # phase 3: broadcast and apply
                    if owners[k] == rank:
                        buf = updates.pop(k).contiguous()
                        if buf.dtype != torch.bfloat16:
                            buf = buf.to(torch.bfloat16)
                    else:
                        buf = torch.empty(tuple(p.shape), dtype=torch.bfloat16, device=p.to_local().device)
                    dist.broadcast(buf, src=dist.get_global_rank(pg, owners[k]), group=pg)
                    self._apply_muon_update(g, p, buf, True, False)
                    buf = None

    # ------------------------------------------------------------------
    # checkpoint: distributed mode keeps momentum on the owner only
    # ------------------------------------------------------------------
    def _rank_local_checkpoint_applies(self) -> bool:
        # exact: every rank holds the same full-matrix state; distributed: consolidated below
        return self.sharded_mode == "approx"

    def state_dict(self):
        """Native state dict; in ``distributed`` mode the owners' momentum is gathered so that every
        rank returns the same, complete (consolidated) checkpoint, loadable at any world size
        (reference ``gefen_muon.py:2110-2284``).  Collective: every rank of the mesh must call it."""
        sd = super().state_dict()
        if self.sharded_mode == "distributed":
            groups = []
            stable = 0
            pgs = {}
            for g in self.param_groups:
                entries = []
                for p in g["params"]:
                    pg, world, _r = self._process_group_of(p)
                    if pg is not None and world > 1:
                        pgs[id(pg)] = (pg, world)
                    st = self.state.get(p, {})
                    entries.append({"saved_id": stable, "name": self._param_name(p),
                                    "shape": tuple(p.shape),
                                    "owner": stable_distributed_owner(stable, max(1, world)),
                                    "state_keys": tuple(sorted(str(k) for k in st)),
                                    "initialized": any(str(k) != "name" for k in st)})
                    stable += 1
                groups.append({"world_size": max((self._process_group_of(p)[1] for p in g["params"]),
                                                 default=1), "params": entries})
            consolidated = False
            if len(pgs) == 1:
                import torch.distributed as dist

                (pg, world), = pgs.values()

                def to_cpu(v):
                    return v.detach().cpu() if torch.is_tensor(v) else v

                mine = {k: {kk: to_cpu(vv) for kk, vv in st.items()} for k, st in sd["state"].items()}
                gathered = [None] * world
                dist.all_gather_object(gathered, mine, group=pg)
                merged = {}
                for part in gathered:                      # non-owners may hold a few scalar keys:
                    for k, st in part.items():             # the owner's entry wins
                        merged.setdefault(k, st)
                for k in list(merged):
                    own = gathered[stable_distributed_owner(int(k), world)].get(k)
                    if own is not None:
                        merged[k] = own
                sd["state"] = {k: merged[k] for k in sorted(merged)}
                for grp in groups:
                    for e in grp["params"]:
                        st = merged.get(e["saved_id"], {})
                        e["state_keys"] = tuple(sorted(str(k) for k in st))
                        e["initialized"] = any(str(k) != "name" for k in st)
                consolidated = True
            sd["gefen_muon_distributed"] = {"version": 2, "ownership": "stable_full_param_index_v1",
                                            "consolidated": consolidated, "groups": groups}
        return sd

    def _validate_distributed_manifest(self, sd, manifest) -> None:
        """A consolidated ``distributed`` checkpoint says, per matrix, who owned it at which world size
        and which state it carries.  Everything that can be checked against the live optimizer is
        checked before the load starts: version and ownership rule, the consolidated flag, one entry
        per live parameter in order with the same name and global shape, owners that follow the
        ownership rule, and initialised entries whose momentum is present and sized for the full
        matrix (reference ``gefen_muon.py:2609-2748``)."""
        def refuse(why):
            return ValueError("GefenMuon.load_state_dict refused the distributed checkpoint: " + why)

        if not isinstance(manifest, dict):
            raise refuse("the manifest is not a mapping")
        if manifest.get("version") not in (1, 2):
            raise refuse("manifest version {!r}, expected 1 or 2".format(manifest.get("version")))
        if manifest.get("ownership") != "stable_full_param_index_v1":
            raise refuse("ownership scheme {!r}, expected 'stable_full_param_index_v1'".format(
                manifest.get("ownership")))
        saved_state = sd.get("state", {})
        if not isinstance(saved_state, dict):
            raise refuse("the 'state' payload is not a mapping")
        if manifest.get("consolidated") is not True:
            # only the saving rank's own matrices are inside: usable on the same single rank only
            if any(self._process_group_of(p)[1] > 1 for g in self.param_groups for p in g["params"]):
                raise refuse("the checkpoint is not consolidated (it holds one rank's momentum only)")
        if manifest.get("version") == 1:
            return
        groups = manifest.get("groups")
        if not isinstance(groups, (list, tuple)):
            raise refuse("the owner manifest is missing or is not a list")
        entries = []
        for gi, grp in enumerate(groups):
            if not isinstance(grp, dict) or not isinstance(grp.get("params"), (list, tuple)):
                raise refuse("manifest group {} is malformed".format(gi))
            ws = grp.get("world_size")
            if isinstance(ws, bool) or not isinstance(ws, int) or ws < 1:
                raise refuse("manifest group {} has world_size {!r}".format(gi, ws))
            for e in grp["params"]:
                if not isinstance(e, dict):
                    raise refuse("manifest group {} holds a malformed parameter entry".format(gi))
                entries.append((ws, e))
        live = [p for g in self.param_groups for p in g["params"]]
        if len(entries) != len(live):
            raise refuse("the manifest lists {} parameters, the optimizer has {}".format(len(entries), len(live)))
        saved_ids = [pid for g in sd.get("param_groups", ()) for pid in g.get("params", ())]
        for pos, ((ws, e), p) in enumerate(zip(entries, live)):
            sid = e.get("saved_id")
            if isinstance(sid, bool) or not isinstance(sid, int) or sid != pos:
                raise refuse("entry {} carries saved_id {!r}".format(pos, sid))
            if e.get("name") != self._param_name(p):
                raise refuse("entry {} is {!r}, the live parameter is {!r}".format(
                    pos, e.get("name"), self._param_name(p)))
            shape = e.get("shape")
            if not isinstance(shape, (list, tuple)) or tuple(int(d) for d in shape) != tuple(p.shape):
                raise refuse("{} was saved with shape {}, the live parameter has {}".format(
                    e.get("name"), shape, tuple(p.shape)))
            if e.get("owner") != stable_distributed_owner(pos, ws):
                raise refuse("{} names owner {!r}; the ownership rule gives {} at world size {}".format(
                    e.get("name"), e.get("owner"), stable_distributed_owner(pos, ws), ws))
            keys = e.get("state_keys")
            if not isinstance(keys, (list, tuple)) or not all(isinstance(k, str) for k in keys):
                raise refuse("{} has malformed state_keys".format(e.get("name")))
            st = saved_state.get(saved_ids[pos] if pos < len(saved_ids) else pos)
            if e.get("initialized"):
                if not isinstance(st, dict) or "m_codebook" not in st or "m_magnitude" not in st:
                    raise refuse("{} is marked initialised but its momentum is missing".format(e.get("name")))
                missing = [k for k in keys if k not in {str(x) for x in st}]
                if missing:
                    raise refuse("{} lacks the state keys {}".format(e.get("name"), missing))
                if torch.is_tensor(st["m_codebook"]) and st["m_codebook"].numel() != p.numel():
                    raise refuse("the momentum of {} holds {} elements, the full matrix has {}".format(
                        e.get("name"), st["m_codebook"].numel(), p.numel()))
            elif isinstance(st, dict) and "m_codebook" in st:
                raise refuse("{} carries momentum but is marked uninitialised".format(e.get("name")))

    def load_state_dict(self, state_dict) -> None:
        """Loads a native checkpoint; after a consolidated ``distributed`` checkpoint every rank
        keeps only the momentum of the matrices it owns at the current world size."""
        sd = dict(state_dict)
        manifest = sd.pop("gefen_muon_distributed", None)
        if manifest is not None:
            self._validate_distributed_manifest(sd, manifest)     # before anything live is touched
        super().load_state_dict(sd)
        if self.sharded_mode == "distributed":
            stable = 0
            for g in self.param_groups:
                for p in g["params"]:
                    pg, world, rank = self._process_group_of(p)
                    if pg is not None and world > 1 and stable_distributed_owner(stable, world) != rank:
                        self.state.pop(p, None)
                    stable += 1
