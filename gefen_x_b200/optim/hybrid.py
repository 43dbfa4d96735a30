"""``GefenMuonHybrid``: Muon for hidden matrices + a backup optimizer for everything else.

The composite owns two child optimizers (``GefenMuon`` and either ``Gefen`` or
``torch.optim.AdamW``) and presents them as one ``torch.optim.Optimizer``-like
object: ``param_groups`` is the live concatenation of the children's groups (LR
schedulers work on it), ``step`` runs the backup then Muon after a joint
pre-collective failure agreement, checkpoints are ``{"muon", "backup",
"backup_optimizer"}`` and are loaded in two phases so that a failure in either
half leaves both untouched.

Parity: reference ``src/gefen/hybrid.py`` (constructor forms ``:228-329``, routing
view ``:91``, step ``:693-776``, checkpoint ``:778-1000``, ``from_model``
``:1020-1032``).
"""
from __future__ import annotations

import copy
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.nn as nn

from ..parallel.control import raise_if_any_rank_failed
from .gefen import Gefen
from .muon import GefenMuon
from .params import (DEFAULT_BACKUP_SUBSTRINGS, split_named_for_muon, split_params_for_muon,
                     validate_split)


_ZERO_HINT = ("GefenMuonHybrid cannot run under DeepSpeed ZeRO: ZeRO replaces the parameters with flat 1-D fp32 "
              "partitions that Muon's 2-D Newton-Schulz step cannot use, and it keeps its bookkeeping in "
              "optimizer.state under those partitions. Use plain Gefen with DeepSpeed ZeRO.")


class _MergedState(dict):
    """``optimizer.state`` of the hybrid: a live view that routes every access to the child that
    owned the parameter at construction.  Reads of a known parameter auto-create in the owning
    child (torch's defaultdict behaviour); a key that is not one of the hybrid's parameters
    raises a ``KeyError`` that names the usual cause, an optimizer wrapper that swapped in flat
    partitions (reference ``hybrid.py`` state view).  The underlying ``dict`` stays empty."""

    def __init__(self, children):
        super().__init__()
        self._children = [c for c in children if c is not None]
        self._owner_of = {id(p): (p, c) for c in self._children for g in c.param_groups for p in g["params"]}

    def _owner(self, p):
        hit = self._owner_of.get(id(p))
        if hit is None or hit[0] is not p:
            raise KeyError("optimizer.state[<{} of shape {}>]: not a parameter of this optimizer. {}".format(
                type(p).__name__, tuple(getattr(p, "shape", ())), _ZERO_HINT))
        return hit[1]

    def _known(self, p) -> bool:
        hit = self._owner_of.get(id(p))
        return hit is not None and hit[0] is p

    def __getitem__(self, p):
        return self._owner(p).state[p]

    def __setitem__(self, p, value):
        self._owner(p).state[p] = value

    def __delitem__(self, p):
        del self._owner(p).state[p]

    def get(self, p, default=None):
        if not self._known(p):
            return default
        st = self._owner(p).state
        return st[p] if p in st else default

    def __contains__(self, p):
        return self._known(p) and p in self._owner(p).state

    def __iter__(self):
        for c in self._children:
            yield from list(c.state)

    def __len__(self):
        return sum(len(c.state) for c in self._children)

    def __bool__(self):
        return len(self) > 0

    def keys(self):
        return list(iter(self))

    def items(self):
        return [(p, st) for c in self._children for p, st in c.state.items()]

    def values(self):
        return [st for c in self._children for st in c.state.values()]

    def setdefault(self, p, default=None):
        st = self._owner(p).state
        if p in st:
            return st[p]
        st[p] = default
        return default

    def update(self, *args, **kwargs):
        for p, value in dict(*args, **kwargs).items():
            self[p] = value

    _MISSING = object()

    def pop(self, p, default=_MISSING):
        st = self._owner(p).state
        if p in st:
            value = st[p]
            del st[p]
            return value
        if default is _MergedState._MISSING:
            raise KeyError(p)
        return default

    def popitem(self):
        raise NotImplementedError("popitem is not defined on the hybrid's merged state view")

    def clear(self):
        for c in self._children:
            c.state.clear()

    def __repr__(self):
        return "_MergedState({} entries)".format(len(self))


class GefenMuonHybrid(torch.optim.Optimizer):
    """See the module docstring.  Call forms: ``(muon_named, backup_named, lr=...)``,
    ``(model, lr=...)`` or ``(named_parameters_iterable, lr=...)``."""

    def __init__(self, muon_named_params, backup_named_params=None, *, lr, backup_substrings=None,
                 muon_lr=None, backup_lr=None, backup_optimizer: str = "gefen",
                 weight_decay: float = 0.0, muon_weight_decay=None, backup_weight_decay=None,
                 no_decay_substrings=(), backup_1d_period_one: bool = False,
                 backup_2d_period_one: bool = False, betas=(0.9, 0.999), eps: float = 1e-8,
                 fused: bool = True, momentum: float = 0.95, nesterov: bool = True, ns_steps: int = 5,
                 ns_schedule: Optional[str] = "tuned3", adjust_lr_fn: Optional[str] = "match_rms_adamw",
                 sharded_mode: str = "exact", fp8_ns: bool = False, fp8_ns_compile: bool = True,
                 batched_ns: bool = False, batched_ns_workspace_bytes: int = 256 << 20,
                 stochastic_round: bool = False, deterministic: bool = False, normuon: bool = True,
                 normuon_beta2: float = 0.95, normuon_eps: float = 1e-8, cautious: bool = False,
                 capturable: bool = False, verbose: bool = False):
        if not isinstance(deterministic, bool):
            raise TypeError("deterministic must be a bool")
        if backup_optimizer not in ("gefen", "adamw"):
            raise ValueError("backup_optimizer must be 'gefen' or 'adamw', got {!r}".format(backup_optimizer))
        if adjust_lr_fn in (None, "original"):
            # Muon-native scaling leaves the matrices on another lr footing than the backup half
            # (reference hybrid.py:395-412): say so instead of silently mis-scaling one half
            import warnings

            warnings.warn("GefenMuonHybrid: adjust_lr_fn={!r} uses Muon-native LR scaling, so an AdamW-scale lr "
                          "will mis-scale the 2D Muon matrices relative to the backup half. Use "
                          "adjust_lr_fn='match_rms_adamw' (the default) to share one AdamW-scale lr, or set "
                          "muon_lr explicitly.".format(adjust_lr_fn), stacklevel=2)
        model = None
        if backup_named_params is None:
            subs = DEFAULT_BACKUP_SUBSTRINGS if backup_substrings is None else tuple(backup_substrings)
            if isinstance(muon_named_params, nn.Module):
                model = muon_named_params
                muon_named, backup_named = split_params_for_muon(model, subs)
            else:
                items = list(muon_named_params)
                if items and isinstance(items[0], torch.Tensor):
                    raise TypeError(
                        "Bare tensors can't be routed by name: pass (name, param) pairs, a model, or use "
                        "GefenMuonHybrid.from_model(model, ...)")
                muon_named, backup_named = split_named_for_muon(items, subs)
        else:
            if backup_substrings is not None:
                raise TypeError("backup_substrings is only valid with the single-argument form (a model or "
                                "one list of named parameters); the two-list form is already routed")
            muon_named, backup_named = list(muon_named_params), list(backup_named_params)
        muon_named, backup_named = validate_split(muon_named, backup_named, model)
        if not muon_named and not backup_named:
            raise ValueError("optimizer got an empty parameter list")
        every = list(muon_named) + list(backup_named)
        if not muon_named and every and all(p.numel() == 0 for _, p in every):
            raise ValueError(
                "GefenMuonHybrid got only zero-numel parameters: this is what DeepSpeed ZeRO stage 3 "
                "(zero.Init) leaves before the optimizer is built, and it would silently give a backup-only "
                "optimizer without the Muon half. Use plain Gefen with ZeRO stage 3.")

        self.backup_optimizer = backup_optimizer
        self.defaults = dict(lr=lr, weight_decay=weight_decay)
        m_lr = lr if muon_lr is None else muon_lr
        b_lr = lr if backup_lr is None else backup_lr
        m_wd = weight_decay if muon_weight_decay is None else muon_weight_decay
        b_wd = weight_decay if backup_weight_decay is None else backup_weight_decay

        self.muon: Optional[GefenMuon] = None
        if muon_named:
            self.muon = GefenMuon(
                muon_named, lr=m_lr, weight_decay=m_wd, momentum=momentum, nesterov=nesterov,
                ns_steps=ns_steps, ns_schedule=ns_schedule, adjust_lr_fn=adjust_lr_fn, fused=fused,
                sharded_mode=sharded_mode, fp8_ns=fp8_ns, fp8_ns_compile=fp8_ns_compile,
                batched_ns=batched_ns, batched_ns_workspace_bytes=batched_ns_workspace_bytes,
                stochastic_round=stochastic_round, deterministic=deterministic, normuon=normuon,
                normuon_beta2=normuon_beta2, normuon_eps=normuon_eps, cautious=cautious,
                capturable=capturable, verbose=verbose)
        self.backup = None
        if backup_named:
            nd = tuple(s.lower() for s in no_decay_substrings)
            decay = [(n, p) for n, p in backup_named if not any(s in n.lower() for s in nd)]
            no_decay = [(n, p) for n, p in backup_named if any(s in n.lower() for s in nd)]
            if backup_optimizer == "gefen":
                groups = []
                if decay:
                    groups.append({"params": decay, "weight_decay": b_wd})
                if no_decay:
                    groups.append({"params": no_decay, "weight_decay": 0.0})
                # the backup never uses the factored second moment: embeddings / heads are sharded
                # by rows under FSDP and the reference pins it off as well (hybrid.py:515-518)
                self.backup = Gefen(groups, lr=b_lr, betas=betas, eps=eps, fused=fused,
                                    factored_v_2d=False, force_1d_period_one=backup_1d_period_one,
                                    force_2d_period_one=backup_2d_period_one,
                                    stochastic_round=stochastic_round, deterministic=deterministic,
                                    capturable=capturable, verbose=verbose)
            else:
                groups = []
                if decay:
                    groups.append({"params": [p for _, p in decay], "param_names": [n for n, _ in decay],
                                   "weight_decay": b_wd})
                if no_decay:
                    groups.append({"params": [p for _, p in no_decay], "param_names": [n for n, _ in no_decay],
                                   "weight_decay": 0.0})
                # the execution flags are forwarded as given (reference hybrid.py: AdamW backup)
                self.backup = torch.optim.AdamW(groups, lr=b_lr, betas=betas, eps=eps, fused=bool(fused),
                                                capturable=bool(capturable))
        self.state = _MergedState([self.muon, self.backup])
        # torch.optim.Optimizer.__init__ is deliberately not called: groups and state are live views
        # of the children's, so a scheduler's in-place ``group["lr"] = ...`` reaches them.  The hook
        # registries that torch.optim, LR schedulers and wrappers introspect are set by hand, and
        # step / state_dict / load_state_dict below dispatch them (reference ``hybrid.py:566-577``).
        from collections import OrderedDict

        self.defaults = self.children[0].defaults
        self._optimizer_step_pre_hooks = OrderedDict()
        self._optimizer_step_post_hooks = OrderedDict()
        self._optimizer_state_dict_pre_hooks = OrderedDict()
        self._optimizer_state_dict_post_hooks = OrderedDict()
        self._optimizer_load_state_dict_pre_hooks = OrderedDict()
        self._optimizer_load_state_dict_post_hooks = OrderedDict()

    def __repr__(self) -> str:
        count = lambda c: 0 if c is None else sum(len(g["params"]) for g in c.param_groups)  # noqa: E731
        return "{}(muon_params={}, backup_params={}, backup_optimizer={!r})".format(
            type(self).__name__, count(self.muon), count(self.backup), self.backup_optimizer)

    @classmethod
    def from_model(cls, model: nn.Module, **kwargs) -> "GefenMuonHybrid":
        subs = kwargs.pop("backup_substrings", DEFAULT_BACKUP_SUBSTRINGS)
        muon_named, backup_named = split_params_for_muon(model, subs)
        validate_split(muon_named, backup_named, model)
        return cls(muon_named, backup_named, **kwargs)

    # ------------------------------------------------------------------
    @property
    def children(self):
        return [c for c in (self.muon, self.backup) if c is not None]

    @property
    def param_groups(self):
        """Live concatenation of the children's groups (mutating a group dict reaches the child)."""
        out = []
        for c in self.children:
            out.extend(c.param_groups)
        return out

    @param_groups.setter
    def param_groups(self, value):
        raise TypeError("GefenMuonHybrid.param_groups is a live view of the children's groups and cannot be "
                        "assigned (DeepSpeed ZeRO's optimizer step does this). " + _ZERO_HINT)

    def add_param_group(self, param_group):
        raise NotImplementedError(
            "GefenMuonHybrid routes parameters at construction; build a new hybrid to add parameters")

    def zero_grad(self, set_to_none: bool = True) -> None:
        for c in self.children:
            c.zero_grad(set_to_none=set_to_none)

    def _process_groups(self):
        pgs, seen = [], set()
        for c in self.children:
            for g in c.param_groups:
                for p in g["params"]:
                    mesh = getattr(p, "device_mesh", None)
                    if mesh is None:
                        continue
                    for d in range(mesh.ndim):
                        pg = mesh.get_group(d)
                        if id(pg) not in seen:
                            seen.add(id(pg))
                            pgs.append(pg)
        return pgs

    @torch.compiler.disable
    @torch.no_grad()
    def step(self, closure=None):
        # instance step hooks with torch's calling convention: hook(optimizer, args, kwargs), args
        # being the raw call arguments (self first); a pre-hook may return replacements
        args, kwargs = ((self, closure) if closure is not None else (self,)), {}
        for h in list(self._optimizer_step_pre_hooks.values()):
            res = h(self, args, kwargs)
            if res is not None:
                if not (isinstance(res, tuple) and len(res) == 2):
                    raise RuntimeError("{}.step pre hook must return None or a tuple of (new_args, new_kwargs), "
                                       "but got {}.".format(type(self).__name__, res))
                args, kwargs = res
        closure = args[1] if len(args) > 1 else kwargs.get("closure")
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # one agreement over the union of both children's meshes before either mutates
        local_exc = None
        try:
            from .gefen import _assert_gradients_structurally_valid

            for c in self.children:
                _assert_gradients_structurally_valid(c)
        except Exception as exc:  # noqa: BLE001
            local_exc = exc
        pgs = self._process_groups()
        if pgs:
            raise_if_any_rank_failed(local_exc, pgs, "GefenMuonHybrid step")
        elif local_exc is not None:
            raise local_exc
        # AMP controls attached to the composite are forwarded to the children
        for attr in ("found_inf", "grad_scale"):
            if hasattr(self, attr):
                for c in self.children:
                    setattr(c, attr, getattr(self, attr))
        try:
            if self.backup is not None:
                self.backup.step()
            if self.muon is not None:
                self.muon._gefen_hybrid_precollective_preflight = True
                try:
                    self.muon.step()
                finally:
                    self.muon._gefen_hybrid_precollective_preflight = False
        finally:
            for attr in ("found_inf", "grad_scale"):
                for c in self.children:
                    if hasattr(c, attr) and hasattr(self, attr):
                        delattr(c, attr)
        for h in list(self._optimizer_step_post_hooks.values()):
            h(self, args, kwargs)
        return loss

    @property
    def _step_supports_amp_scaling(self) -> bool:
        return any(getattr(c, "_step_supports_amp_scaling", False) for c in self.children)

    # ------------------------------------------------------------------
    def state_dict(self) -> Dict[str, Any]:
        for h in list(self._optimizer_state_dict_pre_hooks.values()):
            h(self)
        sd = {
            "muon": self.muon.state_dict() if self.muon is not None else None,
            "backup": self.backup.state_dict() if self.backup is not None else None,
            "backup_optimizer": self.backup_optimizer,
        }
        for h in list(self._optimizer_state_dict_post_hooks.values()):
            res = h(self, sd)
            if res is not None:
                sd = res
        return sd

    def load_state_dict(self, state_dict) -> None:
        """Two-phase load: both halves are restored on shadow copies first; only when both
        succeeded are the results swapped in."""
        for h in list(self._optimizer_load_state_dict_pre_hooks.values()):
            res = h(self, state_dict)
            if res is not None:
                state_dict = res
        if not isinstance(state_dict, dict) or "muon" not in state_dict or "backup" not in state_dict:
            raise ValueError("not a GefenMuonHybrid checkpoint (expected keys 'muon' and 'backup')")
        saved_kind = state_dict.get("backup_optimizer", "gefen")
        if saved_kind != self.backup_optimizer:
            raise ValueError(
                "checkpoint was written with backup_optimizer={!r} but this hybrid uses {!r}".format(
                    saved_kind, self.backup_optimizer))
        if (state_dict["muon"] is None) != (self.muon is None) or \
                (state_dict["backup"] is None) != (self.backup is None):
            raise ValueError("checkpoint halves do not match this hybrid's muon/backup split")
        staged = []
        for child, sd in ((self.muon, state_dict["muon"]), (self.backup, state_dict["backup"])):
            if child is None:
                continue
            if isinstance(child, Gefen):
                shadow = object.__new__(type(child))
                shadow.__dict__.update(child.__dict__)
                shadow.state = copy.copy(child.state)
                shadow.param_groups = [dict(g, params=list(g["params"])) for g in child.param_groups]
                shadow._fast = None
                shadow._plan_cache = None
                shadow.load_state_dict(sd)
                staged.append((child, shadow))
            else:
                snapshot = copy.deepcopy(child.local_state_dict() if hasattr(child, "local_state_dict") else child.state_dict())
                staged.append((child, ("torch", sd, snapshot)))
        done = []
        try:
            for child, shadow in staged:
                if isinstance(shadow, tuple):
                    child.load_state_dict(shadow[1])
                    done.append((child, shadow[2]))
        except Exception:
            for child, snap in done:
                child.load_state_dict(snap)
            raise
        for child, shadow in staged:
            if not isinstance(shadow, tuple):
                child.__dict__.update(shadow.__dict__)
        for h in list(self._optimizer_load_state_dict_post_hooks.values()):
            h(self)

    def state_bytes(self) -> int:
        total = 0
        for c in self.children:
            if isinstance(c, Gefen):
                total += c.state_bytes()
            else:
                for st in c.state.values():
                    total += sum(v.numel() * v.element_size() for v in st.values() if torch.is_tensor(v))
        return total
