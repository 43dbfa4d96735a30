"""``torch.distributed.checkpoint`` adapter that reshards plain-Gefen state N -> M ranks.

The compact state (uint8 indices + per-block magnitudes / second moments) is tied
to the local shard's block geometry, so it is published as *dense* fp32
``Shard(0)`` tensors (``momentum`` = codeword x magnitude, ``second_moment`` =
block value repeated per element) under flat keys; DCP then reshards them like any
other tensor.  On load every rank re-derives a period for its new local shard,
re-learns its codebook from the dense momentum and re-quantises.

Key schema (format version 2, identical to the reference's, ``src/gefen/dcp.py:1119-1169``):
``format_version, global_step, deterministic, slot_count, group_count,
param_identities, param_group_hypers`` and per slot
``slot_%08d.{initialized, step, vmean_step, momentum, second_moment}``.
Requirements, as in the reference (``dcp.py:584-670``): plain ``Gefen`` with
``factored_v_2d=False`` and ``capturable=False``, caller-provided parameter names,
parameters that are ``Shard(0)`` DTensors on the 1-D default-world mesh (or plain
tensors in a single process).

Memory: the dense tensors are never all alive during a save.  ``state_dict()``
publishes zero-storage stand-ins (:class:`~gefen_x_b200.ckpt.lazy.LazyShard`);
:class:`GefenSavePlanner` expands one at a time when the writer asks for it, copies
it to the host through one pinned staging buffer and drops the device copy, so the
device-side transient is one slot's dense form (4 bytes per element of the largest
local shard) instead of 8 bytes per local parameter (reference
``src/gefen/dcp.py:162-391``, ``:1423-1475``, ``:1540-1554``).  Without the planner
the save is still correct, at the eager cost.  Before a save or a load all ranks
agree, with one small all-reduce, on a digest of the slot layout (names, groups,
shapes), so that ranks with different layouts fail before DCP assembles one tensor
from different parameters (reference ``dcp.py:775-785``).

Extension used by the sharded runtime (``parallel.fsdp``): ``geometry=`` places
plain row-shard tensors (not DTensors) in their global tensors, and
``allow_factored=True`` also publishes the factored second moment
(``second_moment_row`` sharded by rows, ``second_moment_col`` replicated,
``factored_step``), which that runtime keeps consistent across its shards.
"""
from __future__ import annotations

import hashlib
import threading
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

from ..optim.gefen import Gefen, _local
from ..parallel.control import control_device, raise_if_any_rank_failed
from ..quant import codebook as _cbk
from ..quant import partitioning as _part
from .lazy import LazyShard, PinnedStaging, row_shard_geometry

FORMAT_VERSION = 2


def _is_dtensor(t) -> bool:
    return hasattr(t, "device_mesh") and hasattr(t, "placements")


def dense_momentum(codebook: torch.Tensor, state: Dict[str, Any], shape) -> torch.Tensor:
    """fp32 momentum of a local shard: ``codebook[idx] * magnitude``."""
    idx = state["m_codebook"]
    cb = codebook.to(idx.device)
    if idx.is_cuda and idx.is_contiguous():
        from ..ops import _ext, quant as _q

        if _ext.available():
            period = idx.numel() // max(1, state["m_magnitude"].numel())
            return _q.dequantize(idx, state["m_magnitude"], cb, period, torch.float32).reshape(shape)
    return (_cbk.dequantize_indices(cb, idx, torch.float32) * state["m_magnitude"]).reshape(shape)


def dense_second_moment(state: Dict[str, Any], shape) -> torch.Tensor:
    """fp32 second moment of a local shard: the block value repeated over its block."""
    vmean = state["vmean"]
    period = int(state["automatic_period"])
    return vmean.reshape(-1, 1).expand(-1, period).reshape(shape).contiguous()


def choose_period(optimizer: Gefen, name: str, parameter, second: torch.Tensor) -> int:
    """Block period of a resharded local shard from its dense second moment (a grad^2 proxy);
    the optimizer's period-one gates win (reference ``dcp.py:430-472``)."""
    if optimizer._force_1d_period_one and parameter.ndim == 1:
        return 1
    if optimizer._force_2d_period_one and parameter.ndim == 2:
        return 1
    if optimizer._period_one_substrings and any(s in str(name).lower()
                                                 for s in optimizer._period_one_substrings):
        return 1
    flat = second.reshape(-1)
    if flat.numel() < 8:
        return 1
    return _part.find_period_by_block_variance(
        flat.detach().float().cpu(), print_results=False, parameter_name=name,
        parameter_shape=tuple(_local(parameter).shape), backend="cpu", input_is_squared=True)


def reblock(codebook: torch.Tensor, momentum: torch.Tensor, second: Optional[torch.Tensor], period: int):
    """Dense fp32 shard -> ``(m_codebook, m_magnitude, vmean)`` for the new blocking
    (``vmean`` is None when no dense second moment is given)."""
    flat = momentum.reshape(-1).float()
    cb = codebook.to(device=flat.device, dtype=torch.float32)
    blocks = flat.view(-1, period)
    mag = blocks.abs().amax(dim=1, keepdim=True)
    inv = torch.where(mag > 0, 1.0 / mag, torch.zeros_like(mag))
    idx = _cbk.nearest_codebook_indices(cb, blocks * inv)
    vmean = None
    if second is not None:
        vmean = second.reshape(-1).float().view(-1, period).mean(dim=1, keepdim=True)
    return idx, mag, vmean


class GefenDCPState:
    """``Stateful`` wrapper: ``dcp.save({"optimizer": GefenDCPState(opt)})`` / ``dcp.load(...)``.

    ``geometry(p) -> (global_shape, offsets, sizes)`` (optional) places a plain local tensor
    inside its global tensor when the shards are not DTensors; ``allow_factored`` admits the
    factored second moment (see the module docstring).
    """

    def __init__(self, optimizer: Gefen, *, dense_device: Optional[torch.device] = None,
                 geometry: Optional[Callable[[torch.Tensor], Tuple[tuple, tuple, tuple]]] = None,
                 allow_factored: bool = False, process_group=None):
        if not isinstance(optimizer, Gefen) or type(optimizer).__name__ != "Gefen":
            raise TypeError("GefenDCPState wraps a plain Gefen optimizer")
        self.optimizer = optimizer
        self.dense_device = dense_device
        self.geometry = geometry
        self.allow_factored = bool(allow_factored)
        self.process_group = process_group
        self._slots = self._validate_layout()
        self._published: Dict[str, Any] = {}

    # ------------------------------------------------------------------
    def _world(self) -> int:
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            return 1
        return dist.get_world_size(self.process_group)

    def _validate_layout(self) -> List[Tuple[int, int, str, torch.Tensor]]:
        opt = self.optimizer
        if opt.capturable:
            raise RuntimeError("GefenDCPState does not support capturable=True; checkpoint with "
                               "capturable=False")
        if opt._factored_v_2d and not self.allow_factored:
            raise RuntimeError(
                "GefenDCPState does not support factored_v_2d=True: the factored row/column second "
                "moment is not shard-addressable. Construct the optimizer with factored_v_2d=False "
                "for DCP resharding.")
        slots, index = [], 0
        world = self._world()
        for gi, group in enumerate(opt.param_groups):
            names = group.get("param_names")
            if names is None or len(names) != len(group["params"]):
                raise RuntimeError("GefenDCPState requires caller-provided stable param_names on every group")
            for name, p in zip(names, group["params"]):
                if opt._param_name_is_synthesized(p):
                    raise RuntimeError(
                        "GefenDCPState requires caller-provided stable parameter names, but slot {} "
                        "carries the positional name {!r} that Gefen synthesized".format(index, name))
                if _is_dtensor(p):
                    mesh = p.device_mesh
                    if mesh.ndim != 1 or mesh.size() != world:
                        raise RuntimeError("GefenDCPState supports only a one-dimensional default-world DeviceMesh")
                    if mesh.mesh.flatten().tolist() != list(range(world)):
                        raise RuntimeError("GefenDCPState supports only the canonical rank order 0..N-1")
                    if len(p.placements) != 1 or type(p.placements[0]).__name__ != "Shard" \
                            or p.placements[0].dim != 0:
                        raise RuntimeError("GefenDCPState supports only one-dimensional Shard(0) parameters")
                elif world > 1 and self.geometry is None:
                    raise RuntimeError("GefenDCPState requires every parameter to be a DTensor when "
                                       "more than one rank participates")
                slots.append((index, gi, str(name), p))
                index += 1
        if not slots:
            raise RuntimeError("GefenDCPState requires at least one parameter")
        if len({s[2] for s in slots}) != len(slots):
            raise RuntimeError("GefenDCPState requires unique parameter names")
        return slots

    @staticmethod
    def _key(index: int, field: str) -> str:
        return "slot_{:08d}.{}".format(index, field)

    # -- geometry of one slot ------------------------------------------------------------
    def _geometry_of(self, p) -> Tuple[tuple, tuple, tuple]:
        """``(global_shape, offsets, sizes)`` of this rank's part of ``p``."""
        if _is_dtensor(p):
            world = p.device_mesh.size(0)
            rank = p.device_mesh.get_local_rank(0)
            offsets, sizes = row_shard_geometry(tuple(p.shape), world, rank)
            local = tuple(p.to_local().shape)
            if local != sizes:                      # an uneven split torch chose differently: trust the tensor
                from torch.distributed.tensor._utils import compute_local_shape_and_global_offset

                sz, off = compute_local_shape_and_global_offset(p.shape, p.device_mesh, p.placements)
                offsets, sizes = tuple(int(o) for o in off), tuple(int(s) for s in sz)
            return tuple(p.shape), offsets, sizes
        if self.geometry is not None:
            g = self.geometry(p)
            if g is not None:
                return tuple(g[0]), tuple(g[1]), tuple(g[2])
        shape = tuple(p.shape)
        return shape, (0,) * len(shape), shape

    def _global_shape(self, p) -> tuple:
        return self._geometry_of(p)[0]

    def _identities(self) -> List[Dict[str, Any]]:
        return [{"name": n, "group": gi, "shape": [int(d) for d in self._global_shape(p)]}
                for _, gi, n, p in self._slots]

    def _process_groups(self):
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.process_group) > 1:
            return [self.process_group]
        return []

    def _agree_on_layout(self) -> None:
        """All ranks must present the same slots in the same order: one all-reduce (MIN over the
        digest words and their negations gives the group-wide minimum and maximum) compares a
        sha256 of the (name, group, global shape) list."""
        import torch.distributed as dist

        pgs = self._process_groups()
        if not pgs:
            return
        canonical = repr([(d["name"], d["group"], tuple(d["shape"])) for d in self._identities()]).encode()
        digest = hashlib.sha256(canonical).digest()[:16]
        words = [int.from_bytes(digest[i:i + 4], "big") for i in range(0, 16, 4)]     # 32-bit pieces: no overflow
        packed = torch.tensor(words + [-w for w in words], dtype=torch.int64, device=control_device(pgs[0]))
        dist.all_reduce(packed, op=dist.ReduceOp.MIN, group=pgs[0])
        vals = packed.tolist()
        if vals[:4] != [-v for v in vals[4:]]:
            raise RuntimeError(
                "GefenDCPState: ranks hold different parameter layouts (name / group / shape) for the same "
                "positional slots, so one global tensor would be assembled from different parameters. "
                "Build every rank's optimizer from the same named parameters in the same group order.")

    # ------------------------------------------------------------------
    def _lazy(self, p, build: Callable[[], torch.Tensor], *, row_vector: bool = False) -> Any:
        """Stand-in for a dense fp32 tensor laid out like ``p`` (or like its rows)."""
        gshape, offsets, sizes = self._geometry_of(p)
        if row_vector:
            gshape, offsets, sizes = gshape[:1], offsets[:1], sizes[:1]
        device = self.dense_device if self.dense_device is not None else _local(p).device
        dd = self.dense_device

        def materialize():
            t = build()
            return t.to(dd) if dd is not None else t

        return LazyShard(gshape, offsets, sizes, materialize, dtype=torch.float32, device=device)

    def state_dict(self) -> Dict[str, Any]:
        exc, out = None, None
        try:
            out = self._build_state_dict()
        except Exception as e:  # noqa: BLE001
            exc = e
        pgs = self._process_groups()
        if pgs:
            raise_if_any_rank_failed(exc, pgs, "GefenDCPState.state_dict")
            self._agree_on_layout()
        elif exc is not None:
            raise exc
        self._published = out
        return out

    def _build_state_dict(self) -> Dict[str, Any]:
        opt = self.optimizer
        out: Dict[str, Any] = {
            "format_version": torch.tensor(FORMAT_VERSION, dtype=torch.int64),
            "global_step": torch.tensor(int(opt._gefen_global_step), dtype=torch.int64),
            "deterministic": torch.tensor(int(bool(opt._deterministic)), dtype=torch.uint8),
            "slot_count": torch.tensor(len(self._slots), dtype=torch.int64),
            "group_count": torch.tensor(len(opt.param_groups), dtype=torch.int64),
            "param_identities": self._identities(),
            "param_group_hypers": [{"lr": float(g["lr"]), "beta1": g["beta1"], "beta2": g["beta2"],
                                    "eps": g["eps"], "weight_decay": g["weight_decay"]}
                                   for g in opt.param_groups],
        }
        for index, _gi, _name, p in self._slots:
            st = opt.state.get(p) or {}
            local = _local(p)
            factored = "v_row" in st
            has_v = factored or "vmean" in st
            init = "m_codebook" in st and has_v and local.numel() > 0
            if factored and not self.allow_factored:
                raise RuntimeError("GefenDCPState found a factored second moment; construct the optimizer with "
                                   "factored_v_2d=False for DCP resharding")
            out[self._key(index, "initialized")] = torch.tensor(int(init), dtype=torch.uint8)
            out[self._key(index, "step")] = torch.tensor(int(st.get("step", 0)), dtype=torch.int64)
            out[self._key(index, "vmean_step")] = torch.tensor(
                int(st.get("vmean_step", st.get("factored_step", st.get("step", 0)))), dtype=torch.int64)
            shape, dev = tuple(local.shape), local.device

            def zeros(shape=shape, dev=dev):
                return torch.zeros(shape, dtype=torch.float32, device=dev)

            if init:
                # the closures read the live state at write time: one dense tensor at a time
                out[self._key(index, "momentum")] = self._lazy(
                    p, lambda st=st, shape=shape: dense_momentum(opt._gefen_codebook, st, shape))
            else:
                out[self._key(index, "momentum")] = self._lazy(p, zeros)
            if self.allow_factored and p.ndim == 2 and (factored or not init) and opt._factored_v_2d:
                rows, cols = shape
                out[self._key(index, "factored_step")] = torch.tensor(int(st.get("factored_step", 0)),
                                                                      dtype=torch.int64)
                out[self._key(index, "second_moment_row")] = self._lazy(
                    p, (lambda st=st: st["v_row"].float().reshape(-1)) if factored else
                    (lambda rows=rows, dev=dev: torch.zeros(rows, dtype=torch.float32, device=dev)),
                    row_vector=True)
                vcol = st["v_col"].detach().float().cpu().clone() if factored else torch.zeros(cols)
                out[self._key(index, "second_moment_col")] = vcol
            elif init:
                out[self._key(index, "second_moment")] = self._lazy(
                    p, lambda st=st, shape=shape: dense_second_moment(st, shape))
            else:
                out[self._key(index, "second_moment")] = self._lazy(p, zeros)
        return out

    # ------------------------------------------------------------------
    def load_state_dict(self, state_dict: Dict[str, Any]) -> None:
        exc, staged = None, None
        try:
            staged = self._stage_load(state_dict)
        except Exception as e:  # noqa: BLE001
            exc = e
        pgs = self._process_groups()
        if pgs:
            raise_if_any_rank_failed(exc, pgs, "GefenDCPState.load_state_dict")
        elif exc is not None:
            raise exc
        self._commit(staged)

    @staticmethod
    def _loaded_tensor(value, device, shape) -> torch.Tensor:
        """What DCP delivered for one dense entry: the filled stand-in buffer, a DTensor's local part
        (checkpoints loaded into eager dense destinations) or a plain tensor."""
        if isinstance(value, LazyShard):
            t = value.loaded()
            if t is None:
                raise ValueError("a dense shard of the checkpoint was not loaded")
            return t.to(device).reshape(shape)
        return _local(value).to(device).reshape(shape)

    def _stage_load(self, sd: Dict[str, Any]):
        opt = self.optimizer
        if int(sd["format_version"]) != FORMAT_VERSION:
            raise ValueError("unsupported GefenDCPState format_version {}".format(int(sd["format_version"])))
        if int(sd["slot_count"]) != len(self._slots):
            raise ValueError("checkpoint has {} slots, optimizer has {}".format(
                int(sd["slot_count"]), len(self._slots)))
        if int(sd["group_count"]) != len(opt.param_groups):
            raise ValueError("checkpoint has {} groups, optimizer has {}".format(
                int(sd["group_count"]), len(opt.param_groups)))
        if bool(int(sd["deterministic"])) != bool(opt._deterministic):
            raise ValueError("checkpoint deterministic policy differs from the optimizer's")
        ids = sd["param_identities"]
        for (index, gi, name, p), ident in zip(self._slots, ids):
            if ident["name"] != name or int(ident["group"]) != gi or \
                    tuple(ident["shape"]) != tuple(self._global_shape(p)):
                raise ValueError("slot {} identity mismatch: checkpoint {}, optimizer {}".format(
                    index, ident, (name, gi, tuple(self._global_shape(p)))))
        # pass 1: periods of the new local shards; the dense momentum feeds the codebook histogram
        plan = []
        for index, _gi, name, p in self._slots:
            init = bool(int(sd[self._key(index, "initialized")]))
            local = _local(p)
            if not init or local.numel() == 0:
                plan.append(None)
                continue
            mom = self._loaded_tensor(sd[self._key(index, "momentum")], local.device, local.shape)
            if not bool(torch.isfinite(mom).all()):
                raise ValueError("checkpoint momentum of {} is not finite".format(name))
            factored = self._key(index, "second_moment_row") in sd and self.allow_factored
            if factored:
                v_row = self._loaded_tensor(sd[self._key(index, "second_moment_row")], local.device,
                                            (local.shape[0],))
                v_col = sd[self._key(index, "second_moment_col")].to(local.device).float().reshape(-1)
                sec = None
                proxy = (v_row[:, None] * v_col[None, :])        # rank-1 estimate of grad^2, for the period
            else:
                sec = self._loaded_tensor(sd[self._key(index, "second_moment")], local.device, local.shape)
                proxy = sec
            if not bool(torch.isfinite(proxy).all()) or bool((proxy < 0).any()):
                raise ValueError("checkpoint second moment of {} is not finite and non-negative".format(name))
            period = choose_period(opt, name, p, proxy)
            if local.numel() % period:
                period = 1
            plan.append(dict(mom=mom, sec=sec, period=period,
                             v_row=v_row if factored else None, v_col=v_col if factored else None))
            del proxy
        items = [(n, d["mom"].reshape(-1), d["period"], d["mom"]) for (_i, _g, n, _p), d in zip(self._slots, plan)
                 if d is not None]
        codebook = None
        if items:
            codebook = _cbk.learn_codebook_from_grad_periods(
                items, opt._gefen_codebook_device(), reduce_counts=opt._histogram_reducer)
        # pass 2: re-quantise slot by slot, dropping each dense form as soon as it is consumed
        staged_states = []
        for (index, _gi, name, p), d in zip(self._slots, plan):
            if d is None:
                staged_states.append(None)
                continue
            idx, mag, vmean = reblock(codebook, d["mom"], d["sec"], d["period"])
            st = {"automatic_period": d["period"], "m_codebook": idx, "m_magnitude": mag,
                  "step": int(sd[self._key(index, "step")])}
            if d["v_row"] is not None:
                st["v_row"], st["v_col"] = d["v_row"].clone(), d["v_col"].clone()
                st["factored_step"] = int(sd[self._key(index, "factored_step")])
            else:
                st["vmean"] = vmean
                st["vmean_step"] = int(sd[self._key(index, "vmean_step")])
            staged_states.append(st)
            d.clear()
            for field in ("momentum", "second_moment", "second_moment_row"):
                v = sd.get(self._key(index, field))
                if isinstance(v, LazyShard):
                    v._gx_cache = None
        return dict(states=staged_states, codebook=codebook, global_step=int(sd["global_step"]),
                    hypers=sd["param_group_hypers"])

    def _commit(self, staged) -> None:
        opt = self.optimizer
        for (index, _gi, name, p), st in zip(self._slots, staged["states"]):
            live = opt.state[p]
            for k in ("automatic_period", "m_codebook", "m_magnitude", "vmean", "step", "vmean_step",
                      "v_row", "v_col", "factored_step"):
                live.pop(k, None)
            live["name"] = name
            if st is not None:
                live.update(st)
        for g, h in zip(opt.param_groups, staged["hypers"]):
            for k in ("lr", "beta1", "beta2", "eps", "weight_decay"):
                if k in h and not torch.is_tensor(g.get(k)):
                    g[k] = h[k]
        opt._gefen_global_step = staged["global_step"]
        opt._set_codebook(staged["codebook"])
        opt._fast = None
        if opt._plan_cache is not None:
            opt._plan_cache.clear()


def _planner_base():
    from torch.distributed.checkpoint import DefaultSavePlanner

    return DefaultSavePlanner


def _writer_base():
    from torch.distributed.checkpoint import FileSystemWriter

    return FileSystemWriter


class GefenSavePlanner(_planner_base()):
    """Save planner that keeps the save of a :class:`GefenDCPState` memory-bounded.

    When the writer asks for the data of a write item that is a stand-in, the dense form of that
    one slot is built, copied to the host through a reusable pinned buffer and dropped on the
    device, all under a lock, so however many writer threads run, at most one dense slot exists
    on the device at a time (reference ``src/gefen/dcp.py:1478-1554``).  Requires the default
    ``flatten_state_dict=True``: stand-ins are addressed by their flattened dotted names.
    """

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        if not self.flatten_state_dict:
            raise ValueError("GefenSavePlanner requires flatten_state_dict=True (the default): stand-ins are "
                             "addressed by their flattened names; without flattening DCP would try to pickle "
                             "the whole optimizer mapping")
        self._gx_lock = threading.Lock()
        self._gx_staging = PinnedStaging()

    def set_up_planner(self, state_dict, storage_meta=None, is_coordinator=False):
        # named arguments on purpose: dcp.save inspects this signature for ``storage_meta``
        super().set_up_planner(state_dict, storage_meta, is_coordinator)

    def resolve_data(self, write_item):
        entry = self.state_dict.get(write_item.index.fqn)
        if isinstance(entry, LazyShard):
            with self._gx_lock:
                return entry.resolve_uncached(self._gx_staging)
        return super().resolve_data(write_item)


def _strip_stand_ins(tree, staged, prefix=()):
    """Copy of ``tree`` without its stand-ins; each is snapshotted to the host into ``staged[path]``
    (one dense form alive at a time)."""
    out = dict(tree)
    for key, value in tree.items():
        path = prefix + (key,)
        if isinstance(value, LazyShard):
            staged[path] = value.staged_to_host()
            del out[key]
        elif isinstance(value, dict):
            out[key] = _strip_stand_ins(value, staged, path)
    return out


def _put_back(tree, staged):
    out = dict(tree)
    for path, shard in staged.items():
        node = out
        for key in path[:-1]:
            node[key] = dict(node[key])
            node = node[key]
        node[path[-1]] = shard
    return out


class GefenFileSystemWriter(_writer_base()):
    """File-system writer that can stage a :class:`GefenDCPState` for ``async_save``.

    ``async_save`` first copies the state dict to the host and writes from a background thread.
    Torch's staging asks every entry for a host copy of itself, which a stand-in without data
    cannot give; this writer expands the stand-ins itself, one slot at a time, into host
    snapshots that keep publishing the slot's global shape and chunk offsets, and leaves the
    rest to torch (reference ``src/gefen/dcp.py:1599-1619``).  The synchronous ``dcp.save`` does
    not stage and works with any writer.
    """

    def __init__(self, path, *args, **kwargs):
        kwargs.setdefault("single_file_per_rank", True)
        super().__init__(path, *args, **kwargs)

    def stage(self, state_dict):
        staged: Dict[tuple, LazyShard] = {}
        stripped = _strip_stand_ins(state_dict, staged)
        return _put_back(super().stage(stripped), staged)
