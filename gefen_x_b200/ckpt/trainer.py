"""Checkpoints of the sharded runtime (:class:`gefen_x_b200.parallel.fsdp.ShardedTrainer`).

Two forms:

* **native, rank-local** (``trainer.state_dict()`` / ``load_state_dict``): this rank's weight shards,
  the native state dict of its optimizer and the step count, ordinary tensors that ``torch.save``
  takes.  Same topology only; resuming from it continues bit for bit.
* **resharding** (``trainer.save_checkpoint(path)`` / ``load_checkpoint(path)``): a
  ``torch.distributed.checkpoint`` directory.  The weight shards are published in place (stand-ins
  that point at the live shard memory with the parameter's global shape and this rank's row
  offsets); the optimizer state goes under the GefenDCPState keys (reference
  ``src/gefen/dcp.py:1119-1169``) as dense fp32 momentum and second moment that exist one slot at a
  time while the planner writes them.  The factored second moment, which this runtime keeps
  consistent across its row shards, is published as ``second_moment_row`` (row-sharded) and
  ``second_moment_col`` (replicated).  Loading works on any number of ranks: every rank reads the
  rows it owns now, re-derives the block period of its new shards, learns the codebook from the
  dense momentum and re-quantises (reference ``src/gefen/dcp.py:1224-1420``).

The Muon hybrid keeps its momentum on the matrix owners as full matrices; its checkpoint is the
native one only.
"""
from __future__ import annotations

from typing import Any, Dict

import torch

from .dcp import GefenDCPState, GefenFileSystemWriter, GefenSavePlanner
from .lazy import LazyShard

FORMAT = "gefen_x_b200.sharded_trainer.v1"


def _identity(tr) -> Dict[str, Any]:
    cfg = tr.cfg
    return {"format": FORMAT, "model": dict(cfg.__dict__), "dtype": str(tr.dtype), "hybrid": bool(tr.hybrid)}


def _check_identity(tr, ident: Dict[str, Any], *, same_world: bool) -> None:
    if ident.get("format") != FORMAT:
        raise ValueError("not a sharded-trainer checkpoint: format {!r}".format(ident.get("format")))
    mine = _identity(tr)
    for key in ("vocab_size", "hidden", "n_layers", "n_heads", "n_kv_heads", "head_dim", "ffn", "qk_norm",
                "tie_embeddings"):
        if ident["model"].get(key) != mine["model"].get(key):
            raise ValueError("checkpoint model differs from the trainer's in {}: {} vs {}".format(
                key, ident["model"].get(key), mine["model"].get(key)))
    if ident.get("dtype") != mine["dtype"] or bool(ident.get("hybrid")) != mine["hybrid"]:
        raise ValueError("checkpoint dtype / optimizer kind differs from the trainer's")
    if same_world and (ident.get("world"), ident.get("rank")) != (tr.world, tr.rank):
        raise ValueError("a rank-local checkpoint reloads on the same topology only: saved on rank {} of {}, "
                         "loading on rank {} of {} (use save_checkpoint / load_checkpoint to reshard)".format(
                             ident.get("rank"), ident.get("world"), tr.rank, tr.world))


# --------------------------------------------------------------------------
# native, rank-local
# --------------------------------------------------------------------------
def native_state_dict(tr) -> Dict[str, Any]:
    ident = _identity(tr)
    ident.update(world=tr.world, rank=tr.rank)
    weights = {}
    for g in tr.all_groups:
        n = g.shard_numel[tr.rank] if tr.world > 1 else g.full_numel
        weights[g.name] = g.shard_w[:n].detach().clone()
    # a snapshot: the optimizer's own state dict refers to the live state tensors, which the kernels
    # keep updating in place
    out = {"identity": ident, "step_count": int(tr.step_count), "weights": weights,
           "optimizer": _snapshot(tr.opt.state_dict())}
    if tr.muon is not None:
        out["muon"] = _snapshot(tr.muon.opt.state_dict())
    return out


def _snapshot(obj):
    if torch.is_tensor(obj):
        return obj.detach().clone()
    if isinstance(obj, dict):
        return {k: _snapshot(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_snapshot(v) for v in obj)
    return obj


def load_native_state_dict(tr, state: Dict[str, Any]) -> None:
    _check_identity(tr, state["identity"], same_world=True)
    for g in tr.all_groups:                       # validate everything before touching anything
        n = g.shard_numel[tr.rank] if tr.world > 1 else g.full_numel
        w = state["weights"].get(g.name)
        if w is None or w.numel() != n or w.dtype != g.shard_w.dtype:
            raise ValueError("checkpoint weights of group {} do not fit this rank's shard".format(g.name))
    tr.opt.load_state_dict(state["optimizer"])    # atomic by itself: validates, then publishes
    if tr.muon is not None:
        if "muon" not in state:
            raise ValueError("checkpoint carries no Muon state")
        tr.muon.opt.load_state_dict(state["muon"])
    for g in tr.all_groups:
        n = g.shard_numel[tr.rank] if tr.world > 1 else g.full_numel
        g.shard_w[:n].copy_(state["weights"][g.name].to(g.shard_w.device))
    tr.step_count = int(state["step_count"])
    tr._after_restore()


# --------------------------------------------------------------------------
# resharding (torch.distributed.checkpoint)
# --------------------------------------------------------------------------
def _geometry(tr):
    """``p -> (global shape, offsets, sizes)`` for the optimizer's shard views."""
    def geometry(p):
        meta = tr._param_meta.get(p)
        if meta is None:
            return None
        _g, sp = meta
        r0 = min(sp.rows, tr.rank * sp.rows_per) if tr.world > 1 else 0
        rows = sp.shard_rows[tr.rank] if tr.world > 1 else sp.rows
        shape = tuple(sp.shape)
        return shape, (r0,) + (0,) * (len(shape) - 1), (rows,) + shape[1:]

    return geometry


class TrainerDCPState:
    """``Stateful`` view of a :class:`ShardedTrainer` for ``torch.distributed.checkpoint``."""

    def __init__(self, trainer):
        if trainer.hybrid:
            raise RuntimeError("the resharding checkpoint covers the Gefen optimizer; the Muon hybrid keeps "
                               "full-matrix momentum on the owners: use state_dict() / load_state_dict()")
        self.tr = trainer
        self.opt_state = GefenDCPState(trainer.opt, geometry=_geometry(trainer), allow_factored=True,
                                       process_group=trainer.process_group)

    def _weight_entries(self) -> Dict[str, Any]:
        tr = self.tr
        geometry = _geometry(tr)
        out = {}
        for name, view in tr.named_shards:
            shape, offsets, sizes = geometry(view)
            # no copy: the stand-in resolves to the live shard, which a load fills in place
            out[name] = LazyShard(shape, offsets, sizes, lambda v=view: v, dtype=view.dtype,
                                  device=view.device, dense_cost=False)
        return out

    def state_dict(self) -> Dict[str, Any]:
        tr = self.tr
        return {"identity": _identity(tr),
                "step_count": torch.tensor(int(tr.step_count), dtype=torch.int64),
                "weights": self._weight_entries(),
                "optimizer": self.opt_state.state_dict()}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        tr = self.tr
        _check_identity(tr, state["identity"], same_world=False)
        self.opt_state.load_state_dict(state["optimizer"])      # validates on every rank before committing
        tr.step_count = int(state["step_count"])
        tr._after_restore()


def save_checkpoint(tr, path: str, *, async_save: bool = False):
    import torch.distributed.checkpoint as dcp

    state = {"trainer": TrainerDCPState(tr).state_dict()}
    writer = GefenFileSystemWriter(path)
    if async_save:
        return dcp.async_save(state, storage_writer=writer, planner=GefenSavePlanner(),
                              process_group=tr.process_group)
    dcp.save(state, storage_writer=writer, planner=GefenSavePlanner(), process_group=tr.process_group)
    return None


def load_checkpoint(tr, path: str) -> None:
    import torch.distributed.checkpoint as dcp

    wrapper = TrainerDCPState(tr)
    # the optimizer must have state objects to load into: an untrained optimizer publishes zero
    # placeholders of the right geometry, which is all the load needs as destinations
    state = {"trainer": wrapper.state_dict()}
    dcp.load(state, checkpoint_id=path, process_group=tr.process_group)
    wrapper.load_state_dict(state["trainer"])
