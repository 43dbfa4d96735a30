"""Muon for row-sharded matrices over peer memory: gather -> Newton–Schulz -> scatter.

Every hidden matrix has one owner rank (stable index modulo world, the reference's
ownership rule, ``src/gefen/gefen_muon.py:26-32``).  Per step:

1. *gather + reduce*: the owner sums the full matrix out of every peer's unsharded
   gradient staging buffer with peer loads (the reduction of the data-parallel gradient
   and the gather of the sharded matrix are one kernel), overlapped with backward;
2. the owner advances its quantised momentum (``momentum_emit`` kernels) and runs the
   Newton–Schulz chain on the tcgen05 GEMM, writing the bf16 update into its arena;
3. *scatter*: after one flag exchange every rank pulls the rows of each update that its
   parameter shard holds straight from the owner's arena inside the apply kernel
   (``scatter_apply``), so the orthogonalised matrix is never broadcast as a whole.

The reference's ``sharded_mode="distributed"`` does the same work with an all-gather of
every gradient and a full-matrix broadcast per matrix through NCCL
(``src/gefen/gefen_muon.py:1821-1900``).  Momentum state lives on the owner only.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import update as U
from ..ops._ext import ops
from ..optim.muon import GefenMuon, adjust_lr_ratio, stable_distributed_owner
from ..optim.params import is_muon_param


class _ApplySeg(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p), ("u", ctypes.c_void_p), ("alpha", ctypes.c_float),
                ("wd_factor", ctypes.c_float)]


def muon_specs(groups) -> List[Tuple[int, object]]:
    """``(group index, spec)`` of every Muon-routed matrix in stable (registration) order."""
    out = []
    for gi, g in enumerate(groups):
        for sp in g.specs:
            if len(sp.shape) == 2 and is_muon_param(sp.name, torch.empty(0, 0)):
                out.append((gi, sp))
    return out


def owned_bytes(groups, world: int, esz: int) -> int:
    """Largest number of update bytes any rank owns (size of the per-rank update region)."""
    per_rank = [0] * world
    for i, (_gi, sp) in enumerate(muon_specs(groups)):
        per_rank[stable_distributed_owner(i, world)] += (sp.rows * sp.cols * esz + 255) // 256 * 256
    return max(per_rank) if per_rank else 0


class ShardedMuon:
    def __init__(self, trainer, *, lr: float, weight_decay: float, region, region_off: int, **muon_kwargs):
        self.tr = trainer
        tr = trainer
        self.world, self.rank = tr.world, tr.rank
        esz = torch.empty((), dtype=tr.dtype).element_size()
        self.specs = muon_specs(tr.all_groups)
        named, self.keys = [], []
        cursor = [0] * self.world
        self.entries = []                       # per matrix: dict(gi, sp, owner, key, u_off, ...)
        for i, (gi, sp) in enumerate(self.specs):
            g = tr.all_groups[gi]
            owner = stable_distributed_owner(i, self.world)
            rows = sp.shard_rows[self.rank]
            off = sp.shard_off[self.rank]
            key = g.shard_w[off:off + rows * sp.cols].view(rows, sp.cols)
            u_off = cursor[owner]
            cursor[owner] += (sp.rows * sp.cols * esz + 255) // 256 * 256
            self.entries.append(dict(gi=gi, sp=sp, owner=owner, key=key, u_off=u_off))
            named.append((sp.name, key))
        self.region, self.region_off = region, region_off
        self.opt = GefenMuon(named, lr=lr, weight_decay=weight_decay, fused=tr.device.type == "cuda",
                             **muon_kwargs)
        self.opt._external_grad_scale = tr.clip_coef[0:1] if tr.clip else None
        self.owned = [e for e in self.entries if e["owner"] == self.rank]
        for e in self.owned:
            sp = e["sp"]
            e["full_grad"] = torch.zeros(sp.rows, sp.cols, dtype=tr.dtype, device=tr.device)
            e["update"] = self.region[e["u_off"]:e["u_off"] + sp.rows * sp.cols * esz].view(tr.dtype).view(
                sp.rows, sp.cols)
        self.by_group: Dict[int, list] = {}
        for e in self.owned:
            self.by_group.setdefault(e["gi"], []).append(e)
        self._apply_table = None
        self._apply_key = None

    # -- step 1: gather + reduce the owned matrices of one group (reduce stream) ------------
    def reduce_group(self, gi: int) -> None:
        tr = self.tr
        esz = torch.empty((), dtype=tr.dtype).element_size()
        g = tr.all_groups[gi]
        for e in self.by_group.get(gi, ()):
            sp = e["sp"]
            if self.world > 1:
                ptrs = tr.arena.peer_ptrs(g.full_g_off + sp.full_off * esz)
            else:
                ptrs = [g.full_g.data_ptr() + sp.full_off * esz]
            U.reduce_sources(e["full_grad"], ptrs, sp.rows * sp.cols, 1.0 / self.world,
                             tr.norm_partials if tr.clip else None, tr.dtype, tr.device)

    # -- steps 2 and 3 ------------------------------------------------------------------------
    def _build_apply_table(self, lr: float):
        tr = self.tr
        esz = torch.empty((), dtype=tr.dtype).element_size()
        group = self.opt.param_groups[0]
        segs, prefix = [], [0]
        for e in self.entries:
            sp = e["sp"]
            rows = sp.shard_rows[self.rank]
            n = rows * sp.cols
            if n == 0:
                continue
            if n % 8:
                raise ValueError("Muon shard of {} is not a multiple of 8 elements".format(sp.name))
            r0 = min(sp.rows, self.rank * sp.rows_per)
            if self.world > 1:
                base = tr.arena.base_ptrs[e["owner"]] + self.region_off + e["u_off"]
            else:
                base = self.region.data_ptr() + e["u_off"]
            ratio = adjust_lr_ratio(group["adjust_lr_fn"], sp.shape)
            segs.append((e["key"].data_ptr(), base + r0 * sp.cols * esz, lr * ratio,
                         1.0 - lr * group["weight_decay"]))
            prefix.append(prefix[-1] + n // 8)
        arr = (_ApplySeg * len(segs))()
        for i, (p, u, a, w) in enumerate(segs):
            arr[i].p, arr[i].u, arr[i].alpha, arr[i].wd_factor = p, u, a, w
        return (torch.frombuffer(arr, dtype=torch.uint8).clone().to(tr.device), len(segs),
                torch.tensor(prefix, dtype=torch.int64, device=tr.device), prefix[-1])

    @torch.no_grad()
    def step(self, t: int) -> None:
        tr = self.tr
        opt = self.opt
        group = opt.param_groups[0]
        if opt._gefen_codebook is None:
            self._learn_codebook()
        for e in self.owned:
            upd = opt._compute_muon_update(group, e["sp"].name, e["key"], e["full_grad"])
            e["update"].copy_(upd)
        opt._gefen_global_step += 1
        if self.world > 1:
            tr.flags.signal(tr.SLOT_MUON, t)
            tr.flags.wait(tr.SLOT_MUON, t)
        lr = opt._lr_scalar(group)
        key = (lr, group["weight_decay"], group["adjust_lr_fn"])
        if self._apply_key != key:
            self._apply_table = self._build_apply_table(lr)
            self._apply_key = key
        segs, n, prefix, total = self._apply_table
        ops().comm_scatter_apply(segs, n, prefix, total, 296)

    def _learn_codebook(self) -> None:
        """First step: periods and one codebook from the owned full gradients (histogram summed
        over the ranks so that every owner quantises with the same codebook)."""
        from ..quant import codebook as _cbk

        opt = self.opt
        items = []
        for e in self.owned:
            g = e["full_grad"]
            st = opt.state[e["key"]]
            period = opt._resolve_automatic_period(e["sp"].name, e["key"], g)
            st["automatic_period"] = period
            items.append((e["sp"].name, g.reshape(-1), period, g))
        cb = _cbk.learn_codebook_from_grad_periods(
            items, tr_device(self.tr), reduce_counts=self.tr._host_allreduce if self.world > 1 else None)
        if cb is None:        # a rank that owns nothing still needs the shared codebook
            counts = torch.zeros(_cbk.HISTOGRAM_BINS, dtype=torch.int64)
            counts = self.tr._host_allreduce(counts)
            cb = _cbk.exact_dp(_cbk.histogram_stats_from_counts(counts), _cbk.NUM_CODEWORDS).to(
                tr_device(self.tr))
        opt._set_codebook(cb)

    def state_bytes(self) -> int:
        return self.opt.state_bytes()


def tr_device(trainer) -> torch.device:
    return trainer.device
