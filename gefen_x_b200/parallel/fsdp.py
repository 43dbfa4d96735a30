"""Sharded training runtime (ZeRO-3 / FSDP2-style ``Shard(0)``) over peer memory.

One process per GPU.  Every logical parameter is split by rows over the ranks
(the placement torch FSDP2 uses); a rank stores its row slices, the optimizer
state for them, and an unsharded bf16 gradient staging buffer per layer group in
a symmetric arena that every peer maps.  A step is

* forward / backward, layer by layer, on the manual layer functions of
  ``models.decoder``; the weights of the next layer are pulled from the peers'
  shards by a copy kernel on a side stream while the current layer computes
  (all-gather by peer loads, no library collective);
* gradient reduction fused into the optimizer: this rank's slices of every
  peer's staging buffer are summed inside the update kernels
  (``rs_mode="fused"``), or once, overlapped with backward, into a bf16 shard
  stash together with the sum of squares needed for global-norm clipping
  (``rs_mode="stash"``, the default when clipping is on);
* one multi-tensor ``Gefen`` step on the shards, with the column statistics of
  the factored second moment summed across the shards inside the kernel.

The reference has no runtime of its own: its FSDP2 runs use torch's
``fully_shard`` (reference ``src/gefen/tools/find_lr.py:467-474``,
``benchmarks/sharding-sweep/fsdp2_convergence.py:196-201``) and step the local
shards after backward (``src/gefen/gefen.py:3496-3499``).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..models.decoder import (ModelConfig, layer_backward, layer_forward, layer_numel,
                              layer_param_specs, layer_views)
from ..ops import gemm as G
from ..ops import model as M
from ..ops import update as U
from ..ops._ext import DTYPE_CODE, ops
from .symm import FlagBoard, SymmetricArena


@dataclass
class ParamSpec:
    name: str
    shape: Tuple[int, ...]
    full_off: int            # element offset inside the group's unsharded buffer
    rows: int
    cols: int                # elements per row
    rows_per: int            # ceil(rows / world)
    shard_off: List[int]     # per rank: element offset inside that rank's shard buffer
    shard_rows: List[int]    # per rank: rows held


class Group:
    """A set of parameters gathered / reduced together (one decoder layer, or the embeddings)."""

    def __init__(self, name: str, named_shapes: List[Tuple[str, Tuple[int, ...]]], world: int):
        self.name = name
        self.specs: List[ParamSpec] = []
        off = 0
        shard_cursor = [0] * world
        for pname, shape in named_shapes:
            rows = int(shape[0])
            cols = int(math.prod(shape[1:])) if len(shape) > 1 else 1
            rows_per = (rows + world - 1) // world
            s_off, s_rows = [], []
            for r in range(world):
                r0 = min(rows, r * rows_per)
                r1 = min(rows, (r + 1) * rows_per)
                s_off.append(shard_cursor[r])
                s_rows.append(r1 - r0)
                shard_cursor[r] += (r1 - r0) * cols
            self.specs.append(ParamSpec(pname, tuple(shape), off, rows, cols, rows_per, s_off, s_rows))
            off += rows * cols
        self.full_numel = off
        self.shard_numel = shard_cursor          # per rank
        self.max_shard = max(shard_cursor)
        # tensors, filled by the trainer
        self.shard_w: Optional[torch.Tensor] = None
        self.shard_w_off = 0
        self.full_w: Optional[torch.Tensor] = None
        self.full_g: Optional[torch.Tensor] = None
        self.full_g_off = 0
        self.stash_g: Optional[torch.Tensor] = None
        self.gather_tables = None

    def local_slice(self, spec: ParamSpec, rank: int) -> Tuple[int, int]:
        """Element range of ``rank``'s rows of ``spec`` inside the unsharded buffer."""
        r0 = min(spec.rows, rank * spec.rows_per)
        return spec.full_off + r0 * spec.cols, spec.shard_rows[rank] * spec.cols


class _ReduceSeg(ctypes.Structure):
    _fields_ = [("dst", ctypes.c_void_p), ("src", ctypes.c_void_p * 8)]


class _GatherSeg(ctypes.Structure):
    _fields_ = [("src_off", ctypes.c_longlong), ("dst_off", ctypes.c_longlong),
                ("src_rank", ctypes.c_int), ("pad", ctypes.c_int)]


def embed_group_shapes(cfg: ModelConfig) -> List[Tuple[str, Tuple[int, ...]]]:
    shapes = [("model.embed_tokens.weight", (cfg.vocab_size, cfg.hidden)),
              ("model.norm.weight", (cfg.hidden,))]
    if not cfg.tie_embeddings:
        shapes.append(("lm_head.weight", (cfg.vocab_size, cfg.hidden)))
    return shapes


class ShardedTrainer:
    """Train a :class:`~gefen_x_b200.models.decoder.ModelConfig` decoder on ``world`` GPUs.

    ``step(tokens, targets)`` takes host (ideally pinned) or device int64 tensors of
    shape ``[B, S]`` holding this rank's micro-batch, runs forward, backward,
    gradient reduction, clipping and the optimizer step, and returns the mean loss
    of the local batch as a 0-dim device tensor.
    """

    def __init__(self, cfg: ModelConfig, *, device=None, dtype=torch.bfloat16, world: int = 1,
                 rank: int = 0, group=None, lr: float = 6e-6, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, clip_grad_norm: Optional[float] = 1.0,
                 factored_v_2d: bool = True, rs_mode: Optional[str] = None, seed: int = 0,
                 optimizer: str = "gefen", global_codebook: bool = True, gather_ctas: int = 64,
                 wait_iters: int = 8_000_000, opt_kwargs: Optional[dict] = None,
                 ag_gemm: bool = False, ag_fetch_ctas: int = 32, muon_kwargs: Optional[dict] = None,
                 gather_mode: str = "ce", reduce_ctas: int = 148, reduce_mode: str = "ce",
                 sparse_embedding: bool = True, embed_capacity: int = 16384, nvls: Optional[bool] = None,
                 gemm_schedule: str = "auto", copy_lanes: int = 4, context_parallel: int = 1):
        if int(context_parallel) != 1:
            # The hook for splitting a sequence over ranks (ring / blockwise attention): the reference has
            # no sequence parallelism either and every benchmark configuration is 2048 tokens.
            raise NotImplementedError("context_parallel > 1 (sequence parallelism) is not implemented; "
                                      "sequences are processed whole on each rank")
        self.cfg = cfg
        self.copy_lanes = max(1, int(copy_lanes))   # auxiliary streams of the copy-engine transfers
        self.world, self.rank = int(world), int(rank)
        self.device = torch.device(device if device is not None else
                                   ("cuda" if torch.cuda.is_available() else "cpu"))
        self.dtype = dtype
        self.clip = clip_grad_norm
        self.rs_mode = rs_mode or ("stash" if (clip_grad_norm or self.world == 1) else "fused")
        if self.rs_mode not in ("stash", "fused"):
            raise ValueError("rs_mode must be 'stash' or 'fused'")
        self.gather_ctas = gather_ctas
        if gather_mode not in ("ce", "kernel"):
            raise ValueError("gather_mode must be 'ce' (copy engines) or 'kernel' (peer loads)")
        self.gather_mode = gather_mode
        if reduce_mode not in ("ce", "kernel"):
            raise ValueError("reduce_mode must be 'ce' (copy engines + local sum) or 'kernel' (peer loads)")
        self.reduce_mode = reduce_mode
        self._reduce_stage: Optional[torch.Tensor] = None
        self.reduce_ctas = max(1, min(int(reduce_ctas), 2048))
        self._copy_tables: Dict[tuple, torch.Tensor] = {}
        self.ag_gemm = bool(ag_gemm) and int(world) > 1
        self.ag_fetch_ctas = int(ag_fetch_ctas)
        # Untied token embedding on several ranks: only the rows of the batch's tokens are fetched from
        # their owners, and only those rows of the gradient are reduced (``embed_capacity`` = the most
        # tokens a rank may pass to one step); otherwise the table is gathered / reduced densely.
        self.sparse_embed = (bool(sparse_embedding) and int(world) > 1 and not cfg.tie_embeddings
                             and dtype == torch.bfloat16 and cfg.hidden % 8 == 0)
        self.embed_capacity = int(embed_capacity)
        self.step_count = 0           # optimisation steps taken (restored by a checkpoint)
        self._epoch = 0               # steps run by this process: the value the arrival flags count up to
        self.process_group = group
        cuda = self.device.type == "cuda"
        esz = torch.empty((), dtype=dtype).element_size()
        if world > U.MAX_SRC:
            raise ValueError("at most {} ranks per node".format(U.MAX_SRC))

        # ---- layout ------------------------------------------------------
        layer_shapes = [(n, s) for n, (_, s) in layer_param_specs(cfg).items()]
        self.groups: List[Group] = []
        for i in range(cfg.n_layers):
            self.groups.append(Group("layers.{}".format(i),
                                     [("model.layers.{}.{}".format(i, n), s) for n, s in layer_shapes],
                                     world))
        self.embed_group = Group("embed", embed_group_shapes(cfg), world)
        self.all_groups = self.groups + [self.embed_group]
        for g in self.all_groups:
            for sp in g.specs:
                for r in range(world):
                    if (sp.shard_rows[r] * sp.cols * esz) % 16 and world > 1:
                        raise ValueError(
                            "shard of {} on rank {} is not a multiple of 16 bytes; pick a world "
                            "size that divides its rows".format(sp.name, r))

        # ---- arena ---------------------------------------------------------
        n2d = sum(1 for g in self.all_groups for sp in g.specs if len(sp.shape) == 2)
        xchg_floats = sum(2 * (sp.cols + 1) for g in self.all_groups for sp in g.specs
                          if len(sp.shape) == 2)
        n_flag_slots = len(self.all_groups) + 5 + n2d
        arena_bytes = 0
        if world > 1:
            arena_bytes += sum((g.max_shard + g.full_numel) * esz + 2048 for g in self.all_groups)
            arena_bytes += xchg_floats * 4 + n_flag_slots * world * 4 + n2d * 512 + (1 << 20)
            if self.sparse_embed:
                arena_bytes += self.embed_capacity * (cfg.hidden * esz + 8) + 4096
        else:
            arena_bytes = 1 << 12
        self.hybrid = optimizer == "muon_hybrid"
        muon_region_bytes = 0
        if self.hybrid:
            from .muon_sharded import owned_bytes

            muon_region_bytes = owned_bytes(self.all_groups, world, esz)
            arena_bytes += muon_region_bytes + 4096
        self.arena = SymmetricArena(arena_bytes, self.device, world, rank, group)
        # Gradient reduce-scatter through NVSwitch (multimem.ld_reduce on the arena's multicast mapping):
        # a rank then receives its shard's bytes once instead of once per peer.  An option (nvls=True, or
        # GEFENX_NVLS=1 with nvls=None): measured slower than the staged peer copies on 2 GPUs and level
        # with them on 8.  NCCL_NVLS_ENABLE=0 also keeps it off (multi-rank failure tests must run without
        # it: a rank that dies while its memory is bound to a multicast object disturbs the other
        # ranks' GPUs).
        import os

        env_on = os.environ.get("GEFENX_NVLS", "0") == "1" and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"
        want = env_on if nvls is None else bool(nvls)
        self.nvls = bool(want and self.arena.mc_base and dtype == torch.bfloat16 and world > 1)
        if nvls and not self.nvls and world > 1:
            raise RuntimeError("nvls=True, but the symmetric arena has no multicast mapping on this system "
                               "(or the dtype is not bf16)")
        if world > 1 and cuda:
            # with several ranks, kernels of the communication streams (gradient reduce-scatter, copies)
            # share SMs with the products: let the pairs draw tiles dynamically instead of a fixed split
            from ..ops import tcgemm as _tcgemm

            _tcgemm.set_dynamic_schedule(gemm_schedule != "static")
        elif cuda and gemm_schedule == "dynamic":
            from ..ops import tcgemm as _tcgemm

            _tcgemm.set_dynamic_schedule(True)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.flags = FlagBoard(self.arena, n_flag_slots, self.status, wait_iters)
        self.wait_iters = int(wait_iters)
        # flag slots: [0, n_groups) gradients of group ready; then named slots
        self.SLOT_PARAMS = len(self.all_groups)
        self.SLOT_NORM = len(self.all_groups) + 1
        self.SLOT_MUON = len(self.all_groups) + 2
        self.SLOT_HEAD = len(self.all_groups) + 3      # arrival of the head's gradients (early reduction)
        self.SLOT_EMBED = len(self.all_groups) + 4     # token ids + embedding-gradient rows published
        self._muon_region = None
        if self.hybrid:
            self._muon_region, self._muon_region_off = self.arena.alloc(max(muon_region_bytes, 256), torch.uint8)
        self._next_param_slot = len(self.all_groups) + 5

        # ---- buffers -------------------------------------------------------
        for g in self.all_groups:
            if world > 1:
                g.shard_w, g.shard_w_off = self.arena.alloc(g.max_shard, dtype)
                g.full_g, g.full_g_off = self.arena.alloc(g.full_numel, dtype)
                g.stash_g = torch.zeros(g.shard_numel[rank], dtype=dtype, device=self.device) \
                    if self.rs_mode == "stash" else None
            else:
                g.shard_w = torch.empty(g.full_numel, dtype=dtype, device=self.device)
                g.full_w = g.shard_w
                g.full_g = torch.zeros(g.full_numel, dtype=dtype, device=self.device)
        if world > 1:
            n_ring = min(3, cfg.n_layers)
            self.ring = [torch.empty(self.groups[0].full_numel, dtype=dtype, device=self.device)
                         for _ in range(n_ring)]
            self.ring_owner = [-1] * n_ring
            self.embed_group.full_w = torch.empty(self.embed_group.full_numel, dtype=dtype,
                                                  device=self.device)
            self.norm_slot, self.norm_slot_off = self.arena.alloc(2, torch.float32)
            if self.sparse_embed:
                self._tok_ids, self._tok_ids_off = self.arena.alloc(self.embed_capacity, torch.int64)
                self._tok_grad, self._tok_grad_off = self.arena.alloc(self.embed_capacity * cfg.hidden, dtype)
                sp0 = self.embed_group.specs[0]
                assert sp0.name == "model.embed_tokens.weight"
                self._embed_grad = torch.zeros(sp0.shard_rows[rank], cfg.hidden, dtype=dtype, device=self.device)
        self._init_weights(seed)
        if world > 1:
            for g in self.all_groups:
                self._build_gather_tables(g)
            if self.ag_gemm:
                for g in self.groups:
                    self._build_ag_tables(g)
                n = self.groups[0].ag_tables["n_segs"]
                self._ag_flags = [torch.zeros(n, dtype=torch.int32, device=self.device) for _ in self.ring]
                self._ag_count = [torch.zeros(n, dtype=torch.int32, device=self.device) for _ in self.ring]
                self._ag_launches = [0] * len(self.ring)

        # ---- streams -------------------------------------------------------
        if cuda:
            self.comm_stream = torch.cuda.Stream(device=self.device)
            self.reduce_stream = torch.cuda.Stream(device=self.device)
        else:
            self.comm_stream = self.reduce_stream = None
        self._layer_done: Dict[int, torch.cuda.Event] = {}
        self._gather_done: Dict[int, torch.cuda.Event] = {}
        self.norm_partials = torch.zeros(2048, dtype=torch.float32, device=self.device)
        self.norm_local = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.norm_total = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.clip_coef = torch.ones(2, dtype=torch.float32, device=self.device)
        self._rope = None
        self._tok_dev = None
        self._trace: Optional[List[Tuple[str, "torch.cuda.Event"]]] = None

        # ---- optimizer -----------------------------------------------------
        self.muon = None
        self._build_optimizer(optimizer, lr, betas, eps, weight_decay, factored_v_2d,
                              global_codebook, opt_kwargs or {}, muon_kwargs or {})
        if world > 1:
            self.arena.barrier()

    # ------------------------------------------------------------------
    def _init_weights(self, seed: int) -> None:
        """Same full-model random init on every rank (seeded), each rank keeps its rows."""
        cfg = self.cfg
        gen = torch.Generator(device=self.device).manual_seed(int(seed))
        for gi, g in enumerate(self.all_groups):
            full = torch.empty(g.full_numel, dtype=torch.float32, device=self.device)
            for sp in g.specs:
                seg = full[sp.full_off:sp.full_off + sp.rows * sp.cols]
                if sp.name.endswith("norm.weight") or "layernorm" in sp.name:
                    seg.fill_(1.0)
                else:
                    seg.normal_(0.0, cfg.init_std, generator=gen)
            full = full.to(self.dtype)
            if self.world == 1:
                g.shard_w.copy_(full)
            else:
                for sp in g.specs:
                    src_off, n = g.local_slice(sp, self.rank)
                    dst = sp.shard_off[self.rank]
                    g.shard_w[dst:dst + n].copy_(full[src_off:src_off + n])
            del full

    _QKV = ("self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight")

    def _build_ag_tables(self, g: Group) -> None:
        """Tables of the all-gather-fused QKV projection of one layer: the q/k/v row shards in
        arrival order (own rank first, then ring order), where they land in the staging matrix,
        and the order in which the GEMM visits its column blocks."""
        esz = torch.empty((), dtype=self.dtype).element_size()
        H = self.cfg.hidden
        qkv = [sp for sp in g.specs if sp.name.endswith(self._QKV)]
        segs, meta = [], []
        for d in range(self.world):
            r = (self.rank + d) % self.world
            for sp in qkv:
                n = sp.shard_rows[r] * sp.cols
                if n == 0:
                    continue
                dst_off, _ = g.local_slice(sp, r)
                row0 = dst_off // H
                segs.append((g.shard_w_off + sp.shard_off[r] * esz, dst_off * esz, r))
                meta.append((n * esz // 16, row0, sp.shard_rows[r]))
        n_rows = self.cfg.q_dim + 2 * self.cfg.kv_dim
        n_tiles = (n_rows + 255) // 256
        arrival = []
        for t in range(n_tiles):
            lo, hi = t * 256, min(n_rows, (t + 1) * 256)
            last = max(i for i, (_u, r0, nr) in enumerate(meta) if r0 < hi and r0 + nr > lo)
            arrival.append((last, t))
        order = [t for _a, t in sorted(arrival)]
        arr = (_GatherSeg * len(segs))()
        for i, (so, do, r) in enumerate(segs):
            arr[i].src_off, arr[i].dst_off, arr[i].src_rank = so, do, r
        g.ag_tables = dict(
            segs=torch.frombuffer(arr, dtype=torch.uint8).clone().to(self.device), n_segs=len(segs),
            meta=torch.tensor(meta, dtype=torch.int64, device=self.device),
            order=torch.tensor(order, dtype=torch.int32, device=self.device), n_rows=n_rows)

    def _qkv_fn(self, li: int, flat: torch.Tensor):
        """The fused projection of layer ``li``: fetches the q/k/v shards into ``flat`` and
        multiplies as they arrive."""
        g = self.groups[li]
        slot = li % len(self.ring)
        tab = g.ag_tables
        wqkv = flat[:tab["n_rows"] * self.cfg.hidden].view(tab["n_rows"], self.cfg.hidden)

        def fn(h1: torch.Tensor) -> torch.Tensor:
            self._ag_launches[slot] += 1
            k = self._ag_launches[slot]
            out = torch.empty(h1.shape[0], tab["n_rows"], dtype=h1.dtype, device=h1.device)
            ops().gemm_ag_bf16(h1, wqkv, out, self.arena.base_ptrs, tab["segs"], tab["meta"], tab["order"],
                               self._ag_flags[slot], self._ag_count[slot], k, k * self.ag_fetch_ctas,
                               self.ag_fetch_ctas, self.status)
            return out

        return fn

    def _build_gather_tables(self, g: Group) -> None:
        esz = torch.empty((), dtype=self.dtype).element_size()
        if self.ag_gemm and g is not self.embed_group:
            g.gather_tables_rest = self._gather_table_for(
                g, [sp for sp in g.specs if not sp.name.endswith(self._QKV)])
        g.gather_tables = self._gather_table_for(g, g.specs)
        if g is self.embed_group and not self.cfg.tie_embeddings:
            # the untied head (and the final norm) are not needed before the end of forward: their
            # gather is issued behind the first layers', off the critical path of the step start
            late = [sp for sp in g.specs if sp.name in self._LATE_EMBED]
            first = [] if self.sparse_embed else [sp for sp in g.specs if sp not in late]
            g.gather_tables_first = self._gather_table_for(g, first)
            g.gather_tables_late = self._gather_table_for(g, late)

    def _gather_table_for(self, g: Group, specs):
        esz = torch.empty((), dtype=self.dtype).element_size()
        segs, prefix = [], [0]
        for sp in specs:
            for r in range(self.world):
                n = sp.shard_rows[r] * sp.cols
                if n == 0:
                    continue
                dst_off, _ = g.local_slice(sp, r)
                segs.append((g.shard_w_off + sp.shard_off[r] * esz, dst_off * esz, r))
                prefix.append(prefix[-1] + n * esz // 16)
        if not segs:
            return (torch.zeros(1, dtype=torch.uint8, device=self.device), 0,
                    torch.zeros(1, dtype=torch.int64, device=self.device), 0, [])
        arr = (_GatherSeg * len(segs))()
        for i, (so, do, r) in enumerate(segs):
            arr[i].src_off, arr[i].dst_off, arr[i].src_rank = so, do, r
        host = torch.frombuffer(arr, dtype=torch.uint8).clone()
        copies = [(do, r, so, (prefix[i + 1] - prefix[i]) * 16) for i, (so, do, r) in enumerate(segs)]
        return (host.to(self.device), len(segs),
                torch.tensor(prefix, dtype=torch.int64, device=self.device), prefix[-1], copies)

    def _build_reduce_table(self, g: Group, part: str = "all"):
        """Slices of this rank's shard inside every rank's unsharded gradient buffer (one launch
        reduces them all); Muon-routed matrices are reduced by their owners instead.

        ``reduce_mode="kernel"``: the kernel sums the slices with peer loads.  ``"ce"``: the copy
        engines first bring the peers' slices into local staging (no SM is taken from the backward
        GEMMs while the bytes cross NVLink), then the same kernel sums local memory."""
        esz = torch.empty((), dtype=self.dtype).element_size()
        base = self.arena.base_ptrs
        staged = self.reduce_mode == "ce" and not self.nvls
        if staged and self._reduce_stage is None:
            need = 0
            for gg in self.all_groups:
                own = sum(sp.shard_rows[self.rank] * sp.cols for sp in gg.specs
                          if sp.name not in self._muon_names)
                need = max(need, (own * esz + 255) // 256 * 256 + 256 * len(gg.specs))
            self._reduce_stage = torch.empty(max(1, (self.world - 1) * need), dtype=torch.uint8,
                                             device=self.device)
            self._reduce_stage_stride = need
        segs, prefix, copies = [], [0], []
        cursor = 0
        for sp in g.specs:
            n = sp.shard_rows[self.rank] * sp.cols
            if n == 0 or sp.name in self._muon_names:
                continue
            if self.sparse_embed and sp.name == "model.embed_tokens.weight":
                continue                    # reduced row-wise from the peers' token lists instead
            if (part == "early" and sp.name not in self._LATE_EMBED) or \
                    (part == "rest" and sp.name in self._LATE_EMBED):
                continue
            src_off, _ = g.local_slice(sp, self.rank)
            arena_off = g.full_g_off + src_off * esz
            dst = 0
            if self.rs_mode == "stash":
                off = sp.shard_off[self.rank]
                dst = g.stash_g.data_ptr() + off * esz
            srcs = []
            slot = 0
            if self.nvls:
                srcs = [self.arena.mc_ptr(arena_off)] + [0] * (self.world - 1)
            for r in range(self.world if not self.nvls else 0):
                if r == self.rank or not staged:
                    srcs.append(base[r] + arena_off)
                else:
                    sptr = self._reduce_stage.data_ptr() + slot * self._reduce_stage_stride + cursor
                    copies.append((sptr, base[r] + arena_off, n * esz))
                    srcs.append(sptr)
                    slot += 1
            cursor += (n * esz + 255) // 256 * 256
            segs.append((dst, srcs))
            prefix.append(prefix[-1] + n * esz // 16)
        arr = (_ReduceSeg * max(1, len(segs)))()
        for i, (d, srcs) in enumerate(segs):
            arr[i].dst = d
            for r, ptr in enumerate(srcs):
                arr[i].src[r] = ptr
        host = torch.frombuffer(arr, dtype=torch.uint8).clone()
        copy_table = torch.tensor(copies, dtype=torch.int64).reshape(-1, 3) if copies else None
        return (host.to(self.device), len(segs),
                torch.tensor(prefix, dtype=torch.int64, device=self.device), prefix[-1], copy_table)

    # ------------------------------------------------------------------
    # optimizer wiring
    # ------------------------------------------------------------------
    def _build_optimizer(self, kind, lr, betas, eps, weight_decay, factored_v_2d, global_codebook,
                         opt_kwargs, muon_kwargs) -> None:
        from ..optim.gefen import Gefen
        from ..optim.params import is_muon_param

        named = []
        self._param_meta: Dict[torch.Tensor, Tuple[Group, ParamSpec]] = {}
        self._grad_cache: Dict[torch.Tensor, object] = {}
        self._muon_names = set()
        for g in self.all_groups:
            for sp in g.specs:
                if self.hybrid and len(sp.shape) == 2 and is_muon_param(sp.name, torch.empty(0, 0)):
                    self._muon_names.add(sp.name)
                    continue
                rows = sp.shard_rows[self.rank]
                off = sp.shard_off[self.rank]
                view = g.shard_w[off:off + rows * sp.cols]
                view = view.view(rows, *sp.shape[1:]) if len(sp.shape) > 1 else view
                named.append((sp.name, view))
                self._param_meta[view] = (g, sp)
        self.named_shards = named
        if kind not in ("gefen", "muon_hybrid"):
            raise ValueError("ShardedTrainer drives 'gefen' or 'muon_hybrid'; got {!r}".format(kind))
        fused = self.device.type == "cuda"
        if self.hybrid:
            # Muon on the hidden matrices (owner-computed, see parallel.muon_sharded); the Gefen
            # backup (embeddings, head, norms) keeps the block second moment as in the reference
            from .muon_sharded import ShardedMuon

            mk = dict(ns_schedule="tuned3", adjust_lr_fn="match_rms_adamw", normuon=True)
            mk.update(muon_kwargs)
            m_lr = mk.pop("lr", lr)
            m_wd = mk.pop("weight_decay", weight_decay)
            factored_v_2d = False
            self.muon = ShardedMuon(self, lr=m_lr, weight_decay=m_wd, region=self._muon_region,
                                    region_off=self._muon_region_off, **mk)
        self.opt = Gefen(named, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         factored_v_2d=factored_v_2d, fused=fused, **opt_kwargs)
        self.opt._grad_source = self._grad_source
        self._align_wanted = True               # first step, and the first one after a restore
        self.opt._pre_launch_hook = self._align_ranks
        self.opt._external_grad_scale = self.clip_coef[0:1] if self.clip else None
        if self.world > 1:
            self._exchange: Dict[torch.Tensor, U.ShardExchange] = {}
            for view, (g, sp) in self._param_meta.items():
                if len(sp.shape) != 2:
                    continue
                slot, slot_off = self.arena.alloc(2 * (sp.cols + 1), torch.float32)
                flag_slot = self._next_param_slot
                self._next_param_slot += 1
                row = self.flags.row_ptrs(flag_slot)
                self._exchange[view] = U.ShardExchange(
                    total_rows=sp.rows, world=self.world, rank=self.rank,
                    xchg_local=slot.data_ptr(), xchg_peer=self.arena.peer_ptrs(slot_off),
                    flag_local=row[self.rank], flag_peer=row,
                    reduce_cols=self._host_allreduce, reduce_scalar=self._host_allreduce)
            self.opt._shard_info = lambda p: self._exchange.get(p)
            if global_codebook:
                self.opt._histogram_reducer = self._host_allreduce

    def _align_ranks(self, heavy: bool = True) -> None:
        """Host barrier before the kernels of a step whose preparation ran long on the host.

        The first step (period search, codebook learning), a codebook refresh and the first step
        after a restore take seconds of host time that differs between ranks; the kernels that
        follow wait for their peers with a bounded budget, so the ranks are aligned first.  All of
        these happen at the same step on every rank.  A step that merely rebuilds a launch plan
        (``heavy`` false) does not meet here: such a rebuild may concern one rank only, the others
        would never join the barrier, and it is short enough for their bounded waits.
        """
        if self.world > 1 and (heavy or self._align_wanted):
            import torch.distributed as dist

            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.process_group)
        self._align_wanted = False

    def _host_allreduce(self, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist

        if self.world == 1:
            return t
        dev = t.device
        backend = str(dist.get_backend(self.process_group)).lower()
        work = t.to(self.device) if ("nccl" in backend and "gloo" not in backend) else t.cpu()
        dist.all_reduce(work, group=self.process_group)
        return work.to(dev)

    def _grad_source(self, p):
        """Gradient of shard ``p``: a local tensor, or the peers' slices to be summed in-kernel."""
        cached = self._grad_cache.get(p)
        if cached is not None:
            return cached
        meta = self._param_meta.get(p)
        if meta is None:
            return None
        src = self._make_grad_source(p, meta)
        self._grad_cache[p] = src
        return src

    def _make_grad_source(self, p, meta):
        g, sp = meta
        rows = sp.shard_rows[self.rank]
        n = rows * sp.cols
        shape = (rows,) + tuple(sp.shape[1:])
        if self.world == 1:
            return _LocalGrad(g.full_g[sp.full_off:sp.full_off + n].view(shape))
        if self.sparse_embed and sp.name == "model.embed_tokens.weight":
            return _LocalGrad(self._embed_grad.view(shape))
        if self.rs_mode == "stash":
            off = sp.shard_off[self.rank]
            return _LocalGrad(g.stash_g[off:off + n].view(shape))
        esz = p.element_size()
        src_off, _ = g.local_slice(sp, self.rank)
        ptrs = self.arena.peer_ptrs(g.full_g_off + src_off * esz)
        mc = self.arena.mc_ptr(g.full_g_off + src_off * esz) if self.nvls else 0
        return U.PeerGrad(ptrs=ptrs, shape=shape, dtype=p.dtype, device=self.device,
                          scale=1.0 / self.world, mc_ptr=mc)

    # ------------------------------------------------------------------
    # parameter gather (all-gather by peer loads)
    # ------------------------------------------------------------------
    _LATE_EMBED = ("lm_head.weight", "model.norm.weight")

    def _gather_into(self, g: Group, dst: torch.Tensor, rest_only: bool = False, part: str = "all") -> None:
        if part == "first":
            tables = g.gather_tables_first
        elif part == "late":
            tables = g.gather_tables_late
        else:
            tables = g.gather_tables_rest if rest_only else g.gather_tables
        segs, n_segs, prefix, total, copies = tables
        if n_segs == 0:
            return
        if self.gather_mode == "ce":
            key = (id(g), dst.data_ptr(), bool(rest_only), part)
            table = self._copy_tables.get(key)
            if table is None:
                base = self.arena.base_ptrs
                table = torch.tensor([[dst.data_ptr() + do, base[r] + so, nb] for do, r, so, nb in copies],
                                     dtype=torch.int64).reshape(-1, 3)
                self._copy_tables[key] = table
            ops().comm_copy_list(table, self.device.index or 0, self.copy_lanes)
            return
        ops().comm_gather(self.arena.base_ptrs, segs, n_segs, dst, prefix, total, self.gather_ctas)

    def _ensure_layer(self, li: int, rest_only: bool = False) -> torch.Tensor:
        """Make layer ``li``'s unsharded weights available; returns the flat buffer.

        The copy runs on the communication stream; the compute stream waits on
        its event.  A ring slot is reused only after the layer that last
        occupied it has finished computing.
        """
        g = self.groups[li]
        if self.world == 1:
            return g.full_w
        slot = li % len(self.ring)
        if self.ring_owner[slot] != li:
            prev = self.ring_owner[slot]
            with torch.cuda.stream(self.comm_stream):
                if prev >= 0 and prev in self._layer_done:
                    self.comm_stream.wait_event(self._layer_done[prev])
                self._gather_into(g, self.ring[slot], rest_only)
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
                self._gather_done[li] = ev
            self.ring_owner[slot] = li
        return self.ring[slot]

    def _wait_layer(self, li: int) -> None:
        if self.world > 1 and li in self._gather_done:
            torch.cuda.current_stream().wait_event(self._gather_done[li])

    def _mark_layer_done(self, li: int) -> None:
        if self.world > 1:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream())
            self._layer_done[li] = ev

    # ------------------------------------------------------------------
    # gradient reduction (reduce-scatter by peer loads) and the clip norm
    # ------------------------------------------------------------------
    def _reduce_group(self, gi: int, part: str = "all") -> None:
        """Reduce-scatter the gradients of group ``gi``.  ``part`` splits the embedding group:
        ``"early"`` = head and final norm (complete right after the head's backward), ``"rest"`` =
        the token embedding (complete at the very end); each part has its own arrival flags."""
        g = self.all_groups[gi]
        t = self._epoch
        code_dev = self.device
        if self.world == 1:
            if self.hybrid:
                esz = g.full_g.element_size()
                if self.clip:
                    for sp in g.specs:
                        if sp.name not in self._muon_names:
                            U.reduce_sources(None, [g.full_g.data_ptr() + sp.full_off * esz],
                                             sp.rows * sp.cols, 1.0, self.norm_partials, self.dtype, code_dev)
                self.muon.reduce_group(gi)
            elif self.clip and self.device.type != "cuda":
                self.norm_partials[0] += g.full_g.float().square().sum()
            elif self.clip and getattr(self, "_fused_norm", False):
                pass            # already summed by the gradient products' epilogues (see step)
            elif self.clip:
                U.reduce_sources(None, [g.full_g.data_ptr()], g.full_numel, 1.0, self.norm_partials,
                                 self.dtype, code_dev)
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        with torch.cuda.stream(self.reduce_stream):
            self.reduce_stream.wait_event(ev)
            slot = self.SLOT_HEAD if part == "early" else gi
            self.flags.signal(slot, t)
            self.flags.wait(slot, t)
            if self.rs_mode == "stash" or self.clip:
                if not hasattr(g, "reduce_tables"):
                    g.reduce_tables = {}
                if part not in g.reduce_tables:
                    g.reduce_tables[part] = self._build_reduce_table(g, part)
                segs, n_segs, prefix, total, copy_table = g.reduce_tables[part]
                if copy_table is not None:
                    ops().comm_copy_list(copy_table, self.device.index or 0, self.copy_lanes)
                if n_segs:
                    ops().comm_reduce_segments(self.world, segs, n_segs, prefix, total,
                                               1.0 / self.world, self.norm_partials if self.clip else None,
                                               self.reduce_ctas, U.DTYPE_CODE[self.dtype], self.nvls)
            if self.hybrid and part != "early":
                self.muon.reduce_group(gi)

    def _reduce_embedding_rows(self, tok_flat: torch.Tensor, dx2d: torch.Tensor, t: int) -> None:
        """Sparse reduce-scatter of the token-embedding gradient: every rank publishes its token ids
        and gradient rows in its arena; every rank then adds, from all ranks' lists, the rows it
        owns into its (zeroed) gradient shard -- a few megabytes over NVLink instead of the table."""
        n = tok_flat.numel()
        self._tok_ids[:n].copy_(tok_flat)
        self._tok_grad[:n * self.cfg.hidden].copy_(dx2d.reshape(-1))
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        sp0 = self.embed_group.specs[0]
        with torch.cuda.stream(self.reduce_stream):
            self.reduce_stream.wait_event(ev)
            self.flags.signal(self.SLOT_EMBED, t)
            self.flags.wait(self.SLOT_EMBED, t)
            self._embed_grad.zero_()
            ops().comm_scatter_add_rows(self.arena.peer_ptrs(self._tok_ids_off),
                                        self.arena.peer_ptrs(self._tok_grad_off), n,
                                        min(sp0.rows, self.rank * sp0.rows_per), 1.0 / self.world,
                                        self._embed_grad)
            if self.clip and self._embed_grad.numel():
                U.reduce_sources(None, [self._embed_grad.data_ptr()], self._embed_grad.numel(), 1.0,
                                 self.norm_partials, self.dtype, self.device)

    def _finish_norm(self) -> None:
        """Global gradient norm -> clip coefficient on the device (no host sync)."""
        if not self.clip:
            return
        if self.world == 1 and self.device.type != "cuda":
            norm = self.norm_partials.sum().sqrt()
            self.clip_coef[1] = norm
            self.clip_coef[0] = torch.clamp(float(self.clip) / (norm + 1e-6), max=1.0)
            return
        if self.world == 1:
            U.clip_coef(self.norm_partials, float(self.clip), self.clip_coef)
            return
        with torch.cuda.stream(self.reduce_stream):
            torch.sum(self.norm_partials, dim=0, keepdim=True, out=self.norm_local)
            ops().comm_allreduce_scalar(self.arena.peer_ptrs(self.norm_slot_off),
                                        self.flags.row_ptrs(self.SLOT_NORM), self.rank,
                                        self.norm_local, self.norm_total, self._epoch,
                                        self.wait_iters, self.status)
            U.clip_coef(self.norm_total, float(self.clip), self.clip_coef)

    # ------------------------------------------------------------------
    # one training step
    # ------------------------------------------------------------------
    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def _embed_views(self, flat: torch.Tensor) -> Dict[str, torch.Tensor]:
        out = {}
        for sp in self.embed_group.specs:
            out[sp.name] = flat[sp.full_off:sp.full_off + sp.rows * sp.cols].view(sp.shape)
        return out

    # ------------------------------------------------------------------
    # device-side step trace (CUDA events on the compute stream)
    # ------------------------------------------------------------------
    nvtx = False          # set True to emit an NVTX mark at every phase boundary (for timeline tools)

    def _mark(self, name: str) -> None:
        if self.nvtx and self.device.type == "cuda":
            torch.cuda.nvtx.mark("gefen_x:" + name)
        if self._trace is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream())
            self._trace.append((name, ev))

    def traced_step(self, tokens: torch.Tensor, targets: torch.Tensor) -> Tuple[torch.Tensor, Dict[str, float]]:
        """One step with CUDA events at every phase boundary of the compute stream.

        Returns the loss and milliseconds per phase: ``fwd_compute`` / ``bwd_compute`` (inside the
        layers), ``fwd_wait`` / ``bwd_wait`` (compute stream idle until a layer's gathered weights
        arrived), ``embed_wait``, ``head``, ``tail_wait`` (waiting for the last gradient reductions
        and the clip norm), ``optimizer`` and ``total``.  Synchronises the device.
        """
        if self.device.type != "cuda":
            raise RuntimeError("traced_step needs a CUDA device")
        self._trace = []
        try:
            loss = self.step(tokens, targets)
            torch.cuda.synchronize(self.device)
            marks = self._trace
        finally:
            self._trace = None
        out: Dict[str, float] = {k: 0.0 for k in ("embed_wait", "fwd_wait", "fwd_compute", "head", "bwd_wait",
                                                  "bwd_compute", "tail_wait", "optimizer")}
        for (n0, e0), (n1, e1) in zip(marks[:-1], marks[1:]):
            dt = e0.elapsed_time(e1)
            if n1 == "embed_ready":
                out["embed_wait"] += dt
            elif n1.startswith("f.start"):
                out["fwd_wait"] += dt
            elif n1.startswith("f.end"):
                out["fwd_compute"] += dt
            elif n1 == "head.end":
                out["head"] += dt
            elif n1.startswith("b.start"):
                out["bwd_wait"] += dt
            elif n1.startswith("b.end") or n1 == "bwd.end":
                out["bwd_compute"] += dt
            elif n1 == "reduce.done":
                out["tail_wait"] += dt
            elif n1 == "opt.end":
                out["optimizer"] += dt
        out["total"] = marks[0][1].elapsed_time(marks[-1][1])
        return loss, out

    @torch.no_grad()
    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        cfg, L = self.cfg, self.cfg.n_layers
        self.step_count += 1
        self._epoch += 1
        t = self._epoch
        tok = self._to_device(tokens)
        tgt = self._to_device(targets)
        B, S = tok.shape
        T = B * S
        if self._rope is None or self._rope[0] != S:
            self._rope = (S,) + M.rope_tables(S, cfg.head_dim, cfg.rope_theta, self.device)
        cos, sin = self._rope[1], self._rope[2]
        multi = self.world > 1
        eg = self.embed_group
        self._mark("begin")
        if self.clip:
            if multi:
                with torch.cuda.stream(self.reduce_stream):
                    self.norm_partials.zero_()
            else:
                self.norm_partials.zero_()
        split_embed = False
        tok_flat = tok.reshape(-1).contiguous()
        x_rows = torch.empty(T, cfg.hidden, dtype=self.dtype, device=self.device) if self.sparse_embed else None
        if multi:
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                if t > 1:
                    self.flags.wait(self.SLOT_PARAMS, t - 1)
                split_embed = hasattr(eg, "gather_tables_late")
                if self.sparse_embed:
                    if T > self.embed_capacity:
                        raise ValueError("{} tokens per step exceed embed_capacity={}".format(T, self.embed_capacity))
                    sp0 = eg.specs[0]
                    esz = x_rows.element_size()
                    ops().comm_gather_rows(self.arena.peer_ptrs(eg.shard_w_off + sp0.shard_off[self.rank] * esz),
                                           sp0.rows_per, sp0.rows, tok_flat, x_rows)
                else:
                    self._gather_into(eg, eg.full_w, part="first" if split_embed else "all")
                ev = torch.cuda.Event()
                ev.record(self.comm_stream)
            self._ensure_layer(0)
            torch.cuda.current_stream().wait_event(ev)
        head_ready = None
        # single GPU with clipping: the weight-gradient products add their sums of squares to the norm
        # partials in their epilogues, so no extra pass over the gradients is needed afterwards
        fused_norm = bool(self.clip) and not multi and not self.hybrid and self.device.type == "cuda"
        G.set_grad_sumsq(self.norm_partials if fused_norm else None)
        self._fused_norm = fused_norm
        self._mark("embed_ready")
        ew = self._embed_views(eg.full_w)
        egrad = self._embed_views(eg.full_g)
        emb_w = ew["model.embed_tokens.weight"]
        head_w = emb_w if cfg.tie_embeddings else ew["lm_head.weight"]

        # ---- forward ---------------------------------------------------
        if self.sparse_embed:
            x = x_rows.view(B, S, cfg.hidden)
        else:
            x = emb_w.index_select(0, tok_flat).view(B, S, cfg.hidden)
        saved: List[Optional[dict]] = []
        fused = self.ag_gemm
        for li in range(L):
            flat = self._ensure_layer(li, rest_only=fused)
            if li + 1 < L:
                self._ensure_layer(li + 1, rest_only=fused)
            if multi and split_embed and li == min(1, L - 1):
                with torch.cuda.stream(self.comm_stream):      # behind the first layers' gathers
                    self._gather_into(eg, eg.full_w, part="late")
                    head_ready = torch.cuda.Event()
                    head_ready.record(self.comm_stream)
            self._wait_layer(li)
            self._mark("f.start")
            x, sv = layer_forward(cfg, layer_views(cfg, flat), x, cos, sin, save=True,
                                  qkv_fn=self._qkv_fn(li, flat) if fused else None)
            saved.append(sv)
            self._mark("f.end")
            self._mark_layer_done(li)

        # ---- head: final norm, logits, loss, and their backward -----------
        if head_ready is not None:
            torch.cuda.current_stream().wait_event(head_ready)
        x2d = x.reshape(T, cfg.hidden)
        hN, rstdN = M.rmsnorm_fwd(x2d, ew["model.norm.weight"], cfg.rms_eps)
        logits = G.mm_nt(hN, head_w)
        loss_rows = M.xent_fwd_bwd_(logits, tgt, 1.0 / T)
        loss = loss_rows.sum() / T
        dhN = G.mm_nn(logits, head_w)
        head_grad = egrad["model.embed_tokens.weight"] if cfg.tie_embeddings else egrad["lm_head.weight"]
        if cfg.tie_embeddings:
            G.mm_tn(logits, hN, out=head_grad)        # the token gradients are added below: norm taken after
        else:
            G.mm_tn_wgrad(logits, hN, head_grad)
        del logits
        if not cfg.tie_embeddings and not self.sparse_embed:
            egrad["model.embed_tokens.weight"].zero_()
        dx2d, dnorm = M.rmsnorm_bwd(dhN, x2d, ew["model.norm.weight"], rstdN)
        egrad["model.norm.weight"].copy_(dnorm)
        if fused_norm:
            G.add_sumsq(egrad["model.norm.weight"], self.norm_partials)
        dx = dx2d.view(B, S, cfg.hidden)
        if multi and not cfg.tie_embeddings:
            # the head's and the final norm's gradients are complete: reduce them under backward
            self._reduce_group(len(self.all_groups) - 1, part="early")
        self._mark("head.end")

        # ---- backward ----------------------------------------------------
        for li in range(L - 1, -1, -1):
            flat = self._ensure_layer(li)
            if li - 1 >= 0:
                self._ensure_layer(li - 1)
            self._wait_layer(li)
            self._mark("b.start")
            g = self.groups[li]
            dx = layer_backward(cfg, layer_views(cfg, flat), layer_views(cfg, g.full_g), saved[li],
                                dx, cos, sin)
            saved[li] = None
            self._mark("b.end")
            self._mark_layer_done(li)
            self._reduce_group(li)
        if self.sparse_embed:
            self._reduce_embedding_rows(tok_flat, dx.reshape(T, cfg.hidden), t)
        else:
            egrad["model.embed_tokens.weight"].index_add_(0, tok_flat, dx.reshape(T, cfg.hidden))
        if fused_norm:
            G.add_sumsq(egrad["model.embed_tokens.weight"], self.norm_partials)
        G.set_grad_sumsq(None)
        self._mark("bwd.end")
        if not self.sparse_embed:
            self._reduce_group(len(self.all_groups) - 1,
                               part="rest" if (multi and not cfg.tie_embeddings) else "all")
        self._finish_norm()
        if multi:
            torch.cuda.current_stream().wait_stream(self.reduce_stream)
        self._mark("reduce.done")

        # ---- optimizer ---------------------------------------------------
        self.opt._exchange_epoch = t
        self.opt.step()
        if self.muon is not None:
            self.muon.step(t)
        self._mark("opt.end")
        if multi:
            self.flags.signal(self.SLOT_PARAMS, t)
            self.ring_owner = [-1] * len(self.ring)
            self._gather_done.clear()
            self._layer_done.clear()
        return loss

    # ------------------------------------------------------------------
    # checkpoints
    # ------------------------------------------------------------------
    def state_dict(self) -> Dict[str, object]:
        """This rank's part of the run: its weight shards, its optimizer state (native Gefen format)
        and the step count.  Same topology only (the same ``world`` and model); a run restored from it
        continues bit for bit.  For a checkpoint that reloads on another number of ranks use
        :meth:`save_checkpoint` (reference: native format ``src/gefen/gefen.py:4558-4707``)."""
        from ..ckpt import trainer as _ck

        return _ck.native_state_dict(self)

    def load_state_dict(self, state: Dict[str, object]) -> None:
        from ..ckpt import trainer as _ck

        _ck.load_native_state_dict(self, state)

    def save_checkpoint(self, path: str, *, async_save: bool = False):
        """Write a resharding checkpoint with ``torch.distributed.checkpoint``: weight shards as they
        are, optimizer state under the GefenDCPState keys as dense tensors that are expanded one slot
        at a time while writing.  Collective: every rank calls it.  Reloads with
        :meth:`load_checkpoint` on any number of ranks (reference ``src/gefen/dcp.py:1068-1169``)."""
        from ..ckpt import trainer as _ck

        return _ck.save_checkpoint(self, path, async_save=async_save)

    def load_checkpoint(self, path: str) -> None:
        from ..ckpt import trainer as _ck

        _ck.load_checkpoint(self, path)

    def _after_restore(self) -> None:
        """Make restored shards visible to the peers and restart the parameter-arrival protocol."""
        self._grad_cache.clear()
        self._align_wanted = True
        self.opt._fast = None
        if self.opt._plan_cache is not None:
            self.opt._plan_cache.clear()
        if self.world > 1:
            self.ring_owner = [-1] * len(self.ring)
            self._gather_done.clear()
            self._layer_done.clear()
            torch.cuda.synchronize(self.device)
            # the next step waits for "parameters of epoch t - 1 are in place" on every peer
            self.flags.signal(self.SLOT_PARAMS, self._epoch)
            self.arena.barrier()

    def check_status(self) -> None:
        """Raise if any kernel recorded a timed-out peer wait (reads one int from the device)."""
        code = int(self.status.item())
        for dev, c in self.opt.kernel_status().items():
            code = max(code, c)
        broken = self.arena.check_guards()
        if broken:
            raise RuntimeError(
                "gefen_x_b200: {} guard line(s) behind symmetric-arena buffers were overwritten (first "
                "at byte offset {}): a kernel wrote past its buffer".format(len(broken), broken[0]))
        if code != 0:
            raise RuntimeError(
                "gefen_x_b200: a bounded wait on a peer ran out (status {}); a rank is missing "
                "or far behind".format(code))

    def num_params(self) -> int:
        return sum(g.full_numel for g in self.all_groups)

    def state_bytes_per_param(self) -> float:
        """Optimizer-state bytes held by this rank divided by the parameters it owns."""
        own = sum(g.shard_numel[self.rank] for g in self.all_groups)
        total = self.opt.state_bytes() + (self.muon.state_bytes() if self.muon is not None else 0)
        return total / max(1, own)


class _LocalGrad(U.LocalGrad):
    pass
