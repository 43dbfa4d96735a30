"""``Gefen``: AdamW-style optimizer with ~1 byte/parameter of state.

First moment: one ``uint8`` codebook index per element plus one fp32 magnitude
per block of ``automatic_period`` elements.  Second moment: one fp32 value per
block (``vmean``) or, for 2-D parameters with ``factored_v_2d``, Adafactor-style
row/column statistics (``v_row``/``v_col``).  The block period and the
optimizer-wide 256-entry codebook are learned from the first step's gradients
and then frozen.

Public surface, defaults, state keys and the checkpoint schema follow the
reference (``src/gefen/gefen.py``: constructor ``:1074-1092``, param groups
``:1388-1528``, step ``:5709-5839``, native ``state_dict`` ``:4558-4707``, load
``:5456-5705``).  The execution model differs: on CUDA every parameter is
stepped by the sm_100a kernels of ``csrc/update.cu`` which read their
per-step scalars either from launch arguments or, under ``capturable``, from one
stacked device buffer refreshed by a handful of tensor ops per step; CPU tensors
go through ``optim.functional``.  A gradient may also be supplied as a set of
peer slices (``parallel.fsdp``), in which case the same kernels sum the peers'
bf16 slices while they update (reduce-scatter fused into the step).
"""
from __future__ import annotations

import logging
import math
import os
import warnings
from collections import defaultdict
from itertools import chain
from typing import Any, Dict, Iterable, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ..parallel.control import (
    synchronize_step_control_range as _synchronize_step_control_range,
    synchronize_step_failure as _synchronize_step_failure,
)
from ..quant import codebook as _cbk
from ..quant import partitioning as _part
from . import functional as F_

logger = logging.getLogger(__name__)

# Module-level switches (reference gefen.py:86-89).  FIND_PERIOD_BACKEND: None =
# pick from the gradient's device ("cuda_kernel" on CUDA, "cpu" otherwise).
FIND_PERIOD_BACKEND: Optional[str] = None
FUSE_AUTOMATIC_VMEAN_UPDATE = True
FUSE_GEFEN_AUTOMATIC_STEP = True
FUSE_HISTOGRAM_FOR_EXACT = True
# Chunk sizes of the reference's torch statements (``gefen.py:206-285``), kept as names for code that
# reads them; the statements here chunk at ``quant.codebook._SEARCH_CHUNK``.
GEFEN_CODEBOOK_SEARCH_CHUNK = 1 << 23
GEFEN_DEQUANT_GATHER_CHUNK = 1 << 23
GEFEN_EXACT_HISTOGRAM_CHUNK = 1 << 28
GEFEN_MOMENTUM_UPDATE_CHUNK = 1 << 23
GEFEN_NONFUSED_FOREACH_BUDGET = int(os.environ.get("GEFEN_NONFUSED_FOREACH_BUDGET", str(1 << 25)))

_SYNTH_KEY = "param_names_synthesized"
_RANK_LOCAL_PAYLOAD_PREFIX = "_gefen_rank_local_payload_"
_RANK_LOCAL_MEMBER_KEY = "_gefen_rank_local_member"
_RANK_LOCAL_FORMAT = "rank_local_dtensor_v2"
_RANK_LOCAL_METADATA_VERSION = 3
_LOCAL_SNAPSHOT_KEY = "gefen_local_snapshot"
_META_KEY = "_gefen_checkpoint_metadata"
_COUNTER_KEYS = ("step", "vmean_step", "factored_step", "normuon_step")
_SCRATCH_KEYS = ("stepsize", "_h_buf", "_capt_row", "_capt_dev", "_fx_scratch")


# --------------------------------------------------------------------------
# AMP (GradScaler) protocol
# --------------------------------------------------------------------------
def _amp_native_scaling_required(optimizer) -> bool:
    """True when GradScaler must hand ``found_inf``/``grad_scale`` to ``step``.

    Needed only when a parameter or its gradient is stored in fp16 (the unscale
    is then folded into the update kernels in fp32 instead of being applied to
    fp16 gradients in place).  bf16/fp32 training keeps GradScaler's own
    unscale-and-skip path.  Reference: ``gefen.py:1233-1239``.
    """
    for group in optimizer.param_groups:
        for p in group["params"]:
            if p.dtype == torch.float16:
                return True
            g = p.grad
            if g is not None and g.dtype == torch.float16:
                return True
    return False


def _amp_step_controls(optimizer):
    found_inf = getattr(optimizer, "found_inf", None)
    overflow = False
    if found_inf is not None:
        if torch.is_tensor(found_inf):
            if found_inf.numel() != 1:
                raise RuntimeError(
                    "GradScaler supplied a non-scalar found_inf tensor with shape {}".format(
                        tuple(found_inf.shape)))
            overflow = bool(found_inf.detach().item())
        else:
            overflow = bool(found_inf)
    grad_scale = getattr(optimizer, "grad_scale", None)
    if torch.is_tensor(grad_scale):
        if grad_scale.numel() != 1:
            raise RuntimeError(
                "GradScaler supplied a non-scalar grad_scale tensor with shape {}".format(
                    tuple(grad_scale.shape)))
        scale = float(grad_scale.detach().item())
    elif grad_scale is not None:
        scale = float(grad_scale)
    else:
        scale = 0.0
    if grad_scale is not None and (not math.isfinite(scale) or scale <= 0.0):
        raise RuntimeError("GradScaler supplied a non-finite or non-positive grad_scale")
    return overflow, grad_scale, scale


def _optimizer_process_groups(optimizer) -> List[Any]:
    """Process groups of every DTensor mesh dimension the optimizer's params live on."""
    groups, seen = [], set()
    for group in optimizer.param_groups:
        for p in group["params"]:
            mesh = getattr(p, "device_mesh", None)
            if mesh is None:
                continue
            for dim in range(mesh.ndim):
                pg = mesh.get_group(dim)
                if id(pg) not in seen:
                    seen.add(id(pg))
                    groups.append(pg)
    return groups


@torch.no_grad()
def _amp_prepare_optimizer_step(optimizer) -> bool:
    """Honour ``GradScaler``'s ``found_inf`` / ``grad_scale`` attributes.

    Returns False when the step must be skipped (overflow on any rank sharing a
    mesh with this optimizer).  Otherwise stores ``1 / grad_scale`` in
    ``optimizer._pending_grad_scale`` so that the update folds the unscale into
    its fp32 gradient load.  Nothing is mutated before the decision.
    Reference: ``gefen.py:652-707``.
    """
    overflow, grad_scale, scale = _amp_step_controls(optimizer)
    pgs = _optimizer_process_groups(optimizer)
    if pgs:
        lo = (float(overflow), scale)
        hi = (float(overflow), scale)
        for pg in pgs:
            lo, hi = _synchronize_step_control_range(lo, hi, pg)
        overflow = hi[0] > 0
        if lo[1] != hi[1]:
            raise RuntimeError("GradScaler grad_scale differs across ranks: {} vs {}".format(lo[1], hi[1]))
    if overflow:
        return False
    if grad_scale is not None and scale != 1.0:
        optimizer._pending_grad_scale = 1.0 / scale
    return True


def _assert_gradients_structurally_valid(optimizer) -> None:
    """Reject unsupported gradients before anything is mutated (reference ``gefen.py:897``)."""
    for group in optimizer.param_groups:
        for p in group["params"]:
            g = p.grad
            if g is None:
                continue
            if getattr(g, "is_sparse", False):
                raise RuntimeError("Gefen does not support sparse gradients")
            if torch.is_complex(g) or torch.is_complex(p):
                raise RuntimeError("Gefen does not support complex gradients")
            if tuple(g.shape) != tuple(p.shape):
                raise RuntimeError(
                    "gradient shape {} does not match parameter shape {}".format(
                        tuple(g.shape), tuple(p.shape)))
            gl = g.to_local() if hasattr(g, "to_local") else g
            pl = p.to_local() if hasattr(p, "to_local") else p
            if gl.device != pl.device:
                raise RuntimeError(
                    "parameter on {} has its gradient on {}".format(pl.device, gl.device))


def _local(t: torch.Tensor) -> torch.Tensor:
    if hasattr(t, "to_local"):
        t = t.to_local()
    if hasattr(t, "wait"):
        t = t.wait()
    return t


def _ext_available() -> bool:
    from ..ops._ext import available

    return available()



# ---------------------------------------------------------------------------
# Module-level functions under the reference's names (``gefen.py:97-517``): the
# single-tensor statements of the optimizer, usable on any device.
# ---------------------------------------------------------------------------
def automatic_partition_view(flat_tensor: torch.Tensor, period: int) -> torch.Tensor:
    """``[numel / period, period]`` view of a flat tensor."""
    return F_.partition_view(flat_tensor, period)


def automatic_partition_reduce(flat_tensor: torch.Tensor, period: int, reduce_op: str) -> torch.Tensor:
    view = automatic_partition_view(flat_tensor, period)
    if reduce_op == "mean":
        return view.mean(dim=1, keepdim=True)
    if reduce_op == "max":
        return view.max(dim=1, keepdim=True).values
    raise ValueError("Unexpected reduce_op: {}".format(reduce_op))


def automatic_vmean_update(vmean: torch.Tensor, grad_view: torch.Tensor, beta2: float, *, use_fused: bool) -> None:
    """``vmean = beta2 * vmean + (1 - beta2) * mean_block(g^2)`` in place.  ``use_fused`` asks for
    CUDA tensors and squares in fp32 (the rule of the fused kernels and of ``Gefen.step`` here);
    otherwise the reference's non-fused statement runs (``gefen.py:152-196``)."""
    if use_fused:
        if grad_view.device.type != "cuda" or vmean.device.type != "cuda":
            raise ValueError("FUSE_AUTOMATIC_VMEAN_UPDATE requires CUDA grad_view and vmean, got {} and {}".format(
                grad_view.device, vmean.device))
        F_.block_second_moment_(vmean, grad_view, beta2)      # fp32 square, as the fused kernels
        return
    # the reference's non-fused statement: the square stays in the gradient's dtype (fp16 is
    # promoted, its squares overflow), the fp32 running mean absorbs the increment
    g = grad_view.float() if grad_view.dtype == torch.float16 else grad_view
    vmean.mul_(beta2).add_(torch.mean(g * g, dim=1, keepdim=True), alpha=1 - beta2)


def gefen_nearest_codebook_indices(codebook: torch.Tensor, normalized_vals: torch.Tensor) -> torch.Tensor:
    if codebook.device != normalized_vals.device:
        raise ValueError("Gefen codebook device {} does not match normalized_vals device {}.".format(
            codebook.device, normalized_vals.device))
    return _cbk.nearest_codebook_indices(codebook, normalized_vals)


def gefen_dequantize_unpacked_indices(codebook: torch.Tensor, stored_indices: torch.Tensor,
                                      like_tensor: torch.Tensor) -> torch.Tensor:
    return _cbk.dequantize_indices(codebook, stored_indices, like_tensor.dtype).to(like_tensor.device)


def gefen_set_unpacked_indices(stored_indices: torch.Tensor, indices: torch.Tensor) -> None:
    stored_indices.copy_(indices.to(torch.uint8))


def gefen_automatic_fused_update(*, p: torch.Tensor, grad_view: torch.Tensor, m_codebook: torch.Tensor,
                                 m_magnitude: torch.Tensor, stepsize: torch.Tensor, codebook: torch.Tensor,
                                 packed_indices: bool, beta1: float, lr: float) -> None:
    """One tensor's momentum EMA + requantisation + parameter update for a given ``stepsize``
    (``[blocks, 1]`` or broadcastable to ``[blocks, period]``).  CUDA tensors only, as in the
    reference (``gefen.py:382-415``); whole steps go through the multi-tensor kernels instead."""
    if grad_view.device.type != "cuda":
        raise ValueError("Fused automatic Gefen update requires CUDA tensors.")
    if codebook.device != grad_view.device:
        raise ValueError("Gefen codebook device {} does not match grad_view device {}.".format(
            codebook.device, grad_view.device))
    if packed_indices:
        raise ValueError("packed (sub-byte) indices are not supported: indices are one byte per element")
    q = F_.momentum_requantize_(codebook, m_codebook, m_magnitude, grad_view, beta1)
    F_.apply_update_(p, q, stepsize, lr, 1.0)


def learn_gefen_exact_codebook_from_grad_periods(*, grad_periods, codebook_device, num_codebooks: int,
                                                 force_endpoints: bool, verbose: bool,
                                                 compute_mse_logging: bool = True,
                                                 use_fused_histogram: Optional[bool] = None):
    """Exact 1-D k-means codebook over the histogram of ``(name, flat_grad, period, grad)`` items."""
    return _cbk.learn_codebook_from_grad_periods(grad_periods, codebook_device=codebook_device,
                                                 num_codebooks=num_codebooks, force_endpoints=force_endpoints,
                                                 verbose=bool(verbose and compute_mse_logging))


class Gefen(torch.optim.Optimizer):
    """Memory-efficient AdamW replacement (quantised momentum, shared/factored v).

    Arguments mirror ``torch.optim.AdamW`` plus:

    * ``fused`` – use the sm_100a kernels for CUDA tensors (default).  CPU
      tensors always use the decomposed torch path.
    * ``force_1d_period_one`` / ``force_2d_period_one`` / ``period_one_substrings``
      – force per-element state (period 1) for the matching parameters.
    * ``factored_v_2d`` – factored second moment for plain 2-D parameters.
    * ``codebook_refresh_every`` – re-learn the codebook every N steps and
      re-quantise the stored momentum onto it.
    * ``stochastic_round`` – stochastic codeword rounding (kernels only).
    * ``deterministic`` – fixed-order reductions only (replica-exact).
    * ``capturable`` – device-resident step counters/scalars so that ``step``
      can be captured in a CUDA graph after an eager first step.

    ``params`` may hold tensors, ``(name, tensor)`` pairs or group dicts.
    """

    def __init__(
        self,
        params: Iterable[Union[nn.Parameter, Tuple[str, nn.Parameter], Dict[str, Any]]],
        lr: Union[float, torch.Tensor] = 1e-3,
        betas: Tuple[float, float] = (0.9, 0.999),
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        *,
        fused: bool = True,
        force_1d_period_one: bool = False,
        force_2d_period_one: bool = False,
        period_one_substrings: Tuple[str, ...] = (),
        factored_v_2d: bool = True,
        codebook_refresh_every: int = 0,
        stochastic_round: bool = False,
        deterministic: bool = False,
        capturable: bool = False,
        verbose: bool = False,
    ):
        if not isinstance(deterministic, bool):
            raise TypeError("deterministic must be a bool")
        if deterministic and factored_v_2d and stochastic_round:
            raise ValueError(
                "deterministic=True with factored_v_2d=True cannot honor stochastic_round=True: "
                "the replica-exact factored path uses deterministic nearest-codeword "
                "quantization. Disable stochastic rounding or factored_v_2d.")
        if fused and not torch.cuda.is_available():
            warnings.warn(
                "Gefen optimizer got fused=True, but CUDA is not available. "
                "Changing fused to False.", UserWarning, stacklevel=2)
            fused = False
        if codebook_refresh_every < 0:
            raise ValueError(
                "codebook_refresh_every must be >= 0 but is: {}".format(codebook_refresh_every))
        if capturable and codebook_refresh_every:
            raise ValueError(
                "capturable=True is incompatible with codebook_refresh_every>0: the periodic "
                "codebook re-learn is host-driven and cannot run inside a replayed CUDA graph.")
        self._validate_group_options(lr, betas, eps, weight_decay)
        logger.info("Initializing Gefen optimizer (fused=%s).", fused)

        self.fused = fused
        self._fused_build_ok: Optional[bool] = None
        self._force_1d_period_one = force_1d_period_one
        self._force_2d_period_one = force_2d_period_one
        self._period_one_substrings = tuple(s.lower() for s in period_one_substrings)
        self._factored_v_2d = factored_v_2d
        self._deterministic = deterministic
        self._codebook_refresh_every = codebook_refresh_every
        self.capturable = capturable
        self._stochastic_round = stochastic_round
        if stochastic_round and not fused:
            warnings.warn(
                "stochastic_round=True is honored only by the fused CUDA kernels; the "
                "non-fused / CPU path uses deterministic nearest rounding, so the flag is "
                "a no-op here.", RuntimeWarning, stacklevel=2)
        self.verbose = verbose

        self._gefen_codebook: Optional[torch.Tensor] = None
        self._gefen_codebook_by_device: Dict[torch.device, torch.Tensor] = {}
        self._gefen_codebook_lut_by_device: Dict[torch.device, torch.Tensor] = {}
        self._gefen_thresholds_by_device: Dict[torch.device, torch.Tensor] = {}
        self._gefen_global_step = 0
        self._gefen_global_step_by_device: Dict[torch.device, torch.Tensor] = {}
        self._capt: Dict[torch.device, Dict[str, Any]] = {}
        self._pending_grad_scale: Optional[float] = None
        # Optional hooks installed by the sharded runtime (parallel.fsdp):
        #   _grad_source(p) -> object describing peer gradient slices, or None
        #   _shard_info(p)  -> (total_rows, exchange) for Shard(0) factored params
        self._grad_source = None
        self._shard_info = None
        self._histogram_reducer = None
        self._external_grad_scale: Optional[torch.Tensor] = None
        self._exchange_epoch = 0
        # called as hook(heavy) before the kernels of a step that went through the full host path;
        # heavy: this step searched periods or learned / refreshed the codebook (seconds of host work,
        # at the same step on every rank), as opposed to merely rebuilding a launch plan
        self._pre_launch_hook = None
        self._heavy_prep = False
        self._fast = None
        self._fused_meta: Dict[Any, list] = {}
        self._slow_params = 0
        self._plan_cache = None
        self._fused_items: Dict[Any, list] = {}
        self._fused_copyback: list = []
        self._status_by_device: Dict[torch.device, torch.Tensor] = {}

        self._param_names: Dict[torch.Tensor, str] = {}
        self._synthesized_param_names: Dict[torch.Tensor, bool] = {}
        defaults = dict(lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay)
        super().__init__(self._normalize_param_groups(params), defaults)

    # ------------------------------------------------------------------
    # construction helpers
    # ------------------------------------------------------------------
    @staticmethod
    def _normalize_param_groups(params):
        groups = [params] if isinstance(params, torch.Tensor) else list(params)
        if len(groups) == 0:
            raise ValueError("optimizer got an empty parameter list")
        if isinstance(groups[0], dict):
            return groups
        return [{"params": groups, "_gefen_implicit_group": True}]

    @staticmethod
    def _validate_group_options(lr, betas, eps, weight_decay):
        if torch.is_tensor(lr) and lr.numel() != 1:
            raise ValueError("lr as a Tensor must be 1-element, got numel={}".format(lr.numel()))
        if not 0.0 <= lr:
            raise ValueError("Invalid learning rate: {}".format(lr))
        if not math.isfinite(eps) or eps <= 0.0:
            raise ValueError("Invalid epsilon value (eps must be finite and > 0): {}".format(eps))
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError("Invalid beta parameter at index 0: {}".format(betas[0]))
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError("Invalid beta parameter at index 1: {}".format(betas[1]))
        if not 0.0 <= weight_decay:
            raise ValueError("Invalid weight_decay value: {}".format(weight_decay))

    @staticmethod
    def _iter_params_with_names(params):
        if isinstance(params, torch.Tensor):
            params = [params]
        for item in params:
            if isinstance(item, torch.Tensor):
                name, p = None, item
            elif isinstance(item, (tuple, list)) and len(item) == 2 and isinstance(item[1], torch.Tensor):
                name, p = item
            else:
                raise TypeError(
                    "Gefen parameters must be tensors or (name, tensor) pairs, got {!r}".format(
                        type(item)))
            if torch.is_complex(p):
                raise ValueError("Gefen does not support complex parameters")
            yield name, p

    @staticmethod
    def _unique_name(base: str, taken) -> str:
        if base not in taken:
            return base
        i = 1
        while "{}_{}".format(base, i) in taken:
            i += 1
        return "{}_{}".format(base, i)

    def add_param_group(self, param_group):
        """Register a group; all-or-nothing (reference ``gefen.py:1388-1528``)."""
        if not isinstance(param_group, dict):
            raise TypeError("param_group must be a dict, got {}".format(type(param_group).__name__))
        if "params" not in param_group:
            raise ValueError("Gefen parameter group is missing the 'params' key.")
        d = self.defaults
        lr = param_group.get("lr", d["lr"])
        if "betas" in param_group:
            betas = param_group["betas"]
        else:
            betas = (param_group.get("beta1", d["beta1"]), param_group.get("beta2", d["beta2"]))
        eps = param_group.get("eps", d["eps"])
        wd = param_group.get("weight_decay", d["weight_decay"])
        self._validate_group_options(lr, betas, eps, wd)
        named = list(self._iter_params_with_names(param_group["params"]))
        if not named:
            raise ValueError("optimizer got an empty parameter list")
        consumed = ("params", "name", "lr", "betas", "beta1", "beta2", "eps", "weight_decay",
                    "param_names", _SYNTH_KEY, "_gefen_implicit_group")
        extra = {k: v for k, v in param_group.items() if k not in consumed}
        taken = set(self._param_names.values())
        existing = set()
        for g in self.param_groups:
            existing.update(g["params"])
        gi = len(self.param_groups)
        gname = param_group.get("name")
        implicit = bool(param_group.get("_gefen_implicit_group", False))
        params, names, synth = [], [], []
        batch = set()
        for i, (name, p) in enumerate(named):
            if p in existing or p in batch:
                raise ValueError("some parameters appear in more than one parameter group")
            batch.add(p)
            s = False
            if name is None:
                if gname is not None and len(named) == 1:
                    base = str(gname).lower()
                    name = self._unique_name(base, taken)
                    s = name != base
                elif implicit:
                    name = self._unique_name("param_{}".format(len(self._param_names) + i), taken)
                    s = True
                else:
                    name = self._unique_name("group_{}_param_{}".format(gi, i), taken)
                    s = True
            else:
                name = str(name).lower()
            params.append(p)
            names.append(name)
            synth.append(s)
            taken.add(name)
        group = dict(extra)
        if gname is not None:
            group["name"] = str(gname).lower()
        elif len(names) == 1:
            group["name"] = names[0]
        group.update({"params": params, "param_names": names, _SYNTH_KEY: synth, "lr": lr,
                      "beta1": betas[0], "beta2": betas[1], "eps": eps, "weight_decay": wd})
        super().add_param_group(group)
        for p, n, s in zip(params, names, synth):
            self._param_names[p] = n
            self._synthesized_param_names[p] = s
            self.state[p]["name"] = n
        self._capt.clear()
        self._fast = None

    def _param_name(self, p) -> str:
        n = self._param_names.get(p)
        if n is None:
            st = self.state.get(p)
            n = st.get("name") if st else None
        if n is None:
            n = self._unique_name("param_{}".format(len(self._param_names)), set(self._param_names.values()))
            self._param_names[p] = n
            self._synthesized_param_names[p] = True
        return n

    def _param_name_is_synthesized(self, p) -> bool:
        return bool(self._synthesized_param_names.get(p, True))

    def _iter_group_params_with_names(self, group):
        for p in group["params"]:
            yield self._param_name(p), p

    # ------------------------------------------------------------------
    # codebook, period
    # ------------------------------------------------------------------
    @property
    def _step_supports_amp_scaling(self) -> bool:
        return _amp_native_scaling_required(self)

    def _fused_for(self, t: torch.Tensor) -> bool:
        """Whether tensor ``t`` is stepped by the CUDA kernels."""
        if not (self.fused and FUSE_GEFEN_AUTOMATIC_STEP):
            return False
        if not t.is_cuda or t.dtype == torch.float64:
            return False
        if self._deterministic and self._factored_v_2d and t.dim() == 2:
            # the two-phase kernels sum row / column statistics with atomics (order not fixed);
            # the replica-exact policy takes the fixed-order torch statement for those tensors
            return False
        if self._fused_build_ok is None:
            from ..ops import update as _u

            # On a CUDA device the extension is mandatory: raise rather than
            # silently running the slow torch path.
            self._fused_build_ok = _u.available(required=True)
        return bool(self._fused_build_ok)

    def _gefen_codebook_device(self) -> torch.device:
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is not None:
                    return _local(p.grad).device
        for group in self.param_groups:
            for p in group["params"]:
                return _local(p).device
        return torch.device("cpu")

    def _gefen_codebook_on(self, device) -> Optional[torch.Tensor]:
        if self._gefen_codebook is None:
            return None
        device = torch.device(device)
        cb = self._gefen_codebook_by_device.get(device)
        if cb is None:
            cb = self._gefen_codebook.to(device=device, dtype=torch.float32).contiguous()
            self._gefen_codebook_by_device[device] = cb
        return cb

    def _gefen_codebook_lut_on(self, device) -> torch.Tensor:
        device = torch.device(device)
        lut = self._gefen_codebook_lut_by_device.get(device)
        if lut is None:
            lut = _cbk.packed_search_lut(self._gefen_codebook_on(device))
            self._gefen_codebook_lut_by_device[device] = lut
        return lut

    def _gefen_thresholds_on(self, device) -> torch.Tensor:
        device = torch.device(device)
        thr = self._gefen_thresholds_by_device.get(device)
        if thr is None:
            thr = _cbk.padded_thresholds(self._gefen_codebook_on(device))
            self._gefen_thresholds_by_device[device] = thr
        return thr

    def _set_codebook(self, cb: Optional[torch.Tensor]) -> None:
        self._gefen_codebook = cb
        self._gefen_codebook_by_device.clear()
        self._gefen_codebook_lut_by_device.clear()
        self._gefen_thresholds_by_device.clear()

    def _resolve_automatic_period(self, name: str, p: torch.Tensor, grad: torch.Tensor) -> int:
        if self._force_1d_period_one and p.ndim == 1:
            return 1
        if self._force_2d_period_one and p.ndim == 2:
            return 1
        if self._period_one_substrings:
            lname = str(name).lower()
            if any(s in lname for s in self._period_one_substrings):
                return 1
        return self._predict_period_from_grad_sq(name, p, grad)

    def _predict_period_from_grad_sq(self, name: str, p: torch.Tensor, grad: torch.Tensor) -> int:
        self._heavy_prep = True
        g = _local(grad).detach()
        backend = FIND_PERIOD_BACKEND
        if backend is None:
            backend = "cuda_kernel" if g.is_cuda else "cpu"
        if backend == "cuda_kernel" and not self._fused_for(g):
            backend = "gpu" if g.is_cuda else "cpu"
        shape = tuple(_local(p).shape)
        if backend == "cuda_kernel":
            return _part.find_period_by_block_variance(
                g.reshape(-1), print_results=False, parameter_name=name, parameter_shape=shape,
                backend=backend, input_is_squared=False)
        if backend == "cpu":
            vals = g.float().square().reshape(-1).cpu()
        elif backend == "gpu":
            if not g.is_cuda:
                raise ValueError("FIND_PERIOD_BACKEND='gpu' requires a CUDA tensor")
            vals = g.float().square().reshape(-1)
        else:
            raise ValueError("Unexpected FIND_PERIOD_BACKEND: {}".format(backend))
        return _part.find_period_by_block_variance(
            vals, print_results=False, parameter_name=name, parameter_shape=shape,
            backend=backend, input_is_squared=True)

    def _grad_of(self, p) -> Optional[torch.Tensor]:
        """Local gradient tensor used for period/codebook learning."""
        if self._grad_source is not None:
            src = self._grad_source(p)
            if src is not None:
                return src.materialize()
        g = p.grad
        return None if g is None else _local(g).detach()

    def _iter_gefen_grad_periods(self, reuse_existing_periods: bool = False):
        for group in self.param_groups:
            for name, p in self._iter_group_params_with_names(group):
                grad = self._grad_of(p)
                if grad is None:
                    continue
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
                if flat.numel() % period:
                    raise ValueError(
                        "Automatic partition period {} does not divide parameter {} with numel {} "
                        "while learning Gefen codebook".format(period, name, flat.numel()))
                yield name, flat, period, grad

    def _learn_gefen_exact_codebook(self, reuse_existing_periods: bool = False,
                                    compute_mse_logging: bool = True) -> Optional[torch.Tensor]:
        self._heavy_prep = True
        return _cbk.learn_codebook_from_grad_periods(
            self._iter_gefen_grad_periods(reuse_existing_periods),
            codebook_device=self._gefen_codebook_device(),
            num_codebooks=_cbk.NUM_CODEWORDS,
            force_endpoints=True,
            verbose=self.verbose and compute_mse_logging,
            reduce_counts=self._histogram_reducer,
        )

    def _resuming_from_checkpoint(self) -> bool:
        return any("automatic_period" in self.state.get(p, {})
                   for g in self.param_groups for p in g["params"])

    def _maybe_refresh_gefen_codebook(self) -> None:
        if self._gefen_codebook is not None:
            dev = self._gefen_codebook_device()
            if self._gefen_codebook.device != dev:
                self._set_codebook(self._gefen_codebook.to(dev))
            return
        cb = self._learn_gefen_exact_codebook(reuse_existing_periods=self._resuming_from_checkpoint())
        if cb is not None:
            self._set_codebook(cb)

    def _maybe_save_gefen_grad_histogram(self) -> None:
        """Dump the histogram of the block-normalised gradients at the optimizer steps listed in
        ``quant.codebook.LIST_STEPS_SAVE_HIST_GRAD`` (off unless set; reference
        ``gefen.py:3095-3155``).  CUDA gradients are binned by the histogram kernel."""
        steps = getattr(_cbk, "LIST_STEPS_SAVE_HIST_GRAD", None)
        if steps is None:
            return
        if self.capturable and steps:
            raise ValueError("capturable=True is incompatible with LIST_STEPS_SAVE_HIST_GRAD: histogram "
                             "collection and file output are host-driven")
        if self._gefen_global_step not in steps:
            return
        prefix = getattr(_cbk, "SAVE_CODEBOOK_PREFIX", None)
        if prefix is None:
            raise ValueError("LIST_STEPS_SAVE_HIST_GRAD requires SAVE_CODEBOOK_PREFIX to be set.")
        if self._gefen_codebook is None:
            raise ValueError("Expected Gefen codebook to be initialized before saving gradient histogram.")
        bins = self._gefen_codebook.numel() * 16
        counts = torch.zeros(bins, dtype=torch.float32)
        total = 0
        for _, flat, period, _ in self._iter_gefen_grad_periods(reuse_existing_periods=True):
            counts.add_(_cbk.block_normalised_histogram(flat, period, bins).cpu().float())
            total += flat.numel()
        if total == 0:
            raise ValueError("Cannot save Gefen gradient histogram because no gradients were available.")
        _cbk.save_distribution_histogram_pt_from_counts(
            hist=counts, prefix=prefix, suffix="grad_hist_step_{}".format(self._gefen_global_step),
            num_samples=total)

    def _refresh_codebook_with_requant(self) -> None:
        """Re-learn the codebook and move every stored index onto it (atomic).

        Reference ``gefen.py:3020-3061``: indices are dequantised with the
        codebook that wrote them, re-searched in the new one and committed only
        after every parameter has been staged.
        """
        old = self._gefen_codebook
        if old is None:
            return
        new = self._learn_gefen_exact_codebook(reuse_existing_periods=True, compute_mse_logging=False)
        if new is None:
            return
        staged = []
        for group in self.param_groups:
            for p in group["params"]:
                st = self.state.get(p)
                if not st or "m_codebook" not in st:
                    continue
                dev = st["m_codebook"].device
                if dev.type == "cuda" and st["m_codebook"].is_contiguous() and _ext_available():
                    staged.append((st["m_codebook"], None))        # remapped in place below (no temporaries)
                    continue
                coeffs = _cbk.dequantize_indices(old.to(dev), st["m_codebook"], torch.float32)
                staged.append((st["m_codebook"], _cbk.nearest_codebook_indices(new.to(dev), coeffs)))
        # the new index of a stored value depends only on its old index: one 256-entry table
        index_map = _cbk.nearest_codebook_indices(new.cpu(), old.cpu().float()).to(torch.uint8)
        for dst, idx in staged:
            if idx is None:
                from ..ops import quant as _q

                _q.remap_indices_(dst, index_map)
            else:
                dst.copy_(idx)
        self._set_codebook(new)

    # ------------------------------------------------------------------
    # counters / capturable scalars
    # ------------------------------------------------------------------
    def _new_step_counter(self, device):
        if self.capturable:
            return torch.zeros((), dtype=torch.float32, device=device)
        return 0

    def _lr_scalar(self, group) -> float:
        """The group's learning rate as a Python float.  A tensor learning rate is read back (a
        device-to-host synchronisation for a CUDA tensor) once per value, not once per parameter: the
        read is cached on the tensor's identity and version counter, which every in-place update of
        a scheduler bumps (reference ``gefen_muon.py`` ``_lr_scalar`` / ``_lr_scalar_cache``)."""
        lr = group["lr"]
        if not torch.is_tensor(lr):
            return float(lr)
        cache = self.__dict__.setdefault("_lr_scalar_cache", {})
        hit = cache.get(id(group))
        if hit is not None and hit[0] is lr and hit[1] == lr._version:
            return hit[2]
        val = float(lr.item())
        cache[id(group)] = (lr, lr._version, val)        # holding the tensor keeps its identity unique
        return val

    @staticmethod
    def _colocate_param_state_(state, device) -> None:
        """Move state tensors stranded on another device (CPU-offload paging)."""
        for k, v in list(state.items()):
            if torch.is_tensor(v) and v.device != device:
                state[k] = v.to(device)

    def _capt_registry(self, device) -> Dict[str, Any]:
        """Stacked device buffers holding every parameter's counters and kernel scalars.

        ``steps[0, i]`` is the second-moment counter (``vmean_step`` or
        ``factored_step``), ``steps[1, i]`` the momentum counter; ``scal[i]`` is
        ``[lr, 1/sqrt(bc2) | 1/bc2, 1/bc1, 1 - lr*wd]``.  The per-parameter
        state entries are views into ``steps`` so that one vectorised refresh
        serves all parameters (reference ``gefen.py:2095-2204``, ``:2440-2465``).
        """
        reg = self._capt.get(device)
        if reg is not None:
            return reg
        entries = []
        for gi, group in enumerate(self.param_groups):
            for p in group["params"]:
                st = self.state.get(p)
                if not st or "step" not in st:
                    continue
                if _local(p).device != device:
                    continue
                entries.append((gi, p, st))
        n = len(entries)
        steps = torch.zeros(2, max(n, 1), dtype=torch.float32, device=device)
        scal = torch.zeros(max(n, 1), 4, dtype=torch.float32, device=device)
        kind = torch.zeros(max(n, 1), dtype=torch.bool, device=device)
        b1 = torch.zeros(max(n, 1), dtype=torch.float32, device=device)
        b2 = torch.zeros(max(n, 1), dtype=torch.float32, device=device)
        wd = torch.zeros(max(n, 1), dtype=torch.float32, device=device)
        gidx = torch.zeros(max(n, 1), dtype=torch.long, device=device)
        rows = {}
        h_kind, h_b1, h_b2, h_wd, h_g, h_s0, h_s1 = [], [], [], [], [], [], []
        for i, (gi, p, st) in enumerate(entries):
            group = self.param_groups[gi]
            vkey = "factored_step" if "v_row" in st else "vmean_step"
            h_kind.append("v_row" in st)
            h_b1.append(group["beta1"])
            h_b2.append(group["beta2"])
            h_wd.append(group["weight_decay"])
            h_g.append(gi)
            h_s0.append(float(st.get(vkey, st["step"])))
            h_s1.append(float(st["step"]))
            rows[p] = i
        if n:
            kind[:n] = torch.tensor(h_kind, device=device)
            b1[:n] = torch.tensor(h_b1, dtype=torch.float32, device=device)
            b2[:n] = torch.tensor(h_b2, dtype=torch.float32, device=device)
            wd[:n] = torch.tensor(h_wd, dtype=torch.float32, device=device)
            gidx[:n] = torch.tensor(h_g, device=device)
            steps[0, :n] = torch.tensor(h_s0, dtype=torch.float32, device=device)
            steps[1, :n] = torch.tensor(h_s1, dtype=torch.float32, device=device)
        for i, (gi, p, st) in enumerate(entries):
            vkey = "factored_step" if "v_row" in st else "vmean_step"
            st[vkey] = steps[0, i]
            st["step"] = steps[1, i]
            st["_capt_row"] = i
            st["_capt_dev"] = device
        reg = dict(steps=steps, scal=scal, kind=kind, b1=b1, b2=b2, wd=wd, gidx=gidx, rows=rows,
                   n=n, active=None, active_key=None,
                   lr_buf=torch.zeros(len(self.param_groups), dtype=torch.float32, device=device))
        self._capt[device] = reg
        return reg

    def _capt_refresh(self, device, active_params) -> None:
        """Advance the counters of the stepping parameters and recompute all scalar rows."""
        reg = self._capt_registry(device)
        if reg["n"] == 0:
            return
        key = tuple(id(p) for p in active_params)
        if reg["active_key"] != key:
            mask = torch.zeros(reg["steps"].shape[1], dtype=torch.float32)
            for p in active_params:
                r = reg["rows"].get(p)
                if r is not None:
                    mask[r] = 1.0
            reg["active"] = mask.to(device)
            reg["active_key"] = key
        for gi, group in enumerate(self.param_groups):
            lr = group["lr"]
            if torch.is_tensor(lr):
                reg["lr_buf"][gi].copy_(lr.reshape(()), non_blocking=True)
            else:
                reg["lr_buf"][gi].fill_(float(lr))
        steps, scal = reg["steps"], reg["scal"]
        steps.add_(reg["active"])
        lr = reg["lr_buf"].index_select(0, reg["gidx"])
        bc1 = 1.0 - torch.pow(reg["b1"], steps[1].clamp(min=1.0))
        bc2 = 1.0 - torch.pow(reg["b2"], steps[0].clamp(min=1.0))
        scal[:, 0] = lr
        scal[:, 1] = torch.where(reg["kind"], 1.0 / bc2, 1.0 / bc2.sqrt())
        scal[:, 2] = 1.0 / bc1
        scal[:, 3] = 1.0 - lr * reg["wd"]

    def _ensure_global_step_device(self, device) -> torch.Tensor:
        t = self._gefen_global_step_by_device.get(device)
        if t is None:
            t = torch.full((), float(self._gefen_global_step), dtype=torch.float64, device=device)
            self._gefen_global_step_by_device[device] = t
        return t

    def _synchronize_gefen_global_step_for_checkpoint(self) -> None:
        """Graph replays do not run Python: read the device counter back before saving."""
        if not self.capturable:
            return
        for t in self._gefen_global_step_by_device.values():
            self._gefen_global_step = max(self._gefen_global_step, int(round(float(t.item()))))

    def _assert_capturable_if_capturing(self) -> None:
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            if not self.capturable:
                raise RuntimeError(
                    "Gefen.step() is being captured in a CUDA graph but capturable=False")
            if self._gefen_codebook is None:
                raise RuntimeError(
                    "Gefen.step() must run eagerly once (codebook learning is host-driven) "
                    "before it can be captured")

    def _kernel_rng_seed(self) -> int:
        return int(self._gefen_global_step)

    def _kernel_rng_seed_on(self, device):
        """``(host seed, device seed)`` of the stochastic-rounding hash for a launch on ``device``.

        Eager steps pass the global step by value.  A capturable optimizer passes 0 and the
        device-resident global-step counter instead: a captured launch replays with the same
        arguments, so a host value would freeze the noise into a per-element bias, while the
        device counter advances inside the captured region (reference ``gefen.py:1770-1890``
        keeps a device seed per device for the same reason).  Both give the same seed at the
        same step."""
        if not self._stochastic_round:
            return None, None
        if self.capturable and device.type == "cuda":
            return 0, self._ensure_global_step_device(device)
        return self._kernel_rng_seed(), None

    # ------------------------------------------------------------------
    # per-parameter state
    # ------------------------------------------------------------------
    def _init_gefen_state(self, state, grad_view: torch.Tensor) -> None:
        state["m_codebook"] = torch.zeros(grad_view.shape, dtype=torch.uint8, device=grad_view.device)
        state["m_magnitude"] = torch.zeros(grad_view.shape[0], 1, dtype=torch.float32,
                                           device=grad_view.device)

    def _ensure_state(self, name: str, p: torch.Tensor, p_local: torch.Tensor,
                      grad: Optional[torch.Tensor], factored: bool) -> Dict[str, Any]:
        """Create (first step) or complete (after a resume) the state of one parameter."""
        state = self.state[p]
        numel = p_local.numel()
        dev = p_local.device
        if "step" not in state:
            if "automatic_period" in state:
                period = state["automatic_period"]
            elif numel == 1:
                period = 1
            else:
                g = grad if grad is not None else self._grad_of(p)
                period = self._resolve_automatic_period(name, p, g)
            if numel % period:
                raise ValueError(
                    "Automatic partition period {} does not divide parameter {} with numel {}".format(
                        period, name, numel))
            state["automatic_period"] = period
            state["step"] = self._new_step_counter(dev)
            nb = numel // period
            state["m_codebook"] = torch.zeros(nb, period, dtype=torch.uint8, device=dev)
            state["m_magnitude"] = torch.zeros(nb, 1, dtype=torch.float32, device=dev)
            self._capt.pop(dev, None)
        period = state["automatic_period"]
        if factored:
            if "v_row" not in state:
                state["v_row"] = torch.zeros(p_local.shape[0], dtype=torch.float32, device=dev)
                state["v_col"] = torch.zeros(p_local.shape[1], dtype=torch.float32, device=dev)
                state["factored_step"] = self._new_step_counter(dev)
                self._capt.pop(dev, None)
        else:
            if "vmean" not in state:
                state["vmean"] = torch.zeros(numel // period, 1, dtype=torch.float32, device=dev)
                state["vmean_step"] = self._new_step_counter(dev)
                self._capt.pop(dev, None)
            elif "vmean_step" not in state:
                s = state["step"]
                state["vmean_step"] = s.clone() if torch.is_tensor(s) else s
        self._colocate_param_state_(state, dev)
        return state

    def _is_factored(self, p) -> bool:
        if not self._factored_v_2d or p.ndim != 2:
            return False
        # DTensor shards keep the block path: row/column statistics of a local
        # shard are only meaningful with the cross-shard reduction that the
        # sharded runtime (parallel.fsdp) supplies through ``_shard_info``.
        return not hasattr(p, "placements")

    # ------------------------------------------------------------------
    # the step
    # ------------------------------------------------------------------
    def _step_param(self, group, name: str, p: torch.Tensor) -> None:
        src = self._grad_source(p) if self._grad_source is not None else None
        grad = None
        if src is not None and hasattr(src, "tensor"):
            grad, src = src.tensor, None
        elif src is None:
            if p.grad is None:
                return
            grad = _local(p.grad).detach()
        p_local = _local(p)
        if p_local.numel() == 0:
            return
        factored = self._is_factored(p)
        state = self._ensure_state(name, p, p_local, grad, factored)
        period = state["automatic_period"]
        vkey = "factored_step" if factored else "vmean_step"
        if not self.capturable:
            state["step"] += 1
            state[vkey] += 1
        beta1, beta2, eps = group["beta1"], group["beta2"], group["eps"]
        gscale = self._external_grad_scale if self._external_grad_scale is not None \
            else self._pending_grad_scale
        use_kernel = self._fused_for(p_local)
        shard = self._shard_info(p) if (self._shard_info is not None and factored) else None

        if use_kernel:
            from ..ops import update as _u

            dev = p_local.device
            if self.capturable:
                reg = self._capt_registry(dev)
                scal_ptr = reg["scal"].data_ptr() + 16 * reg["rows"][p]
                host = (0.0, 1.0, 1.0, 1.0)
            else:
                lr = self._lr_scalar(group)
                bc1 = 1.0 - beta1 ** state["step"]
                bc2 = 1.0 - beta2 ** state[vkey]
                host = (lr, (1.0 / bc2) if factored else (1.0 / math.sqrt(bc2)), 1.0 / bc1,
                        1.0 - lr * group["weight_decay"])
                scal_ptr = 0
            work = p_local if p_local.is_contiguous() else p_local.contiguous()
            if work is not p_local:
                self._fused_copyback.append((p_local, work))
            gsrc = src if src is not None else grad
            if src is None and not grad.is_contiguous():
                gsrc = grad.contiguous()
            if factored and work.dim() != 2:
                raise ValueError("factored update expects a 2-D parameter")
            row_only = (not factored) and not self._deterministic and \
                _u.two_phase_block(period, work.numel() // period)
            item = _u.Item(p=work, grad=gsrc, state=state, period=period, beta1=beta1, beta2=beta2,
                           eps=eps, scalars=host, scal_ptr=scal_ptr, shard=shard, row_only=row_only)
            kind = "factored" if (factored or row_only) else "block"
            mc = bool(getattr(gsrc, "mc_ptr", 0)) and kind == "factored" and not self._stochastic_round
            if getattr(gsrc, "mc_ptr", 0) and not mc:
                import dataclasses

                item.grad = dataclasses.replace(gsrc, mc_ptr=0)      # peer loads: this path cannot use multicast
            # gradients that arrive through an NVLS multicast address form a plan of their own (it runs
            # the kernel instantiation that reads them with multimem.ld_reduce)
            key = (kind + ("+mc" if mc else ""), dev, work.dtype)
            self._fused_items.setdefault(key, []).append(item)
            self._fused_meta.setdefault(key, []).append((p, group, state, vkey, factored))
            return

        # decomposed path (CPU, fp64, fused disabled)
        self._slow_params += 1
        if grad is None:
            grad = src.materialize()
        cb = self._gefen_codebook_on(p_local.device)
        if cb is None:
            raise ValueError("Expected Gefen codebook to be initialized before the update.")
        lr = group["lr"]
        if torch.is_tensor(lr) and not self.capturable:
            lr = self._lr_scalar(group)
        if torch.is_tensor(lr) and lr.device != p_local.device:
            lr = lr.to(p_local.device)
        bc1 = 1 - beta1 ** state["step"]
        bc2 = 1 - beta2 ** state[vkey]
        wdf = 1.0 - lr * group["weight_decay"] if group["weight_decay"] > 0.0 else 1.0
        if factored:
            kw = {}
            if shard is not None:
                kw = dict(total_rows=shard.total_rows, reduce_cols=shard.reduce_cols,
                          reduce_scalar=shard.reduce_scalar)
            F_.factored_update_(
                p_local, grad.view(p_local.shape), period, cb, state["m_codebook"],
                state["m_magnitude"], state["v_row"], state["v_col"], beta1=beta1, beta2=beta2,
                eps=eps, lr=lr, weight_decay_factor=wdf, bc1=bc1, bc2=bc2, grad_scale=gscale, **kw)
        else:
            gv = F_.partition_view(grad.reshape(-1), period)
            F_.block_update_(
                p_local, gv, cb, state["m_codebook"], state["m_magnitude"], state["vmean"],
                beta1=beta1, beta2=beta2, eps=eps, lr=lr, weight_decay_factor=wdf, bc1=bc1,
                bc2=bc2, grad_scale=gscale)

    def _flush_fused(self) -> None:
        """Launch the multi-tensor kernels for everything queued by ``_step_param``."""
        if not self._fused_items:
            return
        from ..ops import update as _u

        if self._plan_cache is None:
            self._plan_cache = _u.PlanCache()
        if self._pre_launch_hook is not None:
            heavy, self._heavy_prep = self._heavy_prep, False
            self._pre_launch_hook(heavy)
        for (kind, dev, _dt), items in self._fused_items.items():
            cb = self._gefen_codebook_on(dev)
            if cb is None:
                raise ValueError("Expected Gefen codebook to be initialized before the update.")
            lut = self._gefen_codebook_lut_on(dev)
            gscale = self._grad_scale_tensor(dev)
            plan = self._plan_cache.get_keyed((kind, dev, _dt), kind.split("+")[0], items)
            sr_seed, sr_dev = self._kernel_rng_seed_on(dev)
            plan.run(items, cb, self._gefen_thresholds_on(dev), lut, gscale=gscale, status=self._status_word(dev),
                     sr_seed=sr_seed, sr_seed_dev=sr_dev, epoch=self._exchange_epoch)
        for dst, work in self._fused_copyback:
            dst.copy_(work)

    # -- steady-state fast path ------------------------------------------------
    def _grad_identity(self, p):
        """Cheap identity of the gradient storage of ``p`` (None when it has no gradient)."""
        if self._grad_source is not None:
            src = self._grad_source(p)
            if src is not None:
                t = getattr(src, "tensor", None)
                return t.data_ptr() if t is not None else tuple(src.ptrs)
        g = p.grad
        if g is None:
            return None
        return _local(g).data_ptr()

    def _remember_fast_path(self, active) -> None:
        """After a step in which every stepping parameter went through the kernels with no
        staging copies, remember the plans so that the next steps only refresh scalars."""
        self._fast = None
        if (self.capturable or self._slow_params or self._fused_copyback or not self._fused_items
                or self._codebook_refresh_every or self._plan_cache is None):
            return
        idents = {}
        for g in self.param_groups:
            for p in g["params"]:
                idents[p] = self._grad_identity(p)
        plans = []
        for key, items in self._fused_items.items():
            plan = self._plan_cache._plans.get(key)
            if plan is None:
                return
            plans.append((key, plan, items, self._fused_meta[key]))
        self._fast = dict(idents=idents, plans=plans, n_groups=len(self.param_groups),
                          n_params=sum(len(g["params"]) for g in self.param_groups))

    def _fast_step(self) -> bool:
        f = self._fast
        if f["n_groups"] != len(self.param_groups) or self._pending_grad_scale is not None:
            self._fast = None
            return False
        idents = f["idents"]
        n = 0
        for g in self.param_groups:
            for p in g["params"]:
                n += 1
                if idents.get(p, 0) != self._grad_identity(p):
                    self._fast = None
                    return False
        if n != f["n_params"]:
            self._fast = None
            return False
        # The plans hold raw device addresses of the parameters and of their state: every one of
        # them, and every hyper-parameter baked into the descriptors, must still be what the
        # optimizer holds (parameters re-assigned with ``p.data = ...``, state paged to the host by
        # an offload wrapper or reloaded, betas / eps edited in a group all invalidate the plan).
        for (kind, dev, _dt), plan, items, metas in f["plans"]:
            if not self._fast_plan_still_valid(plan, items, metas, dev):
                self._fast = None
                return False
        for (kind, dev, _dt), plan, items, metas in f["plans"]:
            for it, (p, group, state, vkey, factored) in zip(items, metas):
                state["step"] += 1
                state[vkey] += 1
                lr = self._lr_scalar(group)
                b1, b2 = group["beta1"], group["beta2"]
                bc1 = 1.0 - b1 ** state["step"]
                bc2 = 1.0 - b2 ** state[vkey]
                it.scalars = (lr, (1.0 / bc2) if factored else (1.0 / math.sqrt(bc2)), 1.0 / bc1,
                              1.0 - lr * group["weight_decay"])
            plan.run(items, self._gefen_codebook_on(dev), self._gefen_thresholds_on(dev),
                     self._gefen_codebook_lut_on(dev),
                     gscale=self._grad_scale_tensor(dev), status=self._status_word(dev),
                     sr_seed=self._kernel_rng_seed() if self._stochastic_round else None,
                     epoch=self._exchange_epoch)      # never capturable here: host seed
        return True

    @staticmethod
    def _fast_plan_still_valid(plan, items, metas, dev) -> bool:
        """Whether the live tensors behind a remembered plan are exactly those it was built on."""
        from ..ops import update as _u

        live = []
        for it, (p, group, state, _vkey, _factored) in zip(items, metas):
            p_local = _local(p)
            if p_local.device != dev or not p_local.is_contiguous() or p_local.shape != it.p.shape:
                return False
            for k in ("m_codebook", "m_magnitude", "vmean", "v_row", "v_col"):
                t = state.get(k)
                if t is not None and (not torch.is_tensor(t) or t.device != dev):
                    return False
            if "m_codebook" not in state or "m_magnitude" not in state:
                return False
            live.append(_u.Item(p=p_local, grad=it.grad, state=state, period=state.get("automatic_period", it.period),
                                beta1=group["beta1"], beta2=group["beta2"], eps=group["eps"],
                                scal_ptr=it.scal_ptr, shard=it.shard, row_only=it.row_only, emit=it.emit))
        return _u.Plan.signature_of(live) == plan.signature

    def _grad_scale_tensor(self, device) -> Optional[torch.Tensor]:
        """Device scalar that multiplies every gradient (AMP unscale and/or clip coefficient)."""
        ext = self._external_grad_scale
        if ext is not None:
            return ext
        if self._pending_grad_scale is None:
            return None
        return torch.full((1,), float(self._pending_grad_scale), dtype=torch.float32, device=device)

    def _status_word(self, device) -> torch.Tensor:
        t = self._status_by_device.get(device)
        if t is None:
            t = torch.zeros(1, dtype=torch.int32, device=device)
            self._status_by_device[device] = t
        return t

    def kernel_status(self) -> Dict[torch.device, int]:
        """Status words written by the kernels (0 = ok, 1 = a bounded peer wait timed out)."""
        return {d: int(t.item()) for d, t in self._status_by_device.items()}

    def _has_grad(self, p) -> bool:
        if self._grad_source is not None and self._grad_source(p) is not None:
            return True
        return p.grad is not None

    @torch.compiler.disable
    @torch.no_grad()
    def step(self, closure=None):
        """One optimisation step; ``closure`` (if given) runs first under ``enable_grad``.

        Excluded from ``torch.compile`` tracing: inside a compiled training step it runs eagerly (its
        kernels are launched through pre-built plans of raw device addresses, which a tracer must not
        reorder or drop); to remove the launch overhead capture it in a CUDA graph with
        ``capturable=True``."""
        self._assert_capturable_if_capturing()
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        _assert_gradients_structurally_valid(self)
        self._pending_grad_scale = None
        if (hasattr(self, "found_inf") or hasattr(self, "grad_scale")) and \
                not _amp_prepare_optimizer_step(self):
            return loss
        try:
            self._maybe_refresh_gefen_codebook()
            self._maybe_save_gefen_grad_histogram()
            if (self._codebook_refresh_every and self._gefen_global_step > 0
                    and self._gefen_global_step % self._codebook_refresh_every == 0):
                self._refresh_codebook_with_requant()

            if self._fast is not None and self._fast_step():
                self._advance_gefen_global_step()
                return loss
            active = [(g, n, p) for g in self.param_groups
                      for n, p in self._iter_group_params_with_names(g) if self._has_grad(p)]
            if self.capturable:
                # State must exist before the stacked counters can alias it.
                by_dev: Dict[torch.device, list] = {}
                for g, n, p in active:
                    pl = _local(p)
                    if pl.numel() == 0:
                        continue
                    self._ensure_state(n, p, pl, None, self._is_factored(p))
                    by_dev.setdefault(pl.device, []).append(p)
                for dev, plist in by_dev.items():
                    self._capt_refresh(dev, plist)
            self._fused_items = {}
            self._fused_copyback = []
            self._fused_meta = {}
            self._slow_params = 0
            for g, n, p in active:
                self._step_param(g, n, p)
            self._flush_fused()
            self._remember_fast_path(active)
        finally:
            self._pending_grad_scale = None
            self._fused_items = {}
            self._fused_copyback = []
        self._advance_gefen_global_step()
        return loss

    def _advance_gefen_global_step(self) -> None:
        if self.capturable:
            devs = {(_local(p)).device for g in self.param_groups for p in g["params"]}
            for d in devs:
                self._ensure_global_step_device(d).add_(1)
        self._gefen_global_step += 1

    # ------------------------------------------------------------------
    # checkpointing (native format)
    # ------------------------------------------------------------------
    def _checkpoint_device_anchor(self) -> torch.Tensor:
        return torch.zeros(1, dtype=torch.uint8, device=self._gefen_codebook_device())

    def state_dict(self) -> Dict[str, Any]:
        """torch ``{"state", "param_groups"}`` plus ``gefen_global_step``,
        ``gefen_deterministic``, ``gefen_codebook``; every group mirrors these in
        ``_gefen_checkpoint_metadata`` so that tools which keep only the two
        standard keys cannot drop the codebook (reference ``gefen.py:4558-4707``)."""
        self._synchronize_gefen_global_step_for_checkpoint()
        reachable = {p for g in self.param_groups for p in g["params"]}
        orphaned = [p for p in self.state if p not in reachable]
        withheld = [(p, self.state.pop(p)) for p in orphaned]
        try:
            sd = super().state_dict()
        finally:
            for p, st in withheld:
                self.state.setdefault(p, st)

        def compact(v):
            if torch.is_tensor(v) and (
                    v.storage_offset() != 0
                    or v.untyped_storage().nbytes() != v.numel() * v.element_size()):
                return v.detach().clone()
            return v

        sd["state"] = {
            pid: ({k: compact(v) for k, v in st.items() if k not in _SCRATCH_KEYS}
                  if isinstance(st, dict) else st)
            for pid, st in sd["state"].items()
        }
        sd["gefen_global_step"] = self._gefen_global_step
        sd["gefen_deterministic"] = self._deterministic
        sd["gefen_codebook"] = self._gefen_codebook
        meta = {
            "format_version": 1,
            "global_step": self._gefen_global_step,
            "codebook": self._gefen_codebook,
            "deterministic": self._deterministic,
            "device_anchor": self._checkpoint_device_anchor(),
        }
        for g in sd["param_groups"]:
            g[_META_KEY] = meta
        ctx = None if getattr(self, "_local_state_dict_only", False) else self._rank_local_context()
        if ctx is not None:
            sd = self._attach_rank_local_payloads(sd, ctx)
        elif getattr(self, "_local_state_dict_only", False) and self._uses_rank_local_sharded_state():
            sd[_LOCAL_SNAPSHOT_KEY] = True          # this rank's own state: loadable on this rank only
        return sd

    def local_state_dict(self) -> Dict[str, Any]:
        """This rank's native state dict without any collective (snapshots, rollbacks)."""
        self._local_state_dict_only = True
        try:
            return self.state_dict()
        finally:
            self._local_state_dict_only = False

    # -- rank-local checkpoints of row-sharded (DTensor) parameters ---------------------------
    #
    # Schema of the reference (``gefen.py:4183-4556`` save, ``:5205-5454`` load), so that files move
    # between the two packages: the per-parameter states are replaced by one carrier entry (the
    # first saved id) holding a ``_gefen_rank_local_payload_<rank>`` uint8 tensor per rank (a
    # ``torch.save`` of that rank's payload dict) and member markers on the others; every group's
    # ``_gefen_checkpoint_metadata`` (format_version 3) carries the marker with the world, the mesh
    # and every rank's parameter signature.  Same topology only.
    def _rank_local_checkpoint_applies(self) -> bool:
        """Whether per-rank state differs between ranks (plain Gefen on shards: yes)."""
        return True

    @staticmethod
    def _is_dtensor_parameter(p) -> bool:
        return hasattr(p, "to_local") and hasattr(p, "placements") and hasattr(p, "device_mesh")

    def _uses_rank_local_sharded_state(self) -> bool:
        if not self._rank_local_checkpoint_applies():
            return False
        return any(self._is_dtensor_parameter(p) for g in self.param_groups for p in g["params"])

    @staticmethod
    def _placement_signature(placement) -> Dict[str, Any]:
        out = {"type": type(placement).__name__, "module": type(placement).__module__}
        for attr in ("dim", "split_factor"):
            v = getattr(placement, attr, None)
            if v is not None:
                out[attr] = int(v)
        op = getattr(placement, "reduce_op", None)
        if op is not None:
            out["reduce_op"] = str(op)
        return out

    @staticmethod
    def _mesh_signature(mesh) -> Dict[str, Any]:
        return {"device_type": str(mesh.device_type), "shape": list(mesh.shape),
                "dim_names": list(mesh.mesh_dim_names or ()),
                "ranks": [int(r) for r in mesh.mesh.detach().cpu().reshape(-1).tolist()]}

    def _rank_local_context(self):
        """World, ranks and mesh of a rank-local checkpoint, or None when the state is not
        rank-local.  One 1-D mesh spanning the default process group, the same for every DTensor
        parameter; anything else is refused (reference ``gefen.py:4091-4181``)."""
        if not self._uses_rank_local_sharded_state():
            return None
        import torch.distributed as dist

        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("Gefen rank-local DTensor checkpointing requires an initialized "
                               "default distributed process group")
        dts = [p for g in self.param_groups for p in g["params"] if self._is_dtensor_parameter(p)]
        mesh = dts[0].device_mesh
        sig = self._mesh_signature(mesh)
        if len(sig["shape"]) != 1:
            raise RuntimeError("Gefen rank-local optimizer checkpoints support only one 1-D DeviceMesh "
                               "spanning the default process group; use GefenDCPState for other layouts")
        if any(self._mesh_signature(p.device_mesh) != sig for p in dts[1:]):
            raise RuntimeError("Gefen rank-local optimizer checkpoints require every DTensor parameter "
                               "to use the same 1-D DeviceMesh")
        world = dist.get_world_size()
        ranks = list(range(world))
        if sig["shape"] != [world] or sorted(sig["ranks"]) != ranks:
            raise RuntimeError("Gefen rank-local optimizer checkpoints do not support DeviceMesh "
                               "subgroups; the one-dimensional mesh must span the default world")
        pg = mesh.get_group()
        coord = mesh.get_coordinate()
        if coord is None:
            raise RuntimeError("The current rank is not a member of Gefen's checkpoint DeviceMesh")
        return {"world_size": world, "global_rank": dist.get_rank(),
                "group_rank": dist.get_group_rank(pg, dist.get_rank()), "world_ranks": ranks,
                "mesh": sig, "coordinate": [int(c) for c in coord]}

    def _rank_local_signature(self) -> List[Dict[str, Any]]:
        """What binds a payload to a topology: per parameter its position, name, global and local
        shape, dtype, placements and mesh (reference ``gefen.py:4219-4274``)."""
        out = []
        for gi, g in enumerate(self.param_groups):
            names = g.get("param_names") or []
            for pi, p in enumerate(g["params"]):
                name = str(names[pi] if pi < len(names) else self._param_names.get(p, "")).lower()
                item = {"identifier": "group_{}_param_{}_{}".format(gi, pi, name), "group": gi, "param": pi,
                        "name": name}
                if not self._is_dtensor_parameter(p):
                    item.update({"sharded": False, "shape": list(p.shape), "local_shape": list(p.shape),
                                 "dtype": str(p.dtype), "requires_grad": bool(p.requires_grad),
                                 "sharded_mode": g.get("sharded_mode")})
                else:
                    local = _local(p)
                    coord = p.device_mesh.get_coordinate()
                    item.update({"sharded": True, "shape": list(p.shape), "local_shape": list(local.shape),
                                 "dtype": str(p.dtype), "local_dtype": str(local.dtype),
                                 "requires_grad": bool(p.requires_grad),
                                 "placements": [self._placement_signature(pl) for pl in p.placements],
                                 "mesh": self._mesh_signature(p.device_mesh),
                                 "coordinate": None if coord is None else list(coord),
                                 "sharded_mode": g.get("sharded_mode")})
                out.append(item)
        return out

    @staticmethod
    def _rank_local_manifest(signature):
        keys = ("identifier", "group", "param", "name", "sharded", "shape", "dtype", "requires_grad",
                "sharded_mode")
        return [{k: item.get(k) for k in keys} for item in signature]

    def _attach_rank_local_payloads(self, sd, ctx):
        """Replace this rank's states by the rank-indexed payloads of all ranks (collective)."""
        import io

        import torch.distributed as dist

        world, rank = ctx["world_size"], ctx["global_rank"]
        saved_ids = list(sd["state"])
        signature = self._rank_local_signature()
        manifest = self._rank_local_manifest(signature)
        control = {"saved_ids": saved_ids, "manifest": manifest, "signature": signature,
                   "global_step": int(self._gefen_global_step), "deterministic": bool(self._deterministic)}
        controls = [None] * world
        dist.all_gather_object(controls, control)
        if any(c["saved_ids"] != saved_ids for c in controls):
            raise RuntimeError("Gefen DTensor checkpoint requires identical optimizer parameter ordering "
                               "on every rank; got state keys {}".format([c["saved_ids"] for c in controls]))
        if any(c["manifest"] != manifest for c in controls):
            raise RuntimeError("Gefen DTensor checkpoint parameter identifiers, names, dtypes, or global "
                               "shapes differ across ranks")
        if len({c["global_step"] for c in controls}) != 1:
            raise RuntimeError("Gefen rank-local checkpoint global_step differs across ranks: {}".format(
                [c["global_step"] for c in controls]))
        if len({c["deterministic"] for c in controls}) != 1:
            raise RuntimeError("Gefen rank-local checkpoint deterministic policy differs across ranks")

        def to_cpu(v):
            if torch.is_tensor(v):
                return _local(v).detach().cpu().contiguous()
            if isinstance(v, dict):
                return {k: to_cpu(x) for k, x in v.items()}
            if isinstance(v, (list, tuple)):
                return type(v)(to_cpu(x) for x in v)
            return v

        payload = {"format": _RANK_LOCAL_FORMAT, "global_rank": rank, "group_rank": ctx["group_rank"],
                   "world_size": world, "world_ranks": ctx["world_ranks"], "mesh": ctx["mesh"],
                   "signature": signature, "parameter_manifest": manifest,
                   "global_step": control["global_step"], "deterministic": control["deterministic"],
                   "states": [to_cpu(sd["state"][i]) for i in saved_ids],
                   "codebook": to_cpu(self._gefen_codebook)}
        buf = io.BytesIO()
        torch.save(payload, buf)
        blobs = [None] * world
        dist.all_gather_object(blobs, buf.getvalue())
        carrier = {"name": 0}
        for r in ctx["world_ranks"]:
            carrier[_RANK_LOCAL_PAYLOAD_PREFIX + str(r)] = torch.frombuffer(bytearray(blobs[r]),
                                                                           dtype=torch.uint8).clone()
        out = dict(sd)
        out["state"] = {sid: (dict(carrier) if i == 0 else {"name": 0, _RANK_LOCAL_MEMBER_KEY: True})
                        for i, sid in enumerate(saved_ids)}
        marker = {"format": _RANK_LOCAL_FORMAT, "world_size": world, "world_ranks": ctx["world_ranks"],
                  "mesh": ctx["mesh"], "signatures": {str(r): controls[r]["signature"] for r in ctx["world_ranks"]},
                  "parameter_manifest": manifest, "global_step": control["global_step"],
                  "deterministic": control["deterministic"]}
        meta = {"format_version": _RANK_LOCAL_METADATA_VERSION, "global_step": control["global_step"],
                "codebook": None, "deterministic": control["deterministic"],
                "device_anchor": torch.zeros(1, dtype=torch.uint8), "rank_local_sharded_state": marker}
        out["param_groups"] = [dict(g) for g in sd["param_groups"]]
        for g in out["param_groups"]:
            g[_META_KEY] = meta
        # a raw state dict must not carry one rank's codebook as if it applied to every payload
        out["gefen_codebook"] = None
        return out

    def _select_rank_local_payload(self, state_dict):
        """This rank's native state dict out of a ``rank_local_dtensor_v2`` checkpoint, after the
        topology checks; other checkpoints pass through, except a full / untagged one into
        rank-local state, which is refused (it would give every rank one rank's blocks)."""
        if not isinstance(state_dict, dict):
            return state_dict
        groups = state_dict.get("param_groups", ())
        metas = [g.get(_META_KEY) for g in groups if isinstance(g, dict)]
        markers = [m.get("rank_local_sharded_state") for m in metas
                   if isinstance(m, dict) and m.get("rank_local_sharded_state") is not None]
        states = state_dict.get("state", {}) or {}

        def wrapped(st):
            return isinstance(st, dict) and (_RANK_LOCAL_MEMBER_KEY in st or any(
                isinstance(k, str) and k.startswith(_RANK_LOCAL_PAYLOAD_PREFIX) for k in st))

        if not markers:
            if any(wrapped(st) for st in states.values()):
                raise ValueError("Gefen checkpoint carries rank-local DTensor payloads but is missing "
                                 "their topology metadata")
            local_snapshot = state_dict.get(_LOCAL_SNAPSHOT_KEY) is True
            if (not local_snapshot and self._uses_rank_local_sharded_state()
                    and any(isinstance(st, dict) and "m_codebook" in st for st in states.values())):
                raise ValueError(
                    "Cannot safely load an untagged/full Gefen checkpoint into rank-local DTensor "
                    "optimizer state: it holds one rank's codebook and block state. Re-save from the "
                    "original run with state_dict() on every rank ({} payloads).".format(_RANK_LOCAL_FORMAT))
            if local_snapshot:
                state_dict = {k: v for k, v in state_dict.items() if k != _LOCAL_SNAPSHOT_KEY}
            return state_dict
        if len(markers) != len(groups):
            raise ValueError("Gefen rank-local DTensor checkpoint metadata is present on only some "
                             "parameter groups")
        marker = markers[0]
        if not isinstance(marker, dict) or any(m != marker for m in markers[1:]):
            raise ValueError("Gefen rank-local checkpoint parameter groups carry inconsistent markers")
        if marker.get("format") != _RANK_LOCAL_FORMAT:
            raise ValueError("Unsupported Gefen rank-local checkpoint format: {!r}".format(marker.get("format")))
        if not self._uses_rank_local_sharded_state():
            raise ValueError("A rank-local DTensor Gefen checkpoint can only load into the same sharded "
                             "optimizer topology; use GefenDCPState to reshard")
        try:
            ctx = self._rank_local_context()
        except RuntimeError as exc:
            raise ValueError(str(exc)) from exc
        world, rank = ctx["world_size"], ctx["global_rank"]
        if marker.get("world_size") != world:
            raise ValueError("Gefen rank-local DTensor checkpoints require the same world size; "
                             "checkpoint={} current={}".format(marker.get("world_size"), world))
        if marker.get("world_ranks") != ctx["world_ranks"]:
            raise ValueError("Gefen rank-local checkpoint default-world rank membership differs")
        if marker.get("mesh") != ctx["mesh"]:
            raise ValueError("Gefen rank-local checkpoint DeviceMesh differs")
        rank_keys = {str(r) for r in ctx["world_ranks"]}
        signatures = marker.get("signatures")
        if not isinstance(signatures, dict) or set(signatures) != rank_keys:
            raise ValueError("Gefen rank-local checkpoint has invalid signatures")
        signature = self._rank_local_signature()
        if signatures[str(rank)] != signature:
            raise ValueError("Gefen rank-local DTensor checkpoint topology differs on rank {}: "
                             "checkpoint={!r} current={!r}".format(rank, signatures[str(rank)], signature))
        manifest = self._rank_local_manifest(signature)
        if marker.get("parameter_manifest") != manifest:
            raise ValueError("Gefen rank-local checkpoint ordered parameter manifest differs")
        step, det = marker.get("global_step"), marker.get("deterministic")
        if type(step) is not int or step < 0:
            raise ValueError("Gefen rank-local checkpoint has invalid global_step")
        if type(det) is not bool:
            raise ValueError("Gefen rank-local checkpoint has invalid deterministic policy")
        saved_ids = list(chain.from_iterable(g.get("params", ()) for g in groups))
        if len(set(saved_ids)) != len(saved_ids):
            raise ValueError("Gefen rank-local checkpoint contains duplicate outer parameter IDs")
        want_keys = {_RANK_LOCAL_PAYLOAD_PREFIX + str(r) for r in ctx["world_ranks"]}
        blobs = None
        for sid in saved_ids:
            st = states.get(sid)
            if not isinstance(st, dict):
                raise ValueError("Gefen rank-local checkpoint is missing parameter state {!r}".format(sid))
            carrier = {k for k in st if isinstance(k, str) and k.startswith(_RANK_LOCAL_PAYLOAD_PREFIX)}
            if set(st) - carrier - {_RANK_LOCAL_MEMBER_KEY, "name"} or st.get("name") != 0:
                raise ValueError("Gefen rank-local checkpoint parameter state has an invalid schema: "
                                 "{!r}".format(sorted(map(str, st))))
            if carrier:
                if _RANK_LOCAL_MEMBER_KEY in st or carrier != want_keys or blobs is not None:
                    raise ValueError("Gefen rank-local checkpoint carrier has missing, unexpected or "
                                     "repeated per-rank payload keys")
                blobs = {str(r): st[_RANK_LOCAL_PAYLOAD_PREFIX + str(r)] for r in ctx["world_ranks"]}
            elif st.get(_RANK_LOCAL_MEMBER_KEY) is not True:
                raise ValueError("Gefen rank-local checkpoint has an invalid member marker")
        if blobs is None or any(not torch.is_tensor(b) for b in blobs.values()):
            raise ValueError("Gefen rank-local checkpoint has invalid rank payloads")
        blob = blobs[str(rank)]
        if blob.dtype != torch.uint8 or blob.dim() != 1:
            raise ValueError("Gefen rank-local checkpoint payload must be a 1-D uint8 tensor")
        import io

        try:
            payload = torch.load(io.BytesIO(blob.detach().cpu().contiguous().numpy().tobytes()),
                                 map_location="cpu", weights_only=True)
        except Exception as exc:
            raise ValueError("Gefen rank-local checkpoint payload is invalid") from exc
        keys = {"format", "global_rank", "group_rank", "world_size", "world_ranks", "mesh", "signature",
                "parameter_manifest", "global_step", "deterministic", "states", "codebook"}
        if not isinstance(payload, dict) or set(payload) != keys:
            raise ValueError("Gefen rank-local checkpoint payload has an invalid schema")
        bound = (payload["format"] == _RANK_LOCAL_FORMAT and payload["global_rank"] == rank
                 and payload["group_rank"] == ctx["group_rank"] and payload["world_size"] == world
                 and payload["world_ranks"] == ctx["world_ranks"] and payload["mesh"] == ctx["mesh"]
                 and payload["signature"] == signature and payload["parameter_manifest"] == manifest
                 and payload["global_step"] == step and payload["deterministic"] == det)
        if not bound:
            raise ValueError("Gefen rank-local checkpoint payload rank/topology/parameter binding differs")
        sel = payload["states"]
        if not isinstance(sel, list) or len(sel) != len(saved_ids) or any(not isinstance(x, dict) for x in sel):
            raise ValueError("Gefen rank-local checkpoint payload states do not match the parameters")
        for st in sel:
            if "m_codebook" in st:
                idx, mag = st["m_codebook"], st.get("m_magnitude")
                if (not torch.is_tensor(idx) or idx.dtype != torch.uint8 or not torch.is_tensor(mag)
                        or mag.dtype != torch.float32 or "step" not in st or "automatic_period" not in st
                        or not bool(torch.isfinite(mag).all())):
                    raise ValueError("Gefen rank-local checkpoint momentum state is incomplete or invalid")
        out = dict(state_dict)
        out["state"] = dict(zip(saved_ids, sel))
        out["gefen_global_step"] = step
        out["gefen_codebook"] = payload["codebook"]
        out["gefen_deterministic"] = det
        out["param_groups"] = []
        for g in groups:
            g = dict(g)
            m = dict(g[_META_KEY])
            m.update(global_step=step, codebook=payload["codebook"], deterministic=det)
            m.pop("rank_local_sharded_state", None)
            g[_META_KEY] = m
            out["param_groups"].append(g)
        return out

    @staticmethod
    def _same_codebook(a, b) -> bool:
        return a is b or (torch.is_tensor(a) and torch.is_tensor(b)
                          and a.shape == b.shape and torch.equal(a.cpu(), b.cpu()))

    @staticmethod
    def _pack_legacy_param_groups_for_load(self_groups, state_dict):
        """Old checkpoints stored one group per parameter; fold them onto the live groups.

        Reference ``gefen.py:4715-4773``.  Applies only when the saved group
        count equals the live parameter count, exceeds the live group count and
        every saved group holds exactly one parameter.
        """
        saved = state_dict["param_groups"]
        live_counts = [len(g["params"]) for g in self_groups]
        if len(saved) == len(self_groups) or len(saved) != sum(live_counts):
            return state_dict
        if any(len(g["params"]) != 1 for g in saved):
            return state_dict
        packed, cursor = [], 0
        for n in live_counts:
            chunk = saved[cursor:cursor + n]
            cursor += n
            merged = dict(chunk[0])
            merged["params"] = [g["params"][0] for g in chunk]
            merged["param_names"] = [
                (g.get("param_names") or [g.get("name")])[0] for g in chunk]
            merged[_SYNTH_KEY] = [bool((g.get(_SYNTH_KEY) or [True])[0]) for g in chunk]
            merged.pop("name", None)
            packed.append(merged)
        out = dict(state_dict)
        out["param_groups"] = packed
        return out

    def _parse_checkpoint_header(self, state_dict):
        """Split a checkpoint into (clean torch state dict, global step, codebook)."""
        sd = dict(state_dict)
        sd["param_groups"] = [dict(g) for g in sd.get("param_groups", ())]
        metas = []
        for g in sd["param_groups"]:
            m = g.pop(_META_KEY, None)
            if m is not None:
                metas.append(m)
        step = sd.pop("gefen_global_step", None)
        cb = sd.pop("gefen_codebook", None)
        has_det = "gefen_deterministic" in sd
        det = sd.pop("gefen_deterministic", None)
        if has_det and type(det) is not bool:
            raise ValueError(
                "Gefen checkpoint top-level deterministic policy must be a bool, got {!r}".format(det))
        if metas:
            if len(metas) != len(sd["param_groups"]):
                raise ValueError("Gefen checkpoint metadata is present on only some parameter groups")
            first = metas[0]
            if first.get("format_version") not in (1, 2, 3):
                raise ValueError(
                    "Unsupported Gefen checkpoint metadata format_version: {}".format(
                        first.get("format_version")))
            for m in metas:
                if "deterministic" in m and type(m["deterministic"]) is not bool:
                    raise ValueError(
                        "Gefen checkpoint parameter-group deterministic policy must be a bool, "
                        "got {!r}".format(m["deterministic"]))
            for m in metas[1:]:
                if (m.get("global_step") != first.get("global_step")
                        or not self._same_codebook(m.get("codebook"), first.get("codebook"))
                        or m.get("deterministic") != first.get("deterministic")):
                    raise ValueError(
                        "Gefen checkpoint parameter groups carry inconsistent optimizer metadata")
            if step is None:
                step = first.get("global_step", 0)
            elif step != first.get("global_step", 0):
                raise ValueError(
                    "Gefen checkpoint top-level and parameter-group global steps disagree")
            if cb is None:
                cb = first.get("codebook")
            elif not self._same_codebook(cb, first.get("codebook")):
                raise ValueError(
                    "Gefen checkpoint top-level and parameter-group codebooks disagree")
            mdet = first.get("deterministic")
            if det is None:
                det = mdet
            elif mdet is not None and det != mdet:
                raise ValueError(
                    "Gefen checkpoint top-level and parameter-group deterministic policies disagree")
        if det is not None and det != self._deterministic:
            raise ValueError(
                "Gefen checkpoint deterministic={!r}, but this optimizer was constructed with "
                "deterministic={!r}. Resuming under a different replica-determinism policy "
                "requires an intentional state migration or a fresh optimizer restart; refusing "
                "to change the policy silently.".format(det, self._deterministic))
        if step is None:
            step = 0
        quantised = any(isinstance(s, dict) and "m_codebook" in s
                        for s in (sd.get("state", {}) or {}).values())
        if quantised and cb is None:
            raise ValueError(
                "Gefen checkpoint contains quantized momentum indices but no frozen codebook. "
                "Loading it would reinterpret the restored indices with a different codebook and "
                "silently corrupt optimizer state. Resume from an unmodified Gefen checkpoint or "
                "a DCP checkpoint written by a version that preserves _gefen_checkpoint_metadata.")
        self._validate_native_states(sd.get("state", {}) or {}, cb)
        sd = self._pack_legacy_param_groups_for_load(self.param_groups, sd)
        self._validate_state_shapes(sd)
        return sd, step, cb

    def _state_shape_for(self, p) -> Optional[Tuple[int, ...]]:
        """Shape the quantised state of ``p`` is laid out for (subclasses whose state follows the
        full matrix of a sharded parameter return None to skip the check)."""
        return tuple(_local(p).shape)

    def _validate_state_shapes(self, sd) -> None:
        """Saved state tensors must fit the live parameters: the update kernels address the state
        through raw pointers with sizes derived from the parameter, so a checkpoint whose
        ``m_codebook`` / ``m_magnitude`` / ``vmean`` / ``v_row`` / ``v_col`` have other sizes would be
        read and written out of bounds on the next step.  Checked before any live mutation
        (reference ``gefen.py:4986-5190``)."""
        saved_groups = sd.get("param_groups", ())
        if len(saved_groups) != len(self.param_groups):
            return                      # torch's own loader reports the group mismatch
        states = sd.get("state", {}) or {}
        for sg, lg in zip(saved_groups, self.param_groups):
            if len(sg.get("params", ())) != len(lg["params"]):
                return
            for pid, p in zip(sg["params"], lg["params"]):
                st = states.get(pid)
                if not isinstance(st, dict) or "m_codebook" not in st:
                    continue
                shape = self._state_shape_for(p)
                if shape is None:
                    continue
                numel = 1
                for d in shape:
                    numel *= int(d)
                if numel == 0:
                    continue
                name = self._param_names.get(p, str(pid))
                period = st.get("automatic_period")
                what = "Gefen checkpoint state of {}".format(name)
                if not isinstance(period, int) or period < 1 or numel % period:
                    raise ValueError("{}: automatic_period {!r} does not divide the parameter's {} "
                                     "elements".format(what, period, numel))
                nb = numel // period
                idx, mag = st["m_codebook"], st["m_magnitude"]
                if tuple(idx.shape) != (nb, period):
                    raise ValueError("{}: m_codebook has shape {}, the parameter needs {}".format(
                        what, tuple(idx.shape), (nb, period)))
                if mag.numel() != nb:
                    raise ValueError("{}: m_magnitude holds {} values, the parameter needs {}".format(
                        what, mag.numel(), nb))
                if "vmean" in st and st["vmean"].numel() != nb:
                    raise ValueError("{}: vmean holds {} values, the parameter needs {}".format(
                        what, st["vmean"].numel(), nb))
                if "v_row" in st:
                    if len(shape) != 2 or st["v_row"].numel() != shape[0] or st["v_col"].numel() != shape[1]:
                        raise ValueError("{}: v_row / v_col hold {} / {} values, the parameter has shape {}".format(
                            what, st["v_row"].numel(), st["v_col"].numel(), shape))
                if "normuon_v" in st and st["normuon_v"].numel() != shape[0]:
                    raise ValueError("{}: normuon_v holds {} values, the parameter has {} rows".format(
                        what, st["normuon_v"].numel(), shape[0]))

    @staticmethod
    def _validate_counter(name: str, value) -> float:
        """A step counter of a checkpoint: a non-negative whole number held as an int, a float or a
        one-element non-boolean tensor (reference ``gefen.py:4923-4950``)."""
        if torch.is_tensor(value):
            if value.numel() != 1 or value.dtype == torch.bool:
                raise ValueError("Gefen checkpoint counter {} must be a one-element numeric tensor".format(name))
            value = value.reshape(()).item()
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ValueError("Gefen checkpoint counter {} must be numeric, got {!r}".format(name, type(value)))
        if not math.isfinite(value) or value < 0 or float(value) != float(int(value)):
            raise ValueError("Gefen checkpoint counter {} must be a non-negative whole number, got {}".format(
                name, value))
        return float(value)

    @classmethod
    def _validate_native_states(cls, states, codebook) -> None:
        """Reject a malformed checkpoint before anything live is touched: counters, period, index
        dtype, magnitudes and second moments finite and non-negative, complete momentum /
        factored / NorMuon groups of keys, a sorted finite 256-entry codebook in [-1, 1]
        (reference ``gefen.py:4896-5203``)."""

        def non_negative(name, t):
            if not torch.is_tensor(t) or not t.is_floating_point() or not bool(torch.isfinite(t).all()) \
                    or not bool((t >= 0).all()):
                raise ValueError("Gefen checkpoint {} must be a finite non-negative floating tensor".format(name))

        quantised = False
        for st in states.values():
            if not isinstance(st, dict):
                continue
            for key in _COUNTER_KEYS:
                if key in st:
                    cls._validate_counter(key, st[key])
            if "automatic_period" in st:
                period = st["automatic_period"]
                if isinstance(period, bool) or not isinstance(period, int) or period < 1:
                    raise ValueError("Gefen checkpoint automatic_period must be a positive int, got {!r}".format(period))
            has_idx, has_mag = "m_codebook" in st, "m_magnitude" in st
            if has_idx != has_mag:
                raise ValueError("Gefen checkpoint momentum state is incomplete")
            moments = [k for k in ("vmean", "v_row", "v_col", "normuon_v") if k in st]
            if not has_idx and (moments or "step" in st):
                raise ValueError("Gefen checkpoint carries optimizer state without its quantized momentum")
            if has_idx:
                quantised = True
                if not torch.is_tensor(st["m_codebook"]) or st["m_codebook"].dtype != torch.uint8:
                    raise ValueError("Gefen checkpoint m_codebook must be a uint8 tensor")
                non_negative("m_magnitude", st["m_magnitude"])
                if "step" not in st or "automatic_period" not in st:
                    raise ValueError("Gefen checkpoint momentum state is missing step or automatic_period")
            if ("v_row" in st) != ("v_col" in st) or ("v_row" in st) != ("factored_step" in st):
                raise ValueError("Gefen checkpoint factored second moment is incomplete")
            if ("normuon_v" in st) != ("normuon_step" in st):
                raise ValueError("Gefen checkpoint NorMuon state is incomplete")
            for key in moments:
                non_negative(key, st[key])
        if quantised and codebook is not None:
            cb = codebook
            ok = (torch.is_tensor(cb) and cb.dim() == 1 and cb.numel() == _cbk.NUM_CODEWORDS and cb.is_floating_point()
                  and bool(torch.isfinite(cb).all()) and float(cb.min()) >= -1.0 and float(cb.max()) <= 1.0
                  and bool((cb[1:] >= cb[:-1]).all()))
            if not ok:
                raise ValueError("Gefen checkpoint codebook must be a sorted finite tensor of {} values in "
                                 "[-1, 1]".format(_cbk.NUM_CODEWORDS))

    def _restore_into(self, target: "Gefen", sd, step, cb) -> None:
        """Run the whole load on ``target`` (a shadow of ``self`` during staging)."""
        saved_state = sd.get("state", {}) or {}
        torch.optim.Optimizer.load_state_dict(target, sd)
        target._gefen_global_step = int(step)
        target._gefen_global_step_by_device = {}
        target._capt = {}
        target._gefen_codebook = cb
        target._gefen_codebook_by_device = {}
        target._gefen_codebook_lut_by_device = {}
        target._gefen_thresholds_by_device = {}
        # torch casts every floating state tensor to the parameter's dtype; put
        # the fp32 moments and uint8 indices back in their saved dtypes.
        id_map = dict(zip(chain.from_iterable(g["params"] for g in sd["param_groups"]),
                          chain.from_iterable(g["params"] for g in target.param_groups)))
        for pid, saved in saved_state.items():
            p = id_map.get(pid)
            live = target.state.get(p) if p is not None else None
            if live is None or not isinstance(saved, dict):
                continue
            for k, v in saved.items():
                if not torch.is_tensor(v):
                    continue
                cur = live.get(k)
                if torch.is_tensor(cur) and cur.dtype == v.dtype:
                    continue
                dev = cur.device if torch.is_tensor(cur) else _local(p).device
                live[k] = v.to(device=dev, dtype=v.dtype)
        for g in target.param_groups:
            for p in g["params"]:
                st = target.state.get(p)
                if not st:
                    continue
                for k in _COUNTER_KEYS:
                    if k not in st:
                        continue
                    v = st[k]
                    if target.capturable:
                        dev = _local(p).device
                        if not torch.is_tensor(v):
                            st[k] = torch.full((), float(v), dtype=torch.float32, device=dev)
                        else:
                            st[k] = v.to(device=dev, dtype=torch.float32).reshape(()).clone()
                    elif torch.is_tensor(v):
                        st[k] = int(v.item())
        # names: the live optimizer's registry wins; state carries it for tools.
        target._param_names = {}
        target._synthesized_param_names = {}
        for g in target.param_groups:
            names = g.get("param_names") or []
            synth = g.get(_SYNTH_KEY) or []
            for i, p in enumerate(g["params"]):
                live_name = self._param_names.get(p)
                n = live_name if live_name is not None else (
                    names[i] if i < len(names) else "param_{}".format(len(target._param_names)))
                target._param_names[p] = n
                target._synthesized_param_names[p] = self._synthesized_param_names.get(
                    p, bool(synth[i]) if i < len(synth) else True)
                target.state[p]["name"] = n
            g["param_names"] = [target._param_names[p] for p in g["params"]]
            g[_SYNTH_KEY] = [target._synthesized_param_names[p] for p in g["params"]]

    def load_state_dict(self, state_dict) -> None:
        """Restore a native checkpoint atomically.

        The load runs on a shadow optimizer object that shares nothing mutable
        with ``self``; only after it fully succeeded are the results swapped in,
        so a failing load leaves the live optimizer untouched (reference
        ``gefen.py:4818-4856``).
        """
        # instance load hooks fire once, on this optimizer: pre-hooks before the transaction (they may
        # replace the state dict), post-hooks only after a successful commit
        for hook in list(getattr(self, "_optimizer_load_state_dict_pre_hooks", {}).values()):
            replaced = hook(self, state_dict)
            if replaced is not None:
                state_dict = replaced
        state_dict = self._select_rank_local_payload(state_dict)
        sd, step, cb = self._parse_checkpoint_header(state_dict)
        shadow = object.__new__(type(self))
        shadow.__dict__.update(self.__dict__)
        shadow._optimizer_load_state_dict_pre_hooks = type(self._optimizer_load_state_dict_pre_hooks)()
        shadow._optimizer_load_state_dict_post_hooks = type(self._optimizer_load_state_dict_post_hooks)()
        shadow.state = defaultdict(dict)
        for p, st in self.state.items():
            shadow.state[p] = dict(st)
        shadow.param_groups = [dict(g, params=list(g["params"])) for g in self.param_groups]
        self._restore_into(shadow, sd, step, cb)
        # publish
        self._fast = None
        if self._plan_cache is not None:
            self._plan_cache.clear()
        self.state = shadow.state
        self.param_groups = shadow.param_groups
        for attr in ("_gefen_global_step", "_gefen_global_step_by_device",
                     "_capt", "_gefen_codebook", "_gefen_codebook_by_device",
                     "_gefen_codebook_lut_by_device", "_gefen_thresholds_by_device", "_param_names", "_synthesized_param_names"):
            setattr(self, attr, getattr(shadow, attr))
        for hook in list(self._optimizer_load_state_dict_post_hooks.values()):
            hook(self)

    # ------------------------------------------------------------------
    # introspection
    # ------------------------------------------------------------------
    def state_bytes(self) -> int:
        """Bytes held in tensors of ``self.state`` (the "B/param state" numerator)."""
        total, seen = 0, set()
        for st in self.state.values():
            for k, v in st.items():
                if torch.is_tensor(v) and k not in _SCRATCH_KEYS:
                    key = (v.untyped_storage().data_ptr(), v.storage_offset(), v.numel())
                    if key in seen:
                        continue
                    seen.add(key)
                    total += v.numel() * v.element_size()
        return total
