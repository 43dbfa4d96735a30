"""Host side of the multi-tensor update kernels (``csrc/update.cu``).

A *plan* is the device-resident description of every tensor that one launch
sequence updates: an array of ``TensorDesc`` records, the tile prefix table and
one scratch arena.  Plans are cached by the optimizer and rebuilt only when a
pointer or a geometry changes, so a steady-state step costs one small pinned
host->device copy of the per-step scalars plus one operator call per plan.

The reference steps one parameter per kernel launch sequence through pybind
entry points (reference ``src/gefen/kernels/automatic_gefen_fused.py:581-771``).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ._ext import DTYPE_CODE, available, ops

MAX_SRC = 8
_THREADS = 256
DEFAULT_WAIT_ITERS = 4_000_000  # ~1 s of polling with 64 ns back-off


class TensorDesc(ctypes.Structure):
    """Mirror of ``gx::TensorDesc`` (csrc/update.h); size checked against the library."""

    _fields_ = [
        ("p", ctypes.c_void_p),
        ("g", ctypes.c_void_p * MAX_SRC),
        ("idx", ctypes.c_void_p),
        ("mag", ctypes.c_void_p),
        ("mag_new", ctypes.c_void_p),
        ("v0", ctypes.c_void_p),
        ("v1", ctypes.c_void_p),
        ("row_sq", ctypes.c_void_p),
        ("col_sq", ctypes.c_void_p),
        ("rfac", ctypes.c_void_p),
        ("cfac", ctypes.c_void_p),
        ("scal", ctypes.c_void_p),
        ("xchg_local", ctypes.c_void_p),
        ("xchg_peer", ctypes.c_void_p * MAX_SRC),
        ("flag_local", ctypes.c_void_p),
        ("flag_peer", ctypes.c_void_p * MAX_SRC),
        ("numel", ctypes.c_longlong),
        ("nb", ctypes.c_longlong),
        ("rows", ctypes.c_int),
        ("cols", ctypes.c_int),
        ("period", ctypes.c_int),
        ("total_rows", ctypes.c_int),
        ("n_src", ctypes.c_int),
        ("blk_mode", ctypes.c_int),
        ("tcols", ctypes.c_int),
        ("trows", ctypes.c_int),
        ("n_col_tiles", ctypes.c_int),
        ("rows_per_tile", ctypes.c_int),
        ("mode", ctypes.c_int),
        ("vec", ctypes.c_int),
        ("world", ctypes.c_int),
        ("rank", ctypes.c_int),
        ("row_only", ctypes.c_int),
        ("g_multimem", ctypes.c_int),
        ("beta1", ctypes.c_float),
        ("omb1", ctypes.c_float),
        ("beta2", ctypes.c_float),
        ("omb2", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("src_scale", ctypes.c_float),
    ]


def _desc_stride() -> int:
    n = ctypes.sizeof(TensorDesc)
    return (n + 15) // 16 * 16


_checked = False


def _check_layout() -> None:
    global _checked
    if _checked:
        return
    want = int(ops().desc_size())
    if want != _desc_stride():
        raise RuntimeError(
            "TensorDesc layout mismatch: python {} bytes, library {} bytes".format(
                _desc_stride(), want))
    _checked = True


@dataclass
class PeerGrad:
    """A gradient given as slices inside several (peer) buffers.

    ``ptrs[s]`` is the device address of this rank's slice inside source ``s``;
    the kernels use ``round(sum_s src_s * scale)``.  ``materialize`` returns that
    value as a local tensor (used for the first-step analysis and the CPU path).
    """

    ptrs: Sequence[int]
    shape: Tuple[int, ...]
    dtype: torch.dtype
    device: torch.device
    scale: float = 1.0
    _cache: Any = None
    # NVLS: multicast address of the same slice (0 = none).  The two-phase bf16 kernels then read the
    # gradient with multimem.ld_reduce (in-switch sum) instead of one peer load per rank.
    mc_ptr: int = 0

    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n

    def materialize(self) -> torch.Tensor:
        out = torch.empty(self.shape, dtype=self.dtype, device=self.device)
        ops().reduce_sources(out, list(self.ptrs), out.numel(), float(self.scale), None,
                             DTYPE_CODE[self.dtype], self.device.index or 0)
        return out


class LocalGrad:
    """A gradient that already is a local tensor, handed to the optimizer out of band."""

    def __init__(self, tensor: torch.Tensor):
        self.tensor = tensor

    def materialize(self) -> torch.Tensor:
        return self.tensor


@dataclass
class ShardExchange:
    """Where a ``Shard(0)`` factored tensor publishes / reads its column statistics."""

    total_rows: int
    world: int = 1
    rank: int = 0
    xchg_local: int = 0
    xchg_peer: Sequence[int] = ()
    flag_local: int = 0
    flag_peer: Sequence[int] = ()
    # host-side reductions for the decomposed path
    reduce_cols: Any = None
    reduce_scalar: Any = None


@dataclass
class Item:
    """One tensor of a plan."""

    p: torch.Tensor                   # contiguous local parameter (shard)
    grad: Any                         # torch.Tensor (contiguous) or PeerGrad
    state: Dict[str, Any]
    period: int
    beta1: float
    beta2: float
    eps: float
    scalars: Tuple[float, float, float, float] = (0.0, 1.0, 1.0, 1.0)
    scal_ptr: int = 0                 # device address of the scalar row (capturable), or 0
    shard: Optional[ShardExchange] = None
    row_only: bool = False            # block-path tensor run through the two-phase kernels
    emit: int = 0                     # 2: write the dense new momentum into p (Muon); 3: + Nesterov


def two_phase_block(period: int, nb: int) -> bool:
    """Block-path tensors whose blocks are long and few go through the two-phase kernels
    (many CTAs per block) instead of the one-worker-per-block kernel."""
    return period >= 1024 and nb < 2048


_STREAMING = True
_WIDE = False


def set_wide_chunks(on: bool) -> None:
    """Whether new streamed plans whose block periods are multiples of 16 use 16 elements per thread
    (two consumer groups per SM instead of three).  Off by default: measured 3% faster on a
    128256 x 4096 matrix and 6-15% slower on 4096 x 14336 and smaller ones."""
    global _WIDE
    _WIDE = bool(on)



def set_streaming(on: bool) -> None:
    """Whether new plans of 2-byte tensors may take the streamed kernels (shared-memory rings fed by
    bulk async copies).  Off: the register-pipelined fast kernels.  Both compute the same values."""
    global _STREAMING
    _STREAMING = bool(on)


def _lut_single(lut: torch.Tensor) -> bool:
    """Whether no bucket of the packed search table holds more than one decision threshold.  The
    streamed apply kernel resolves a value with one comparison and has no full search; a codebook
    with codewords closer than a bucket (1.2e-4 of the normalised range) goes to the
    register-pipelined kernels instead.  The answer is remembered on the table tensor itself (it
    lives and dies with it); reading it synchronises once per codebook.  During stream capture an
    unknown table counts as not single."""
    hit = getattr(lut, "_gx_single_threshold_buckets", None)
    if hit is None:
        if lut.is_cuda and torch.cuda.is_current_stream_capturing():
            return False
        hit = bool((((lut.to(torch.int32) & 0xFFFF) >> 8).max() <= 1).item())
        try:
            lut._gx_single_threshold_buckets = hit
        except AttributeError:
            pass
    return hit


def _aligned(ptr: int, n: int) -> bool:
    return ptr % n == 0


def _row_only_cols(period: int, numel: Optional[int] = None) -> int:
    """Column count of the matrix view of a row-only tensor.

    Long blocks: a divisor of the period, so that a row never straddles two blocks, near 2048
    elements (one 256-thread row of 8-wide chunks) so that long blocks are cut into many rows and
    every CTA tile holds full 16-row columns; multiples of 16 are preferred (rows then start where
    the bulk copies of the streamed kernels may start).  Short blocks (with ``numel`` given): several
    whole blocks per row, up to 2048 elements, again a multiple of 16 if one exists, so that a
    tensor of many tiny blocks is not walked as rows of a few elements."""
    if period > 4096 and period % 8 == 0:
        best = None
        for c in range(4096, 255, -8):
            if period % c == 0:
                chunks = c // 8
                waste = min((chunks + t - 1) // t * t - chunks for t in (256, 128, 64, 32))
                key = (waste, c % 16 != 0)
                if best is None or key < best[0]:
                    best = (key, c)
                    if key == (0, False):
                        break
        return best[1] if best is not None else period
    if numel is not None and period < 1024 and period % 8 == 0 and numel % period == 0:
        nb = numel // period
        for k in range(min(nb, 2048 // period), 1, -1):
            if nb % k == 0 and (period * k) % 16 == 0:
                return period * k
    return period


def _pick_tcols(chunks: int) -> int:
    best, best_waste = 256, None
    for t in (256, 128, 64, 32):
        waste = (chunks + t - 1) // t * t - chunks
        if best_waste is None or waste < best_waste:
            best, best_waste = t, waste
    return best


def check_state_shapes(st: Dict[str, Any], shape: Tuple[int, ...], period: int, *, factored: bool,
                       emit: bool = False, what: str = "Gefen state") -> None:
    """The kernels index the state through raw pointers with sizes derived from the parameter: a state
    tensor of another size would be read or written out of bounds.  Raises ``ValueError`` unless
    ``m_codebook`` is a contiguous ``[numel / P, P]`` uint8 tensor, ``m_magnitude`` (and ``vmean``) hold
    ``numel / P`` values and ``v_row`` / ``v_col`` match the parameter's rows / columns."""
    numel = 1
    for d in shape:
        numel *= int(d)
    if not isinstance(period, int) or period < 1 or numel % period:
        raise ValueError("{}: period {!r} does not divide {} elements".format(what, period, numel))
    nb = numel // period
    idx, mag = st.get("m_codebook"), st.get("m_magnitude")
    if not torch.is_tensor(idx) or tuple(idx.shape) != (nb, period) or not idx.is_contiguous():
        raise ValueError("{}: m_codebook must be a contiguous [{}, {}] tensor, got {}".format(
            what, nb, period, tuple(idx.shape) if torch.is_tensor(idx) else type(idx)))
    if not torch.is_tensor(mag) or mag.numel() != nb or not mag.is_contiguous():
        raise ValueError("{}: m_magnitude must hold {} contiguous values".format(what, nb))
    if emit:
        return
    if factored:
        if len(shape) != 2:
            raise ValueError("{}: the factored second moment needs a 2-D parameter".format(what))
        vr, vc = st.get("v_row"), st.get("v_col")
        if not torch.is_tensor(vr) or vr.numel() != shape[0] or not vr.is_contiguous() or \
                not torch.is_tensor(vc) or vc.numel() != shape[1] or not vc.is_contiguous():
            raise ValueError("{}: v_row / v_col must hold {} / {} contiguous values".format(what, shape[0], shape[1]))
    else:
        vm = st.get("vmean")
        if not torch.is_tensor(vm) or vm.numel() != nb or not vm.is_contiguous():
            raise ValueError("{}: vmean must hold {} contiguous values".format(what, nb))


class Plan:
    """Device tables for one (device, kind, dtype) group of tensors."""

    def __init__(self, kind: str, items: List[Item], device: torch.device, dtype: torch.dtype):
        _check_layout()
        self.kind = kind
        self.device = device
        self.dtype = dtype
        self.n = len(items)
        self.signature = self.signature_of(items)
        stride = _desc_stride()
        # scratch arena
        sizes = []
        for it in items:
            if kind == "factored":
                nb = it.p.numel() // it.period
                if it.row_only or it.emit:
                    cols = _row_only_cols(it.period, it.p.numel())
                    rows = it.p.numel() // cols
                    sizes.append((nb, nb, cols, nb, cols, rows))   # row statistics are per block
                else:
                    rows, cols = it.p.shape
                    sizes.append((nb, rows, cols, rows, cols, rows))
            else:
                sizes.append((0, 0, 0, 0, 0, 0))
        _up4 = lambda n: (n + 3) // 4 * 4                    # every scratch array starts 16-byte aligned
        total = sum(sum(_up4(x) for x in s[:5]) for s in sizes)
        # Work tiles: 256 threads x 8 elements x tile_k rows, the same for every tensor of the plan so
        # that equal tile counts mean equal work.  CTAs take contiguous tile ranges (consecutive row
        # tiles of a column tile run as one pipelined loop), so small tiles cost nothing: the tile is
        # shrunk until the plan has enough tiles to balance the CTAs.
        tile_k = 16
        if kind == "factored":
            def _tiles(k):
                t = 0
                for (_nb, _nr, nc, _a, _b, rows) in sizes:
                    chunks = (nc + 7) // 8
                    tc = _pick_tcols(chunks)
                    tr = _THREADS // tc
                    t += ((chunks + tc - 1) // tc) * ((rows + tr * k - 1) // (tr * k))
                return t
            while tile_k > 1 and _tiles(tile_k) < 8192:
                tile_k //= 2
        self.scratch = torch.zeros(max(total, 1), dtype=torch.float32, device=device)
        self.scal_dev = torch.zeros(self.n, 4, dtype=torch.float32, device=device)
        self._uploaded_scalars = None          # what scal_dev holds (constant for momentum-emit plans)
        buf = (ctypes.c_ubyte * (stride * self.n))()
        tile_start = [0]
        # NVLS: every gradient of the plan has a multicast address and qualifies for the 8-wide bf16
        # kernels, which are the ones that can read it (multimem.ld_reduce); otherwise peer loads
        use_mc = kind == "factored" and dtype == torch.bfloat16 and all(
            isinstance(it.grad, PeerGrad) and it.grad.mc_ptr and not it.emit and it.grad.mc_ptr % 16 == 0
            and it.p.numel() < 2 ** 31 - 1 and it.period % 8 == 0 and it.p.data_ptr() % 16 == 0
            and it.state["m_codebook"].data_ptr() % 8 == 0
            and ((_row_only_cols(it.period, it.p.numel()) if it.row_only else it.p.shape[-1]) % 8 == 0)
            for it in items)
        base = self.scratch.data_ptr()
        cursor = 0
        self._keepalive = []
        for i, it in enumerate(items):
            d = TensorDesc.from_buffer(buf, i * stride)
            p = it.p
            st = it.state
            check_state_shapes(st, tuple(p.shape), it.period, emit=bool(it.emit),
                               factored=(kind == "factored" and not it.row_only and not it.emit))
            d.p = p.data_ptr()
            d.g_multimem = 0
            if use_mc:
                srcs = [int(it.grad.mc_ptr)]
                d.src_scale = float(it.grad.scale)
                d.g_multimem = 1
            elif isinstance(it.grad, PeerGrad):
                srcs = list(it.grad.ptrs)
                d.src_scale = float(it.grad.scale)
            else:
                srcs = [it.grad.data_ptr()]
                d.src_scale = 1.0
            if not 1 <= len(srcs) <= MAX_SRC:
                raise ValueError("a gradient needs 1..{} sources".format(MAX_SRC))
            for s, ptr in enumerate(srcs):
                d.g[s] = ptr
            d.n_src = len(srcs)
            d.idx = st["m_codebook"].data_ptr()
            d.mag = st["m_magnitude"].data_ptr()
            d.numel = p.numel()
            d.period = it.period
            d.nb = p.numel() // it.period
            d.beta1 = it.beta1
            d.omb1 = 1.0 - it.beta1
            d.beta2 = it.beta2
            d.omb2 = 1.0 - it.beta2
            d.eps = it.eps
            d.scal = it.scal_ptr if it.scal_ptr else self.scal_dev.data_ptr() + 16 * i
            esz = p.element_size()
            ptr_ok = _aligned(p.data_ptr(), 16) and all(_aligned(s, 16) for s in srcs) and \
                _aligned(st["m_codebook"].data_ptr(), 8)
            if kind == "factored":
                nb, nr, nc, _, _, rows = sizes[i]
                cols = nc
                d.rows, d.cols = rows, cols
                d.row_only = int(it.emit) if it.emit else int(it.row_only)
                if it.emit:
                    d.total_rows = rows
                    d.v0 = st["m_magnitude"].data_ptr()      # unused by the emit path
                    d.v1 = st["m_magnitude"].data_ptr()
                elif it.row_only:
                    d.total_rows = rows
                    d.v0 = st["vmean"].data_ptr()
                    d.v1 = st["vmean"].data_ptr()
                else:
                    d.total_rows = it.shard.total_rows if it.shard is not None else rows
                    d.v0 = st["v_row"].data_ptr()
                    d.v1 = st["v_col"].data_ptr()
                d.mag_new = base + 4 * cursor; cursor += _up4(nb)
                d.row_sq = base + 4 * cursor; cursor += _up4(nr)
                d.col_sq = base + 4 * cursor; cursor += _up4(nc)
                d.rfac = base + 4 * cursor; cursor += _up4(nr)
                d.cfac = base + 4 * cursor; cursor += _up4(nc)
                P = it.period
                if P == cols:
                    d.blk_mode = 0
                elif cols % P == 0:
                    d.blk_mode = 1
                elif P % cols == 0:
                    d.blk_mode = 2
                else:
                    d.blk_mode = 3
                vec = ptr_ok and cols % 8 == 0 and P % 8 == 0 and (cols * esz) % 16 == 0
                d.vec = int(vec)
                unit = 8 if vec else 1
                chunks = (cols + unit - 1) // unit
                d.tcols = _pick_tcols(chunks)
                d.trows = _THREADS // d.tcols
                d.n_col_tiles = (chunks + d.tcols - 1) // d.tcols
                d.rows_per_tile = d.trows * tile_k
                n_row_tiles = (rows + d.rows_per_tile - 1) // d.rows_per_tile
                tiles = d.n_col_tiles * n_row_tiles
                sh = None if (it.row_only or it.emit) else it.shard
                if sh is not None and sh.world > 1:
                    d.world, d.rank = sh.world, sh.rank
                    d.xchg_local = sh.xchg_local
                    d.flag_local = sh.flag_local
                    for r in range(sh.world):
                        d.xchg_peer[r] = sh.xchg_peer[r]
                        d.flag_peer[r] = sh.flag_peer[r]
                else:
                    d.world, d.rank = 1, 0
            else:
                d.v0 = st["vmean"].data_ptr()
                d.rows, d.cols = int(d.nb), it.period
                d.total_rows = int(d.nb)
                P = it.period
                if P < 32:
                    d.mode = 0
                    tiles = (d.nb + _THREADS - 1) // _THREADS
                elif P < 1024:
                    d.mode = 1
                    tiles = (d.nb + 7) // 8
                else:
                    d.mode = 2
                    tiles = d.nb
                d.vec = int(ptr_ok and P % 8 == 0 and d.mode > 0)
                d.world, d.rank = 1, 0
            if tile_start[-1] + tiles >= 2 ** 31:
                raise ValueError("plan too large for 32-bit tile indices")
            tile_start.append(tile_start[-1] + int(tiles))
        self.total_tiles = tile_start[-1]
        host = torch.frombuffer(buf, dtype=torch.uint8).clone()
        self.descs = host.to(device)
        self.tile_start = torch.tensor(tile_start, dtype=torch.int32).to(device)
        self.uses_host_scalars = any(not it.scal_ptr for it in items)
        stride_ = _desc_stride()
        self.fast = int(kind == "factored" and all(
            TensorDesc.from_buffer(buf, i * stride_).vec == 1 and TensorDesc.from_buffer(buf, i * stride_).n_src == 1
            and TensorDesc.from_buffer(buf, i * stride_).numel < 2 ** 31 - 1
            for i in range(self.n)))
        if use_mc:
            if not self.fast:
                raise RuntimeError("internal: a multicast plan did not qualify for the fast kernels")
            self.fast = 2
        elif self.fast and _STREAMING and dtype in (torch.bfloat16, torch.float16) and all(
                self._stream_ok(TensorDesc.from_buffer(buf, i * stride_)) for i in range(self.n)):
            # the streamed kernels: rows are brought into shared memory by bulk async copies, whose
            # source addresses and sizes must be multiples of 16 bytes for all three arrays
            self.fast = 3
            # 16 elements per thread when no 16-element chunk can straddle two blocks; the kernels derive
            # that tile geometry from the 8-wide fields with the rule below, the prefix goes behind the
            # 8-wide one
            descs_ = [TensorDesc.from_buffer(buf, i * stride_) for i in range(self.n)]
            if _WIDE and all(d.period % 16 == 0 for d in descs_):
                wide = [0]
                for d in descs_:
                    chunks = d.cols // 16
                    tc = _pick_tcols(chunks)
                    rows_per_tile = (_THREADS // tc) * (d.rows_per_tile // d.trows)
                    wide.append(wide[-1] + ((chunks + tc - 1) // tc) * ((d.rows + rows_per_tile - 1) // rows_per_tile))
                if wide[-1] < 2 ** 31:
                    self.fast = 4
                    self.tile_start = torch.tensor(tile_start + wide, dtype=torch.int32).to(device)

    @staticmethod
    def _stream_ok(d) -> bool:
        ptrs = (d.idx, d.p, d.g[0])            # ctypes gives None for a null pointer (storage-less test tensors)
        return d.row_only < 2 and d.cols % 16 == 0 and all((x or 0) % 16 == 0 for x in ptrs)

    @staticmethod
    def signature_of(items: List[Item]):
        sig = []
        for it in items:
            g = it.grad
            gp = (tuple(g.ptrs) + (int(g.mc_ptr),)) if isinstance(g, PeerGrad) else (g.data_ptr(),)
            st = it.state
            sig.append((it.p.data_ptr(), gp, st["m_codebook"].data_ptr(), st["m_magnitude"].data_ptr(),
                        (st["v_row"] if "v_row" in st else st.get("vmean", st["m_magnitude"])).data_ptr(),
                        st["v_col"].data_ptr() if "v_col" in st else 0,
                        it.period, it.scal_ptr, tuple(it.p.shape), it.beta1, it.beta2, it.eps, it.row_only, it.emit))
        return tuple(sig)

    def run(self, items: List[Item], codebook: torch.Tensor, thr: torch.Tensor, lut: torch.Tensor, *,
            gscale: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None,
            sr_seed: Optional[int] = None, wait_iters: int = DEFAULT_WAIT_ITERS,
            phases: int = 7, epoch: int = 0, sr_seed_dev: Optional[torch.Tensor] = None) -> None:
        """``sr_seed`` switches stochastic rounding on; ``sr_seed_dev`` (a float64 device scalar) is
        added to it inside the kernels, so that CUDA-graph replays, which re-run the launch with
        the same arguments, still draw fresh noise as long as the counter advances on the device."""
        if self.uses_host_scalars and (phases & 1 or self.kind == "block"):
            scalars = tuple(tuple(it.scalars) for it in items)
            if scalars != self._uploaded_scalars:
                if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
                    # a captured host-to-device copy would replay from host memory that is gone
                    raise RuntimeError("the per-step scalars of this plan live on the host and changed: run the "
                                       "step with capturable=True (device-resident scalars) to capture it")
                # A fresh pageable tensor per upload: the runtime stages it before the call
                # returns, so the host may run ahead of the device without racing on it.
                h = torch.tensor(scalars, dtype=torch.float32)
                self.scal_dev.copy_(h, non_blocking=True)
                self._uploaded_scalars = scalars
        code = DTYPE_CODE[self.dtype]
        seed = 0 if sr_seed is None else int(sr_seed)
        if self.kind == "factored":
            fast = int(self.fast)
            if fast >= 3 and not _lut_single(lut):
                fast = 1
            ops().factored_update(self.descs, self.tile_start, self.n, self.total_tiles, codebook, thr, lut,
                                  gscale, status, code, seed, sr_seed is not None, int(wait_iters),
                                  int(phases), int(epoch) & 0x7FFFFFFF, fast, sr_seed_dev)
        else:
            ops().block_update(self.descs, self.tile_start, self.n, self.total_tiles, codebook, thr, lut,
                               gscale, status, code, seed, sr_seed is not None, sr_seed_dev)


class PlanCache:
    """Plans keyed by (kind, device, dtype); rebuilt when a signature changes."""

    def __init__(self):
        self._plans: Dict[Any, Plan] = {}
        self.rebuilds = 0

    def get(self, kind: str, items: List[Item]) -> Plan:
        p0 = items[0].p
        key = (kind, p0.device, p0.dtype)
        sig = Plan.signature_of(items)
        plan = self._plans.get(key)
        if plan is None or plan.signature != sig:
            plan = Plan(kind, items, p0.device, p0.dtype)
            self._plans[key] = plan
            self.rebuilds += 1
        return plan

    def get_keyed(self, key, kind: str, items: List[Item]) -> Plan:
        """Like :meth:`get` but with a caller-chosen cache key (one plan per tensor)."""
        sig = Plan.signature_of(items)
        plan = self._plans.get(key)
        if plan is None or plan.signature != sig:
            plan = Plan(kind, items, items[0].p.device, items[0].p.dtype)
            self._plans[key] = plan
            self.rebuilds += 1
        return plan

    def clear(self) -> None:
        self._plans.clear()


_EMIT_CACHE = PlanCache()


def momentum_emit(grad, state: Dict[str, Any], out: torch.Tensor, codebook: torch.Tensor,
                  thr: torch.Tensor, lut: torch.Tensor, *, beta: float, nesterov: bool,
                  gscale: Optional[torch.Tensor] = None, cache: Optional["PlanCache"] = None) -> torch.Tensor:
    """Muon momentum on the GPU: advance the quantised EMA of ``grad`` (in ``state``) and write the
    dense new momentum (with the Nesterov look-ahead if asked) into ``out`` (same dtype as grad)."""
    item = Item(p=out.view(-1), grad=grad.reshape(-1) if torch.is_tensor(grad) else grad, state=state,
                period=int(state["automatic_period"]), beta1=beta, beta2=0.0, eps=0.0,
                emit=3 if nesterov else 2)
    cache = cache if cache is not None else _EMIT_CACHE
    plan = cache.get_keyed(("emit", id(state)), "factored", [item])
    plan.run([item], codebook, thr, lut, gscale=gscale)
    return out


def reduce_sources(out: Optional[torch.Tensor], ptrs: Sequence[int], numel: int, scale: float,
                   partials: Optional[torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
    ops().reduce_sources(out, list(ptrs), int(numel), float(scale), partials, DTYPE_CODE[dtype],
                         device.index or 0)


def clip_coef(partials: torch.Tensor, max_norm: float, coef: torch.Tensor) -> None:
    ops().clip_coef(partials, float(max_norm), coef)
