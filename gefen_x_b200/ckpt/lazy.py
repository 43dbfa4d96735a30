"""Zero-storage stand-ins for sharded tensors in ``torch.distributed.checkpoint``.

DCP plans a save from *metadata* (global shape, this rank's chunk) and asks for the
bytes of one write item at a time, so a dense fp32 view of quantised optimizer state
does not have to exist for the whole write.  :class:`LazyShard` is a tensor wrapper
subclass without storage that publishes a global shape and the offsets / sizes of
this rank's chunk through torch's checkpointable protocol
(``__create_write_items__`` / ``__create_chunk_list__`` / ``__get_tensor_shard__``)
and builds the local data only when asked:

* on **save**, :class:`~gefen_x_b200.ckpt.dcp.GefenSavePlanner` resolves one stand-in
  at a time, under a lock, through a reusable pinned staging buffer, and hands the
  writer a host copy; the device-side expansion is dropped before the next one
  starts, so the transient is one slot's dense form instead of all of them;
* on **load**, ``__get_tensor_shard__`` returns one cached destination buffer that
  DCP fills in place and the owner reads back.

Unlike the reference's stand-in (reference ``src/gefen/dcp.py:162-391``), which takes
its geometry from a DTensor parameter, the geometry here is explicit, so the same
class also publishes the plain row-shard tensors of the sharded runtime
(``parallel.fsdp``), which are not DTensors.

``LazyShard.accounting`` counts the bytes of dense expansions alive at any time; the
tests use it to check the memory bound without a GPU.
"""
from __future__ import annotations

import threading
import weakref
from typing import Callable, Optional, Sequence, Tuple

import torch


class _Accounting:
    """Bytes of materialised dense tensors currently alive, and their high-water mark."""

    def __init__(self):
        self._lock = threading.Lock()
        self.live = 0
        self.peak = 0

    def track(self, t: torch.Tensor) -> torch.Tensor:
        n = t.numel() * t.element_size()
        with self._lock:
            self.live += n
            self.peak = max(self.peak, self.live)
        weakref.finalize(t, self._release, n)
        return t

    def _release(self, n: int) -> None:
        with self._lock:
            self.live -= n

    def reset(self) -> None:
        with self._lock:
            self.live = 0
            self.peak = 0


class PinnedStaging:
    """One reusable page-locked buffer for device -> host copies of dense expansions.

    A copy through pinned memory runs at full PCIe bandwidth and does not synchronise the
    whole device; the result handed out is pageable (copied once more on the host), so the
    writer threads may hold many of them without draining the page-locked pool (reference
    ``src/gefen/dcp.py:1423-1475``).
    """

    def __init__(self, max_bytes: int = 1 << 28):
        self.max_bytes = int(max_bytes)
        self._buf: Optional[torch.Tensor] = None

    def _buffer(self, nbytes: int) -> Optional[torch.Tensor]:
        if not torch.cuda.is_available():
            return None
        if self._buf is None or self._buf.numel() < min(nbytes, self.max_bytes):
            want = min(max(nbytes, 1 << 20), self.max_bytes)
            try:
                self._buf = torch.empty(want, dtype=torch.uint8, pin_memory=True)
            except RuntimeError:
                self._buf = None
        return self._buf

    def to_host(self, dense: torch.Tensor) -> torch.Tensor:
        """Host copy of ``dense`` (a contiguous device tensor), made in buffer-sized pieces."""
        if dense.device.type == "cpu":
            return dense
        out = torch.empty(dense.shape, dtype=dense.dtype, device="cpu")
        src = dense.contiguous().view(-1).view(torch.uint8)
        dst = out.view(-1).view(torch.uint8)
        buf = self._buffer(src.numel())
        if buf is None:
            dst.copy_(src)
            return out
        step = buf.numel()
        for off in range(0, src.numel(), step):
            n = min(step, src.numel() - off)
            buf[:n].copy_(src[off:off + n], non_blocking=True)
            torch.cuda.current_stream(dense.device).synchronize()
            dst[off:off + n].copy_(buf[:n])
        return out


class LazyShard(torch.Tensor):
    """Stand-in for this rank's chunk ``[offsets, offsets + sizes)`` of a tensor of ``global_shape``.

    ``materialize()`` returns the local data (shape ``sizes``); it is called at write time
    (uncached) or once for a load destination (cached).  ``sizes`` with a zero entry means this
    rank holds nothing of the tensor: no write item and no read request is produced for it.
    """

    accounting = _Accounting()

    @staticmethod
    def __new__(cls, global_shape: Sequence[int], offsets: Sequence[int], sizes: Sequence[int],
                materialize: Callable[[], torch.Tensor], *, dtype=torch.float32, device="cpu",
                dense_cost: bool = True):
        t = torch.Tensor._make_wrapper_subclass(cls, tuple(int(d) for d in global_shape), dtype=dtype,
                                                device=torch.device(device), requires_grad=False)
        t._gx_offsets = tuple(int(o) for o in offsets)
        t._gx_sizes = tuple(int(s) for s in sizes)
        t._gx_materialize = materialize
        t._gx_cache = None
        t._gx_dense_cost = bool(dense_cost)      # False: materialize returns a view of live memory
        return t

    def __init__(self, *args, **kwargs):
        pass

    # -- nothing but the checkpoint protocol may touch a stand-in ---------------------------
    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        if func in (torch.Tensor.to, torch.Tensor.cpu, torch.Tensor.cuda):
            raise RuntimeError(
                "a gefen_x_b200 checkpoint stand-in carries no data and cannot be moved between devices; "
                "torch.distributed.checkpoint.async_save needs storage_writer=GefenFileSystemWriter(path), "
                "which expands the stand-ins one at a time while staging")
        return super().__torch_function__(func, types, args, kwargs or {})

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        if func is torch.ops.aten.is_pinned.default:
            return False
        raise RuntimeError(
            "a gefen_x_b200 checkpoint stand-in cannot execute {}: it carries no data of its own and is "
            "resolved only through torch.distributed.checkpoint's save / load protocol (use the "
            "optimizer's own state_dict() for ordinary tensors)".format(func))

    def __repr__(self, *, tensor_contents=None):
        return "LazyShard(global_shape={}, offsets={}, sizes={}, dtype={}, {})".format(
            tuple(self.shape), getattr(self, "_gx_offsets", None), getattr(self, "_gx_sizes", None), self.dtype,
            "materialised" if getattr(self, "_gx_cache", None) is not None else "unmaterialised")

    def __reduce_ex__(self, protocol):
        raise TypeError("a gefen_x_b200 checkpoint stand-in cannot be pickled; save it with "
                        "torch.distributed.checkpoint, or use the optimizer's own state_dict()")

    # -- geometry -----------------------------------------------------------------------------
    @property
    def local_numel(self) -> int:
        n = 1
        for s in self._gx_sizes:
            n *= s
        return n

    def local_nbytes(self) -> int:
        return self.local_numel * self.element_size()

    def _chunk(self):
        from torch.distributed.checkpoint.metadata import ChunkStorageMetadata

        return ChunkStorageMetadata(offsets=torch.Size(self._gx_offsets), sizes=torch.Size(self._gx_sizes))

    # -- data ----------------------------------------------------------------------------------
    def _dense(self) -> torch.Tensor:
        t = self._gx_materialize()
        if tuple(t.shape) != self._gx_sizes:
            t = t.reshape(self._gx_sizes)
        if self._gx_dense_cost:
            LazyShard.accounting.track(t)
        return t

    def resolve_uncached(self, staging: Optional[PinnedStaging] = None) -> torch.Tensor:
        """The local data on the host, for the writer; nothing is retained here."""
        dense = self._dense()
        if dense.device.type == "cpu":
            return dense
        host = (staging or PinnedStaging()).to_host(dense)
        del dense
        return host

    def staged_to_host(self) -> "LazyShard":
        """A stand-in with the same geometry whose data is a host snapshot taken now (async save)."""
        host = self.resolve_uncached()
        if host.device.type == "cpu" and not self._gx_dense_cost:
            host = host.clone()                   # a view of live memory: snapshot it
        return LazyShard(self.shape, self._gx_offsets, self._gx_sizes, lambda: host, dtype=self.dtype,
                         device="cpu", dense_cost=False)

    # -- torch.distributed.checkpoint protocol ----------------------------------------------
    def __create_write_items__(self, fqn, obj):
        from torch.distributed.checkpoint.metadata import MetadataIndex, TensorProperties
        from torch.distributed.checkpoint.planner import TensorWriteData, WriteItem, WriteItemType

        if self.local_numel == 0:
            return []
        chunk = self._chunk()
        return [WriteItem(index=MetadataIndex(fqn, chunk.offsets), type=WriteItemType.SHARD,
                          tensor_data=TensorWriteData(chunk=chunk, properties=TensorProperties(dtype=self.dtype),
                                                      size=self.size()))]

    def __create_chunk_list__(self):
        return [] if self.local_numel == 0 else [self._chunk()]

    def __get_tensor_shard__(self, index):
        # the load destination: DCP copies into it in place, so it must stay the same buffer
        if self._gx_cache is None:
            self._gx_cache = self._dense()
        return self._gx_cache

    def loaded(self) -> Optional[torch.Tensor]:
        """What a load wrote into this stand-in (None when nothing was requested)."""
        return self._gx_cache


def row_shard_geometry(global_shape: Sequence[int], world: int, rank: int) -> Tuple[Tuple[int, ...], Tuple[int, ...]]:
    """``(offsets, sizes)`` of rank ``rank``'s rows under the ``Shard(0)`` split torch FSDP2 uses
    (``ceil(rows / world)`` rows per rank, the last ranks possibly short or empty)."""
    rows = int(global_shape[0])
    per = (rows + world - 1) // world
    r0 = min(rows, rank * per)
    r1 = min(rows, (rank + 1) * per)
    offsets = (r0,) + (0,) * (len(global_shape) - 1)
    sizes = (r1 - r0,) + tuple(int(d) for d in global_shape[1:])
    return offsets, sizes
