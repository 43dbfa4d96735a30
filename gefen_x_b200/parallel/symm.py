"""Symmetric arena: one identically laid-out allocation per rank, mapped by every peer.

All buffers that another GPU reads or writes (parameter shards, unsharded
gradient staging, exchange slots, flags) are carved out of a single arena that
is allocated with ``torch.distributed._symmetric_memory`` and exchanged once at
start-up; ``peer_ptrs`` then gives the device address of any sub-buffer on every
rank.  With one rank no distributed machinery is touched: the arena is a plain
CUDA (or CPU) tensor.

The reference has no peer-memory layer (its collectives are torch FSDP2's); this
is the transport under ``parallel.fsdp``.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from ..ops._ext import ops

_ALIGN = 256
_GUARD = 64            # bytes of the guard line behind every arena allocation
_GUARD_BYTE = 0xA5


class SymmetricArena:
    def __init__(self, nbytes: int, device: torch.device, world: int = 1, rank: int = 0,
                 group=None):
        self.device = torch.device(device)
        self.world = world
        self.rank = rank
        self.nbytes = (int(nbytes) + _ALIGN - 1) // _ALIGN * _ALIGN
        self._cursor = 0
        self.handle = None
        self.mc_base = 0
        if world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem

            grp = group if group is not None else dist.group.WORLD
            self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            self.handle = symm_mem.rendezvous(self.buf, group=grp)
            off = int(getattr(self.handle, "offset", 0) or 0)      # of this tensor inside its allocation
            self.base_ptrs = [int(p) + off for p in self.handle.buffer_ptrs]
            if self.base_ptrs[rank] != self.buf.data_ptr():
                # the local mapping must be the tensor we write through
                self.base_ptrs[rank] = self.buf.data_ptr()
            # NVLS: the multicast mapping of the whole arena (0 when the fabric or the driver has none).
            # A multimem.ld_reduce at mc_base + offset returns the sum of that location over all ranks.
            try:
                self.mc_base = int(self.handle.multicast_ptr or 0)
                if self.mc_base:
                    self.mc_base += off
            except Exception:           # pragma: no cover - older symmetric-memory handles
                self.mc_base = 0
        else:
            self.buf = torch.empty(self.nbytes, dtype=torch.uint8, device=self.device)
            self.base_ptrs = [self.buf.data_ptr()]
        self.buf.zero_()
        self._guards: List[int] = []

    def alloc(self, numel: int, dtype: torch.dtype) -> Tuple[torch.Tensor, int]:
        """Carve ``numel`` elements; returns (local view, byte offset inside the arena).

        Every allocation is followed by a guard line of ``_GUARD`` bytes holding a fixed pattern:
        a kernel (local or on a peer) that writes past a buffer lands there, and
        :meth:`check_guards` finds it on the host."""
        esz = torch.empty((), dtype=dtype).element_size()
        off = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        nbytes = int(numel) * esz
        guard = (off + nbytes + 15) // 16 * 16
        if guard + _GUARD > self.nbytes:
            raise MemoryError("symmetric arena exhausted: need {} more bytes".format(
                guard + _GUARD - self.nbytes))
        self._cursor = guard + _GUARD
        self.buf[guard:guard + _GUARD].fill_(_GUARD_BYTE)
        self._guards.append(guard)
        view = self.buf[off:off + nbytes].view(dtype)
        return view, off

    def check_guards(self) -> List[int]:
        """Byte offsets of the guard lines that no longer hold their pattern (reads them back)."""
        if not self._guards:
            return []
        idx = torch.tensor(self._guards, dtype=torch.long, device=self.buf.device)
        lines = self.buf[(idx[:, None] + torch.arange(_GUARD, device=self.buf.device)[None, :]).reshape(-1)]
        bad = (lines.view(len(self._guards), _GUARD) != _GUARD_BYTE).any(dim=1).cpu().tolist()
        return [g for g, b in zip(self._guards, bad) if b]

    def mc_ptr(self, byte_offset: int) -> int:
        """Multicast address of ``byte_offset`` (0 when NVLS is not available)."""
        return self.mc_base + int(byte_offset) if self.mc_base else 0

    def peer_ptrs(self, byte_offset: int) -> List[int]:
        return [b + int(byte_offset) for b in self.base_ptrs]

    def barrier(self) -> None:
        """Host-visible barrier over the arena's group (start-up / teardown only)."""
        if self.world > 1:
            import torch.distributed as dist

            torch.cuda.synchronize(self.device)
            dist.barrier()


class FlagBoard:
    """``n_slots x world`` uint32 arrival flags in the arena.

    ``signal(slot, value)`` writes ``value`` into ``[slot][my rank]`` on every
    rank (release, system scope); ``wait(slot, value)`` polls the local row until
    every rank's entry reached ``value``, for at most ``wait_iters`` iterations,
    after which the status word is set and the stream carries on.
    """

    def __init__(self, arena: SymmetricArena, n_slots: int, status: torch.Tensor,
                 wait_iters: int = 4_000_000):
        self.arena = arena
        self.n_slots = n_slots
        self.world = arena.world
        self.status = status
        self.wait_iters = int(wait_iters)
        self.flags, self.off = arena.alloc(n_slots * self.world, torch.int32)
        self.flags.zero_()

    def row_ptrs(self, slot: int) -> List[int]:
        return self.arena.peer_ptrs(self.off + 4 * slot * self.world)

    def signal(self, slot: int, value: int) -> None:
        if self.world == 1:
            return
        ops().comm_signal(self.row_ptrs(slot), self.arena.rank, int(value) & 0x7FFFFFFF,
                          self.arena.device.index or 0)

    def wait(self, slot: int, value: int) -> None:
        if self.world == 1:
            return
        row = self.flags[slot * self.world:(slot + 1) * self.world]
        ops().comm_wait(row, self.world, int(value) & 0x7FFFFFFF, self.wait_iters, self.status)
