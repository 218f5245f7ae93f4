"""Symmetric device buffers over CUDA IPC and the flag protocol used by the fused kernels.

``SymmetricHeap(nbytes, group)`` allocates the same-size device buffer on every rank of the group,
exchanges IPC handles through the process group (host-side plumbing, done once) and maps every
peer's buffer into this process.  ``ptrs[r]`` is rank r's buffer as addressable from here;
``alloc(...)`` gives torch views of the local buffer.  Flags are groups of four u32 words at the
start of the heap -- the flag itself, two last-CTA counters for producer kernels and the round
counter of the waiting side: ``flag_ptrs(slot)`` returns, per rank, the address of the flag word in
that rank's memory; producers add 1 to it on every rank (``csrc/comm.cuh``) and
``wait(slot, signals)`` enqueues a bounded device-side wait for ``signals`` more arrivals than the
previous round had.  The round count lives on the device, so a launch sequence that contains waits
can be captured once in a CUDA graph and replayed.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import check, ptr, stream_handle
from ..ops.functional import status_word
from ..utils.trace import span

FLAG_BYTES = 4096          # 1024 flag / counter words at the start of every heap


class _RawCuda:
    """Minimal ``__cuda_array_interface__`` carrier so torch can view externally owned memory."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3}


class SymmetricHeap:
    def __init__(self, nbytes: int, group: Optional[dist.ProcessGroup] = None, device=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = torch.device(device if device is not None else torch.cuda.current_device())
        self.nbytes = FLAG_BYTES + (int(nbytes) + 255) // 256 * 256
        self.lib = _lib.load()
        local = ctypes.c_void_p()
        check(self.lib.solar_comm_alloc(ctypes.c_longlong(self.nbytes), ctypes.byref(local)), "solar_comm_alloc")
        self.local_ptr = int(local.value)
        handle = (ctypes.c_ubyte * 64)()
        check(self.lib.solar_comm_ipc_handle(ctypes.c_void_p(self.local_ptr), handle), "solar_comm_ipc_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            out = ctypes.c_void_p()
            check(self.lib.solar_comm_ipc_open(buf, ctypes.byref(out)), "solar_comm_ipc_open")
            self.ptrs.append(int(out.value))
        self._bytes = torch.as_tensor(_RawCuda(self.local_ptr, self.nbytes), device=self.device)
        self._cursor = FLAG_BYTES
        self._next_slot = 0
        dist.barrier(group=group)

    # -- memory ---------------------------------------------------------------------------
    def alloc(self, shape, dtype=torch.bfloat16):
        """Carve a tensor out of the local buffer (same offset on every rank); returns (tensor, offset)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._cursor + 255) // 256 * 256
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {off + nbytes} of {self.nbytes} bytes")
        self._cursor = off + nbytes
        return self._bytes[off:off + nbytes].view(dtype).view(*shape), off

    def peer_ptr_array(self, offset: int):
        """``void*[world]``: address of ``offset`` in every rank's buffer (as seen from this process)."""
        return (ctypes.c_void_p * self.world)(*[p + offset for p in self.ptrs])

    # -- flags ----------------------------------------------------------------------------
    def new_flag(self) -> int:
        """A flag group: word ``slot`` is the flag, ``slot + 1`` / ``slot + 2`` are last-CTA counters for up to two
        producer kernels that may run at the same time, ``slot + 3`` is the waiting side's round counter."""
        slot = self._next_slot
        self._next_slot += 4
        if self._next_slot * 4 > FLAG_BYTES:
            raise MemoryError("out of flag slots")
        return slot

    def flag_ptrs(self, slot: int):
        return (ctypes.c_void_p * self.world)(*[p + 4 * slot for p in self.ptrs])

    def counter_ptr(self, slot: int, which: int = 0):
        return ctypes.c_void_p(self.local_ptr + 4 * (slot + 1 + int(which)))

    def epoch_ptr(self, slot: int):
        return ctypes.c_void_p(self.local_ptr + 4 * (slot + 3))

    def wait(self, slot: int, signals: Optional[int] = None, limit_seconds: float = 20.0) -> None:
        """Bounded device-side wait until ``signals`` (default: one per rank) more arrivals than the previous
        round's total have reached this rank's flag word.  On a timeout the kernel sets the status word and
        returns; ``ops.read_status`` / ``ops.check_status`` report it."""
        add = self.world if signals is None else int(signals)
        with span("comm_wait"):
            self._wait_launch(slot, add, limit_seconds)

    def _wait_launch(self, slot: int, add: int, limit_seconds: float) -> None:
        check(self.lib.solar_comm_wait_round(ctypes.c_void_p(self.local_ptr + 4 * slot), self.epoch_ptr(slot),
                                             ctypes.c_uint(add), ptr(status_word(self.device)),
                                             ctypes.c_double(limit_seconds), stream_handle()),
              "solar_comm_wait_round")
        _lib.count("comm_wait")

    def signal(self, slot: int) -> None:
        """Add 1 to the flag word of ``slot`` on every rank, ordered after everything enqueued so far."""
        check(self.lib.solar_comm_signal(self.flag_ptrs(slot), ctypes.c_int(self.world), stream_handle()),
              "solar_comm_signal")
        _lib.count("comm_signal")

    def new_allsum(self, n: int):
        """A small all-reduce (sum of ``n <= 256`` fp32 values over the ranks) that runs as one kernel of this
        library; returns a callable ``(src, out) -> out``."""
        table, off = self.alloc((2, self.world, int(n)), torch.float32)
        slot = self.new_flag()
        tables = self.peer_ptr_array(off)
        flags = self.flag_ptrs(slot)

        def allsum(src: torch.Tensor, out: torch.Tensor, limit_seconds: float = 20.0) -> torch.Tensor:
            assert src.dtype == torch.float32 and out.dtype == torch.float32 and src.numel() == n == out.numel()
            check(self.lib.solar_comm_allsum(ptr(src), ctypes.c_int(n), tables, flags, ctypes.c_int(self.world),
                                             ctypes.c_int(self.rank), self.epoch_ptr(slot), ptr(out),
                                             ptr(status_word(self.device)), ctypes.c_double(limit_seconds),
                                             stream_handle()), "solar_comm_allsum")
            _lib.count("comm_allsum")
            return out

        allsum.table = table
        return allsum

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.group is not None or dist.is_initialized():
            dist.barrier(group=self.group)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.lib.solar_comm_ipc_close(ctypes.c_void_p(p))
        self.lib.solar_comm_free(ctypes.c_void_p(self.local_ptr))
        self.ptrs = []
