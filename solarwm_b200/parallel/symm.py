"""Symmetric device buffers over CUDA IPC and the flag protocol used by the fused kernels.

``SymmetricHeap(nbytes, group)`` allocates the same-size device buffer on every rank of the group,
exchanges IPC handles through the process group (host-side plumbing, done once) and maps every
peer's buffer into this process.  ``ptrs[r]`` is rank r's buffer as addressable from here;
``tensor(...)`` gives torch views of the local buffer.  Flags are u32 words at the start of the
heap: ``flag_ptrs(slot)`` returns, per rank, the address of that slot in the rank's memory;
producers add 1 to it on every rank (``csrc/comm.cuh``) and ``wait(slot, expected)`` enqueues a
bounded device-side wait on the local word.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import check, ptr, stream_handle
from ..ops.functional import status_word

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
        self._flag_epoch: dict[int, int] = {}
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
        slot = self._next_slot
        self._next_slot += 2           # slot: the flag word; slot + 1: the producer's local CTA counter
        if self._next_slot * 4 > FLAG_BYTES:
            raise MemoryError("out of flag slots")
        self._flag_epoch[slot] = 0
        return slot

    def flag_ptrs(self, slot: int):
        return (ctypes.c_void_p * self.world)(*[p + 4 * slot for p in self.ptrs])

    def counter_ptr(self, slot: int):
        return ctypes.c_void_p(self.local_ptr + 4 * (slot + 1))

    def expect(self, slot: int, signals_per_round: Optional[int] = None) -> int:
        """Advance the slot's epoch and return the value the local flag must reach."""
        self._flag_epoch[slot] += signals_per_round if signals_per_round is not None else self.world
        return self._flag_epoch[slot]

    def wait(self, slot: int, expected: int, limit_seconds: float = 20.0) -> None:
        check(self.lib.solar_comm_wait(ctypes.c_void_p(self.local_ptr + 4 * slot), ctypes.c_uint(expected & 0xFFFFFFFF),
                                       ptr(status_word(self.device)), ctypes.c_double(limit_seconds), stream_handle()),
              "solar_comm_wait")
        _lib.count("comm_wait")

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        if self.group is not None or dist.is_initialized():
            dist.barrier(group=self.group)
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                self.lib.solar_comm_ipc_close(ctypes.c_void_p(p))
        self.lib.solar_comm_free(ctypes.c_void_p(self.local_ptr))
        self.ptrs = []
