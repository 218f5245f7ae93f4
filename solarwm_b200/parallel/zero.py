"""ZeRO / FSDP-style sharding of the optimizer over flat units.

Every rank of the shard group keeps the full bf16 parameters (needed by its forward anyway) and
the full fp32 ``main_grad`` buffers, but owns the fp32 master weights, both Adam moments and the EMA
of one contiguous ``1 / world`` shard of every flat buffer.  One ``step``:

    reduce-scatter   this rank's shard of every gradient buffer = sum over ranks
    clip             global norm from the shard sums of squares (one scalar all-reduce)
    AdamW            fused kernel on the shard
    all-gather       refreshed bf16 parameters back into every rank's buffer

Two transports:

* ``collective``: ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` of the process group
  (NCCL on GPUs; on gloo, which has no reduce-scatter, an all-reduce followed by a local slice).
  This is what the reference gets from FSDP1 (solar/backends/wan22/runtime/distributed.py:73-123).
* ``fused``: parameter and gradient buffers live in a ``SymmetricHeap``; ``solar_zero_reduce`` pulls
  the shard from every peer over NVLink while summing, ``solar_zero_adamw_push`` applies Adam and
  stores the new bf16 parameters straight into every peer's buffer (``csrc/zero.cu``).  Two flag
  rounds fence the step: "my gradients are complete" before the pull and "my pushes have landed"
  after it.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, Optional

import torch
import torch.distributed as dist

from .. import ops
from ..engine.optim import FlatAdamW
from ..ops import _lib
from ..ops._lib import check, ptr, stream_handle


class ZeroAdamW(FlatAdamW):
    def __init__(self, units: Iterable, group=None, *, transport: str = "collective", heap=None, replica_group=None,
                 **kw):
        """``group``: the ranks one copy of the optimizer state is sharded over.  ``replica_group`` (hybrid
        sharding): the ranks that hold the SAME shard in other shard groups (e.g. one per node); the reduced
        gradient shard is summed over it before the update, so every replica applies the identical step."""
        self.group = group
        self.replica_group = replica_group
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        units = list(units)
        for u in units:
            if u.numel_m % (4 * world) or u.numel_v % (4 * world):
                raise ValueError("flat units must be padded to a multiple of 4 * shard world (FlatUnit pad_to)")
        self.transport = transport
        self.heap = heap
        self._heap_off = {}
        if transport == "fused":
            if heap is None:
                raise ValueError("the fused transport needs a SymmetricHeap")
            for i, u in enumerate(units):
                u.ensure_grads()
                flat, off_p = heap.alloc((u.numel_m,), u.flat.dtype)
                flat_v, off_pv = heap.alloc((u.numel_v,), u.flat_v.dtype)
                grad, off_g = heap.alloc((u.numel_m,), torch.float32)
                grad_v, off_gv = heap.alloc((u.numel_v,), torch.float32)
                u.move_(flat, flat_v)
                u.move_grads_(grad, grad_v)
                self._heap_off[i] = {"m": (off_p, off_g), "v": (off_pv, off_gv)}
            self._flag_grads = heap.new_flag()
            self._flag_params = heap.new_flag()
            self._lib = _lib.load()
        super().__init__(units, shard_rank=rank, shard_world=world, **kw)
        self.world, self.rank = world, rank

    # ------------------------------------------------------------------------------------
    def _buffers(self):
        for i, (u, st) in enumerate(zip(self.units, self.state)):
            for key, buf, g in (("m", u.flat, u.grad), ("v", u.flat_v, u.grad_v)):
                yield i, key, buf, g, st[key]

    def _signal_and_wait(self, slot: int) -> None:
        h = self.heap
        check(self._lib.solar_comm_signal(h.flag_ptrs(slot), ctypes.c_int(h.world), stream_handle()), "solar_comm_signal")
        _lib.count("comm_signal")
        h.wait(slot, h.expect(slot))

    def reduce_scatter_grads(self) -> torch.Tensor:
        """Leaves the group-summed gradient in this rank's shard of every ``main_grad`` buffer and
        returns the (device) sum of squares of the local shards."""
        self._norm_sq.zero_()
        if self.world == 1:
            return self.local_grad_sumsq()
        if self.transport == "fused":
            self._signal_and_wait(self._flag_grads)          # every rank's backward is complete
            for i, key, buf, g, s in self._buffers():
                a, b = s["range"]
                off_g = self._heap_off[i][key][1]
                out = self._reduced(i, key, b - a, g.device)
                check(self._lib.solar_zero_reduce(self.heap.peer_ptr_array(off_g), ctypes.c_int(self.world),
                                                  ctypes.c_longlong(a), ctypes.c_longlong(b - a), ptr(out),
                                                  ptr(self._norm_sq), ctypes.c_int(0), stream_handle()),
                      "solar_zero_reduce")
                _lib.count("zero_reduce")
            return self._norm_sq
        backend = dist.get_backend(self.group)
        for i, key, buf, g, s in self._buffers():
            a, b = s["range"]
            if backend == "gloo":
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
            else:
                dist.reduce_scatter_tensor(g[a:b], g, op=dist.ReduceOp.SUM, group=self.group)
        return self.local_grad_sumsq()

    def _reduced(self, i, key, n, device):
        store = self.__dict__.setdefault("_reduced_bufs", {})
        if (i, key) not in store:
            store[(i, key)] = torch.empty(n, dtype=torch.float32, device=device)
        return store[(i, key)]

    def _replica_sum(self) -> None:
        """Hybrid sharding: sum this rank's reduced gradient shards over its replica group."""
        if self.replica_group is None or dist.get_world_size(self.replica_group) == 1:
            return
        for i, key, buf, g, s in self._buffers():
            a, b = s["range"]
            shard = self._reduced(i, key, b - a, g.device) if (self.transport == "fused" and self.world > 1) else g[a:b]
            dist.all_reduce(shard, op=dist.ReduceOp.SUM, group=self.replica_group)

    def global_grad_norm(self, sumsq: torch.Tensor) -> torch.Tensor:
        if self.replica_group is not None and dist.get_world_size(self.replica_group) > 1:
            self._replica_sum()
            sumsq = self._shard_sumsq()              # the shards changed: recompute their sum of squares
        if self.world > 1:
            dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=self.group)
        return sumsq.sqrt()

    def _shard_sumsq(self) -> torch.Tensor:
        first = True
        for i, key, buf, g, s in self._buffers():
            a, b = s["range"]
            shard = self._reduced(i, key, b - a, g.device) if (self.transport == "fused" and self.world > 1) else g[a:b]
            ops.sumsq(shard, out=self._norm_sq, accumulate=not first)
            first = False
        return self._norm_sq

    def step(self) -> None:
        if self.world == 1 or self.transport != "fused":
            super().step()
            if self.world > 1:
                self.all_gather_params()
            return
        self.step_count += 1
        b1, b2 = self.betas
        for i, key, buf, g, s in self._buffers():
            a, b = s["range"]
            off_p = self._heap_off[i][key][0]
            is_bf16 = buf.dtype == torch.bfloat16
            master = s["master"] if s["master"] is not None else buf[a:b]
            if s["master"] is None and not is_bf16:
                # fp32 vector units: the live shard is its own master; push a copy to the peers
                master = self.__dict__.setdefault("_vec_master", {}).setdefault((i, key), buf[a:b].clone())
            check(self._lib.solar_zero_adamw_push(
                self.heap.peer_ptr_array(off_p), ctypes.c_int(1 if is_bf16 else 0), ctypes.c_int(self.world),
                ctypes.c_longlong(a), ctypes.c_longlong(b - a), ptr(master), ptr(s["exp_avg"]), ptr(s["exp_avg_sq"]),
                ptr(self._reduced(i, key, b - a, buf.device)), ptr(s["ema"]) if s["ema"] is not None else None,
                ctypes.c_float(self.lr), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(self.eps),
                ctypes.c_float(self.weight_decay), ctypes.c_int(self.step_count),
                ctypes.c_float(0.0 if self.ema_decay is None else self.ema_decay), ptr(self._scale), ptr(self._skip),
                ctypes.c_int(0), stream_handle()), "solar_zero_adamw_push")
            _lib.count("zero_adamw_push")
        self._signal_and_wait(self._flag_params)              # every rank's pushes have landed here

    def all_gather_params(self) -> None:
        backend = dist.get_backend(self.group)
        for i, key, buf, g, s in self._buffers():
            a, b = s["range"]
            if backend == "gloo":
                parts = [torch.empty(b - a, dtype=buf.dtype, device=buf.device) for _ in range(self.world)]
                dist.all_gather(parts, buf[a:b].contiguous(), group=self.group)
                buf.copy_(torch.cat(parts))
            else:
                dist.all_gather_into_tensor(buf, buf[a:b], group=self.group)

    def sharded_step(self, max_norm: Optional[float]) -> torch.Tensor:
        """reduce-scatter -> global norm -> clip -> AdamW on the shard -> all-gather; returns the norm."""
        norm = self.global_grad_norm(self.reduce_scatter_grads())
        self.set_clip(norm, max_norm)
        self.step()
        return norm
