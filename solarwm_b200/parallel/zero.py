"""ZeRO / FSDP-style sharding of the optimizer over flat units.

Every rank of the shard group keeps the full bf16 parameters (needed by its forward anyway) and
the full fp32 ``main_grad`` buffers, but owns the fp32 master weights, both Adam moments and the EMA
of one contiguous ``1 / world`` shard of every flat buffer.  One ``step``:

    reduce-scatter   this rank's shard of every gradient buffer = sum over ranks
    clip             global norm from the shard sums of squares (one small all-reduce)
    AdamW            fused kernel on the shard
    all-gather       refreshed bf16 parameters back into every rank's buffer

Two transports:

* ``collective``: ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` of the process group
  (NCCL on GPUs; on gloo, which has no reduce-scatter, an all-reduce followed by a local slice).
  This is what the reference gets from FSDP1 (solar/backends/wan22/runtime/distributed.py:73-123).
* ``fused``: parameter and gradient buffers live in a ``SymmetricHeap`` and no library collective runs:

  - reduce-scatter UNDER backward: as soon as a unit's gradients are final (``unit_ready``, called from the
    model's backward as each block finishes) a side stream exchanges a flag round with the peers and
    ``solar_zero_reduce`` pulls this rank's shard from every peer over NVLink while summing (and accumulating the
    sum of squares), so only the last unit's reduction is exposed after backward;
  - the global norm is one kernel (``SymmetricHeap.new_allsum``); a non-zero bounded-wait status word on ANY rank is
    folded into it as infinity, so every rank sees a non-finite norm, skips the update and can stop together;
  - ``solar_zero_adamw_push_multi`` applies AdamW to every shard of every buffer in ONE launch and stores the new
    bf16 parameters straight into every peer's buffer; learning rate and bias corrections are read from device
    memory, so the launch sequence of a step is identical from step to step (CUDA-graph replayable);
  - one flag round ("my pushes have landed") fences the step.
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
from ..ops.functional import status_word
from ..utils.trace import span


def fused_heap_bytes(units, world: int, sharded=(), slots: int = 2) -> int:
    """Bytes of symmetric heap the fused transport needs for ``units``: replicated units hold their bf16 parameters
    and fp32 gradients there; ``sharded`` units hold a ``1 / world`` parameter shard each and share ``slots`` fp32
    gradient buffers of the largest unit's size."""
    sharded_ids = {id(u) for u in sharded}
    total = 1 << 16
    for u in units:
        total += u.numel_v * 8 + 2048
        total += (u.numel_m * 2 // world + 512) if id(u) in sharded_ids else u.numel_m * 6
    if sharded_ids:
        total += slots * (max(u.numel_m for u in sharded) * 4 + 512)
    return total


class ZeroAdamW(FlatAdamW):
    def __init__(self, units: Iterable, group=None, *, transport: str = "collective", heap=None, replica_group=None,
                 reduce_ctas: int = 32, param_shards=None, **kw):
        """``group``: the ranks one copy of the optimizer state is sharded over.  ``replica_group`` (hybrid
        sharding): the ranks that hold the SAME shard in other shard groups (e.g. one per node); the reduced
        gradient shard is summed over it before the update, so every replica applies the identical step.
        ``reduce_ctas``: CTAs of one overlapped reduce launch (a small grid leaves the SMs to backward).
        ``param_shards``: a ``parallel.shard_params.ShardedParameters`` over some of the units (fused transport):
        those units keep only this rank's parameter shard and share gathered / gradient slots; their update writes
        the rank's own shard instead of pushing to every peer."""
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
        self.reduce_ctas = int(reduce_ctas)
        self._heap_off = {}
        self.param_shards = param_shards if (transport == "fused" and world > 1) else None
        self._sharded_units = {}
        if transport == "fused":
            if heap is None:
                raise ValueError("the fused transport needs a SymmetricHeap")
            for i, u in enumerate(units):
                k = None if self.param_shards is None else self.param_shards.index_of(u)
                if k is None:
                    u.ensure_grads()
                flat_v, off_pv = heap.alloc((u.numel_v,), u.flat_v.dtype)
                grad_v, off_gv = heap.alloc((u.numel_v,), torch.float32)
                if k is None:
                    flat, off_p = heap.alloc((u.numel_m,), u.flat.dtype)
                    grad, off_g = heap.alloc((u.numel_m,), torch.float32)
                    u.move_(flat, flat_v)
                    u.move_grads_(grad, grad_v)
                else:
                    # sharded unit: the matrices stay where they are until ``attach`` (the master weights are copied
                    # out of them below); only the small fp32 vectors move into the heap now
                    self._sharded_units[i] = k
                    flat_v.copy_(u.flat_v)
                    u.flat_v = flat_v
                    for name, prm in u.params.items():
                        if u.slots[name].is_vector:
                            prm.data = u.view(name)
                    grad_v.zero_()
                    u.grad_v = grad_v            # the matrix gradients come from the shared slots at ``attach``
                    off_p = self.param_shards.shard_off[k]
                    off_g = self.param_shards.gbuf_off[self.param_shards.slot_of(k)]
                self._heap_off[i] = {"m": (off_p, off_g), "v": (off_pv, off_gv)}
            self._flag_unit = [heap.new_flag() for _ in units]
            self._flag_params = heap.new_flag()
            self._allsum = heap.new_allsum(2)
            self._lib = _lib.load()
        super().__init__(units, shard_rank=rank, shard_world=world, **kw)
        self.world, self.rank = world, rank
        self._reduced_units: set = set()
        self._unit_index = {id(u): i for i, u in enumerate(self.units)}
        if transport == "fused" and world > 1:
            dev = self.units[0].device
            self._comm_stream = torch.cuda.Stream(device=dev)
            self._dyn = torch.zeros(4, dtype=torch.float32, device=dev)
            self._dyn_host = torch.zeros(4, dtype=torch.float32).pin_memory()
            self._norm_in = torch.zeros(2, dtype=torch.float32, device=dev)
            self._norm_out = torch.zeros(2, dtype=torch.float32, device=dev)
            self._host_prepared = False
            if self.param_shards is not None:
                self.param_shards.attach()
            self._build_table()

    # ------------------------------------------------------------------------------------
    def _buffers(self):
        for i, (u, st) in enumerate(zip(self.units, self.state)):
            for key, buf, g in (("m", u.flat, u.grad), ("v", u.flat_v, u.grad_v)):
                yield i, key, buf, g, st[key]

    def _build_table(self) -> None:
        """Device tables of every shard (one entry per flat buffer) for the single-launch AdamW: ``_tables`` is a list
        of (table, segments, chunks, ranks to write to); replicated buffers are pushed to every rank, sharded matrix
        buffers are written into this rank's own parameter shard only."""
        lib = self._lib
        lib.solar_zero_chunk_elems.restype = ctypes.c_longlong
        seg_bytes, chunk = int(lib.solar_zero_segment_bytes()), int(lib.solar_zero_chunk_elems())
        pushed, own = [], []
        for entry in self._buffers():
            i, key = entry[0], entry[1]
            (own if (key == "m" and i in self._sharded_units) else pushed).append(entry)
        self._tables = []
        for entries, to_all in ((pushed, True), (own, False)):
            if not entries:
                continue
            host = (ctypes.c_ubyte * (seg_bytes * len(entries)))()
            chunks = 0
            for idx, (i, key, buf, g, s) in enumerate(entries):
                a, b = s["range"]
                is_bf16 = buf.dtype == torch.bfloat16
                master = s["master"]
                if master is None:
                    if is_bf16:
                        raise ValueError("bf16 buffers need an fp32 master copy")
                    # fp32 vector units: the live shard is its own master; the kernel updates a copy and pushes it
                    master = self.__dict__.setdefault("_vec_master", {}).setdefault((i, key), buf[a:b].clone())
                # an own-shard segment addresses the shard buffer from its first element
                check(lib.solar_zero_segment_fill(host, ctypes.c_int(idx), ctypes.c_longlong(self._heap_off[i][key][0]),
                                                  ctypes.c_longlong(a if to_all else 0), ctypes.c_longlong(b - a),
                                                  ctypes.c_longlong(chunks), ptr(master), ptr(s["exp_avg"]),
                                                  ptr(s["exp_avg_sq"]), ptr(self._reduced(i, key, b - a, buf.device)),
                                                  ptr(s["ema"]) if s["ema"] is not None else None,
                                                  ctypes.c_int(1 if is_bf16 else 0)), "solar_zero_segment_fill")
                chunks += (b - a + chunk - 1) // chunk
            table = torch.frombuffer(bytearray(host), dtype=torch.uint8).clone().to(self.units[0].device)
            self._tables.append((table, len(entries), chunks, to_all))

    # reduce-scatter ------------------------------------------------------------------------
    def unit_ready(self, unit_or_index) -> None:
        """The gradients of one unit are final on this rank: start its reduce-scatter on the side stream.  Called
        from backward (per block) by the model; units nobody announced are reduced by ``reduce_scatter_grads``.
        No-op for the collective transport and for a single rank."""
        if self.transport != "fused" or self.world == 1:
            return
        i = unit_or_index if isinstance(unit_or_index, int) else self._unit_index[id(unit_or_index)]
        if i in self._reduced_units:
            return
        self._reduced_units.add(i)
        self.units[i].finalize_grads()
        main = torch.cuda.current_stream()
        done = torch.cuda.Event()
        done.record(main)
        h, side = self.heap, self._comm_stream
        with torch.cuda.stream(side):
            side.wait_event(done)
            slot = self._flag_unit[i]
            h.signal(slot)                               # this rank's gradients of unit i are complete
            h.wait(slot)                                 # ... and so are every peer's
            u, st = self.units[i], self.state[i]
            for key, g in (("m", u.grad), ("v", u.grad_v)):
                a, b = st[key]["range"]
                out = self._reduced(i, key, b - a, g.device)
                check(self._lib.solar_zero_reduce(h.peer_ptr_array(self._heap_off[i][key][1]), ctypes.c_int(self.world),
                                                  ctypes.c_longlong(a), ctypes.c_longlong(b - a), ptr(out),
                                                  ptr(self._norm_sq), ctypes.c_int(self.reduce_ctas), stream_handle()),
                      "solar_zero_reduce")
                _lib.count("zero_reduce")
            if i in self._sharded_units:
                self.param_shards.gradients_read(self._sharded_units[i])     # the shared gradient slot may be reused

    def reduce_scatter_grads(self) -> torch.Tensor:
        """Leaves the group-summed gradient in this rank's shard of every ``main_grad`` buffer and
        returns the (device) sum of squares of the local shards."""
        if self.world == 1:
            self._norm_sq.zero_()
            return self.local_grad_sumsq()
        if self.transport == "fused":
            for i in sorted(self._reduced_units):
                # a gradient that autograd delivered after the unit's overlapped reduce started would be lost
                late = [n for n, p in self.units[i].params.items() if p.grad is not None]
                if late:
                    raise RuntimeError(f"gradients arrived after unit {i} was announced ready: {late[:3]}")
            with span("zero.reduce_tail"):              # what backward did not hide
                for i in range(len(self.units)):
                    self.unit_ready(i)
                joined = torch.cuda.Event()
                joined.record(self._comm_stream)
                torch.cuda.current_stream().wait_event(joined)
            self._reduced_units.clear()
            return self._norm_sq
        self._norm_sq.zero_()
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
        if self.world > 1 and self.transport == "fused":
            # [sum of squares, "a bounded wait gave up on this rank"] summed over the ranks by one kernel of this
            # library; a failed wait anywhere makes the norm infinite everywhere (the update is then skipped)
            self._norm_in[0:1].copy_(sumsq.view(1))
            self._norm_in[1:2].copy_(status_word(sumsq.device).ne(0).to(torch.float32))
            self._allsum(self._norm_in, self._norm_out)
            total = torch.where(self._norm_out[1] > 0, torch.full_like(self._norm_out[0], float("inf")), self._norm_out[0])
            if sumsq.data_ptr() == self._norm_sq.data_ptr():
                self._norm_sq.zero_()                # consumed: the next step's overlapped reduces add into it again
            return total.sqrt()
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

    # update ----------------------------------------------------------------------------------
    def begin_step_host(self) -> None:
        """Host half of a fused step: advance the step count and stage {lr, 1 - beta1^t, 1 - beta2^t} in pinned
        memory.  ``step`` calls it itself; a caller that REPLAYS a captured step calls it before every replay (the
        captured copy then picks the fresh values up) and sets ``_host_prepared`` while capturing."""
        self.step_count += 1
        b1, b2 = self.betas
        self._dyn_host[0] = self.lr
        self._dyn_host[1] = 1.0 - b1 ** self.step_count
        self._dyn_host[2] = 1.0 - b2 ** self.step_count

    def step(self) -> None:
        if self.world == 1 or self.transport != "fused":
            super().step()
            if self.world > 1:
                self.all_gather_params()
            return
        with span("zero.adamw_push"):
            self._fused_update()

    def _fused_update(self) -> None:
        if not self._host_prepared:
            self.begin_step_host()
        self._dyn.copy_(self._dyn_host, non_blocking=True)
        b1, b2 = self.betas
        h = self.heap
        if self.param_shards is not None:
            self.param_shards.settle()
        for table, n_seg, n_chunks, to_all in self._tables:
            targets = list(h.ptrs) if to_all else [h.local_ptr]
            heaps = (ctypes.c_void_p * len(targets))(*targets)
            check(self._lib.solar_zero_adamw_push_multi(
                ptr(table), ctypes.c_int(n_seg), ctypes.c_longlong(n_chunks), heaps,
                ctypes.c_int(len(targets)), ctypes.c_float(b1), ctypes.c_float(b2), ctypes.c_float(self.eps),
                ctypes.c_float(self.weight_decay), ctypes.c_float(0.0 if self.ema_decay is None else self.ema_decay),
                ptr(self._dyn), ptr(self._scale), ptr(self._skip), ctypes.c_int(0), stream_handle()),
                "solar_zero_adamw_push_multi")
            _lib.count("zero_adamw_push")
        if self.param_shards is not None:
            self.param_shards.invalidate()
        h.signal(self._flag_params)                    # every rank's pushes have landed here
        h.wait(self._flag_params)

    def _live_shard(self, index: int, key: str) -> torch.Tensor:
        k = getattr(self, "_sharded_units", {}).get(index)
        if key == "m" and k is not None:
            return self.param_shards.shard[k]            # a sharded block's matrices live only as this rank's shard
        return super()._live_shard(index, key)

    def adopt_live_weights(self, reset_ema: bool = True) -> None:
        super().adopt_live_weights(reset_ema)
        self.__dict__.pop("_vec_master", None)           # fp32 vector shards are re-cloned at the next step
        if self.param_shards is not None:
            self.param_shards.invalidate()

    def _gather_shard(self, shard: torch.Tensor, total: int) -> torch.Tensor:
        """All ranks' shards of one state tensor, concatenated in rank order (a collective over the shard group)."""
        if self.world == 1:
            return shard
        shard = shard.contiguous()
        if dist.get_backend(self.group) == "gloo":
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard, group=self.group)
            return torch.cat(parts)
        full = torch.empty(total, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard, group=self.group)
        return full

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
