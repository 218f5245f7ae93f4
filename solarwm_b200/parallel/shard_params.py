"""Parameter sharding with just-in-time gathers (own FSDP FULL_SHARD, fused transport only).

Without this module every rank keeps all bf16 parameters and a full fp32 gradient buffer per block; with it a rank
keeps, per transformer block,

  * its ``1 / world`` shard of the block's flat bf16 buffer (in the symmetric heap, where peers can read it),
  * nothing else of the block's parameters or gradients between uses.

``slots`` (default 2) full-size *gathered* buffers and as many full-size fp32 *gradient* buffers are shared by all
blocks: block ``i`` permanently aliases slot ``i mod slots`` (its ``nn.Parameter`` views and ``main_grad`` views point
there and never move), so nothing is re-bound per step and a captured CUDA graph sees fixed addresses.

  gather      ``solar_comm_gather`` pulls the ``world`` shards of a block straight out of the peers' memory over
              NVLink into the block's slot, on a side stream, one block AHEAD of the compute stream (forward: block
              ``i + 1`` lands while block ``i`` runs; backward: block ``i - 1``); the compute stream waits on the
              gather's event just before the block's first GEMM reads the weights.  A slot is refilled only after the
              block that used it has released it (event), and a block that is still resident (the last forward blocks
              at the start of backward, a recomputed block) is not fetched again.
  gradients   the block's wgrad GEMMs write the slot's fp32 buffer; when the block's backward is done the sharded
              optimizer (``parallel/zero.py``) reduce-scatters it under the backward of the blocks below and then
              signals "I have read every rank's copy"; a gradient slot is written again only after that round.
  update      AdamW writes the refreshed bf16 values into the rank's own shard (no push to the peers: the next
              gather is the all-gather); a flag round at the end of the step orders shard updates before gathers.

The reference gets the same memory behaviour from FSDP1 FULL_SHARD with backward prefetch
(solar/backends/wan22/runtime/distributed.py:73-123, sequence_parallel.py:263-287); there the all-gather and the
reduce-scatter are NCCL collectives issued from module hooks.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch

from ..ops import _lib
from ..ops._lib import check, ptr, stream_handle
from ..utils.trace import span


class ShardedParameters:
    def __init__(self, units: Sequence, heap, *, slots: int = 2, gather_ctas: int = 48):
        """``units``: the flat units to shard (the transformer blocks, in execution order; every unit's ``numel_m``
        must be a multiple of ``8 * world``).  ``heap``: the symmetric heap that also carries the optimizer's
        buffers."""
        self.units = list(units)
        self.heap, self.world, self.rank = heap, heap.world, heap.rank
        self.slots = max(2, int(slots))
        self.gather_ctas = int(gather_ctas)
        self.lib = _lib.load()
        dev = self.units[0].device
        for u in self.units:
            if u.numel_m % (8 * self.world):
                raise ValueError("sharded units must be padded to a multiple of 8 * world elements")
        self.shard: List[torch.Tensor] = []
        self.shard_off: List[int] = []
        for u in self.units:
            per = u.numel_m // self.world
            t, off = heap.alloc((per,), u.flat.dtype)
            t.copy_(u.flat[self.rank * per:(self.rank + 1) * per])
            self.shard.append(t)
            self.shard_off.append(off)
        biggest = max(u.numel_m for u in self.units)
        self.gathered = [torch.empty(biggest, dtype=self.units[0].flat.dtype, device=dev) for _ in range(self.slots)]
        self.gbuf, self.gbuf_off = [], []
        for _ in range(self.slots):
            t, off = heap.alloc((biggest,), torch.float32)
            self.gbuf.append(t)
            self.gbuf_off.append(off)
        self.flag_read = [heap.new_flag() for _ in range(self.slots)]   # "every rank has read this gradient slot"
        self.stream = torch.cuda.Stream(device=dev)
        self.resident: List[Optional[int]] = [None] * self.slots
        self._gather_done: List[Optional[torch.cuda.Event]] = [None] * self.slots
        self._slot_free: List[Optional[torch.cuda.Event]] = [None] * self.slots
        self._grad_slot_pending = [False] * self.slots     # a reduce round of this step still reads the slot
        self._index = {id(u): i for i, u in enumerate(self.units)}
        self.attached = False

    # -- set-up -----------------------------------------------------------------------------------------------------
    def index_of(self, unit) -> Optional[int]:
        return self._index.get(id(unit))

    def slot_of(self, i: int) -> int:
        return i % self.slots

    def attach(self) -> None:
        """Point every unit at its slot (parameters and gradients alias the shared buffers from here on) and drop the
        full-size per-unit buffers.  Call after the optimizer has copied its master weights out of them."""
        for i, u in enumerate(self.units):
            s = self.slot_of(i)
            u.flat = self.gathered[s][:u.numel_m]
            for name, p in u.params.items():
                if not u.slots[name].is_vector:
                    p.data = u.view(name)
            u.grad = self.gbuf[s][:u.numel_m]
            u.ensure_grads()
        self.attached = True
        torch.cuda.empty_cache()

    # -- gathers ----------------------------------------------------------------------------------------------------
    def _issue_gather(self, i: int) -> None:
        s = self.slot_of(i)
        side = self.stream
        main = torch.cuda.current_stream()                   # the compute stream (read before switching streams)
        with torch.cuda.stream(side):
            if self._slot_free[s] is not None:
                side.wait_event(self._slot_free[s])          # the slot's previous block is done with it
            else:
                side.wait_stream(main)
            u = self.units[i]
            per_bytes = (u.numel_m // self.world) * u.flat.element_size()
            check(self.lib.solar_comm_gather(ptr(self.gathered[s]), self.heap.peer_ptr_array(self.shard_off[i]),
                                             ctypes.c_int(self.world), ctypes.c_longlong(per_bytes),
                                             ctypes.c_int(self.gather_ctas), stream_handle()), "solar_comm_gather")
            _lib.count("param_gather")
            done = torch.cuda.Event()
            done.record(side)
        self._gather_done[s] = done
        self.resident[s] = i

    def acquire(self, i: int, *, backward: bool = False) -> None:
        """Block ``i`` is about to run on the current stream: make its parameters resident, start the fetch of the
        block that runs next, and (backward) make sure the gradient slot may be overwritten."""
        s = self.slot_of(i)
        with span("fsdp.acquire"):
            if self.resident[s] != i:
                self._issue_gather(i)
            if self._gather_done[s] is not None:
                torch.cuda.current_stream().wait_event(self._gather_done[s])
            nxt = i - 1 if backward else i + 1
            if 0 <= nxt < len(self.units) and self.resident[self.slot_of(nxt)] != nxt:
                self._issue_gather(nxt)
            if backward and self._grad_slot_pending[s]:
                self.heap.wait(self.flag_read[s])            # all ranks finished reading the slot's previous gradients
                self._grad_slot_pending[s] = False

    def release(self, i: int) -> None:
        """Block ``i`` (forward or backward) has been enqueued completely on the current stream."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream())
        self._slot_free[self.slot_of(i)] = ev

    def gradients_read(self, i: int) -> None:
        """Called on the reduce stream after this rank's reduce of block ``i``: tell every rank."""
        s = self.slot_of(i)
        self.heap.signal(self.flag_read[s])
        self._grad_slot_pending[s] = True

    def settle(self) -> None:
        """End of a step, on the current stream: consume the read rounds nobody waited for (the last ``slots`` blocks
        of backward) so that every round's counter advances exactly once per use."""
        for s in range(self.slots):
            if self._grad_slot_pending[s]:
                self.heap.wait(self.flag_read[s])
                self._grad_slot_pending[s] = False

    def reset_events(self) -> None:
        """Forget every recorded event (the device must be idle): a CUDA-graph capture may only wait on events
        recorded inside the capture."""
        self._gather_done = [None] * self.slots
        self._slot_free = [None] * self.slots
        self.resident = [None] * self.slots

    def invalidate(self) -> None:
        """The shards changed (optimizer update): nothing that is gathered is current any more."""
        self.resident = [None] * self.slots

    # -- whole-model views (checkpoints) ----------------------------------------------------------------------------
    def materialize(self, model) -> Dict[str, torch.Tensor]:
        """``model.state_dict()`` for a sharded model: every block is gathered in turn and its tensors are copied to
        the host.  Collective in the sense that every rank must be past its last optimizer update."""
        out: Dict[str, torch.Tensor] = {}
        owner = {}
        for name, p in model.named_parameters():
            unit = getattr(p, "flat_unit", None)
            owner.setdefault(self.index_of(unit) if unit is not None else None, []).append((name, p))
        for idx, named in owner.items():
            if idx is not None:
                torch.cuda.current_stream().synchronize()
                self._slot_free[self.slot_of(idx)] = None
                self.resident[self.slot_of(idx)] = None
                self.acquire_only(idx)
                torch.cuda.current_stream().synchronize()
            for name, p in named:
                out[name] = p.detach().cpu().clone()
        for name, b in model.named_buffers():
            out.setdefault(name, b.detach().cpu().clone())
        self.invalidate()
        return out

    def load_state(self, model, weights) -> None:
        """Inverse of ``materialize``: take this rank's shard of every sharded block out of a full name -> tensor
        mapping (the other parameters are copied in place).  Strict about names and shapes."""
        named = dict(model.named_parameters())
        missing = sorted(set(named) - set(weights))
        extra = sorted(set(weights) - set(named) - {n for n, _ in model.named_buffers()})
        if missing or extra:
            raise KeyError(f"checkpoint weights do not match the model: missing {missing[:3]}, unexpected {extra[:3]}")
        torch.cuda.current_stream().synchronize()
        by_unit: Dict[Optional[int], list] = {}
        for name, p in named.items():
            unit = getattr(p, "flat_unit", None)
            by_unit.setdefault(self.index_of(unit) if unit is not None else None, []).append((name, p))
        with torch.no_grad():
            for idx, items in by_unit.items():
                for name, p in items:
                    if tuple(weights[name].shape) != tuple(p.shape):
                        raise ValueError(f"{name}: checkpoint shape {tuple(weights[name].shape)} != {tuple(p.shape)}")
                    p.copy_(weights[name])                    # sharded blocks: into the block's slot
                if idx is not None:
                    u = self.units[idx]
                    per = u.numel_m // self.world
                    self.shard[idx].copy_(u.flat[self.rank * per:(self.rank + 1) * per])
                    torch.cuda.current_stream().synchronize()
        self.invalidate()

    def acquire_only(self, i: int) -> None:
        s = self.slot_of(i)
        self._issue_gather(i)
        torch.cuda.current_stream().wait_event(self._gather_done[s])
