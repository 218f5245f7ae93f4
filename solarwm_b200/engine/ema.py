"""Exponential moving average of parameters, kept in flat fp32 storage.

Two holders of the same average:

* the flat optimizer (``FlatAdamW(ema_decay=...)`` and its sharded subclass) refreshes one fp32 shadow per flat
  buffer inside the fused AdamW kernel; ``FlatEMAView`` names that shadow parameter by parameter, gathering the
  shards of a sharded optimizer first;
* ``ShardedEMA`` serves modules that are not built on flat units (the Stage-2 student, adapters): it packs the
  selected parameters of whatever shard the rank exposes into ONE fp32 vector and advances it with a pair of
  multi-tensor calls, instead of one ``mul_`` / ``add_`` pair per parameter.

Behaviour contract (reference: solar/training/ema.py:12-116): decay in [0, 1]; ``decay_for_step`` is 0 before the
warm-up step (the shadow then copies the live weights); names and shapes must match the live module on every
update, load and swap; ``swapped_into`` puts the average into the module for validation / saving and restores the
live weights afterwards, also when the body raises.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Dict, List, Mapping, Tuple

from ..errors import BackendContractError


def _unit_interval(value, what: str) -> float:
    v = float(value)
    if not 0.0 <= v <= 1.0:
        raise BackendContractError(f"{what} must be in [0,1]")
    return v


def ema_decay_for_step(*, target_decay: float, global_step: int, warmup_steps: int = 0) -> float:
    decay = _unit_interval(target_decay, "EMA decay")
    step, warm = int(global_step), int(warmup_steps)
    if step < 0 or warm < 0:
        raise BackendContractError("EMA step and warm-up must be non-negative")
    return decay if step >= warm else 0.0


class ShardedEMA:
    """fp32 (or any floating dtype) average of a module's parameters in one packed vector.

    ``layout`` maps a parameter name to ``(offset, shape)`` inside ``flat``; ``shadow`` is the name-keyed view of the
    same storage, so reading ``shadow[name]`` never copies."""

    def __init__(self, module, *, decay: float, device, dtype, trainable_only: bool = False):
        import torch

        self.decay = _unit_interval(decay, "EMA decay")
        if not (isinstance(dtype, torch.dtype) and dtype.is_floating_point):
            raise BackendContractError("EMA dtype must be floating point")
        self.device, self.dtype = torch.device(device), dtype
        self.trainable_only = bool(trainable_only)
        self.num_updates = 0
        self.layout: Dict[str, Tuple[int, tuple]] = {}
        cursor = 0
        picked = self._select(module)
        for name, p in picked:
            self.layout[name] = (cursor, tuple(p.shape))
            cursor += p.numel()
        if not self.layout:
            raise BackendContractError("EMA selected no parameters")
        self.flat = torch.empty(cursor, dtype=dtype, device=self.device)
        self._views: List[Any] = []
        self._bind_views()
        with torch.no_grad():
            for view, (_, p) in zip(self._views, picked):
                view.copy_(p.detach())

    # -- selection and layout checks -----------------------------------------------------------------------------
    def _select(self, module):
        inner = getattr(module, "module", module)
        return [(n, p) for n, p in inner.named_parameters() if p.requires_grad or not self.trainable_only]

    def _bind_views(self) -> None:
        self._views = [self.flat[off:off + _numel(shape)].view(shape) for off, shape in self.layout.values()]

    def _live(self, module):
        """The module's selected parameters in layout order, after checking names and shapes."""
        picked = dict(self._select(module))
        if picked.keys() != self.layout.keys():
            raise BackendContractError("EMA parameter names differ from the live model")
        ordered = []
        for name, (_, shape) in self.layout.items():
            if tuple(picked[name].shape) != shape:
                raise BackendContractError(f"EMA shard layout differs for {name}")
            ordered.append(picked[name])
        return ordered

    @property
    def shadow(self) -> Dict[str, Any]:
        return dict(zip(self.layout, self._views))

    # -- the average -----------------------------------------------------------------------------------------------
    def update(self, module, *, decay=None) -> None:
        import torch

        d = self.decay if decay is None else _unit_interval(decay, "EMA update decay")
        live = self._live(module)
        with torch.no_grad():
            fresh = [p.detach().to(device=self.device, dtype=self.dtype) for p in live]
            torch._foreach_mul_(self._views, d)
            torch._foreach_add_(self._views, fresh, alpha=1.0 - d)
        self.num_updates += 1

    def state_dict(self) -> dict:
        return {name: view.clone() for name, view in zip(self.layout, self._views)}

    def load_state_dict(self, values: Mapping[str, Any], *, num_updates: int) -> None:
        import torch

        if int(num_updates) < 0:
            raise BackendContractError("EMA update count must be non-negative")
        if set(values) != set(self.layout):
            raise BackendContractError("EMA checkpoint names differ from the live layout")
        staged = torch.empty_like(self.flat)
        for name, (off, shape) in self.layout.items():
            v = values[name]
            if tuple(v.shape) != shape or not v.is_floating_point():
                raise BackendContractError(f"EMA checkpoint layout differs for {name}")
            staged[off:off + _numel(shape)].view(shape).copy_(v.detach())
        self.flat = staged                      # all-or-nothing: nothing changes when any entry is refused
        self._bind_views()
        self.num_updates = int(num_updates)

    @contextmanager
    def swapped_into(self, module):
        import torch

        live = self._live(module)
        with torch.no_grad():
            kept = [p.detach().clone() for p in live]
        try:
            with torch.no_grad():
                for p, view in zip(live, self._views):
                    p.copy_(view)
            yield
        finally:
            with torch.no_grad():
                for p, k in zip(live, kept):
                    p.copy_(k)


def _numel(shape) -> int:
    n = 1
    for s in shape:
        n *= int(s)
    return n


class FlatEMAView:
    """Names the flat EMA shadows that the flat optimizer keeps.  With a sharded optimizer ``state_dict`` is a
    collective (every rank of the shard group calls it): the shards are gathered first, so the result is always the
    whole average in the un-sharded layout.  ``gathered``: an ``optimizer.state_dict()`` result to reuse."""

    def __init__(self, model, optimizer, gathered=None):
        if optimizer.ema_decay is None:
            raise BackendContractError("the optimizer was built without an EMA shadow")
        self.model, self.optimizer, self.gathered = model, optimizer, gathered

    def state_dict(self) -> dict:
        return self.optimizer.ema_state_dict(self.model, self.gathered)
