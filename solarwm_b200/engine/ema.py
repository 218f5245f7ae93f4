"""Exponential moving average of parameters.

``ShardedEMA`` keeps an fp32 shadow per named parameter of whatever shards the rank exposes and
offers ``swapped_into`` for EMA validation / saving (reference: solar/training/ema.py:12-116).  When
the flat optimizer is used the shadow is updated inside the fused AdamW kernel instead
(``FlatAdamW(ema_decay=...)``); ``FlatEMAView`` exposes that flat shadow under parameter names so
both paths produce the same ``generator_ema`` state dict.
"""
from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Mapping

from ..errors import BackendContractError


def ema_decay_for_step(*, target_decay: float, global_step: int, warmup_steps: int = 0) -> float:
    decay, step, warm = float(target_decay), int(global_step), int(warmup_steps)
    if not 0 <= decay <= 1 or step < 0 or warm < 0:
        raise BackendContractError("invalid EMA decay/step/warmup")
    return 0.0 if step < warm else decay


class ShardedEMA:
    def __init__(self, module, *, decay: float, device, dtype, trainable_only: bool = False):
        import torch

        if not 0 <= float(decay) <= 1:
            raise BackendContractError("EMA decay must be in [0,1]")
        if not isinstance(dtype, torch.dtype) or not dtype.is_floating_point:
            raise BackendContractError("EMA dtype must be floating point")
        self.decay, self.device, self.dtype = float(decay), torch.device(device), dtype
        self.trainable_only = bool(trainable_only)
        self.num_updates = 0
        self.shadow = {n: p.detach().to(device=self.device, dtype=dtype).clone() for n, p in self._named(module)}
        if not self.shadow:
            raise BackendContractError("EMA selected no parameters")

    def _named(self, module):
        root = getattr(module, "module", module)
        return [(n, p) for n, p in root.named_parameters() if not self.trainable_only or p.requires_grad]

    def _checked(self, module):
        named = self._named(module)
        if {n for n, _ in named} != set(self.shadow):
            raise BackendContractError("EMA parameter names differ from the live model")
        for n, p in named:
            s = self.shadow[n]
            if s.shape != p.shape or s.dtype != self.dtype:
                raise BackendContractError(f"EMA shard layout differs for {n}")
        return named

    def update(self, module, *, decay=None) -> None:
        import torch

        d = self.decay if decay is None else float(decay)
        if not 0 <= d <= 1:
            raise BackendContractError("EMA update decay must be in [0,1]")
        with torch.no_grad():
            for n, p in self._checked(module):
                self.shadow[n].mul_(d).add_(p.detach().to(device=self.device, dtype=self.dtype), alpha=1 - d)
        self.num_updates += 1

    def state_dict(self) -> dict:
        return {n: v.clone() for n, v in self.shadow.items()}

    def load_state_dict(self, values: Mapping[str, Any], *, num_updates: int) -> None:
        if set(values) != set(self.shadow):
            raise BackendContractError("EMA checkpoint names differ from the live layout")
        new = {}
        for n, cur in self.shadow.items():
            v = values[n]
            if v.shape != cur.shape or not v.is_floating_point():
                raise BackendContractError(f"EMA checkpoint layout differs for {n}")
            new[n] = v.detach().to(device=self.device, dtype=self.dtype, copy=True)
        if int(num_updates) < 0:
            raise BackendContractError("EMA update count must be non-negative")
        self.shadow, self.num_updates = new, int(num_updates)

    @contextmanager
    def swapped_into(self, module):
        import torch

        named = self._checked(module)
        live = {n: p.detach().clone() for n, p in named}
        try:
            with torch.no_grad():
                for n, p in named:
                    p.copy_(self.shadow[n].to(device=p.device, dtype=p.dtype))
            yield
        finally:
            with torch.no_grad():
                for n, p in self._named(module):
                    p.copy_(live[n])


class FlatEMAView:
    """Names the flat EMA shadows kept by ``FlatAdamW`` (full, un-sharded layout only)."""

    def __init__(self, model, optimizer):
        self.model, self.optimizer = model, optimizer
        if optimizer.ema_decay is None:
            raise BackendContractError("the optimizer was built without an EMA shadow")
        if optimizer.shard_world != 1:
            raise BackendContractError("gather the EMA shards before naming them")

    def state_dict(self) -> dict:
        out = {}
        units = {id(u): st for u, st in zip(self.optimizer.units, self.optimizer.state)}
        for name, p in self.model.named_parameters():
            unit, slot = p.flat_unit, p.flat_unit.slots[p.flat_name]
            st = units[id(unit)]["v" if slot.is_vector else "m"]
            out[name] = st["ema"][slot.offset:slot.offset + slot.numel].view(slot.shape).clone()
        return out
