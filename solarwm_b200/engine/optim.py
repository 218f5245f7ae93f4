"""Sharded fp32-master AdamW over flat parameter units, one fused kernel launch per buffer.

State per unit (only the slice this rank owns when sharded): fp32 master copy of the bf16
matrices, fp32 first/second moments, optional fp32 EMA shadow.  ``step`` applies decoupled weight
decay, the Adam update, refreshes the bf16 live parameters and the EMA in a single pass over
memory (``csrc/pointwise.cu: adamw_kernel``); the gradient scale (clip coefficient) and a
skip flag are read from device memory, so clipping needs no host round trip.

Reference behaviour: ``FP32MasterAdamW`` (solar/training/optim.py:18-226) loops over parameters
with ~8 element-wise kernels each, ``ShardedEMA.update`` (solar/training/ema.py:71-81) adds a
``mul_/add_`` pair per parameter; both are folded into the one kernel here.
"""
from __future__ import annotations

from typing import Iterable, Mapping, Optional

import torch

from .. import ops


def shard_bounds(numel: int, rank: int, world: int):
    per = numel // world
    assert per * world == numel, "flat units must be padded to a multiple of the shard count"
    return rank * per, (rank + 1) * per


class FlatAdamW:
    def __init__(self, units: Iterable, *, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, shard_rank: int = 0, shard_world: int = 1,
                 ema_decay: Optional[float] = None):
        self.units = list(units)
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), tuple(betas), float(eps), float(weight_decay)
        self.shard_rank, self.shard_world = int(shard_rank), int(shard_world)
        self.ema_decay = ema_decay
        self.step_count = 0
        self.state = []
        for u in self.units:
            entry = {}
            for key, buf in (("m", u.flat), ("v", u.flat_v)):
                a, b = shard_bounds(buf.numel(), self.shard_rank, self.shard_world)
                live = buf[a:b]
                needs_master = live.dtype != torch.float32
                entry[key] = {
                    "range": (a, b),
                    "master": live.float().clone() if needs_master else None,
                    "exp_avg": torch.zeros(b - a, dtype=torch.float32, device=live.device),
                    "exp_avg_sq": torch.zeros(b - a, dtype=torch.float32, device=live.device),
                    "ema": live.float().clone() if ema_decay is not None else None,
                }
            self.state.append(entry)
        dev = self.units[0].device
        self._norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)

    # gradients ---------------------------------------------------------------------------
    def _grad_shards(self):
        for u, st in zip(self.units, self.state):
            for key, g in (("m", u.grad), ("v", u.grad_v)):
                a, b = st[key]["range"]
                yield g[a:b]

    def local_grad_sumsq(self) -> torch.Tensor:
        """Sum of squares of this rank's gradient shards (device scalar, no host sync)."""
        first = True
        for g in self._grad_shards():
            ops.sumsq(g, out=self._norm_sq, accumulate=not first)
            first = False
        return self._norm_sq

    def set_clip(self, total_norm: torch.Tensor, max_norm: Optional[float]) -> None:
        """clip coefficient min(1, max_norm / (norm + 1e-6)); a non-finite norm raises the skip flag."""
        finite = torch.isfinite(total_norm)
        self._skip.copy_((~finite).to(torch.int32).view(1))
        if max_norm is None:
            self._scale.fill_(1.0)
        else:
            self._scale.copy_(torch.clamp(max_norm / (total_norm + 1e-6), max=1.0).view(1))

    # update ------------------------------------------------------------------------------
    def step(self) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        for u, st in zip(self.units, self.state):
            for key, buf, g in (("m", u.flat, u.grad), ("v", u.flat_v, u.grad_v)):
                s = st[key]
                a, b = s["range"]
                live = buf[a:b]
                master = s["master"] if s["master"] is not None else live
                ops.adamw_(master, s["exp_avg"], s["exp_avg_sq"], g[a:b],
                           live=live if s["master"] is not None else None, ema=s["ema"], lr=self.lr,
                           beta1=b1, beta2=b2, eps=self.eps, wd=self.weight_decay, step=self.step_count,
                           grad_scale=self._scale, skip=self._skip,
                           ema_decay=0.0 if self.ema_decay is None else self.ema_decay)

    # state -------------------------------------------------------------------------------
    _STATE_TENSORS = ("master", "exp_avg", "exp_avg_sq", "ema")

    def _gather_shard(self, shard: torch.Tensor, total: int) -> torch.Tensor:
        """The un-sharded tensor a shard belongs to; the unsharded optimizer holds it already.  Sharded
        subclasses make this a collective over their shard group."""
        return shard

    def state_dict(self, keep: bool = True):
        """State in the UN-SHARDED layout: every tensor covers the whole flat buffer, whatever the number of ranks the
        optimizer is sharded over, so that a checkpoint can be resumed at another shard count.  With a sharded
        optimizer this is a collective: every rank of the shard group must call it.  ``keep`` = False on the ranks
        that will not write the checkpoint: they take part in every gather and drop the result instead of copying
        tens of gigabytes to their host memory (their tensors are ``None``)."""
        out = {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
               "weight_decay": self.weight_decay, "layout": "full", "units": []}
        for u, st in zip(self.units, self.state):
            entry = {}
            for key, buf in (("m", u.flat), ("v", u.flat_v)):
                s = st[key]
                entry[key] = {"numel": int(buf.numel())}
                for name in self._STATE_TENSORS:
                    t = s[name]
                    if t is None:
                        entry[key][name] = None
                        continue
                    full = self._gather_shard(t.detach(), buf.numel())
                    entry[key][name] = full.cpu() if keep else None
                    del full
            out["units"].append(entry)
        return out

    def load_state_dict(self, state) -> None:
        """Accepts the un-sharded layout written by ``state_dict`` (each rank copies its own ``[a, b)`` range) and
        refuses a checkpoint whose un-sharded sizes differ from this model's."""
        if state.get("layout") != "full":
            shard = tuple(state.get("shard", (0, 1)))
            if shard != (0, 1):
                raise ValueError("optimizer state was saved as one rank's shard; it cannot be resumed")
        if len(state["units"]) != len(self.state):
            raise ValueError("optimizer state has a different number of flat units")
        self.step_count = int(state["step"])
        for u, st, saved in zip(self.units, self.state, state["units"]):
            for k, buf in (("m", u.flat), ("v", u.flat_v)):
                a, b = st[k]["range"]
                total = int(saved[k].get("numel", buf.numel())) if isinstance(saved[k], dict) else buf.numel()
                if total != buf.numel():
                    raise ValueError(f"optimizer state covers {total} elements, the flat buffer {buf.numel()}")
                for n in self._STATE_TENSORS:
                    mine, theirs = st[k][n], saved[k].get(n)
                    if mine is None or theirs is None:
                        continue
                    if mine.dtype != theirs.dtype:
                        raise ValueError("optimizer state dtype mismatch (casting is refused)")
                    if theirs.numel() != total:
                        raise ValueError("optimizer state tensor does not cover the whole flat buffer")
                    mine.copy_(theirs[a:b])

    # weights that arrive from outside the optimizer ----------------------------------------------------------------
    def _live_shard(self, index: int, key: str) -> torch.Tensor:
        """This rank's range of the live parameters of unit ``index`` (``key``: "m" matrices, "v" vectors)."""
        u = self.units[index]
        a, b = self.state[index][key]["range"]
        return (u.flat if key == "m" else u.flat_v)[a:b]

    @torch.no_grad()
    def adopt_live_weights(self, reset_ema: bool = True) -> None:
        """The live parameters were overwritten from outside (a weights-only checkpoint load): take them as the fp32
        master weights -- otherwise the first step would write the OLD master back over them -- and, with
        ``reset_ema``, restart the EMA shadow from them.  Moments and the step counter are left alone."""
        for i, st in enumerate(self.state):
            for key in ("m", "v"):
                live = self._live_shard(i, key).float()
                if st[key]["master"] is not None:
                    st[key]["master"].copy_(live)
                if reset_ema and st[key]["ema"] is not None:
                    st[key]["ema"].copy_(live)

    @torch.no_grad()
    def load_named_ema(self, model, named: Mapping[str, torch.Tensor]) -> None:
        """EMA shadow from a parameter-name -> tensor mapping (e.g. a checkpoint's averaged weights next to its live
        ones); every rank copies the part of each parameter that falls into its own range.  Strict about names and
        shapes."""
        if self.ema_decay is None:
            raise ValueError("the optimizer was built without an EMA shadow")
        index = {id(u): i for i, u in enumerate(self.units)}
        params = dict(model.named_parameters())
        if set(params) != set(named):
            odd = sorted(set(params) ^ set(named))
            raise ValueError(f"averaged weights do not match the model (e.g. {odd[:4]})")
        for name, p in params.items():
            slot = p.flat_unit.slots[p.flat_name]
            src = named[name]
            if tuple(src.shape) != tuple(slot.shape):
                raise ValueError(f"{name}: averaged weight has shape {tuple(src.shape)}, the model {tuple(slot.shape)}")
            st = self.state[index[id(p.flat_unit)]]["v" if slot.is_vector else "m"]
            a, b = st["range"]
            lo, hi = max(a, slot.offset), min(b, slot.offset + slot.numel)
            if lo < hi:
                st["ema"][lo - a:hi - a].copy_(src.reshape(-1)[lo - slot.offset:hi - slot.offset].to(st["ema"].device, torch.float32))

    @torch.no_grad()
    def load_named_moments(self, model, named: Mapping[str, Mapping[str, torch.Tensor]], step: int) -> None:
        """Adam moments from a per-parameter mapping ``{name: {"exp_avg", "exp_avg_sq"}}`` -- the form a
        ``torch.optim.AdamW`` full state takes once its entries are keyed by parameter name (the reference's
        checkpoints) -- packed into the flat buffers; parameters the mapping does not name keep zero moments only if
        ``named`` is empty for them everywhere, otherwise the mismatch is an error."""
        index = {id(u): i for i, u in enumerate(self.units)}
        params = dict(model.named_parameters())
        if set(params) != set(named):
            odd = sorted(set(params) ^ set(named))
            raise ValueError(f"optimizer entries do not match the model's parameters (e.g. {odd[:4]})")
        for name, p in params.items():
            slot = p.flat_unit.slots[p.flat_name]
            st = self.state[index[id(p.flat_unit)]]["v" if slot.is_vector else "m"]
            a, b = st["range"]
            lo, hi = max(a, slot.offset), min(b, slot.offset + slot.numel)
            for field in ("exp_avg", "exp_avg_sq"):
                src = named[name][field]
                if src.numel() != slot.numel:
                    raise ValueError(f"{name}: {field} has {src.numel()} elements, the parameter {slot.numel}")
                if lo < hi:
                    st[field][lo - a:hi - a].copy_(src.reshape(-1)[lo - slot.offset:hi - slot.offset].to(st[field].device, torch.float32))
        self.step_count = int(step)

    def ema_state_dict(self, model, gathered=None) -> dict:
        """The EMA shadow under the model's parameter names (un-sharded).  ``gathered``: a ``state_dict()`` result to
        take the shadows from (saves a second gather); collective when sharded, like ``state_dict``."""
        if self.ema_decay is None:
            raise ValueError("the optimizer was built without an EMA shadow")
        state = gathered if gathered is not None else self.state_dict()
        by_unit = {id(u): saved for u, saved in zip(self.units, state["units"])}
        out = {}
        for name, p in model.named_parameters():
            unit, slot = p.flat_unit, p.flat_unit.slots[p.flat_name]
            full = by_unit[id(unit)]["v" if slot.is_vector else "m"]["ema"]
            out[name] = full[slot.offset:slot.offset + slot.numel].view(slot.shape).clone()
        return out
