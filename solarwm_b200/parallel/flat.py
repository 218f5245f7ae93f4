"""Flat parameter units.

Each transformer block (and the stem / head) owns ONE contiguous bf16 buffer for its matrices
and biases and ONE contiguous fp32 buffer for its small vectors (norm weights, adaLN
modulation tables); ``nn.Parameter`` objects are views into those buffers, so

* checkpoints keep the reference's per-tensor names (``blocks.3.self_attn.q.weight`` ...),
* fused operands are free: ``q|k|v`` weights are adjacent, so one ``[3*dim, dim]`` view feeds
  a single QKV GEMM,
* gradients land in a flat fp32 ``main_grad`` buffer with the same layout (the wgrad GEMM's
  TMA store writes there directly), which is what the sharded optimizer, the gradient
  reduce-scatter and the norm computation consume without any per-parameter loop,
* a unit is the granularity of sharding (own FSDP: each rank owns ``1/world`` of every
  unit's master/moment buffers).

This replaces FSDP1's FlatParameter machinery used by the reference
(solar/backends/wan22/runtime/distributed.py:73-123).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch
import torch.nn as nn

ALIGN = 64  # elements; keeps every view 128-byte aligned for TMA and vector loads


@dataclass
class Slot:
    name: str
    shape: tuple
    is_vector: bool
    offset: int
    numel: int


def _round_up(n: int, a: int) -> int:
    return (n + a - 1) // a * a


class FlatUnit:
    """Owns the flat buffers of one unit and hands out parameter views."""

    def __init__(self, specs: Sequence[tuple], device, dtype=torch.bfloat16, grad_dtype=torch.float32,
                 pad_to: int = 1):
        self.device = torch.device(device)
        self.dtype = dtype
        self.grad_dtype = grad_dtype
        self.slots: dict[str, Slot] = {}
        off_m = off_v = 0
        for name, shape, is_vector in specs:
            n = 1
            for s in shape:
                n *= int(s)
            if is_vector:
                self.slots[name] = Slot(name, tuple(shape), True, off_v, n)
                off_v = _round_up(off_v + n, ALIGN)
            else:
                self.slots[name] = Slot(name, tuple(shape), False, off_m, n)
                off_m = _round_up(off_m + n, ALIGN)
        pad = ALIGN * max(int(pad_to), 1)
        self.numel_m = _round_up(max(off_m, ALIGN), pad)
        self.numel_v = _round_up(max(off_v, ALIGN), pad)
        vec_dtype = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        self.flat = torch.zeros(self.numel_m, dtype=dtype, device=self.device)
        self.flat_v = torch.zeros(self.numel_v, dtype=vec_dtype, device=self.device)
        self.grad = None
        self.grad_v = None
        self.params: dict[str, nn.Parameter] = {}

    # -- views ---------------------------------------------------------------------------
    def view(self, name: str) -> torch.Tensor:
        s = self.slots[name]
        buf = self.flat_v if s.is_vector else self.flat
        return buf[s.offset:s.offset + s.numel].view(s.shape)

    def span(self, first: str, last: str, shape) -> torch.Tensor:
        """One view covering the adjacent slots ``first..last`` (no padding may sit between)."""
        a, b = self.slots[first], self.slots[last]
        assert a.is_vector == b.is_vector
        buf = self.flat_v if a.is_vector else self.flat
        return buf[a.offset:b.offset + b.numel].view(shape)

    def grad_span(self, first: str, last: str, shape) -> torch.Tensor:
        a, b = self.slots[first], self.slots[last]
        buf = self.grad_v if a.is_vector else self.grad
        return buf[a.offset:b.offset + b.numel].view(shape)

    def parameter(self, name: str) -> nn.Parameter:
        if name not in self.params:
            p = nn.Parameter(self.view(name), requires_grad=True)
            p.flat_unit = self
            p.flat_name = name
            self.params[name] = p
        return self.params[name]

    # -- gradients -----------------------------------------------------------------------
    def ensure_grads(self) -> None:
        if self.grad is None:
            self.grad = torch.zeros(self.numel_m, dtype=self.grad_dtype, device=self.device)
            self.grad_v = torch.zeros(self.numel_v, dtype=torch.float32 if self.flat_v.dtype == torch.float32
                                      else self.grad_dtype, device=self.device)
        for name, p in self.params.items():
            s = self.slots[name]
            buf = self.grad_v if s.is_vector else self.grad
            p.main_grad = buf[s.offset:s.offset + s.numel].view(s.shape)
            p.grad_live = False

    def zero_grads(self, set_to_zero: bool = False) -> None:
        """Mark gradients as unwritten (first write overwrites); optionally clear the buffers."""
        if self.grad is None:
            return
        if set_to_zero:
            self.grad.zero_()
            self.grad_v.zero_()
        for p in self.params.values():
            p.grad_live = False

    def finalize_grads(self) -> None:
        """Zero the slices no kernel wrote this step and fold autograd ``.grad`` into main_grad."""
        for p in self.params.values():
            if p.grad is not None:
                if p.grad_live:
                    p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                else:
                    p.main_grad.copy_(p.grad)
                    p.grad_live = True
                p.grad = None
            if not p.grad_live:
                p.main_grad.zero_()

    def move_grads_(self, grad: torch.Tensor, grad_v: torch.Tensor) -> None:
        """Put the flat gradient buffers onto caller-provided storage (e.g. symmetric memory)."""
        assert grad.numel() == self.numel_m and grad_v.numel() == self.numel_v
        if self.grad is not None:
            grad.copy_(self.grad)
            grad_v.copy_(self.grad_v)
        else:
            grad.zero_()
            grad_v.zero_()
        self.grad, self.grad_v = grad, grad_v
        self.ensure_grads()

    def move_(self, flat: torch.Tensor, flat_v: torch.Tensor) -> None:
        """Re-home the unit onto caller-provided storage (e.g. symmetric memory)."""
        flat.copy_(self.flat)
        flat_v.copy_(self.flat_v)
        self.flat, self.flat_v = flat, flat_v
        for name, p in self.params.items():
            p.data = self.view(name)
