"""FP32-master AdamW for an arbitrary list of (typically bf16 LoRA) parameters.

The parameters are packed once into one contiguous live buffer (each parameter becomes a view), with
fp32 master / first / second moment buffers of the same length, so a step is one fused kernel
launch instead of the reference's per-parameter Python loop of ~8 element-wise kernels
(solar/training/optim.py:18-226; H3 twin solar/backends/minimax_h3/optimizer.py:96-133).
``load_state_dict`` refuses dtype casts, as the reference does."""
from __future__ import annotations

from typing import Iterable, Optional

import torch

from .. import ops


class FP32MasterAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], *, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0):
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("optimizer got no trainable parameters")
        dev, dt = self.params[0].device, self.params[0].dtype
        sizes = [(p.numel() + 63) // 64 * 64 for p in self.params]
        total = sum(sizes)
        self.live = torch.zeros(total, dtype=dt, device=dev)
        self.grad = torch.zeros(total, dtype=torch.float32, device=dev)
        self.offsets = []
        off = 0
        for p, n in zip(self.params, sizes):
            self.live[off:off + p.numel()].copy_(p.data.reshape(-1))
            p.data = self.live[off:off + p.numel()].view(p.shape)
            self.offsets.append(off)
            off += n
        self.master = self.live.float().clone()
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.lr, self.betas, self.eps, self.weight_decay = float(lr), tuple(betas), float(eps), float(weight_decay)
        self.step_count = 0
        self._scale = torch.ones(1, dtype=torch.float32, device=dev)
        self._skip = torch.zeros(1, dtype=torch.int32, device=dev)

    def gather_grads(self) -> torch.Tensor:
        """Copy ``.grad`` of every parameter into the flat fp32 gradient buffer (zeros where absent)."""
        self.grad.zero_()
        for p, off in zip(self.params, self.offsets):
            if p.grad is not None:
                self.grad[off:off + p.numel()].copy_(p.grad.reshape(-1))
        return self.grad

    def clip_(self, max_norm: Optional[float]) -> torch.Tensor:
        norm = ops.sumsq(self.grad).sqrt()
        finite = torch.isfinite(norm)
        self._skip.copy_((~finite).to(torch.int32).view(1))
        if max_norm is not None:
            self._scale.copy_(torch.clamp(max_norm / (norm + 1e-6), max=1.0).view(1))
        return norm

    def step(self) -> None:
        self.step_count += 1
        ops.adamw_(self.master, self.exp_avg, self.exp_avg_sq, self.grad, live=self.live, lr=self.lr, beta1=self.betas[0],
                   beta2=self.betas[1], eps=self.eps, wd=self.weight_decay, step=self.step_count, grad_scale=self._scale,
                   skip=self._skip)

    def zero_grad(self) -> None:
        for p in self.params:
            p.grad = None

    def state_dict(self):
        return {"step": self.step_count, "master": self.master.cpu(), "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu(), "lr": self.lr}

    def load_state_dict(self, state) -> None:
        for name in ("master", "exp_avg", "exp_avg_sq"):
            src, dst = state[name], getattr(self, name)
            if src.dtype != dst.dtype or src.shape != dst.shape:
                raise ValueError(f"optimizer state {name} has a different dtype or shape (casting is refused)")
            dst.copy_(src)
        self.step_count = int(state["step"])
        self.live.copy_(self.master.to(self.live.dtype))
