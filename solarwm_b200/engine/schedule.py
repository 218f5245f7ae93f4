"""Learning-rate schedule: linear warm-up then cosine decay to ``min_lr_ratio``
(reference: solar/training/schedule.py:11-28)."""
from __future__ import annotations

import math


def warmup_cosine_factor(step: int, *, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.1) -> float:
    step = int(step)
    if warmup_steps > 0 and step < warmup_steps:
        return (step + 1) / float(warmup_steps)
    if total_steps <= warmup_steps:
        return 1.0
    progress = min(1.0, max(0.0, (step - warmup_steps) / float(total_steps - warmup_steps)))
    cosine = 0.5 * (1.0 + math.cos(math.pi * progress))
    return min_lr_ratio + (1.0 - min_lr_ratio) * cosine


class WarmupCosine:
    """Stateful wrapper with the ``step`` / ``state_dict`` surface of a torch LR scheduler."""

    def __init__(self, optimizer, *, warmup_steps: int, total_steps: int, min_lr_ratio: float = 0.1):
        self.optimizer = optimizer
        self.warmup_steps, self.total_steps, self.min_lr_ratio = int(warmup_steps), int(total_steps), float(min_lr_ratio)
        self.base_lr = float(optimizer.lr)
        self.last_step = 0
        self._apply()

    def _apply(self):
        self.optimizer.lr = self.base_lr * warmup_cosine_factor(
            self.last_step, warmup_steps=self.warmup_steps, total_steps=self.total_steps,
            min_lr_ratio=self.min_lr_ratio)

    def step(self):
        self.last_step += 1
        self._apply()

    def state_dict(self):
        return {"last_step": self.last_step, "base_lr": self.base_lr}

    def load_state_dict(self, state):
        self.last_step = int(state["last_step"])
        self.base_lr = float(state["base_lr"])
        self._apply()
