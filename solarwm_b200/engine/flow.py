"""Flow-matching schedule and objective math (Wan convention: x_t = (1-s) x0 + s n, target n - x0).

``FlowMatchScheduler`` reproduces the shifted linear schedule and the Gaussian timestep weights
of the reference (solar/backends/wan22/runtime/scheduler.py:60-112); the tensor math itself runs
in the fused scheduler kernel (``ops.add_noise`` / ``flow_to_x0`` / ``euler_step``).
NumPy twins used as CPU oracles mirror solar/backends/wan22/objectives.py:24-91.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .. import ops


def apply_timestep_shift(s, shift: float):
    """s * shift / (1 + (shift - 1) s) on tensors, arrays or floats in [0, 1]."""
    if not math.isfinite(float(shift)) or float(shift) <= 0:
        raise ValueError("shift must be positive and finite")
    if float(shift) == 1.0:
        return s
    return float(shift) * s / (1.0 + (float(shift) - 1.0) * s)


class FlowMatchScheduler:
    def __init__(self, num_train_timesteps: int = 1000, shift: float = 3.0, sigma_max: float = 1.0,
                 sigma_min: float = 0.0, extra_one_step: bool = True):
        self.num_train_timesteps = int(num_train_timesteps)
        self.shift = float(shift)
        self.sigma_max, self.sigma_min = float(sigma_max), float(sigma_min)
        self.extra_one_step = bool(extra_one_step)
        self.set_timesteps(self.num_train_timesteps, training=True)

    def set_timesteps(self, steps: int, training: bool = False) -> None:
        steps = int(steps)
        count = steps + 1 if self.extra_one_step else steps
        s = torch.linspace(self.sigma_max, self.sigma_min, count)
        if self.extra_one_step:
            s = s[:-1]
        self.sigmas = self.shift * s / (1 + (self.shift - 1) * s)
        self.timesteps = self.sigmas * self.num_train_timesteps
        if training:
            w = torch.exp(-2 * ((self.timesteps - steps / 2) / steps) ** 2)
            w = w - w.min()
            self.linear_timesteps_weights = w * (steps / w.sum())

    def _on(self, name: str, device) -> torch.Tensor:
        """The schedule table ``name`` on ``device`` (copied once per table and device, not once per step)."""
        src = getattr(self, name)
        if src.device == torch.device(device):
            return src
        cache = self.__dict__.setdefault("_device_tables", {})
        hit = cache.get((name, str(device)))
        if hit is None or hit[0] is not src:
            hit = (src, src.to(device))
            cache[(name, str(device))] = hit
        return hit[1]

    def indices(self, timestep: torch.Tensor) -> torch.Tensor:
        v = timestep.flatten().float()
        sched = self._on("timesteps", v.device)
        return (sched.unsqueeze(0) - v.unsqueeze(1)).abs().argmin(dim=1)

    def sigma_of(self, timestep: torch.Tensor) -> torch.Tensor:
        return self._on("sigmas", timestep.device)[self.indices(timestep)]

    def training_weight(self, timestep: torch.Tensor) -> torch.Tensor:
        return self._on("linear_timesteps_weights", timestep.device)[self.indices(timestep)]

    def add_noise(self, clean, noise, timestep):
        """clean/noise ``[G, ...]`` with one timestep per leading row -> (x_t, velocity target)."""
        return ops.add_noise(clean, noise, self.sigma_of(timestep).float())


def logit_normal_sigmas(n: int, shift: float, generator=None, device="cpu", mean=0.0, std=1.0):
    """Logit-normal sigma sampling with timestep shift (the training recipe of the Wan-5B-shaped benchmark)."""
    u = torch.randn(n, generator=generator, device=device) * std + mean
    return apply_timestep_shift(torch.sigmoid(u), shift)


def first_frame_loss_mask(batch: int, frames: int, dropped: torch.Tensor) -> torch.Tensor:
    """TI2V: frame 0 is a clean condition and is supervised only when the image is dropped."""
    dropped = torch.as_tensor(dropped, dtype=torch.bool)
    if tuple(dropped.shape) != (batch,):
        raise ValueError(f"dropped must have shape {(batch,)}")
    mask = torch.ones((batch, frames), dtype=torch.bool, device=dropped.device)
    mask[:, 0] = dropped
    return mask


# ---- NumPy twins (oracles) -------------------------------------------------------------
def rectified_interpolate_array(clean, noise, sigma):
    clean = np.asarray(clean, dtype=np.float64)
    noise = np.asarray(noise, dtype=np.float64)
    s = np.asarray(sigma, dtype=np.float64)
    while s.ndim < clean.ndim:
        s = s[..., None]
    return (1.0 - s) * clean + s * noise


def velocity_target_array(clean, noise):
    return np.asarray(noise, dtype=np.float64) - np.asarray(clean, dtype=np.float64)


def weighted_masked_mse_array(pred, target, mask, weight):
    pred = np.asarray(pred, dtype=np.float64)
    target = np.asarray(target, dtype=np.float64)
    m = np.asarray(mask, dtype=bool)
    w = np.asarray(weight, dtype=np.float64)
    while m.ndim < pred.ndim:
        m = m[..., None]
    while w.ndim < pred.ndim:
        w = w[..., None]
    valid = np.broadcast_to(m, pred.shape)
    diff = np.where(valid, pred - target, 0.0)
    return float(((diff ** 2) * w).sum() / max(valid.sum(), 1.0))
