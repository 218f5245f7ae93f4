"""H3 flow convention (data-ward): ``x_t = t x0 + (1 - t) n``, target ``x0 - n``, ``x0 = x_t + (1 - t) v``,
timestep shift 12 for video and 3 for audio, Euler step in fp32
(reference: solar/backends/minimax_h3/torch_flow.py:27-141)."""
from __future__ import annotations

import torch

VIDEO_SHIFT, AUDIO_SHIFT = 12.0, 3.0


def shifted_sigma(u, shift: float):
    """u in [0,1] noise level -> shifted noise level."""
    return shift * u / (1.0 + (shift - 1.0) * u)


def interpolate(x0, noise, t):
    t = torch.as_tensor(t, dtype=torch.float32, device=x0.device)
    return (t * x0.float() + (1.0 - t) * noise.float()).to(x0.dtype)


def target(x0, noise):
    return x0.float() - noise.float()


def x0_from_velocity(x_t, v, t):
    return (x_t.float() + (1.0 - float(t)) * v.float()).to(x_t.dtype)


def rollout_times(steps: int = 4, shift: float = VIDEO_SHIFT):
    """t_k = 1 - sigma_k with sigma from linspace(1, 0, steps + 1) shifted."""
    s = shifted_sigma(torch.linspace(1.0, 0.0, steps + 1), shift)
    return (1.0 - s).tolist()
