"""Two-expert (high-noise / low-noise) operation of the A14B family.

The A14B checkpoints are two dense DiTs of the same architecture; the *high-noise* expert serves
``sigma >= boundary`` and the *low-noise* expert the rest (boundary 0.875 for I2V).  Only one expert
is trained per run: its timesteps are drawn from its own side of the boundary; at inference each
solver step calls the expert that owns the step's sigma, and only that expert has to be resident
(reference: solar/backends/wan22 family profile ``i2v_a14b`` and runtime/inference.py expert switch).

I2V conditioning ``y`` ([B, 4 + z, F, H, W]: a 4-channel first-frame mask plus the VAE latent of the
conditioning frame, zero elsewhere) is concatenated to the noisy latent on the channel axis by
``WanDiT.forward``; ``pack_i2v_condition`` builds it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch

BOUNDARY_I2V = 0.875


def expert_for_sigma(sigma: float, boundary: float = BOUNDARY_I2V) -> str:
    return "high_noise" if float(sigma) >= boundary else "low_noise"


def sample_expert_sigmas(n: int, expert: str, *, boundary: float = BOUNDARY_I2V, shift: float = 5.0,
                         generator=None, device="cpu") -> torch.Tensor:
    """Shifted uniform sigmas restricted to the expert's side of the boundary (rejection-free: the
    unshifted interval that maps onto the side is sampled directly)."""
    if expert not in ("high_noise", "low_noise"):
        raise ValueError(f"unknown expert {expert!r}")
    # invert sigma = s u / (1 + (s - 1) u) at the boundary
    u_b = boundary / (shift - (shift - 1.0) * boundary)
    lo, hi = (u_b, 1.0) if expert == "high_noise" else (0.0, u_b)
    u = lo + (hi - lo) * torch.rand(n, generator=generator, device=device)
    return shift * u / (1.0 + (shift - 1.0) * u)


def pack_i2v_condition(first_frame_latent: torch.Tensor, frames: int) -> torch.Tensor:
    """first_frame_latent [B, z, 1, H, W] -> y [B, 4 + z, F, H, W]."""
    B, z, _, H, W = first_frame_latent.shape
    y = torch.zeros(B, 4 + z, frames, H, W, dtype=first_frame_latent.dtype, device=first_frame_latent.device)
    y[:, :4, 0] = 1.0
    y[:, 4:, :1] = first_frame_latent
    return y


@dataclass
class ExpertPair:
    """Holds up to two models; ``load`` callbacks make an expert resident on demand so that a 180 GB
    device never needs both sets of optimizer state."""
    high_noise: Optional[torch.nn.Module] = None
    low_noise: Optional[torch.nn.Module] = None
    boundary: float = BOUNDARY_I2V
    load: Optional[Callable[[str], torch.nn.Module]] = None

    def model_for(self, sigma: float) -> torch.nn.Module:
        name = expert_for_sigma(sigma, self.boundary)
        m = getattr(self, name)
        if m is None:
            if self.load is None:
                raise RuntimeError(f"expert {name} is not resident and no loader was given")
            m = self.load(name)
            setattr(self, name, m)
        return m

    def __call__(self, x, t, context, **kw):
        """Dispatch on the (single) timestep of the call; per-frame timesteps must lie on one side."""
        sig = (t.float() / 1000.0)
        moving = sig[sig > 0]                      # clean conditioning frames (t = 0) do not vote
        side = moving if moving.numel() else sig
        hi = bool((side >= self.boundary).all())
        lo = bool((side < self.boundary).all())
        if not (hi or lo):
            raise ValueError("timesteps of one call straddle the expert boundary")
        return self.model_for(float(side.flatten()[0]))(x, t, context, **kw)


class TwoExpertTrainer:
    """Flow-matching training of BOTH experts of an A14B-style pair in one run.

    Every step draws the per-video sigma first -- on the host, from a generator that sequence-parallel peers seed
    alike, so that choosing the expert costs no device read -- and then runs the whole step (forward, backward,
    sharded update) on the expert that owns that side of ``boundary``: the high-noise expert for
    ``sigma >= boundary``, the low-noise expert below it.  Each expert is a complete ``WanStage0p5Trainer`` with its
    own sharded optimizer; the two share the sequence-parallel context and the symmetric heap.  With parameter
    sharding only ``1 / world`` of either expert's weights, gradients' reductions and optimizer state is resident.

    The reference trains the high-noise expert alone (its A14B recipe); the boundary switch follows the upstream
    Wan2.2 two-expert inference rule."""

    def __init__(self, high_noise, low_noise, *, boundary: float = BOUNDARY_I2V, shift: float = 5.0, seed: int = 0):
        self.trainers = {"high_noise": high_noise, "low_noise": low_noise}
        # one expert trains per step, so their captured steps can share one pool of activation memory: whichever
        # captures second borrows the first one's pool (two private pools of a 14B step do not fit beside each other)
        high_noise.graph_pool_donor, low_noise.graph_pool_donor = low_noise, high_noise
        self.boundary, self.shift = float(boundary), float(shift)
        self.host_gen = torch.Generator().manual_seed(int(seed) * 100003 + 17)
        self.steps = {"high_noise": 0, "low_noise": 0}
        self.last_expert = None

    def draw_sigma(self, n: int = 1) -> torch.Tensor:
        """Logit-normal sigmas with the timestep shift, on the host."""
        u = torch.sigmoid(torch.randn(n, generator=self.host_gen))
        return self.shift * u / (1.0 + (self.shift - 1.0) * u)

    def train_step(self, batch: dict, sigma: Optional[torch.Tensor] = None) -> torch.Tensor:
        sigma = self.draw_sigma(batch["latents"].shape[0]) if sigma is None else sigma
        sides = {expert_for_sigma(float(s), self.boundary) for s in sigma}
        if len(sides) != 1:
            raise ValueError("the sigmas of one micro-batch straddle the expert boundary (use micro-batch 1)")
        name = sides.pop()
        trainer = self.trainers[name]
        t_video = (sigma * trainer.scheduler.num_train_timesteps).to(torch.float32)
        if batch["latents"].is_cuda:
            t_video = t_video.to(batch["latents"].device)
        elif trainer.device.type == "cuda":
            t_video = t_video.pin_memory()
        self.steps[name] += 1
        self.last_expert = name
        return trainer.train_step({**batch, "t_video": t_video})
