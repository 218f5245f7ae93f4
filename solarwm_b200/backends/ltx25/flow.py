"""LTX rectified-flow objective: shifted logit-normal sigma whose mean grows linearly with the token
count (1024 tokens -> 0.95, 4096 -> 2.05; std 1.0; 10 % uniform samples), first latent frame kept
clean as the image condition, velocity target ``noise - clean``, loss excludes frame 0
(reference: solar/backends/ltx25/torch_flow.py:14-118; NumPy twins in flow.py)."""
from __future__ import annotations


import numpy as np
import torch


def sigma_mean_for_tokens(tokens: int, lo=(1024, 0.95), hi=(4096, 2.05)) -> float:
    (t0, m0), (t1, m1) = lo, hi
    return m0 + (m1 - m0) * (tokens - t0) / (t1 - t0)


def sample_sigmas(batch: int, tokens: int, *, generator=None, device="cpu", std: float = 1.0, uniform_fraction: float = 0.1):
    mu = sigma_mean_for_tokens(tokens)
    z = torch.randn(batch, generator=generator, device=device) * std + mu
    s = torch.sigmoid(z)
    u = torch.rand(batch, generator=generator, device=device)
    pick = torch.rand(batch, generator=generator, device=device) < uniform_fraction
    return torch.where(pick, u, s)


def noisy_input_and_target(clean, noise, sigma):
    """clean/noise [B, C, F, H, W]; sigma [B].  Frame 0 stays clean (per-frame sigma 0)."""
    B, _, F = clean.shape[:3]
    per_frame = sigma.view(B, 1).expand(B, F).clone()
    per_frame[:, 0] = 0.0
    s = per_frame.view(B, 1, F, 1, 1).to(clean.dtype)
    return (1 - s) * clean + s * noise, noise - clean, per_frame


def masked_flow_loss(pred, target):
    """Mean squared error over frames 1.. (frame 0 is the condition)."""
    return (pred[:, :, 1:].float() - target[:, :, 1:].float()).pow(2).mean()


def sigma_mean_for_tokens_array(tokens):
    return 0.95 + (2.05 - 0.95) * (np.asarray(tokens, dtype=np.float64) - 1024.0) / (4096.0 - 1024.0)
