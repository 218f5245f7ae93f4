"""Synthetic sources with the reference's tensor schemas (no dataset can be downloaded where the
benchmarks run): Wan / LTX / H3 preencoded samples in pinned host memory, random camera paths."""
from __future__ import annotations

import numpy as np
import torch


def random_camera_path(frames: int, seed: int = 0, rot_deg: float = 3.0, trans_std: float = 0.1) -> np.ndarray:
    """Per-frame 6-DoF poses: a random-walk SO(3) rotation and translation ~ N(0, trans_std); [T,4,4] C2W."""
    rng = np.random.default_rng(seed)
    out = np.tile(np.eye(4, dtype=np.float64), (frames, 1, 1))
    R, t = np.eye(3), np.zeros(3)
    for i in range(1, frames):
        axis = rng.normal(size=3)
        axis /= np.linalg.norm(axis) + 1e-12
        ang = np.deg2rad(rot_deg) * rng.normal()
        K = np.array([[0, -axis[2], axis[1]], [axis[2], 0, -axis[0]], [-axis[1], axis[0], 0]])
        R = R @ (np.eye(3) + np.sin(ang) * K + (1 - np.cos(ang)) * K @ K)
        t = t + rng.normal(scale=trans_std, size=3)
        out[i, :3, :3], out[i, :3, 3] = R, t
    return out.astype(np.float32)


def wan_sample(frames=31, channels=48, height=44, width=80, text_len=512, text_dim=4096, batch=1, seed=0, pin=True):
    g = torch.Generator().manual_seed(seed)
    lat = torch.randn(batch, frames, channels, height, width, generator=g).to(torch.bfloat16)
    txt = torch.randn(batch, text_len, text_dim, generator=g).to(torch.bfloat16)
    if pin and torch.cuda.is_available():
        lat, txt = lat.pin_memory(), txt.pin_memory()
    return {"latents": lat, "text": txt}


def h3_sample(latent_frames=47, channels=24, height=48, width=84, prompt_len=263, text_dim=5120, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"target_latents": torch.randn(channels, latent_frames, height, width, generator=g).to(torch.bfloat16),
            "anchor_latents": torch.randn(channels, 1, height, width, generator=g).to(torch.bfloat16),
            "prompt_embeds": torch.randn(prompt_len, text_dim, generator=g).to(torch.bfloat16),
            "text_token_tags": (torch.arange(prompt_len) % 2).to(torch.int32),
            "camera_c2w": torch.from_numpy(random_camera_path(latent_frames, seed))}


def ltx_sample(frames=16, channels=128, height=16, width=24, text_len=128, text_dim=4096, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {"latents": torch.randn(1, channels, frames, height, width, generator=g).to(torch.bfloat16),
            "text": torch.randn(1, text_len, text_dim, generator=g).to(torch.bfloat16)}
