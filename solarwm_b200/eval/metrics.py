"""Reference-based video metrics on tensors (no external models).

* ``psnr`` / ``ssim``: per-frame fidelity against a ground-truth clip (Gaussian-window SSIM, 11x11,
  sigma 1.5, on luma).
* ``flicker``: mean absolute temporal difference of the rendered clip minus that of the reference
  (positive = the render flickers more).
* ``edge_errors``: structure adherence -- gradient-magnitude edges of the render against the edges
  of the conditioning clip with a pixel tolerance: missed edges and extra edges as fractions
  (reference: eval/solar_renderer/metrics.py:471-508 uses Canny; a Sobel threshold stands in for
  it here, with the same tolerance dilation).

Model-based scores of the reference (DOVER, VideoScore2, CLIP/DINO embeddings, optical-flow
trackers, a VLM judge) need network weights that are not available offline; their aggregation
(`ratings.py`) is implemented, the scorers are not.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.nn.functional as F


def _luma(x: torch.Tensor) -> torch.Tensor:
    """[T, 3, H, W] in [0, 1] -> [T, 1, H, W]."""
    w = torch.tensor([0.299, 0.587, 0.114], device=x.device, dtype=x.dtype).view(1, 3, 1, 1)
    return (x * w).sum(1, keepdim=True)


def psnr(render: torch.Tensor, truth: torch.Tensor) -> float:
    mse = (render.float() - truth.float()).pow(2).mean(dim=(1, 2, 3)).clamp_min(1e-12)
    return float((10.0 * torch.log10(1.0 / mse)).mean())


def ssim(render: torch.Tensor, truth: torch.Tensor, window: int = 11, sigma: float = 1.5) -> float:
    x, y = _luma(render.float()), _luma(truth.float())
    g = torch.arange(window, dtype=torch.float32, device=x.device) - window // 2
    g = torch.exp(-(g ** 2) / (2 * sigma ** 2))
    g = (g / g.sum()).view(1, 1, -1)
    k = (g.transpose(1, 2) @ g).view(1, 1, window, window)
    mu_x, mu_y = F.conv2d(x, k), F.conv2d(y, k)
    sxx = F.conv2d(x * x, k) - mu_x ** 2
    syy = F.conv2d(y * y, k) - mu_y ** 2
    sxy = F.conv2d(x * y, k) - mu_x * mu_y
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    s = ((2 * mu_x * mu_y + c1) * (2 * sxy + c2)) / ((mu_x ** 2 + mu_y ** 2 + c1) * (sxx + syy + c2))
    return float(s.mean())


def flicker(render: torch.Tensor, truth: torch.Tensor) -> float:
    d = lambda v: (v[1:].float() - v[:-1].float()).abs().mean()   # noqa: E731
    return float(d(render) - d(truth))


def edges(clip: torch.Tensor, level: float = 0.25) -> torch.Tensor:
    """Boolean edge maps [T, H, W] from Sobel gradient magnitude of the luma."""
    y = _luma(clip.float())
    kx = torch.tensor([[-1.0, 0, 1], [-2, 0, 2], [-1, 0, 1]], device=y.device).view(1, 1, 3, 3)
    gx, gy = F.conv2d(y, kx, padding=1), F.conv2d(y, kx.transpose(2, 3), padding=1)
    return (gx ** 2 + gy ** 2).sqrt()[:, 0] > level


def edge_errors(render: torch.Tensor, condition: torch.Tensor, tolerance: int = 2, level: float = 0.25) -> Dict[str, float]:
    made, want = edges(render, level), edges(condition, level)
    grow = lambda m: F.max_pool2d(m.float().unsqueeze(1), 2 * tolerance + 1, 1, tolerance)[:, 0] > 0   # noqa: E731
    missed = (want & ~grow(made)).float().sum() / want.float().sum().clamp_min(1.0)
    extra = (made & ~grow(want)).float().sum() / made.float().sum().clamp_min(1.0)
    return {"missed": float(missed), "extra": float(extra)}


def compute(render: torch.Tensor, truth: torch.Tensor, condition: torch.Tensor = None) -> Dict[str, float]:
    out = {"psnr": psnr(render, truth), "ssim": ssim(render, truth), "flicker": flicker(render, truth)}
    if condition is not None:
        out.update({f"edge_{k}": v for k, v in edge_errors(render, condition).items()})
    return out
