"""Projective positional encoding (PRoPE) for camera-conditioned attention.

For a token seen by camera ``(K, V)`` (intrinsics, world-to-camera view matrix) let
``P = lift(K_norm) @ V`` with ``K_norm = diag(fx, fy, 1)`` (principal point dropped) and ``lift`` the
embedding of a 3x3 into a 4x4.  Every 4-vector of a head's channels is multiplied by

    q <- P^T q        k <- P^-1 k        v <- P^-1 v        attention output <- P o

with ``P^-1 = V^-1 lift(K_norm^-1)`` built in closed form from the rigid inverse, in fp32; without
intrinsics ``P = V`` (GTA form).  The translation of first-frame-relative view matrices can first be
compressed with ``logd4``: ``t <- t * log1p(|t|) / (4 |t|)``.

The per-row matrices feed ``ops.head_norm_rope_prope`` (``csrc/headops.cu``): with ``rot_dims=0`` the
whole 128-channel head is transformed (Wan), with ``rot_dims=96`` only channels [96, 128) (H3).
Reference: solar/backends/wan22/runtime/modeling/camera_prope.py:34-338, runtime/camera.py:29-66.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import ops


def transform_translation(viewmats: torch.Tensor, transform: str = "linear") -> torch.Tensor:
    if transform == "linear":
        return viewmats
    if transform != "logd4":
        raise ValueError(f"unknown camera_translation_transform {transform!r}")
    t = viewmats[..., :3, 3].float()
    n = torch.linalg.vector_norm(t, dim=-1, keepdim=True)
    scale = torch.where(n > 0, torch.log1p(n) / (4.0 * n.clamp_min(torch.finfo(torch.float32).tiny)), torch.zeros_like(n))
    out = viewmats.clone()
    out[..., :3, 3] = (t * scale).to(viewmats.dtype)
    return out


def invert_se3(v: torch.Tensor) -> torch.Tensor:
    R, t = v[..., :3, :3], v[..., :3, 3:]
    out = torch.zeros_like(v)
    out[..., :3, :3] = R.transpose(-1, -2)
    out[..., :3, 3:] = -R.transpose(-1, -2) @ t
    out[..., 3, 3] = 1.0
    return out


def prope_matrices(viewmats: torch.Tensor, Ks: Optional[torch.Tensor] = None, *, transform: str = "linear"
                   ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """viewmats [..., 4, 4], Ks [..., 3, 3] or None -> (P^T, P^-1, P), each fp32 [..., 4, 4]."""
    v = transform_translation(viewmats.float(), transform)
    if Ks is None:
        P, Pinv = v, invert_se3(v)
    else:
        fx, fy = Ks[..., 0, 0].float(), Ks[..., 1, 1].float()
        one = torch.ones_like(fx)
        lift = torch.diag_embed(torch.stack([fx, fy, one, one], dim=-1))
        lift_inv = torch.diag_embed(torch.stack([1.0 / fx, 1.0 / fy, one, one], dim=-1))
        P = lift @ v
        Pinv = invert_se3(v) @ lift_inv
    return P.transpose(-1, -2).contiguous(), Pinv.contiguous(), P.contiguous()


def per_row(mats: torch.Tensor, rows_per_camera: int) -> torch.Tensor:
    """[cameras, 4, 4] -> [cameras * rows_per_camera, 4, 4] (token order: camera-major)."""
    return mats.repeat_interleave(rows_per_camera, dim=0).contiguous()


def apply(x: torch.Tensor, mats: torch.Tensor, heads: int, rot_dims: int = 0) -> torch.Tensor:
    """x [rows, heads * 128]; mats fp32 [rows, 4, 4] -> every 4-vector of channels [rot_dims, 128) of
    each head multiplied by the row's matrix."""
    hd = x.shape[1] // heads
    if hd != 128 and rot_dims == 0 and x.shape[1] % 128 == 0:
        # the matrix acts on every 4-vector of a row alike, so head boundaries do not matter to the camera-only
        # transform: narrower heads (LTX: 64) ride the 128-wide kernel as pseudo-heads
        heads = x.shape[1] // 128
    return ops.head_norm_rope_prope(x, None, None, None, mats.float().contiguous(), heads=heads, rot_dims=rot_dims)
