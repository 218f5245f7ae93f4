"""LTX-shaped video DiT.  The block structure (adaLN scale/shift/gate table + timestep embedding,
full-width q/k RMSNorm + 3-axis RoPE, text cross-attention, GELU-tanh FFN) is the Wan block with
RMSNorm as the pre-modulation norm, patch size 1 and 64-wide heads, so it runs on the same fused
operators (reference: solar/backends/ltx25/torch_model.py:125-371, which wraps the external
``ltx_core`` transformer; dims of the benchmark shape: 28 blocks, 2048 wide, 32 heads x 64,
128-channel latents, 128 text tokens of width 4096)."""
from __future__ import annotations

import torch

from .wan import WanConfig, WanDiT, wan_preset


def ltx_preset(name: str = "ltx_video_2b") -> WanConfig:
    if name == "tiny":
        return WanConfig(model_type="t2v", patch_size=(1, 1, 1), in_dim=16, out_dim=16, dim=128, ffn_dim=256, num_heads=2,
                         num_layers=2, text_dim=64, text_len=16, freq_dim=64, norm_type="rms", cross_attn_norm=False)
    return wan_preset(name)


# The LTX camera path is parameter-free PRoPE with ONE fixed normalised focal length for every frame (the Wan
# training cameras' 969.7-pixel focal on a 1920 x 1080 sensor), not per-sample intrinsics
# (reference: solar/backends/ltx25/torch_prope.py:21-71).
FIXED_FX_NORM = 969.6969696969696 / (960.0 * 2)
FIXED_FY_NORM = 969.6969696969696 / (540.0 * 2)


def ltx_camera_condition(viewmats: torch.Tensor, transform: str = "linear") -> dict:
    """viewmats [B, F, 4, 4] (first-frame-relative world-to-camera) -> the ``y_camera`` argument of ``forward``
    with the fixed intrinsics; ``transform`` is the translation compression ("linear" or "logd4")."""
    if viewmats.dim() != 4 or tuple(viewmats.shape[-2:]) != (4, 4):
        raise ValueError("viewmats must be [B, F, 4, 4]")
    Ks = torch.zeros(*viewmats.shape[:2], 3, 3, dtype=torch.float32, device=viewmats.device)
    Ks[..., 0, 0], Ks[..., 1, 1] = FIXED_FX_NORM, FIXED_FY_NORM
    Ks[..., 0, 2] = Ks[..., 1, 2] = 0.5
    Ks[..., 2, 2] = 1.0
    return {"viewmats": viewmats, "Ks": Ks, "transform": transform}


class LTXDiT(WanDiT):
    """``forward(x [B,C,F,H,W], t [B,F], context [B,T,text_dim])`` -> velocity ``[B,C,F,H,W]``."""

    def __init__(self, cfg: WanConfig = None, device="cpu", dtype=torch.bfloat16, seed=0):
        super().__init__(cfg or ltx_preset(), device=device, dtype=dtype, seed=seed)
