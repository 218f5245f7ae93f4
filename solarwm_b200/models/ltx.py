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


class LTXDiT(WanDiT):
    """``forward(x [B,C,F,H,W], t [B,F], context [B,T,text_dim])`` -> velocity ``[B,C,F,H,W]``."""

    def __init__(self, cfg: WanConfig = None, device="cpu", dtype=torch.bfloat16, seed=0):
        super().__init__(cfg or ltx_preset(), device=device, dtype=dtype, seed=seed)
