"""Causal 3-D convolutional video VAE (Wan-style) with streaming decode.

Building blocks (reference: solar/backends/wan22/runtime/modeling/vae.py:19-868):
  * ``CausalConv3d``: temporal padding on the past side only; in streaming mode the last
    ``kt - 1`` input frames of every convolution are kept in a feature cache so decoding chunk by
    chunk is bit-for-bit the same function as decoding the whole clip
  * ``RMSNormC``: channel RMS norm with a learned gain; ``ResBlock`` (norm-SiLU-conv x2 + skip)
  * ``FrameAttention``: single-head attention over the pixels of each frame
  * ``Upsample``: nearest 2x spatial (+ temporal doubling through a causal conv that emits two
    frames per input frame, the first latent frame excepted)
  * ``Decoder3d`` / ``Encoder3d`` and ``VideoVAE.encode / decode / cached_decode``

On a B200 the stride-1 convolutions of inference (every convolution of the decoder) run on this package's
implicit-GEMM kernel over channels-last activations (``ops.functional.conv3d_channels_last``: tcgen05 MMAs fed
by 4-D TMA box loads whose out-of-range reads supply the spatial and the causal padding); training-time,
strided (encoder down-sampling) and CPU convolutions go through ``torch.nn.functional.conv3d``.  Pixel
conversion uses ``ops.rgb8``.  ``StreamingDecoder`` owns the per-layer caches and is what the
realtime server calls once per generated chunk.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class CausalConv3d(nn.Conv3d):
    def __init__(self, cin, cout, kernel=3, stride=1):
        k = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
        super().__init__(cin, cout, k, stride=stride, padding=0)
        self.pad_t = k[0] - 1
        self.pad_hw = (k[2] // 2, k[2] // 2, k[1] // 2, k[1] // 2)

    def _native_ok(self, x) -> bool:
        # inference on a B200: bf16 activations, stride 1, channel count the TMA strides allow
        return (x.is_cuda and x.dtype == torch.bfloat16 and tuple(self.stride) == (1, 1, 1) and x.shape[1] % 8 == 0
                and not (torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad)))

    def _forward_native(self, x, cache, key):
        """Channels-last implicit-GEMM kernel: no padded copy, the border and the causal history are TMA fills.
        The result is returned as an NCDHW view of channels-last memory, so a following convolution's layout
        change is free."""
        from ..ops import functional as F_

        tag = (self.weight.data_ptr(), self.weight._version, str(x.device))
        if getattr(self, "_packed_tag", None) != tag:
            self._packed = F_.pack_conv_weight(self.weight, self.bias)
            self._packed_tag = tag
        w, b = self._packed
        xc = x.permute(0, 2, 3, 4, 1).contiguous()                      # [B, T, H, W, C]
        ck = None if key is None else key + "#cl"
        outs = []
        hist = cache.get(ck) if (cache is not None and self.pad_t) else None
        for i in range(xc.shape[0]):
            outs.append(F_.conv3d_channels_last(xc[i], w, b, self.kernel_size, history=None if hist is None else hist[i],
                                                out_channels=self.out_channels))
        if cache is not None and self.pad_t:
            full = xc if hist is None else torch.cat([hist, xc], 1)
            if full.shape[1] < self.pad_t:
                full = torch.cat([full.new_zeros(full.shape[0], self.pad_t - full.shape[1], *full.shape[2:]), full], 1)
            cache[ck] = full[:, -self.pad_t:].detach().contiguous()
        return torch.stack(outs).permute(0, 4, 1, 2, 3)

    def forward(self, x, cache: Optional[dict] = None, key: Optional[str] = None):
        """x [B, C, T, H, W].  With a cache dict the temporal left context comes from the previous call."""
        if self._native_ok(x):
            return self._forward_native(x, cache, key)
        x = F.pad(x, self.pad_hw)
        if self.pad_t:
            if cache is not None and key in cache:
                left = cache[key]
            else:
                left = x[:, :, :1].expand(-1, -1, self.pad_t, -1, -1) * 0
            xin = torch.cat([left, x], dim=2)
            if cache is not None:
                cache[key] = xin[:, :, -self.pad_t:].detach()
        else:
            xin = x
        return F.conv3d(xin, self.weight, self.bias, self.stride)


class RMSNormC(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(dim))
        self.scale = dim ** 0.5

    def forward(self, x, silu: bool = False):
        """Channel RMS norm of ``x [B, C, T, H, W]``; ``silu=True`` also applies the activation that follows it in
        every block (one kernel on channels-last bf16 CUDA activations at inference)."""
        C = x.shape[1]
        if (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 5 and C % 8 == 0 and C <= 1024
                and not (torch.is_grad_enabled() and (x.requires_grad or self.gamma.requires_grad))):
            from ..ops import functional as F_

            xc = x.permute(0, 2, 3, 4, 1).contiguous()                  # free when x already is channels-last memory
            return F_.rms_silu_channels_last(xc, self.gamma, silu).permute(0, 4, 1, 2, 3)
        y = F.normalize(x.float(), dim=1).to(x.dtype) * self.scale * self.gamma.view(1, -1, 1, 1, 1).to(x.dtype)
        return F.silu(y) if silu else y


class ResBlock(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.n1, self.c1 = RMSNormC(cin), CausalConv3d(cin, cout)
        self.n2, self.c2 = RMSNormC(cout), CausalConv3d(cout, cout)
        self.skip = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x, cache=None, key=""):
        h = self.c1(self.n1(x, silu=True), cache, key + ".c1")
        h = self.c2(self.n2(h, silu=True), cache, key + ".c2")
        return h + (x if self.skip is None else self.skip(x))


class FrameAttention(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.norm = RMSNormC(dim)
        self.qkv = nn.Conv2d(dim, 3 * dim, 1)
        self.proj = nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def forward(self, x):
        B, C, T, H, W = x.shape
        y = self.norm(x).permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        q, k, v = self.qkv(y).reshape(B * T, 1, 3 * C, H * W).permute(0, 1, 3, 2).chunk(3, dim=-1)
        o = F.scaled_dot_product_attention(q, k, v)
        o = self.proj(o.squeeze(1).permute(0, 2, 1).reshape(B * T, C, H, W))
        return x + o.view(B, T, C, H, W).permute(0, 2, 1, 3, 4)


class AvgDown3D(nn.Module):
    """Parameter-free shortcut of a down-sampling stage: fold ``ft x fs x fs`` neighbourhoods into channels,
    then average channel groups down to ``cout`` (the first temporal group is padded causally)."""

    def __init__(self, cin, cout, factor_t, factor_s):
        super().__init__()
        self.cin, self.cout, self.ft, self.fs = cin, cout, factor_t, factor_s
        self.group = cin * factor_t * factor_s * factor_s // cout

    def forward(self, x):
        B, C, T, H, W = x.shape
        pad_t = (self.ft - T % self.ft) % self.ft
        x = F.pad(x, (0, 0, 0, 0, pad_t, 0))
        T2 = x.shape[2]
        x = x.view(B, C, T2 // self.ft, self.ft, H // self.fs, self.fs, W // self.fs, self.fs)
        x = x.permute(0, 1, 3, 5, 7, 2, 4, 6).reshape(B, C * self.ft * self.fs * self.fs, T2 // self.ft, H // self.fs, W // self.fs)
        return x.view(B, self.cout, self.group, *x.shape[2:]).mean(dim=2)


class DupUp3D(nn.Module):
    """Parameter-free shortcut of an up-sampling stage: repeat channels, then unfold them into ``ft x fs x fs``
    neighbourhoods (the first chunk drops the leading ``ft - 1`` frames, like the learned path)."""

    def __init__(self, cin, cout, factor_t, factor_s):
        super().__init__()
        self.cin, self.cout, self.ft, self.fs = cin, cout, factor_t, factor_s
        self.repeats = cout * factor_t * factor_s * factor_s // cin

    def forward(self, x, first_chunk=False):
        B, C, T, H, W = x.shape
        x = x.repeat_interleave(self.repeats, dim=1)
        x = x.view(B, self.cout, self.ft, self.fs, self.fs, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4)
        x = x.reshape(B, self.cout, T * self.ft, H * self.fs, W * self.fs)
        return x[:, :, self.ft - 1:] if first_chunk else x


class Upsample(nn.Module):
    def __init__(self, dim, temporal: bool):
        super().__init__()
        self.temporal = temporal
        self.conv = nn.Conv2d(dim, dim // 2, 3, padding=1)
        if temporal:
            self.time_conv = CausalConv3d(dim, 2 * dim, (3, 1, 1))

    def forward(self, x, cache=None, key="", first_chunk=True):
        B, C, T, H, W = x.shape
        if self.temporal:
            y = self.time_conv(x, cache, key + ".t")                       # [B, 2C, T, H, W]
            y = y.view(B, 2, C, T, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C, 2 * T, H, W)
            if first_chunk:
                y = y[:, :, 1:]             # the first latent frame maps to a single pixel-time step
            x = y
            T = x.shape[2]
        if (x.is_cuda and x.dtype == torch.bfloat16 and C % 8 == 0
                and not (torch.is_grad_enabled() and (x.requires_grad or self.conv.weight.requires_grad))):
            return self._spatial_native(x)
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        y = self.conv(F.interpolate(y.float(), scale_factor=2.0, mode="nearest").to(x.dtype))
        return y.view(B, T, C // 2, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)

    def _spatial_native(self, x):
        """Nearest 2x in channels-last memory, then the 3 x 3 convolution as a one-frame-deep implicit GEMM."""
        from ..ops import functional as F_

        B, C, T, H, W = x.shape
        w = self.conv.weight
        tag = (w.data_ptr(), w._version, str(x.device))
        if getattr(self, "_packed_tag", None) != tag:
            self._packed = F_.pack_conv_weight(w.unsqueeze(2), self.conv.bias)
            self._packed_tag = tag
        pw, pb = self._packed
        xc = x.permute(0, 2, 3, 4, 1)                                    # [B, T, H, W, C] view
        up = xc.reshape(B, T, H, 1, W, 1, C).expand(B, T, H, 2, W, 2, C).reshape(B, T, 2 * H, 2 * W, C)
        outs = [F_.conv3d_channels_last(up[i], pw, pb, (1, 3, 3), out_channels=C // 2) for i in range(B)]
        return torch.stack(outs).permute(0, 4, 1, 2, 3)


@dataclass
class VAEConfig:
    z_dim: int = 48
    base: int = 64
    temporal_ups: tuple = (True, True, False)     # 4x temporal, 8x spatial (x patch 2 = 16 for Wan-5B)
    out_channels: int = 3


class Decoder3d(nn.Module):
    def __init__(self, cfg: VAEConfig):
        super().__init__()
        n = len(cfg.temporal_ups)
        top = cfg.base * (2 ** n)
        self.conv_in = CausalConv3d(cfg.z_dim, top)
        self.mid1, self.mid_attn, self.mid2 = ResBlock(top, top), FrameAttention(top), ResBlock(top, top)
        self.stages = nn.ModuleList()
        dim = top
        for t in cfg.temporal_ups:
            self.stages.append(nn.ModuleList([ResBlock(dim, dim), ResBlock(dim, dim), Upsample(dim, t)]))
            dim //= 2
        self.norm_out, self.conv_out = RMSNormC(dim), CausalConv3d(dim, cfg.out_channels)

    def forward(self, z, cache=None, first_chunk=True):
        x = self.conv_in(z, cache, "in")
        x = self.mid2(self.mid_attn(self.mid1(x, cache, "m1")), cache, "m2")
        for i, (r1, r2, up) in enumerate(self.stages):
            x = up(r2(r1(x, cache, f"s{i}.r1"), cache, f"s{i}.r2"), cache, f"s{i}.up", first_chunk)
        return self.conv_out(self.norm_out(x, silu=True), cache, "out")


class Encoder3d(nn.Module):
    def __init__(self, cfg: VAEConfig):
        super().__init__()
        n = len(cfg.temporal_ups)
        self.conv_in = CausalConv3d(cfg.out_channels, cfg.base)
        self.stages = nn.ModuleList()
        dim = cfg.base
        for t in reversed(cfg.temporal_ups):
            self.stages.append(nn.ModuleList([ResBlock(dim, 2 * dim),
                                              CausalConv3d(2 * dim, 2 * dim, 3, stride=(2 if t else 1, 2, 2))]))
            dim *= 2
        self.mid = ResBlock(dim, dim)
        self.conv_out = CausalConv3d(dim, 2 * cfg.z_dim, 1)

    def forward(self, x):
        x = self.conv_in(x)
        for res, down in self.stages:
            x = down(res(x))
        return self.conv_out(self.mid(x))


class VideoVAE(nn.Module):
    def __init__(self, cfg: VAEConfig = VAEConfig(), mean: Optional[List[float]] = None, std: Optional[List[float]] = None):
        super().__init__()
        self.cfg = cfg
        self.encoder, self.decoder = Encoder3d(cfg), Decoder3d(cfg)
        self.register_buffer("mean", torch.tensor(mean if mean is not None else [0.0] * cfg.z_dim).view(1, -1, 1, 1, 1))
        self.register_buffer("std", torch.tensor(std if std is not None else [1.0] * cfg.z_dim).view(1, -1, 1, 1, 1))

    @torch.no_grad()
    def encode(self, video):
        """[B, 3, T, H, W] -> normalised latent mean [B, z, T', H', W']"""
        mu = self.encoder(video).chunk(2, dim=1)[0]
        return (mu - self.mean.to(mu)) / self.std.to(mu)

    @torch.no_grad()
    def decode(self, z):
        return self.decoder(z * self.std.to(z) + self.mean.to(z), None, True)


class StreamingDecoder:
    """Chunk-by-chunk decode with a persistent feature cache: ``push(latent chunk)`` returns the newly
    decodable pixel frames; the concatenation over pushes equals ``VideoVAE.decode`` of the whole clip
    (reference: WanVAE_.cached_decode and Wan5BVAE.decode_streaming_chunks, vae.py:706-868,
    components.py:250-289)."""

    def __init__(self, vae: VideoVAE):
        self.vae = vae
        self.cache: dict = {}
        self.first = True

    @torch.no_grad()
    def push(self, z_chunk):
        z = z_chunk * self.vae.std.to(z_chunk) + self.vae.mean.to(z_chunk)
        out = self.vae.decoder(z, self.cache, self.first)
        self.first = False
        return out

    def reset(self) -> None:
        self.cache.clear()
        self.first = True
