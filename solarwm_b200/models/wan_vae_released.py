"""The published Wan video VAEs (Wan2.1: 16 channels, 4 x 8 x 8; Wan2.2: 48 channels, 4 x 16 x 16) in this package's
building blocks, with a loader for the published checkpoints.

Both are causal 3-D convolutional auto-encoders over pixel clips of ``1 + 4k`` frames:

  encoder   [pixel-unshuffle 2 (2.2)] -> conv -> 4 stages of residual blocks, the first three followed by a
            2x spatial down-sampling (zero pad right / bottom, 3 x 3 stride-2 convolution) and, where the stage is
            temporal, a 2x temporal one (the first frame passes, every later pair is folded by a 3-tap stride-2
            convolution that starts at the previous frame) -> residual, per-frame attention, residual -> norm, SiLU,
            conv -> 1 x 1 x 1 convolution; the first half of the channels is the posterior mean
  decoder   1 x 1 x 1 convolution -> conv -> residual, attention, residual -> 4 stages of 3 residual blocks, the first
            three followed by an up-sampling (where temporal: every frame but the first becomes two through a causal
            3-tap convolution with twice the channels; then nearest 2x in space and a 3 x 3 convolution) -> norm, SiLU,
            conv [-> pixel-shuffle 2 (2.2)]

Wan2.2 adds a parameter-free shortcut around each stage (``AvgDown3D`` / ``DupUp3D``) and keeps the channel count
through an up-sampling; in Wan2.1 the up-sampling convolution halves it.

Unlike the published code, which walks the clip one latent frame (four pixel frames) at a time through a list of
per-convolution caches, every module here takes ANY run of frames plus a keyed cache: a whole clip is one pass (the
memory is there), and a stream is the same function called per chunk.  Every convolution is causal, so the two are the
same function; ``tests/test_wan_vae_released.py`` checks that against the reference class, chunked and whole.

``released_names(vae)`` gives our parameter name for every name of the published state dict, ``load_released`` reads a
``.pth`` / ``.safetensors`` file strictly (every tensor used, none missing, shapes equal).  The diffusers naming of the
Wan2.1 VAE is accepted as well.

Reference: solar/backends/wan22/runtime/modeling/vae.py:19-868 (blocks, ``WanVAE_``, ``_video_vae``),
solar/backends/wan22/runtime/components.py:66-424 (``Wan5BVAE``, ``WanA14BVAE``).
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Mapping, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .vae import AvgDown3D, CausalConv3d, DupUp3D, FrameAttention, ResBlock, RMSNormC


@dataclass(frozen=True)
class ReleasedVAEConfig:
    z_dim: int
    enc_dim: int
    dec_dim: int
    mult: Tuple[int, ...] = (1, 2, 4, 4)
    res_blocks: int = 2
    temporal_down: Tuple[bool, ...] = (False, True, True)
    patch: int = 1                     # pixel-unshuffle factor in front of the encoder
    stage_shortcuts: bool = False      # AvgDown3D / DupUp3D around each stage; up-sampling keeps the channel count

    @classmethod
    def wan21(cls, dim: int = 96, z_dim: int = 16):
        return cls(z_dim=z_dim, enc_dim=dim, dec_dim=dim)

    @classmethod
    def wan22(cls, enc_dim: int = 160, dec_dim: int = 256, z_dim: int = 48):
        return cls(z_dim=z_dim, enc_dim=enc_dim, dec_dim=dec_dim, patch=2, stage_shortcuts=True)


def _conv2d_frames(conv: nn.Conv2d, x: torch.Tensor, pad=None) -> torch.Tensor:
    B, C, T, H, W = x.shape
    y = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
    if pad is not None:
        y = F.pad(y, pad)
    y = conv(y)
    return y.view(B, T, *y.shape[1:]).permute(0, 2, 1, 3, 4)


class Down(nn.Module):
    """2x in space, optionally 2x in time."""

    def __init__(self, dim: int, temporal: bool):
        super().__init__()
        self.space = nn.Conv2d(dim, dim, 3, stride=2)
        self.time = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1)) if temporal else None

    def forward(self, x, cache: Optional[dict], key: str):
        x = _conv2d_frames(self.space, x, (0, 1, 0, 1))
        if self.time is None:
            return x
        # the stride-2 fold starts at the last frame of the previous call; the clip's very first frame passes through
        prev = None if cache is None else cache.get(key)
        if cache is not None:
            cache[key] = x[:, :, -1:].detach()
        seq = x if prev is None else torch.cat([prev, x], dim=2)
        if seq.shape[2] % 2 == 0:
            raise ValueError("temporal down-sampling takes 1 + 2k frames at the start of a clip and 2k frames after it")
        folded = F.conv3d(seq, self.time.weight, self.time.bias, self.time.stride) if seq.shape[2] >= 3 else seq[:, :, :0]
        return folded if prev is not None else torch.cat([x[:, :, :1], folded], dim=2)


class Up(nn.Module):
    """Optionally 2x in time (all frames but the clip's first), then 2x in space."""

    def __init__(self, dim: int, out_dim: int, temporal: bool):
        super().__init__()
        self.space = nn.Conv2d(dim, out_dim, 3, padding=1)
        self.time = CausalConv3d(dim, 2 * dim, (3, 1, 1)) if temporal else None

    def forward(self, x, cache: Optional[dict], key: str, first_chunk: bool):
        B, C, T, H, W = x.shape
        if self.time is not None:
            head, rest = (x[:, :, :1], x[:, :, 1:]) if first_chunk else (x[:, :, :0], x)
            if rest.shape[2]:
                y = self.time(rest, cache, key)                              # zero history right after the first frame
                n = rest.shape[2]
                rest = y.reshape(B, 2, C, n, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C, 2 * n, H, W)
            x = torch.cat([head, rest], dim=2)
        T = x.shape[2]
        if (x.is_cuda and x.dtype == torch.bfloat16 and C % 8 == 0 and self.space.out_channels % 8 == 0
                and not torch.is_grad_enabled()):
            return self._space_native(x)
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, C, H, W)
        y = self.space(F.interpolate(y.float(), scale_factor=2.0, mode="nearest-exact").to(x.dtype))
        return y.view(B, T, -1, 2 * H, 2 * W).permute(0, 2, 1, 3, 4)

    def _space_native(self, x):
        """Nearest 2x as a broadcast view of channels-last memory, the 3 x 3 convolution as a one-frame-deep implicit GEMM."""
        from ..ops import functional as F_

        B, C, T, H, W = x.shape
        w = self.space.weight
        tag = (w.data_ptr(), w._version, str(x.device))
        if getattr(self, "_packed_tag", None) != tag:
            self._packed = F_.pack_conv_weight(w.unsqueeze(2), self.space.bias)
            self._packed_tag = tag
        pw, pb = self._packed
        xc = x.permute(0, 2, 3, 4, 1)
        up = xc.reshape(B, T, H, 1, W, 1, C).expand(B, T, H, 2, W, 2, C).reshape(B, T, 2 * H, 2 * W, C)
        outs = [F_.conv3d_channels_last(up[i], pw, pb, (1, 3, 3), out_channels=self.space.out_channels) for i in range(B)]
        return torch.stack(outs).permute(0, 4, 1, 2, 3)


class Stage(nn.Module):
    """``n`` residual blocks, an optional resampler, an optional parameter-free shortcut around both."""

    def __init__(self, cin: int, cout: int, n: int, resample: Optional[nn.Module], shortcut: Optional[nn.Module]):
        super().__init__()
        self.blocks = nn.ModuleList([ResBlock(cin if i == 0 else cout, cout) for i in range(n)])
        self.resample, self.shortcut = resample, shortcut

    def forward(self, x, cache, key, first_chunk=False):
        h = x
        for i, b in enumerate(self.blocks):
            h = b(h, cache, f"{key}.b{i}")
        if isinstance(self.resample, Up):
            h = self.resample(h, cache, key + ".up", first_chunk)
        elif self.resample is not None:
            h = self.resample(h, cache, key + ".down")
        if self.shortcut is None:
            return h
        return h + (self.shortcut(x, first_chunk) if isinstance(self.shortcut, DupUp3D) else self.shortcut(x))


class _Middle(nn.Module):
    def __init__(self, dim):
        super().__init__()
        self.r1, self.attn, self.r2 = ResBlock(dim, dim), FrameAttention(dim), ResBlock(dim, dim)

    def forward(self, x, cache, key):
        return self.r2(self.attn(self.r1(x, cache, key + ".r1")), cache, key + ".r2")


class ReleasedEncoder(nn.Module):
    def __init__(self, c: ReleasedVAEConfig):
        super().__init__()
        dims = [c.enc_dim] + [c.enc_dim * m for m in c.mult]
        self.conv_in = CausalConv3d(3 * c.patch * c.patch, dims[0])
        self.stages = nn.ModuleList()
        last = len(c.mult) - 1
        for i, (a, b) in enumerate(zip(dims[:-1], dims[1:])):
            temporal = i < len(c.temporal_down) and c.temporal_down[i]
            down = Down(b, temporal) if i != last else None
            short = AvgDown3D(a, b, 2 if temporal else 1, 2 if down is not None else 1) if c.stage_shortcuts else None
            self.stages.append(Stage(a, b, c.res_blocks, down, short))
        self.middle = _Middle(dims[-1])
        self.norm_out, self.conv_out = RMSNormC(dims[-1]), CausalConv3d(dims[-1], 2 * c.z_dim)

    def forward(self, x, cache: Optional[dict] = None):
        x = self.conv_in(x, cache, "in")
        for i, s in enumerate(self.stages):
            x = s(x, cache, f"s{i}")
        x = self.middle(x, cache, "mid")
        return self.conv_out(self.norm_out(x, silu=True), cache, "out")


class ReleasedDecoder(nn.Module):
    def __init__(self, c: ReleasedVAEConfig):
        super().__init__()
        dims = [c.dec_dim * c.mult[-1]] + [c.dec_dim * m for m in reversed(c.mult)]
        ups = tuple(reversed(c.temporal_down))
        self.conv_in = CausalConv3d(c.z_dim, dims[0])
        self.middle = _Middle(dims[0])
        self.stages = nn.ModuleList()
        last = len(c.mult) - 1
        carried = dims[0]                                      # channels that arrive at the stage
        for i, b in enumerate(dims[1:]):
            temporal = i < len(ups) and ups[i]
            up_out = b if c.stage_shortcuts else b // 2
            up = Up(b, up_out, temporal) if i != last else None
            short = DupUp3D(carried, b, 2 if temporal else 1, 2) if (c.stage_shortcuts and up is not None) else None
            self.stages.append(Stage(carried, b, c.res_blocks + 1, up, short))
            carried = up_out if up is not None else b
        self.norm_out, self.conv_out = RMSNormC(carried), CausalConv3d(carried, 3 * c.patch * c.patch)

    def forward(self, z, cache: Optional[dict] = None, first_chunk: bool = True):
        x = self.middle(self.conv_in(z, cache, "in"), cache, "mid")
        for i, s in enumerate(self.stages):
            x = s(x, cache, f"s{i}", first_chunk)
        return self.conv_out(self.norm_out(x, silu=True), cache, "out")


def pixel_unshuffle(x, p: int):
    if p == 1:
        return x
    B, C, T, H, W = x.shape
    x = x.view(B, C, T, H // p, p, W // p, p)                  # b c f h q w r -> b (c r q) f h w
    return x.permute(0, 1, 6, 4, 2, 3, 5).reshape(B, C * p * p, T, H // p, W // p)


def pixel_shuffle(x, p: int):
    if p == 1:
        return x
    B, C, T, H, W = x.shape
    x = x.view(B, C // (p * p), p, p, T, H, W)                  # b (c r q) f h w -> b c f (h q) (w r)
    return x.permute(0, 1, 4, 5, 3, 6, 2).reshape(B, C // (p * p), T, H * p, W * p)


class ReleasedVAE(nn.Module):
    """Same ``encode / decode / cfg.z_dim / mean / std / decoder(z, cache, first)`` surface as ``models.vae.VideoVAE``,
    so the codec adapters and ``StreamingDecoder`` take either."""

    def __init__(self, cfg: ReleasedVAEConfig, mean: Optional[Sequence[float]] = None, std: Optional[Sequence[float]] = None):
        super().__init__()
        self.cfg = cfg
        self.encoder_net, self.decoder_net = ReleasedEncoder(cfg), ReleasedDecoder(cfg)
        self.quant = CausalConv3d(2 * cfg.z_dim, 2 * cfg.z_dim, 1)
        self.post_quant = CausalConv3d(cfg.z_dim, cfg.z_dim, 1)
        self.register_buffer("mean", torch.tensor(list(mean) if mean is not None else [0.0] * cfg.z_dim).view(1, -1, 1, 1, 1))
        self.register_buffer("std", torch.tensor(list(std) if std is not None else [1.0] * cfg.z_dim).view(1, -1, 1, 1, 1))

    # the surface StreamingDecoder drives: de-normalised latents in, pixels out
    def decoder(self, z, cache: Optional[dict] = None, first_chunk: bool = True):
        return pixel_shuffle(self.decoder_net(self.post_quant(z), cache, first_chunk), self.cfg.patch)

    def posterior(self, video, cache: Optional[dict] = None):
        """[B, 3, T, H, W] -> (mean, log-variance), un-normalised."""
        return self.quant(self.encoder_net(pixel_unshuffle(video, self.cfg.patch), cache)).chunk(2, dim=1)

    @torch.no_grad()
    def encode(self, video, chunk_frames: Optional[int] = None):
        """Normalised posterior mean.  ``chunk_frames`` (a multiple of 4) bounds the activation memory: the clip is
        walked as ``1 + chunk_frames`` frames and then ``chunk_frames`` at a time with one cache."""
        if (video.shape[2] - 1) % 4:
            raise ValueError("the VAE encodes clips of 1 + 4k frames")
        if chunk_frames is None or video.shape[2] <= 1 + chunk_frames:
            mu = self.posterior(video)[0]
        else:
            if chunk_frames % 4 or chunk_frames <= 0:
                raise ValueError("chunk_frames is a positive multiple of 4")
            cache, parts, start, stop = {}, [], 0, 1 + chunk_frames
            while start < video.shape[2]:
                parts.append(self.posterior(video[:, :, start:stop], cache)[0])
                start, stop = stop, stop + chunk_frames
            mu = torch.cat(parts, dim=2)
        return (mu - self.mean.to(mu)) / self.std.to(mu)

    @torch.no_grad()
    def decode(self, z):
        return self.decoder(z * self.std.to(z) + self.mean.to(z), None, True)


# ---------------------------------------------------------------------------------------------------------------------
# Published names
# ---------------------------------------------------------------------------------------------------------------------
def _res_names(ours: str, theirs: str, block: ResBlock, out: Dict[str, str]) -> None:
    out[f"{theirs}.residual.0.gamma"] = f"{ours}.n1.gamma"
    out[f"{theirs}.residual.3.gamma"] = f"{ours}.n2.gamma"
    for slot, name in ((2, "c1"), (6, "c2")):
        for leaf in ("weight", "bias"):
            out[f"{theirs}.residual.{slot}.{leaf}"] = f"{ours}.{name}.{leaf}"
    if block.skip is not None:
        for leaf in ("weight", "bias"):
            out[f"{theirs}.shortcut.{leaf}"] = f"{ours}.skip.{leaf}"


def _middle_names(ours: str, theirs: str, mid: _Middle, out: Dict[str, str]) -> None:
    _res_names(f"{ours}.r1", f"{theirs}.0", mid.r1, out)
    _res_names(f"{ours}.r2", f"{theirs}.2", mid.r2, out)
    out[f"{theirs}.1.norm.gamma"] = f"{ours}.attn.norm.gamma"
    for leaf in ("weight", "bias"):
        out[f"{theirs}.1.to_qkv.{leaf}"] = f"{ours}.attn.qkv.{leaf}"
        out[f"{theirs}.1.proj.{leaf}"] = f"{ours}.attn.proj.{leaf}"


def released_names(vae: ReleasedVAE) -> Dict[str, str]:
    """published state-dict name -> our parameter name.  Wan2.2 nests each stage (``downsamples.i.downsamples.j``),
    Wan2.1 numbers the blocks and resamplers of all stages in one list."""
    out: Dict[str, str] = {}
    nested = vae.cfg.stage_shortcuts
    for side, net, group in (("encoder", vae.encoder_net, "downsamples"), ("decoder", vae.decoder_net, "upsamples")):
        for leaf in ("weight", "bias"):
            out[f"{side}.conv1.{leaf}"] = f"{side}_net.conv_in.{leaf}"
            out[f"{side}.head.2.{leaf}"] = f"{side}_net.conv_out.{leaf}"
        out[f"{side}.head.0.gamma"] = f"{side}_net.norm_out.gamma"
        _middle_names(f"{side}_net.middle", f"{side}.middle", net.middle, out)
        flat = 0
        for i, stage in enumerate(net.stages):
            for j, block in enumerate(stage.blocks):
                theirs = f"{side}.{group}.{i}.{group}.{j}" if nested else f"{side}.{group}.{flat}"
                _res_names(f"{side}_net.stages.{i}.blocks.{j}", theirs, block, out)
                flat += 1
            if stage.resample is not None:
                theirs = f"{side}.{group}.{i}.{group}.{len(stage.blocks)}" if nested else f"{side}.{group}.{flat}"
                flat += 1
                for leaf in ("weight", "bias"):
                    out[f"{theirs}.resample.1.{leaf}"] = f"{side}_net.stages.{i}.resample.space.{leaf}"
                    if stage.resample.time is not None:
                        out[f"{theirs}.time_conv.{leaf}"] = f"{side}_net.stages.{i}.resample.time.{leaf}"
    for leaf in ("weight", "bias"):
        out[f"conv1.{leaf}"] = f"quant.{leaf}"
        out[f"conv2.{leaf}"] = f"post_quant.{leaf}"
    return out


_DIFFUSERS_RES = {"norm1.gamma": "residual.0.gamma", "conv1.weight": "residual.2.weight", "conv1.bias": "residual.2.bias",
                  "norm2.gamma": "residual.3.gamma", "conv2.weight": "residual.6.weight", "conv2.bias": "residual.6.bias",
                  "conv_shortcut.weight": "shortcut.weight", "conv_shortcut.bias": "shortcut.bias"}


def from_diffusers_wan21(name: str, res_blocks: int = 2) -> str:
    """A name of the diffusers Wan2.1 auto-encoder in the original numbering (what ``released_names`` keys)."""
    fixed = {"quant_conv": "conv1", "post_quant_conv": "conv2"}
    head, _, leaf = name.partition(".")
    if head in fixed:
        return f"{fixed[head]}.{leaf}"
    side = head
    rest = leaf
    for a, b in (("conv_in.", "conv1."), ("conv_out.", "head.2."), ("norm_out.", "head.0.")):
        if rest.startswith(a):
            return f"{side}.{b}{rest[len(a):]}"
    m = re.fullmatch(r"mid_block\.resnets\.(\d)\.(.+)", rest)
    if m:
        return f"{side}.middle.{2 * int(m[1])}.{_DIFFUSERS_RES[m[2]]}"
    m = re.fullmatch(r"mid_block\.attentions\.0\.(.+)", rest)
    if m:
        return f"{side}.middle.1.{m[1]}"
    m = re.fullmatch(r"down_blocks\.(\d+)\.(.+)", rest)                       # the encoder list is already flat
    if m:
        return f"{side}.downsamples.{m[1]}.{_DIFFUSERS_RES.get(m[2], m[2])}"
    per = res_blocks + 2                                                      # 3 residual blocks + 1 resampler
    m = re.fullmatch(r"up_blocks\.(\d+)\.resnets\.(\d+)\.(.+)", rest)
    if m:
        return f"{side}.upsamples.{int(m[1]) * per + int(m[2])}.{_DIFFUSERS_RES[m[3]]}"
    m = re.fullmatch(r"up_blocks\.(\d+)\.upsamplers\.0\.(.+)", rest)
    if m:
        return f"{side}.upsamples.{int(m[1]) * per + res_blocks + 1}.{m[2]}"
    raise KeyError(name)


def adopt_released_state(vae: ReleasedVAE, state: Mapping[str, torch.Tensor]) -> None:
    """Strict: every tensor of ``state`` lands in exactly one parameter and no parameter stays unset."""
    from ..errors import BackendContractError

    names = released_names(vae)
    if not set(names) <= set(state) and any(k.startswith(("encoder.conv_in", "quant_conv")) for k in state):
        try:
            state = {from_diffusers_wan21(k, vae.cfg.res_blocks): v for k, v in state.items()}
        except KeyError as exc:
            raise BackendContractError(f"unknown tensor {exc.args[0]!r} in a diffusers-layout VAE checkpoint") from None
    missing, extra = sorted(set(names) - set(state)), sorted(set(state) - set(names))
    if missing or extra:
        raise BackendContractError(f"VAE checkpoint does not match the architecture: missing {missing[:6]}, unexpected {extra[:6]}")
    own = dict(vae.named_parameters())
    if set(names.values()) != set(own):
        raise BackendContractError("internal: the published-name table does not cover the module")
    with torch.no_grad():
        for theirs, ours in names.items():
            src, dst = state[theirs], own[ours]
            if src.numel() != dst.numel() or (src.dim() == dst.dim() and src.shape != dst.shape):
                raise BackendContractError(f"{theirs}: checkpoint shape {tuple(src.shape)} does not fit {tuple(dst.shape)}")
            dst.copy_(src.reshape(dst.shape))                 # norm gains are stored as [C, 1, 1(, 1)]


def load_released(path, cfg: ReleasedVAEConfig, mean=None, std=None, *, device="cpu", dtype=torch.float32) -> ReleasedVAE:
    """Build the architecture and fill it from a published ``.pth`` (read with ``weights_only``) or ``.safetensors``."""
    from ..errors import BackendContractError

    path = Path(path)
    if not path.is_file():
        raise BackendContractError(f"VAE checkpoint {path} does not exist")
    if path.suffix == ".safetensors":
        from safetensors.torch import load_file

        state = load_file(str(path))
    else:
        state = torch.load(str(path), map_location="cpu", weights_only=True, mmap=True)
    if not isinstance(state, Mapping) or not state:
        raise BackendContractError(f"{path}: not a state dict")
    vae = ReleasedVAE(cfg, mean, std)
    adopt_released_state(vae, state)
    return vae.to(device=device, dtype=dtype).eval().requires_grad_(False)
