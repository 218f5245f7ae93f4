"""Codec adapters of the Wan backends: the video VAE behind a BTCHW contract.

``WanVideoCodec`` wraps ``models.vae.VideoVAE``:

* ``encode(video [B, T, 3, H, W] in [-1, 1]) -> latents [B, T', C, H', W']`` (deterministic: the posterior mean,
  normalised with the per-channel statistics of the checkpoint);
* ``decode(latents) -> video`` clamped to [-1, 1];
* ``decode_streaming_chunks(latents, chunk_latent_frames=60)``: a generator of host BTCHW pieces decoded with ONE
  continuous feature cache across pieces (so the pieces concatenate to exactly the one-shot decode), each checked
  for non-finite pixels before it leaves the device; the cache is cleared at the start and in ``finally``.

``Wan5BVAE`` (48 channels, 4 x 16 x 16 compression) takes its statistics from the checkpoint;
``WanA14BVAE`` (16 channels, 4 x 8 x 8) carries the published Wan2.1 statistics.  ``flow_to_x0`` does the
flow -> clean-sample conversion in fp64 as the reference's scheduler wrapper does.

Reference behaviour: solar/backends/wan22/runtime/components.py:66-330 (``Wan5BVAE``, ``WanA14BVAE``),
:576 (``WanDiffusion``).
"""
from __future__ import annotations

from typing import Iterator, Optional, Sequence

import torch

from ...errors import BackendContractError
from ...models.vae import StreamingDecoder, VAEConfig, VideoVAE


class WanVideoCodec:
    latent_channels: int = 0

    def __init__(self, vae: VideoVAE):
        if vae.cfg.z_dim != self.latent_channels and self.latent_channels:
            raise BackendContractError(f"this codec needs a {self.latent_channels}-channel VAE, got {vae.cfg.z_dim}")
        self.vae = vae.eval().requires_grad_(False)

    @staticmethod
    def _check_btchw(x, channels: Optional[int], what: str):
        if x.ndim != 5 or x.shape[1] <= 0:
            raise BackendContractError(f"{what} must be a non-empty BTCHW tensor")
        if channels is not None and x.shape[2] != channels:
            raise BackendContractError(f"{what} must have {channels} channels, got {x.shape[2]}")

    @torch.no_grad()
    def encode(self, video_btchw: torch.Tensor) -> torch.Tensor:
        self._check_btchw(video_btchw, 3, "video")
        z = self.vae.encode(video_btchw.permute(0, 2, 1, 3, 4))
        return z.permute(0, 2, 1, 3, 4).contiguous()

    @torch.no_grad()
    def decode(self, latents_btchw: torch.Tensor) -> torch.Tensor:
        self._check_btchw(latents_btchw, self.vae.cfg.z_dim, "latents")
        out = self.vae.decode(latents_btchw.permute(0, 2, 1, 3, 4))
        if not bool(torch.isfinite(out).all()):
            raise BackendContractError("VAE decode produced non-finite pixels")
        return out.float().clamp_(-1, 1).permute(0, 2, 1, 3, 4).contiguous()

    @torch.no_grad()
    def decode_streaming_chunks(self, latents_btchw: torch.Tensor, *, chunk_latent_frames: int = 60) -> Iterator[torch.Tensor]:
        self._check_btchw(latents_btchw, self.vae.cfg.z_dim, "latents")
        if latents_btchw.shape[0] != 1:
            raise BackendContractError("streaming decode takes batch size one")
        if chunk_latent_frames <= 0:
            raise BackendContractError("chunk size must be positive")
        clip = latents_btchw.permute(0, 2, 1, 3, 4)                         # [1, C, T, H, W]
        dec = StreamingDecoder(self.vae)
        try:
            for start in range(0, clip.shape[2], chunk_latent_frames):
                piece = dec.push(clip[:, :, start:start + chunk_latent_frames].contiguous())
                if not bool(torch.isfinite(piece).all()):
                    raise BackendContractError("streaming VAE decode produced non-finite pixels")
                yield piece.float().clamp_(-1, 1).permute(0, 2, 1, 3, 4).contiguous().cpu()
                del piece
        finally:
            dec.reset()


class Wan5BVAE(WanVideoCodec):
    """48-channel Wan2.2 VAE (TI2V-5B); statistics come with the checkpoint."""
    latent_channels = 48

    @classmethod
    def build(cls, mean: Sequence[float], std: Sequence[float], base: int = 64):
        if len(mean) != 48 or len(std) != 48:
            raise BackendContractError("the 5B VAE needs 48 per-channel means and standard deviations")
        return cls(VideoVAE(VAEConfig(z_dim=48, base=base, temporal_ups=(True, True, False)), list(mean), list(std)))


class WanA14BVAE(WanVideoCodec):
    """16-channel Wan2.1 VAE used by I2V-A14B, with its published latent statistics."""
    latent_channels = 16
    mean = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
            0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921)
    std = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
           3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160)

    @classmethod
    def build(cls, base: int = 96):
        return cls(VideoVAE(VAEConfig(z_dim=16, base=base, temporal_ups=(True, True, False)), list(cls.mean), list(cls.std)))


def flow_to_x0(x_t: torch.Tensor, flow: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    """x0 = x_t - sigma * v, evaluated in fp64 and returned in the input dtype."""
    s = sigma.to(torch.float64)
    while s.dim() < x_t.dim():
        s = s.unsqueeze(-1)
    return (x_t.to(torch.float64) - s * flow.to(torch.float64)).to(x_t.dtype)


def btchw_to_bcthw(x: torch.Tensor) -> torch.Tensor:
    return x.permute(0, 2, 1, 3, 4).contiguous()


def bcthw_to_btchw(x: torch.Tensor) -> torch.Tensor:
    return x.permute(0, 2, 1, 3, 4).contiguous()
