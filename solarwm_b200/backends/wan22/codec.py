"""Codec adapters of the Wan backends: the video VAE behind a BTCHW contract.

``WanVideoCodec`` wraps ``models.vae.VideoVAE``:

* ``encode(video [B, T, 3, H, W] in [-1, 1]) -> latents [B, T', C, H', W']`` (deterministic: the posterior mean,
  normalised with the per-channel statistics of the checkpoint);
* ``decode(latents) -> video`` clamped to [-1, 1];
* ``decode_streaming_chunks(latents, chunk_latent_frames=60)``: a generator of host BTCHW pieces decoded with ONE
  continuous feature cache across pieces (so the pieces concatenate to exactly the one-shot decode), each checked
  for non-finite pixels before it leaves the device; the cache is cleared at the start and in ``finally``.

``Wan5BVAE`` (48 channels, 4 x 16 x 16 compression) and ``WanA14BVAE`` (16 channels, 4 x 8 x 8) carry the published
latent statistics; ``from_checkpoint`` builds the published topology (``models.wan_vae_released``) and fills it
strictly from the published weight file, ``build`` gives this package's own lighter topology for random-init runs.  ``flow_to_x0`` does the
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
    """48-channel Wan2.2 VAE (TI2V-5B) with its published latent statistics."""
    latent_channels = 48
    mean = (-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891,
            0.1570, -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502,
            -0.2055, -0.0322, 0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313, -0.1649, 0.0117, 0.0723,
            -0.2839, -0.2083, -0.0520, 0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667)
    std = (0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901,
            0.6885, 0.6165, 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659,
            0.7069, 0.5338, 0.4889, 0.4917, 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944,
            0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.0600, 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744)

    @classmethod
    def from_checkpoint(cls, path, *, device="cpu", dtype=torch.float32):
        """The published ``Wan2.2_VAE.pth`` in the published topology (160-wide encoder, 256-wide decoder)."""
        from ...models.wan_vae_released import ReleasedVAEConfig, load_released

        return cls(load_released(path, ReleasedVAEConfig.wan22(), cls.mean, cls.std, device=device, dtype=dtype))

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

    @classmethod
    def from_checkpoint(cls, path, *, device="cpu", dtype=torch.float32):
        """The published ``Wan2.1_VAE.pth`` (original or diffusers tensor names) in the published topology."""
        from ...models.wan_vae_released import ReleasedVAEConfig, load_released

        return cls(load_released(path, ReleasedVAEConfig.wan21(), cls.mean, cls.std, device=device, dtype=dtype))


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
