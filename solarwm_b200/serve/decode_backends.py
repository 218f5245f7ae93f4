"""Decoder switch of the realtime worker: two explicit pixel decoders behind one ``push`` contract.

``conv``  the causal-convolution VAE (``models.vae.StreamingDecoder``; implicit-GEMM convolutions on a B200)
``vit``   the streaming ViT decoder (``models.vit_decoder.StreamingViTDecoder``, tiles dealt to the ranks of the
          decode group and gathered on the device)

``push(index, latent_chunk, on_piece)`` binds the decoder input to rank 0 (a broadcast, although every SP rank
already holds the chunk), decodes its latents one by one, copies each piece to pinned host memory on rank 0,
refuses non-finite pixels and hands the piece to the callback with a monotonic timestamp.  Chunks must arrive in
order.  Returns the milliseconds the call took (reference: deploy/solar_wm/shared/vae/backends.py:47-146).
"""
from __future__ import annotations

import time
from typing import Callable, Dict, Optional

import numpy as np
import torch

KINDS = ("conv", "vit")


def finite_host(value: torch.Tensor) -> bool:
    """Finite check of a host tensor; bf16 is tested on its exponent bits (no fp32 copy)."""
    if value.device.type != "cpu":
        raise ValueError("a host tensor is required")
    value = value.detach()
    if value.dtype == torch.bfloat16:
        bits = value.contiguous().view(torch.int16).numpy().view(np.uint16)
        return not bool(np.any((bits & 0x7F80) == 0x7F80))
    return bool(np.isfinite(value.numpy()).all())


class DecodeBackends:
    def __init__(self, factories: Dict[str, Callable[[], object]], *, rank: int = 0, group=None, pin: Optional[bool] = None):
        """``factories[kind]()`` builds the decoder object (``push(latent [C, h, w]) -> frames or None`` for ``vit``;
        ``push(z [1, C, 1, h, w]) -> frames`` for ``conv``) the first time the kind is started."""
        unknown = set(factories) - set(KINDS)
        if unknown:
            raise ValueError(f"unsupported decoder kinds: {sorted(unknown)}")
        self.factories, self.rank, self.group = factories, rank, group
        self.pin = torch.cuda.is_available() if pin is None else pin
        self.models: Dict[str, object] = {}
        self.kind: Optional[str] = None
        self.next_chunk = 0

    def load(self, kind: str) -> None:
        if kind not in self.factories:
            raise ValueError(f"unsupported decoder {kind!r}")
        if kind not in self.models:
            self.models[kind] = self.factories[kind]()

    def start(self, kind: str) -> None:
        self.load(kind)
        self.kind, self.next_chunk = kind, 0
        self.models[kind].reset()

    def _decode_one(self, z: torch.Tensor):
        """z [C, h, w] -> frames [3, F, H, W] on rank 0 (None elsewhere for the tile-parallel decoder)."""
        dec = self.models[self.kind]
        if self.kind == "vit":
            return dec.push(z)
        out = dec.push(z.unsqueeze(0).unsqueeze(2))
        return out[0] if self.rank == 0 else None

    @torch.no_grad()
    def push(self, index: int, latent: torch.Tensor, on_piece: Callable[[int, int, torch.Tensor, int], None]) -> float:
        """latent [C, n, h, w]; ``on_piece(chunk index, latent offset, host frames [3, F, H, W], monotonic ns)``."""
        if self.kind is None or index != self.next_chunk:
            raise RuntimeError("decoder request reordered")
        started = time.perf_counter()
        if self.group is not None or (torch.distributed.is_available() and torch.distributed.is_initialized()):
            import torch.distributed as dist

            latent = latent.contiguous()
            dist.broadcast(latent, src=0 if self.group is None else dist.get_global_rank(self.group, 0), group=self.group)
        for offset in range(latent.shape[1]):
            frames = self._decode_one(latent[:, offset])
            if self.rank != 0 or frames is None:
                continue
            host = torch.empty(frames.shape, dtype=frames.dtype, device="cpu", pin_memory=self.pin)
            host.copy_(frames, non_blocking=True)
            if frames.is_cuda:
                torch.cuda.current_stream(frames.device).synchronize()
            if not finite_host(host):
                raise FloatingPointError("nonfinite decoder pixels")
            on_piece(index, offset, host, time.monotonic_ns())
        if latent.is_cuda:
            torch.cuda.synchronize(latent.device)
        self.next_chunk += 1
        return (time.perf_counter() - started) * 1000.0

    def finish(self) -> None:
        self.kind = None

    def close(self) -> None:
        self.models.clear()
        self.kind = None
