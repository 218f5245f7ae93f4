"""The fixed audio input of the video-only H3 stages: encoded silence.

The released model is an audio-video model; the world-model stages train and sample it with a SILENT soundtrack: the
audio stream's rows are the audio codec's encoding of silence (one tensor ``[2, 32, L]`` per supported clip length, stored
as ``silence_<frames>f`` in one safetensors file), noised to their own time like any other row, and their prediction is
ignored.  ``silence_rows`` turns the stored tensor into packed rows ``[2 L, 32]`` (channel pair major, time minor, as the
model's audio projection expects).

Reference: load_silence_latents (solar/backends/minimax_h3/artifacts.py:814-842), H3Stage0p5Core.audio_rows.
"""
from __future__ import annotations

from pathlib import Path
from typing import Tuple

import torch

from ...errors import DataContractError

LENGTHS = {153: 255, 158: 263, 170: 283}
AUDIO_SHIFT = 3.0


def load_silence_latents(path, *, pixel_frames: int = 158) -> torch.Tensor:
    src = Path(path)
    if not src.is_file():
        raise DataContractError(f"the silence artifact is missing: {src}")
    if pixel_frames not in LENGTHS:
        raise DataContractError("silence is stored for the 153-, 158- and 170-frame profiles")
    try:
        from safetensors.torch import load_file

        tensors = load_file(str(src), device="cpu")
    except Exception as exc:  # noqa: BLE001 - whatever the parser raises for a damaged file
        raise DataContractError("the silence artifact is not a valid safetensors file") from exc
    key = f"silence_{pixel_frames}f"
    if key not in tensors:
        raise DataContractError(f"the silence artifact lacks {key!r}")
    value = tensors[key].contiguous()
    if tuple(value.shape) != (2, 32, LENGTHS[pixel_frames]) or value.dtype != torch.bfloat16:
        raise DataContractError(f"silence must be bf16 [2, 32, {LENGTHS[pixel_frames]}]")
    if not bool(torch.isfinite(value.float()).all()):
        raise DataContractError("silence contains non-finite values")
    return value


def silence_rows(value: torch.Tensor) -> torch.Tensor:
    """[2, 32, L] -> packed audio rows [2 L, 32]."""
    if value.dim() != 3 or value.shape[0] != 2:
        raise DataContractError("silence is a [2, channels, L] tensor")
    return value.permute(0, 2, 1).reshape(-1, value.shape[1]).contiguous()


def noised_silence(rows: torch.Tensor, generator: torch.Generator, device) -> Tuple[torch.Tensor, float]:
    """The rows at a freshly drawn audio time (shifted as the audio stream's schedule is): ``(rows_t, t_audio)``."""
    from . import flow

    u = torch.rand(1, generator=generator, device=device)
    t = float(1.0 - flow.shifted_sigma(u, AUDIO_SHIFT))
    noise = torch.randn(rows.shape, generator=generator, device=device, dtype=torch.float32)
    return (t * rows.to(device).float() + (1.0 - t) * noise), t
