"""Generated-versus-source comparison views.

``side_by_side`` pads two clips to a common height, trims both to the shorter length and
concatenates them on the width axis with a separator band; ``write_comparison`` encodes the view
through ``serve.media.FrameSink`` (an ffmpeg pipe when the binary exists, a raw RGB8 ``.npy``
stack otherwise) and records a small JSON manifest next to it
(reference: solar/inference/comparison.py:38-276).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping, Optional

import torch


def _fit_height(clip: torch.Tensor, height: int) -> torch.Tensor:
    """clip [T, 3, H, W] in [-1, 1] -> centred on a canvas of the given height (black bars)."""
    T, C, H, W = clip.shape
    if H == height:
        return clip
    canvas = torch.full((T, C, height, W), -1.0, dtype=clip.dtype, device=clip.device)
    top = (height - H) // 2
    canvas[:, :, top:top + H] = clip
    return canvas


def side_by_side(generated: torch.Tensor, source: torch.Tensor, separator: int = 8) -> torch.Tensor:
    """[T, 3, H, W] x 2 -> [T', 3, max(H), Wg + separator + Ws] (T' = shorter clip)."""
    if generated.dim() != 4 or source.dim() != 4 or generated.shape[1] != 3 or source.shape[1] != 3:
        raise ValueError("comparison clips are [T, 3, H, W]")
    T = min(generated.shape[0], source.shape[0])
    H = max(generated.shape[2], source.shape[2])
    g, s = _fit_height(generated[:T].float(), H), _fit_height(source[:T].float().to(generated.device), H)
    band = torch.ones(T, 3, H, separator, device=g.device)
    return torch.cat([g, band, s], dim=3)


def write_comparison(out_dir, generated: torch.Tensor, source: torch.Tensor, *, fps: float = 16.0,
                     meta: Optional[Mapping[str, object]] = None, use_ffmpeg: Optional[bool] = None) -> Mapping[str, object]:
    from ..serve.media import FrameSink

    view = side_by_side(generated, source)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    sink = FrameSink(out, width=view.shape[3], height=view.shape[2], fps=fps, use_ffmpeg=use_ffmpeg)
    for frame in view:
        sink.push(frame)
    info = dict(sink.close())
    info.update({"schema": "solarwm.comparison.v1", "frames": int(view.shape[0]), "layout": "generated|source",
                 **dict(meta or {})})
    (out / "comparison.json").write_text(json.dumps(info, sort_keys=True, default=str))
    return info
