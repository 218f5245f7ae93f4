"""Packed-document layout of the H3 backend: row order, modality tags, timestep groups, native
position grids and camera rows (reference: solar/backends/minimax_h3/layout.py:219-563,
geometry.py:16-255).

Order  [text (Qwen rows) | anchor frame | audio | target video].  Position ids ``[S, 3]``:
  text   (i, 0, 0)
  video  (t, h, w) with the non-uniform temporal grid of the H3 VAE -- per latent the pixel spans
         5/3 * (1, 4, 4, 4, 4) repeating -- offset by the number of text rows, and spatial axes
         ``linspace(left, left + ratio, n, endpoint=False) * 32`` with ``ratio = dim / sqrt(H * W)``
  audio  (origin + j, 0, w_first | w_last)
Timesteps are stored per row GROUP: a table of unique values plus per-row inverse indices, which is
what the adaLN table lookup ``t_idx * 3 + tag`` consumes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

TAG_VIDEO, TAG_TEXT, TAG_AUDIO = 0, 1, 2


def temporal_positions(latent_frames: int, origin: float) -> np.ndarray:
    spans = np.array([1, 4, 4, 4, 4], dtype=np.float64) * (5.0 / 3.0)
    steps = np.concatenate([[0.0], np.cumsum(np.tile(spans, latent_frames // 5 + 2))])[:latent_frames]
    return origin + steps


def spatial_axis(n: int, other: int, left: float = 0.0) -> np.ndarray:
    ratio = n / np.sqrt(float(n) * float(other))
    return np.linspace(left, left + ratio, n, endpoint=False) * 32.0


@dataclass
class PackedLayout:
    tags: torch.Tensor           # [S] int32
    t_index: torch.Tensor        # [S] int32
    timesteps: torch.Tensor      # [T] unique values
    position_ids: torch.Tensor   # [S, 3] float64
    camera_rows: torch.Tensor    # [S] bool: rows that carry a camera matrix
    n_text: int
    n_anchor: int
    n_audio: int
    n_video: int
    rows_per_latent: int


def build_layout(*, n_text: int, latent_frames: int, grid_hw, n_audio: int = 0, anchor_frames: int = 1,
                 t_video: float = 0.5, t_anchor: float = 0.999, t_audio: float = 0.5) -> PackedLayout:
    h, w = grid_hw
    rows = h * w
    n_anchor, n_video = anchor_frames * rows, latent_frames * rows
    S = n_text + n_anchor + n_audio + n_video
    tags = np.concatenate([np.full(n_text, TAG_TEXT), np.full(n_anchor, TAG_VIDEO), np.full(n_audio, TAG_AUDIO),
                           np.full(n_video, TAG_VIDEO)]).astype(np.int32)
    values = [1.0, t_anchor, t_audio, t_video]         # text rows use the clean (t = 1) table entry
    uniq, inverse = np.unique(np.asarray(values, dtype=np.float64), return_inverse=True)
    t_index = np.concatenate([np.full(n_text, inverse[0]), np.full(n_anchor, inverse[1]), np.full(n_audio, inverse[2]),
                              np.full(n_video, inverse[3])]).astype(np.int32)
    pos = np.zeros((S, 3), dtype=np.float64)
    pos[:n_text, 0] = np.arange(n_text)
    ys, xs = spatial_axis(h, w), spatial_axis(w, h)
    grid = np.stack(np.meshgrid(ys, xs, indexing="ij"), -1).reshape(rows, 2)

    def place(start, frames, t_positions):
        for f in range(frames):
            sl = slice(start + f * rows, start + (f + 1) * rows)
            pos[sl, 0] = t_positions[f]
            pos[sl, 1:] = grid

    tpos = temporal_positions(latent_frames + anchor_frames, origin=float(n_text))
    place(n_text, anchor_frames, tpos[:anchor_frames])
    a0 = n_text + n_anchor
    pos[a0:a0 + n_audio, 0] = n_text + np.arange(n_audio)
    pos[a0:a0 + n_audio, 2] = np.where(np.arange(n_audio) < n_audio // 2, xs[0], xs[-1])
    place(a0 + n_audio, latent_frames, tpos[anchor_frames:])
    cam = np.zeros(S, dtype=bool)
    cam[n_text:n_text + n_anchor] = True
    cam[a0 + n_audio:] = True
    return PackedLayout(torch.from_numpy(tags), torch.from_numpy(t_index), torch.from_numpy(uniq).float(),
                        torch.from_numpy(pos), torch.from_numpy(cam), n_text, n_anchor, n_audio, n_video, rows)


def expand_cameras(layout: PackedLayout, w2c_per_latent: torch.Tensor) -> torch.Tensor:
    """[anchor + latent frames, 4, 4] -> per-row view matrices [S, 4, 4] (identity on camera-less rows)."""
    S = layout.tags.shape[0]
    out = torch.eye(4).repeat(S, 1, 1)
    idx = torch.nonzero(layout.camera_rows).flatten()
    frame = torch.arange(idx.numel()) // layout.rows_per_latent
    out[idx] = w2c_per_latent[frame].float()
    return out


def patchify_latents(lat: torch.Tensor) -> torch.Tensor:
    """[C, F, H, W] -> rows [F * H/2 * W/2, C*4] ordered (f, h, w)."""
    C, F, H, W = lat.shape
    return lat.view(C, F, H // 2, 2, W // 2, 2).permute(1, 2, 4, 0, 3, 5).reshape(F * (H // 2) * (W // 2), C * 4)


def unpatchify_rows(rows: torch.Tensor, C: int, F: int, H: int, W: int) -> torch.Tensor:
    return rows.view(F, H // 2, W // 2, C, 2, 2).permute(3, 0, 1, 4, 2, 5).reshape(C, F, H, W)
