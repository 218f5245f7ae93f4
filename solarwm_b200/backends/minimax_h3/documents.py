"""Packed attention documents of the H3 family as a list of typed segments.

``layout.build_layout`` covers what the trainers of this package feed today (text | one anchor frame | audio | target
video).  The released recipes pack more: keyframe anchors at the FIRST and / or LAST frame, *visual observations*
(reference images or clips: "free" ones get a slot of their own on the rotary clock ahead of the clip and keep their
own spatial grid; "aligned" ones sit at given target frames and are laid over a box of the target's canvas, so they
also carry those frames' cameras), and the Stage-1 document that holds every target frame twice (a clean copy for
teacher forcing and the noisy copy that is trained) with identical positions and chunk numbers.

A document is built from segments; every segment contributes rows with a modality tag, a role, ``(t, h, w)`` positions,
the target frame whose camera the row carries (-1: none) and the causal chunk it belongs to (-1: none).
``PackedDocument`` is the concatenation plus the index sets the models and losses ask for.

Position rules (the same numbers ``layout.py`` uses): text rows ``(i, 0, 0)``; video rows ``(t, h, w)`` with the
non-uniform temporal grid 5/3 x (1, 4, 4, 4, 4) per five latents, starting at the clock ``origin`` = number of text rows
plus what the free observations used; spatial axes ``(left + ratio * u) * 32`` with ``ratio = n / sqrt(H W)``,
``left = (1 - ratio) / 2`` for canvas boxes and ``u`` in ``[low, high)`` of the box.

Reference: H3VisualObservationSpec, _base_layout, build_stage0p5_layout, build_stage1_layout
(solar/backends/minimax_h3/layout.py:50-563).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np

from .layout import TAG_AUDIO, TAG_VIDEO, spatial_axis, temporal_positions

ROLE_CONDITION, ROLE_AUDIO, ROLE_CLEAN, ROLE_NOISY = 0, 1, 2, 3
_FRAME = 5.0 / 3.0


@dataclass(frozen=True)
class Observation:
    """One visual observation of ``frames`` latent frames of ``height`` x ``width`` latent pixels.  ``at`` = target
    frame indices (aligned) or None (free); ``boxes`` = ``(x0, y0, x1, y1)`` in the unit canvas, one for all frames or
    one per frame (aligned observations only; default: the whole canvas)."""

    frames: int
    height: int
    width: int
    at: Optional[Tuple[int, ...]] = None
    boxes: Optional[Tuple[Tuple[float, float, float, float], ...]] = None


@dataclass
class _Rows:
    tag: np.ndarray
    role: np.ndarray
    pos: np.ndarray
    camera_frame: np.ndarray
    chunk: np.ndarray
    kind: str


def _rows(n, tag, role, pos, camera_frame=-1, chunk=-1, kind="") -> _Rows:
    full = lambda v: np.broadcast_to(np.asarray(v, dtype=np.int64), (n,)).copy()      # noqa: E731
    return _Rows(full(tag), full(role), np.asarray(pos, dtype=np.float64).reshape(n, 3), full(camera_frame), full(chunk), kind)


def canvas_grid(rows_h: int, rows_w: int, box, target_h: int, target_w: int) -> np.ndarray:
    """``[rows_h * rows_w, 2]`` spatial positions of a frame laid over ``box`` of a ``target_h`` x ``target_w`` canvas."""
    x0, y0, x1, y1 = (float(v) for v in box)
    if not (0.0 <= x0 < x1 <= 1.0 and 0.0 <= y0 < y1 <= 1.0):
        raise ValueError(f"observation box {box} must lie inside the unit canvas")
    axes = []
    for size, low, high, count in ((target_h, y0, y1, rows_h), (target_w, x0, x1, rows_w)):
        ratio = size / np.sqrt(float(target_h) * float(target_w))
        u = low + (high - low) * np.arange(count, dtype=np.float64) / count
        axes.append(((1.0 - ratio) / 2.0 + ratio * u) * 32.0)
    gh, gw = np.meshgrid(axes[0], axes[1], indexing="ij")
    return np.stack([gh.reshape(-1), gw.reshape(-1)], -1)


def frame_grid(rows_h: int, rows_w: int) -> np.ndarray:
    ys, xs = spatial_axis(rows_h, rows_w), spatial_axis(rows_w, rows_h)
    return np.stack(np.meshgrid(ys, xs, indexing="ij"), -1).reshape(rows_h * rows_w, 2)


@dataclass
class PackedDocument:
    tags: np.ndarray              # [S] modality tag per row
    roles: np.ndarray             # [S] ROLE_*
    position_ids: np.ndarray      # [S, 3] float64
    camera_frame: np.ndarray      # [S] target frame whose camera the row carries, -1 for none
    chunk_ids: np.ndarray         # [S] causal chunk of the row, -1 for none
    kinds: Tuple[Tuple[str, int, int], ...]     # (segment kind, first row, one past the last row)
    rows_per_frame: int
    stage: str
    chunk_latent_frames: Optional[int] = None
    window_chunks: Optional[int] = None
    observation_rows: Tuple[int, ...] = ()

    def _where(self, *kinds) -> np.ndarray:
        parts = [np.arange(a, b, dtype=np.int64) for k, a, b in self.kinds if k in kinds]
        return np.concatenate(parts) if parts else np.empty(0, dtype=np.int64)

    text_indices = property(lambda self: self._where("text"))
    audio_indices = property(lambda self: self._where("audio"))
    condition_video_indices = property(lambda self: self._where("anchor", "observation"))
    observation_indices = property(lambda self: self._where("observation"))
    clean_video_indices = property(lambda self: self._where("clean"))
    noisy_video_indices = property(lambda self: self._where("noisy"))
    target_video_indices = noisy_video_indices
    video_indices = property(lambda self: self._where("anchor", "observation", "clean", "noisy"))
    camera_indices = property(lambda self: np.nonzero(self.camera_frame >= 0)[0])

    @property
    def sequence_length(self) -> int:
        return int(self.tags.shape[0])

    @property
    def target_video_output_slice(self) -> slice:
        """The trained rows inside an output that was already filtered to video rows."""
        start = len(self.condition_video_indices) + len(self.clean_video_indices)
        return slice(start, start + len(self.noisy_video_indices))

    def camera_rows(self, w2c_per_frame) -> "np.ndarray":
        """``[frames, 4, 4]`` cameras -> per-row ``[S, 4, 4]`` (identity where a row carries none)."""
        out = np.tile(np.eye(4), (self.sequence_length, 1, 1))
        idx = self.camera_indices
        out[idx] = np.asarray(w2c_per_frame, dtype=np.float64)[self.camera_frame[idx]]
        return out

    def to_layout_tensors(self, device="cpu"):
        import torch

        return {"tags": torch.from_numpy(self.tags.astype(np.int32)).to(device),
                "position_ids": torch.from_numpy(self.position_ids).to(device),
                "roles": torch.from_numpy(self.roles).to(device), "chunk_ids": torch.from_numpy(self.chunk_ids).to(device)}


def _assemble(segments: Sequence[_Rows], **meta) -> PackedDocument:
    kinds, start = [], 0
    for s in segments:
        kinds.append((s.kind, start, start + len(s.tag)))
        start += len(s.tag)
    cat = lambda name: np.concatenate([getattr(s, name) for s in segments])           # noqa: E731
    return PackedDocument(cat("tag"), cat("role"), cat("pos"), cat("camera_frame"), cat("chunk"), tuple(kinds), **meta)


def _condition_segments(text_tags, frames: int, h: int, w: int, anchors: Sequence[str], observations: Sequence[Observation],
                        audio_latents: int, audio_channels: int):
    """Everything in front of the target video, plus the clip's temporal grid and the clock origin."""
    text_tags = np.asarray(text_tags, dtype=np.int64).reshape(-1)
    if frames < 1 or h < 1 or w < 1:
        raise ValueError("the target clip needs at least one frame and one row")
    n_text, rows = int(text_tags.size), h * w
    tpos = np.zeros((n_text, 3))
    tpos[:, 0] = np.arange(n_text)
    segs = [_Rows(text_tags, np.full(n_text, ROLE_CONDITION), tpos, np.full(n_text, -1), np.full(n_text, -1), "text")]
    # free observations advance the clock ahead of the clip
    origin, free_times = float(n_text), []
    for ob in observations:
        if ob.frames < 1 or ob.height < 1 or ob.width < 1:
            raise ValueError(f"{ob} is empty")
        if ob.at is not None and (len(ob.at) != ob.frames or min(ob.at) < 0 or max(ob.at) >= frames):
            raise ValueError(f"{ob} is not aligned with the {frames} target frames")
        if ob.boxes is not None and (ob.at is None or len(ob.boxes) not in (1, ob.frames)):
            raise ValueError(f"{ob}: boxes need target frames, one box for all or one per frame")
        if ob.at is not None:
            free_times.append(None)
        elif ob.frames == 1:
            free_times.append(np.asarray([origin]))
            origin += 1.0
        else:
            free_times.append(temporal_positions(ob.frames, origin))
            origin += float(np.diff(temporal_positions(ob.frames + 1, 0.0)).sum())
    clip_t = temporal_positions(frames, origin)
    grid = frame_grid(h, w)
    for anchor in anchors:
        if anchor == "first":
            t, fid = origin, 0
        elif anchor == "last":
            t, fid = float(temporal_positions(frames + 1, origin)[-1] - _FRAME), frames - 1
        else:
            raise ValueError(f"keyframe anchor must be 'first' or 'last', got {anchor!r}")
        segs.append(_rows(rows, TAG_VIDEO, ROLE_CONDITION, np.concatenate([np.full((rows, 1), t), grid], 1), fid, -1, "anchor"))
    ob_rows = []
    for ob, free in zip(observations, free_times):
        per = ob.height * ob.width
        n = ob.frames * per
        ob_rows.append(n)
        if free is not None:
            times, cams = free, np.full(n, -1)
            spatial = np.tile(frame_grid(ob.height, ob.width), (ob.frames, 1))
        else:
            times, cams = clip_t[np.asarray(ob.at)], np.repeat(np.asarray(ob.at), per)
            boxes = ob.boxes or ((0.0, 0.0, 1.0, 1.0),)
            grids = [canvas_grid(ob.height, ob.width, b, h, w) for b in boxes]
            spatial = np.tile(grids[0], (ob.frames, 1)) if len(grids) == 1 else np.concatenate(grids, 0)
        pos = np.concatenate([np.repeat(times, per)[:, None], spatial], 1)
        segs.append(_Rows(np.full(n, TAG_VIDEO), np.full(n, ROLE_CONDITION), pos, cams, np.full(n, -1), "observation"))
    if audio_latents:
        xs = spatial_axis(w, h)
        n = audio_latents * audio_channels
        pos = np.zeros((n, 3))
        pos[:, 0] = np.tile(origin + np.arange(audio_latents), audio_channels)
        pos[:, 2] = np.repeat(np.asarray([xs[0], xs[-1]])[:audio_channels], audio_latents) if audio_channels <= 2 \
            else np.repeat(np.linspace(xs[0], xs[-1], audio_channels), audio_latents)
        segs.append(_rows(n, TAG_AUDIO, ROLE_AUDIO, pos, -1, -1, "audio"))
    return segs, clip_t, grid, tuple(ob_rows)


def _clip_rows(clip_t, grid, role: int, kind: str, chunk_latent_frames: Optional[int]) -> _Rows:
    frames, rows = len(clip_t), grid.shape[0]
    pos = np.concatenate([np.repeat(clip_t, rows)[:, None], np.tile(grid, (frames, 1))], 1)
    chunk = np.repeat(np.arange(frames) // chunk_latent_frames, rows) if chunk_latent_frames else -1
    return _rows(frames * rows, TAG_VIDEO, role, pos, np.repeat(np.arange(frames), rows), chunk, kind)


def stage0p5_document(text_tags, frames: int, grid_hw, *, anchors: Sequence[str] = ("first",),
                      observations: Sequence[Observation] = (), audio_latents: int = 0, audio_channels: int = 2) -> PackedDocument:
    """Bidirectional document: conditions, then the noisy target clip."""
    h, w = grid_hw
    segs, clip_t, grid, ob_rows = _condition_segments(text_tags, frames, h, w, anchors, observations, audio_latents, audio_channels)
    segs.append(_clip_rows(clip_t, grid, ROLE_NOISY, "noisy", None))
    return _assemble(segs, rows_per_frame=h * w, stage="stage0p5", observation_rows=ob_rows)


def stage1_document(text_tags, frames: int, grid_hw, *, chunk_latent_frames: int = 5, window_chunks: int = 6,
                    anchors: Sequence[str] = ("first",), observations: Sequence[Observation] = (), audio_latents: int = 0,
                    audio_channels: int = 2) -> PackedDocument:
    """Teacher-forcing document: conditions, a CLEAN copy of the clip and the NOISY copy that is trained; both copies
    have the same positions, cameras and chunk numbers."""
    if chunk_latent_frames < 1 or window_chunks < 1 or frames % chunk_latent_frames:
        raise ValueError(f"{frames} frames do not split into chunks of {chunk_latent_frames} (window {window_chunks})")
    h, w = grid_hw
    segs, clip_t, grid, ob_rows = _condition_segments(text_tags, frames, h, w, anchors, observations, audio_latents, audio_channels)
    segs.append(_clip_rows(clip_t, grid, ROLE_CLEAN, "clean", chunk_latent_frames))
    segs.append(_clip_rows(clip_t, grid, ROLE_NOISY, "noisy", chunk_latent_frames))
    return _assemble(segs, rows_per_frame=h * w, stage="stage1", chunk_latent_frames=chunk_latent_frames,
                     window_chunks=window_chunks, observation_rows=ob_rows)
