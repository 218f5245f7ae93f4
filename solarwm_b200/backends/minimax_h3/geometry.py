"""H3 clip geometry and raw-camera decoding: the rules that tie pixel frames, latent frames, cameras and the canvas together.

  frames     the video codec takes ``17 n + 5`` pixel frames and gives ``5 n + 2`` latents; latent ``i`` sits on the source
             frame ``17 (i // 5) + (0, 1, 5, 9, 13)[i % 5]`` (the last, partial period keeps its in-range offsets), so a clip
             is never re-timed: its cameras are simply read at those frames.  158 frames <-> 47 latents.
  audio      25 audio latents per second on the 24 frames-per-second timeline, rounded.
  canvas     heights and widths are multiples of 32; anything else is refused rather than rounded.
  cameras    a camera archive carries absolute camera-to-world (or world-to-camera) poses under one of several names, with a
             tracker status that must be ``ok``; intrinsics arrive as 3 x 3 matrices or ``(fx, fy, cx, cy)`` vectors, one for
             the clip or one per frame, in pixels or already normalised (both focal lengths and principal point at most 4 in
             magnitude means normalised).  They are carried through the resize + crop of the preprocessing and normalised by
             the target canvas; focal lengths outside (0, 4] trip the guard unless the model replaces source focal lengths
             with its fixed ones.  Without any intrinsics the fixed training camera is used.

Reference: solar/backends/minimax_h3/geometry.py:16-260, raw_data.py:104-251.
"""
from __future__ import annotations

import io
from dataclasses import dataclass
from typing import Mapping, Optional, Sequence, Tuple

import numpy as np

from ...errors import DataContractError

PIXELS_PER_PERIOD, LATENTS_PER_PERIOD, PREFIX = 17, 5, 2
OFFSETS = (0, 1, 5, 9, 13)
SEMANTIC_FPS, AUDIO_LATENTS_PER_SECOND = 24.0, 25
FIXED_FOCAL = (969.6969696969696 / 1920.0, 969.6969696969696 / 1080.0)
POSE_KEYS = (("vipe_c2w", False), ("vipe_w2c", True), ("camera_c2w", False), ("c2w", False), ("camera_w2c", True), ("w2c", True))
K_KEYS = ("camera_K", "K", "intrinsics")


def align_pixel_frames(frames: int) -> int:
    """Round up to the next ``17 n + 5``."""
    if frames < 1:
        raise ValueError(f"frames must be positive, got {frames}")
    frames = int(frames)
    return frames + (LATENTS_PER_PERIOD - frames) % PIXELS_PER_PERIOD


def pixel_to_latent_frames(frames: int) -> int:
    if frames < LATENTS_PER_PERIOD or frames % PIXELS_PER_PERIOD != LATENTS_PER_PERIOD:
        raise ValueError(f"pixel frames must be 17 n + 5, got {frames}")
    return (frames - LATENTS_PER_PERIOD) // PIXELS_PER_PERIOD * LATENTS_PER_PERIOD + PREFIX


def latent_to_pixel_frames(latents: int) -> int:
    if latents < PREFIX or (latents - PREFIX) % LATENTS_PER_PERIOD:
        raise ValueError(f"latent frames must be 5 n + 2, got {latents}")
    return (latents - PREFIX) // LATENTS_PER_PERIOD * PIXELS_PER_PERIOD + LATENTS_PER_PERIOD


def latent_pixel_indices(frames: int) -> np.ndarray:
    """The source frame of every latent of a ``17 n + 5`` clip."""
    want = pixel_to_latent_frames(frames)
    i = np.arange(want)
    idx = PIXELS_PER_PERIOD * (i // LATENTS_PER_PERIOD) + np.asarray(OFFSETS)[i % LATENTS_PER_PERIOD]
    if idx[-1] >= frames:
        raise RuntimeError("pixel / latent alignment is inconsistent")
    return idx.astype(np.int64)


def audio_latents_for_video(frames: int, fps: float = SEMANTIC_FPS, per_second: int = AUDIO_LATENTS_PER_SECOND) -> int:
    if frames < 1 or fps <= 0 or per_second <= 0:
        raise ValueError("frames, fps and latents per second must be positive")
    return round(frames / fps * per_second)


def validate_canvas(height: int, width: int, multiple: int = 32) -> Tuple[int, int]:
    if height <= 0 or width <= 0 or multiple <= 0 or height % multiple or width % multiple:
        raise ValueError(f"height and width must be positive multiples of {multiple}, got {(height, width)}")
    return int(height), int(width)


@dataclass(frozen=True)
class ResizeCrop:
    """Source ``source_w x source_h`` resized to ``resized_w x resized_h``, then a ``target_w x target_h`` window cut at
    ``(crop_left, crop_top)``."""
    source_w: int
    source_h: int
    resized_w: int
    resized_h: int
    target_w: int
    target_h: int
    crop_left: int = 0
    crop_top: int = 0

    @classmethod
    def cover(cls, source_w: int, source_h: int, target_w: int, target_h: int) -> "ResizeCrop":
        """Aspect-preserving resize that covers the target, centre crop."""
        scale = max(target_w / source_w, target_h / source_h)
        rw, rh = max(target_w, round(source_w * scale)), max(target_h, round(source_h * scale))
        return cls(source_w, source_h, rw, rh, target_w, target_h, (rw - target_w) // 2, (rh - target_h) // 2)


def fixed_intrinsics(count: int) -> np.ndarray:
    K = np.zeros((count, 3, 3), dtype=np.float32)
    K[:, 0, 0], K[:, 1, 1] = FIXED_FOCAL
    K[:, 0, 2] = K[:, 1, 2] = 0.5
    K[:, 2, 2] = 1.0
    return K


def normalise_intrinsics(candidate, source_indices: Sequence[int], how: ResizeCrop, *, focal_guard: bool = True) -> np.ndarray:
    """Intrinsics of the selected frames on the target canvas, normalised by its size: ``[len(source_indices), 3, 3]``."""
    n, top = len(source_indices), max(source_indices)
    if candidate is None:
        return fixed_intrinsics(n)
    value = np.asarray(candidate, dtype=np.float64)
    pick = np.asarray(source_indices)

    def per_frame(rows, width):
        if rows.shape[0] > top:
            return rows[pick].copy()
        if rows.shape[0] == 1:
            return np.broadcast_to(rows, (n, *width)).copy()
        raise DataContractError("camera intrinsics cannot be aligned to the selected source frames")

    if value.shape == (3, 3):
        K = np.broadcast_to(value, (n, 3, 3)).copy()
    elif value.ndim == 3 and value.shape[1:] == (3, 3):
        K = per_frame(value, (3, 3))
    elif value.shape == (4,) or (value.ndim == 2 and value.shape[1] == 4):
        vec = per_frame(value.reshape(-1, 4), (4,))
        K = np.zeros((n, 3, 3))
        K[:, 0, 0], K[:, 1, 1], K[:, 0, 2], K[:, 1, 2], K[:, 2, 2] = vec[:, 0], vec[:, 1], vec[:, 2], vec[:, 3], 1.0
    else:
        raise DataContractError(f"unsupported camera intrinsics shape {value.shape}")
    already = np.nanmax(np.abs(K[:, (0, 1), (0, 1)])) <= 4 and np.nanmax(np.abs(K[:, (0, 1), (2, 2)])) <= 4
    if already:                                   # normalised by the source size: back to source pixels first
        K[:, 0, :] *= how.source_w
        K[:, 1, :] *= how.source_h
    sx, sy = how.resized_w / how.source_w, how.resized_h / how.source_h
    K[:, 0, 0] *= sx
    K[:, 1, 1] *= sy
    K[:, 0, 2] = K[:, 0, 2] * sx - how.crop_left
    K[:, 1, 2] = K[:, 1, 2] * sy - how.crop_top
    K[:, 0, :] /= how.target_w
    K[:, 1, :] /= how.target_h
    K[:, 2, :] = (0.0, 0.0, 1.0)
    focal = K[:, (0, 1), (0, 1)]
    if not np.isfinite(K).all() or (focal_guard and (np.any(focal <= 0) or np.any(focal > 4))):
        raise DataContractError("camera intrinsics exceed the normalised guards")
    return K.astype(np.float32)


def _invert_rigid(m) -> np.ndarray:
    m = np.asarray(m, dtype=np.float64)
    out = np.tile(np.eye(4), (m.shape[0], 1, 1))
    R = np.transpose(m[:, :3, :3], (0, 2, 1))
    out[:, :3, :3] = R
    out[:, :3, 3] = -np.einsum("nij,nj->ni", R, m[:, :3, 3])
    return out.astype(np.float32)


def _intrinsics_of(archive, extra: Optional[bytes]):
    if extra:
        loaded = np.load(io.BytesIO(extra), allow_pickle=False)
        if isinstance(loaded, np.lib.npyio.NpzFile):
            try:
                for key in K_KEYS:
                    if key in loaded.files:
                        return np.asarray(loaded[key])
                raise DataContractError("the intrinsics archive holds none of camera_K, K, intrinsics")
            finally:
                loaded.close()
        return np.asarray(loaded)
    names = set(archive.files)
    for key in K_KEYS:
        if key in names:
            return np.asarray(archive[key])
    if {"fx", "fy"} <= names:
        fx, fy = np.asarray(archive["fx"]), np.asarray(archive["fy"])
        cx = np.asarray(archive["cx"]) if "cx" in names else 0.5
        cy = np.asarray(archive["cy"]) if "cy" in names else 0.5
        return np.stack(np.broadcast_arrays(fx, fy, cx, cy), axis=-1)
    return None


def decode_camera(camera_bytes: bytes, source_indices: Sequence[int], how: ResizeCrop, *, intrinsics_bytes: Optional[bytes] = None,
                  focal_guard: bool = True):
    """``(absolute c2w [n, 4, 4], normalised K [n, 3, 3])`` of the selected source frames of one clip."""
    with np.load(io.BytesIO(camera_bytes), allow_pickle=False) as archive:
        names = set(archive.files)
        if "vipe_status" in names:
            status = str(np.asarray(archive["vipe_status"]).reshape(-1)[0]).strip().lower()
            if status != "ok":
                raise DataContractError(f"the camera tracker's status is {status!r}")
        for key, inverted in POSE_KEYS:
            if key in names:
                poses = _invert_rigid(archive[key]) if inverted else np.asarray(archive[key], dtype=np.float32)
                break
        else:
            raise DataContractError("the camera archive has no camera-to-world or world-to-camera array")
        K = _intrinsics_of(archive, intrinsics_bytes)
    if poses.ndim != 3 or poses.shape[1:] != (4, 4):
        raise DataContractError("camera poses must be [N, 4, 4]")
    if poses.shape[0] <= max(source_indices):
        raise DataContractError("the camera track is shorter than the selected window")
    c2w = poses[np.asarray(source_indices)].copy()
    if not np.isfinite(c2w).all():
        raise DataContractError("camera poses contain non-finite values")
    return c2w.astype(np.float32), normalise_intrinsics(K, source_indices, how, focal_guard=focal_guard)
