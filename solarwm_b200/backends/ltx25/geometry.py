"""The one clip geometry of the LTX-2.5 recipes and the arithmetic that brings a source clip into it.

A 768 x 512 clip of 153 frames at 24 fps becomes ``[128, 20, 16, 24]`` latents: the causal VAE keeps the first frame
on its own and folds every further 8 frames into one latent (``1 + 8 n`` pixel frames -> ``1 + n`` latents), and shrinks
space by 32.  The cameras that condition latent ``i`` are those of the FIRST pixel frame of its interval: 0, 1, 9, 17,
..., 145.  Sources of another size are cover-resized (the short side meets the target, integer truncation as the
recipe's bicubic resize does it) and centre-cropped; their pinhole intrinsics follow the same resize and crop and are
then normalised by the target size.  A training window is 153 CONSECUTIVE source frames; the source frame rate is not
consulted.

Reference: LTX25Geometry, cover_resize, transform_intrinsics, validate_contiguous_source_indices
(solar/backends/ltx25/geometry.py:18-215).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from ...errors import BackendContractError

PIXEL_FRAMES, HEIGHT, WIDTH = 153, 512, 768
TEMPORAL_FACTOR, SPATIAL_FACTOR, LATENT_CHANNELS, MODEL_FPS = 8, 32, 128, 24.0


def _positive(name: str, value) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, np.integer)) or value <= 0:
        raise BackendContractError(f"{name} must be a positive integer, got {value!r}")
    return int(value)


def latent_frames_of(pixel_frames: int, factor: int = TEMPORAL_FACTOR) -> int:
    frames, factor = _positive("pixel_frames", pixel_frames), _positive("temporal_factor", factor)
    if (frames - 1) % factor:
        raise BackendContractError(f"a causal VAE takes 1 + {factor} n pixel frames, not {frames}")
    return 1 + (frames - 1) // factor


def camera_pixel_indices(pixel_frames: int = PIXEL_FRAMES, factor: int = TEMPORAL_FACTOR) -> Tuple[int, ...]:
    """Pixel frame whose camera conditions each latent: 0, then the first frame of every ``factor``-frame interval."""
    n = latent_frames_of(pixel_frames, factor)
    return (0,) + tuple(1 + i * factor for i in range(n - 1))


@dataclass(frozen=True)
class ClipGeometry:
    pixel_frames: int = PIXEL_FRAMES
    height: int = HEIGHT
    width: int = WIDTH

    def __post_init__(self):
        if (self.pixel_frames, self.height, self.width) != (PIXEL_FRAMES, HEIGHT, WIDTH):
            raise BackendContractError(f"the LTX-2.5 recipes are fixed to {WIDTH}x{HEIGHT}x{PIXEL_FRAMES}f, got "
                                       f"{self.width}x{self.height}x{self.pixel_frames}f")

    latent_frames = property(lambda self: latent_frames_of(self.pixel_frames))
    latent_height = property(lambda self: self.height // SPATIAL_FACTOR)
    latent_width = property(lambda self: self.width // SPATIAL_FACTOR)
    latent_shape = property(lambda self: (LATENT_CHANNELS, self.latent_frames, self.latent_height, self.latent_width))
    first_frame_latent_shape = property(lambda self: (LATENT_CHANNELS, 1, self.latent_height, self.latent_width))
    tokens_per_latent = property(lambda self: self.latent_height * self.latent_width)
    video_tokens = property(lambda self: self.latent_frames * self.tokens_per_latent)
    camera_pixel_indices = property(lambda self: camera_pixel_indices(self.pixel_frames))


STABLE = ClipGeometry()


@dataclass(frozen=True)
class CoverResize:
    source_height: int
    source_width: int
    resized_height: int
    resized_width: int
    crop_top: int
    crop_left: int
    target_height: int = HEIGHT
    target_width: int = WIDTH

    scale_y = property(lambda self: self.resized_height / self.source_height)
    scale_x = property(lambda self: self.resized_width / self.source_width)


def cover_resize(source_height: int, source_width: int) -> CoverResize:
    sh, sw = _positive("source_height", source_height), _positive("source_width", source_width)
    if sw / sh > WIDTH / HEIGHT:                       # wider than the target: heights meet, the width overhangs
        rh, rw = HEIGHT, int(HEIGHT * (sw / sh))
    else:
        rh, rw = int(WIDTH / (sw / sh)), WIDTH
    return CoverResize(sh, sw, rh, rw, (rh - HEIGHT) // 2, (rw - WIDTH) // 2)


def transform_intrinsics(intrinsics, how: CoverResize, *, input_normalized: Optional[bool] = None) -> np.ndarray:
    """One no-skew pinhole matrix through the resize and the crop, normalised by the target size (fx / W, fy / H,
    cx / W, cy / H).  Inputs whose entries are all <= 4 in magnitude are taken as already normalised by the SOURCE size
    unless ``input_normalized`` says otherwise.  The normalised focal length has no upper bound."""
    k = np.asarray(intrinsics, dtype=np.float64)
    if k.shape != (3, 3) or not np.isfinite(k).all():
        raise BackendContractError("intrinsics must be one finite [3, 3] matrix")
    if not np.allclose(k[2], (0.0, 0.0, 1.0), atol=1e-7, rtol=0.0) or abs(k[0, 1]) > 1e-7 or abs(k[1, 0]) > 1e-7:
        raise BackendContractError("intrinsics must be a zero-skew pinhole matrix with bottom row [0, 0, 1]")
    fx, fy, cx, cy = k[0, 0], k[1, 1], k[0, 2], k[1, 2]
    if input_normalized is None:
        input_normalized = bool(max(abs(fx), abs(fy), abs(cx), abs(cy)) <= 4.0)
    if input_normalized:
        fx, cx, fy, cy = fx * how.source_width, cx * how.source_width, fy * how.source_height, cy * how.source_height
    out = np.asarray([[fx * how.scale_x / how.target_width, 0.0, (cx * how.scale_x - how.crop_left) / how.target_width],
                      [0.0, fy * how.scale_y / how.target_height, (cy * how.scale_y - how.crop_top) / how.target_height],
                      [0.0, 0.0, 1.0]], dtype=np.float32)
    if not np.isfinite(out).all() or out[0, 0] <= 0 or out[1, 1] <= 0:
        raise BackendContractError("transformed focal lengths must be finite and positive")
    return out


def check_window(source_indices, *, start: Optional[int] = None) -> np.ndarray:
    """A training window: exactly 153 consecutive, non-negative source frame ordinals (int64)."""
    idx = np.asarray(source_indices)
    if idx.dtype != np.int64 or idx.shape != (PIXEL_FRAMES,):
        raise BackendContractError(f"a window is int64 [{PIXEL_FRAMES}] source ordinals")
    if idx[0] < 0 or not np.all(np.diff(idx) == 1):
        raise BackendContractError("a window holds consecutive, non-negative source ordinals")
    if start is not None and int(idx[0]) != int(start):
        raise BackendContractError("the window does not begin at the declared start frame")
    return idx


def window_cameras(per_pixel_frame, geometry: ClipGeometry = STABLE):
    """``[153, ...]`` per-pixel-frame camera quantities -> ``[20, ...]``: the ones that condition each latent."""
    values = np.asarray(per_pixel_frame)
    if values.shape[0] != geometry.pixel_frames:
        raise BackendContractError(f"expected {geometry.pixel_frames} per-frame cameras, got {values.shape[0]}")
    return values[np.asarray(geometry.camera_pixel_indices)]
