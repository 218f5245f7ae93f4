"""Camera conventions (NumPy, no torch).

* NPZ members ``c2w / w2c / vipe_c2w / vipe_w2c / relative_w2c`` -> ``[T,4,4]`` (pickle refused,
  VIPE status must be ``ok``)
* rigid inverse, first-frame-relative world-to-camera (row 0 must come out as identity)
* ``logd4`` translation compression ``t * log1p(|t|) / (4 |t|)`` for model conditioning
* guards: relative translation norm <= 20 and |entry| <= 20 over the audited prefix
* latent-aligned pixel indices of a causal VAE: frame 0, then every ``temporal_stride``-th frame from 1
* the fixed normalised pinhole intrinsics all backends condition on, and PRoPE projection matrices

Reference: solar/data/camera.py:34-157, solar/backends/wan22/runtime/data.py:34-35,477-536.
"""
from __future__ import annotations

import io
from dataclasses import dataclass
from typing import Optional

import numpy as np

from ..errors import DataContractError

_KEYS = {"c2w": "absolute_c2w", "w2c": "absolute_w2c", "vipe_c2w": "absolute_c2w", "vipe_w2c": "absolute_w2c",
         "relative_w2c": "relative_w2c"}

# fx, fy of the fixed normalised intrinsics K = [[fx,0,.5],[0,fy,.5],[0,0,1]]
FIXED_FX = 969.697 / (2 * 960)
FIXED_FY = 969.697 / (2 * 540)


class CameraGuardError(DataContractError):
    pass


def _matrices(value, name: str) -> np.ndarray:
    m = np.asarray(value)
    if m.ndim != 3 or m.shape[1:] != (4, 4):
        raise DataContractError(f"{name} must have shape [T,4,4], got {m.shape}")
    if not np.isfinite(m).all():
        raise DataContractError(f"{name} contains non-finite values")
    return m


def load_camera_npz(blob: bytes, array_key: str):
    if array_key not in _KEYS:
        raise DataContractError(f"unsupported camera array key {array_key!r}")
    try:
        with np.load(io.BytesIO(blob), allow_pickle=False) as archive:
            if array_key.startswith("vipe_") and "vipe_status" in archive.files:
                status = str(np.asarray(archive["vipe_status"]).reshape(-1)[0]).lower()
                if status != "ok":
                    raise DataContractError(f"VIPE camera status is {status!r}, expected 'ok'")
            if array_key not in archive.files:
                raise DataContractError(f"camera archive lacks declared array {array_key!r}")
            mats = np.asarray(archive[array_key])
    except (OSError, ValueError) as exc:
        raise DataContractError("camera member is not a valid non-pickled NPZ") from exc
    return _matrices(mats, array_key), _KEYS[array_key]


def invert_se3(mats) -> np.ndarray:
    m = _matrices(mats, "SE3")
    out = np.zeros_like(m)
    rt = np.swapaxes(m[:, :3, :3], -1, -2)
    out[:, :3, :3] = rt
    out[:, :3, 3] = -np.einsum("tij,tj->ti", rt, m[:, :3, 3])
    out[:, 3, 3] = 1
    return out


def absolute_c2w(mats, storage: str) -> np.ndarray:
    m = _matrices(mats, "camera")
    if storage == "absolute_c2w":
        return m
    if storage == "absolute_w2c":
        return invert_se3(m)
    raise DataContractError("relative_w2c cannot be converted back to authoritative absolute C2W")


def relative_w2c(mats, storage: str) -> np.ndarray:
    m = _matrices(mats, "camera")
    if storage == "relative_w2c":
        rel = m.copy()
    else:
        c2w = absolute_c2w(m, storage)
        rel = np.matmul(invert_se3(c2w), c2w[0])
    if not np.allclose(rel[0], np.eye(4, dtype=rel.dtype), rtol=1e-5, atol=1e-5):
        raise DataContractError("first relative W2C row is not identity")
    return rel


def relative_c2w(mats, storage: str) -> np.ndarray:
    return invert_se3(relative_w2c(mats, storage))


def transform_translation(relative, transform: str) -> np.ndarray:
    m = _matrices(relative, "relative camera")
    if transform == "linear":
        return m
    if transform != "logd4":
        raise DataContractError(f"unknown camera translation transform {transform!r}")
    out = m.copy()
    dt = np.float64 if m.dtype == np.float64 else np.float32
    t = m[:, :3, 3].astype(dt, copy=False)
    norm = np.linalg.norm(t, axis=-1)
    scale = np.zeros_like(norm)
    nz = norm != 0
    scale[nz] = np.log1p(norm[nz]) / (4.0 * norm[nz])
    out[:, :3, 3] = (t * scale[:, None]).astype(out.dtype, copy=False)
    return out


@dataclass(frozen=True)
class CameraGuards:
    max_rel_translation: Optional[float] = 20.0
    max_camera_abs: Optional[float] = 20.0

    def apply(self, relative, *, audit_rows: Optional[int] = None) -> np.ndarray:
        m = _matrices(relative, "relative camera")
        n = m.shape[0] if audit_rows is None else int(audit_rows)
        if not 1 <= n <= m.shape[0]:
            raise DataContractError("audit_rows is outside the camera trajectory")
        head = m[:n]
        if self.max_rel_translation is not None and \
                float(np.linalg.norm(head[:, :3, 3], axis=-1).max(initial=0.0)) > self.max_rel_translation:
            raise CameraGuardError("relative translation exceeds configured guard")
        if self.max_camera_abs is not None and float(np.abs(head).max(initial=0.0)) > self.max_camera_abs:
            raise CameraGuardError("camera matrix exceeds configured absolute guard")
        return m.copy()


def audited_rows(count: int, fps: float, max_seconds: float) -> int:
    if count == 0:
        return 0
    if not np.isfinite(fps) or fps <= 0 or not np.isfinite(max_seconds) or max_seconds <= 0:
        return count
    return min(count, max(1, int(np.ceil(float(fps) * float(max_seconds)))))


def causal_pixel_indices(pixel_frames: int, temporal_stride: int) -> np.ndarray:
    if pixel_frames < 1 or temporal_stride < 1:
        raise DataContractError("pixel_frames and temporal_stride must be positive")
    if pixel_frames == 1:
        return np.asarray([0], dtype=np.int64)
    return np.asarray([0, *range(1, pixel_frames, temporal_stride)], dtype=np.int64)


def fixed_intrinsics(count: int, dtype=np.float32) -> np.ndarray:
    k = np.array([[FIXED_FX, 0, 0.5], [0, FIXED_FY, 0.5], [0, 0, 1]], dtype=dtype)
    return np.broadcast_to(k, (count, 3, 3)).copy()


def camera_tokens(c2w, *, pixel_frames: int, temporal_stride: int, tokens_per_frame: int, transform: str = "linear",
                  guards: CameraGuards = CameraGuards(), storage: str = "absolute_c2w"):
    """Latent-aligned, first-frame-relative W2C view matrices repeated per token, plus fixed K."""
    idx = causal_pixel_indices(pixel_frames, temporal_stride)
    rel = relative_w2c(np.asarray(c2w, dtype=np.float32), storage)
    rel = guards.apply(rel)[idx]
    rel = transform_translation(rel, transform)
    view = np.repeat(rel, tokens_per_frame, axis=0)
    return {"viewmats": view.astype(np.float32), "K": fixed_intrinsics(view.shape[0])}


def prope_matrices(viewmats, K):
    """PRoPE projection ``P = lift(K') @ view`` per token (principal point dropped) and its inverse.
    Queries use ``P^T``, keys and values ``P^-1``, outputs ``P`` on each 4-vector of a head."""
    view = np.asarray(viewmats, dtype=np.float64)
    k = np.asarray(K, dtype=np.float64)
    lift = np.zeros(view.shape, dtype=np.float64)
    lift[:, 0, 0], lift[:, 1, 1] = k[:, 0, 0], k[:, 1, 1]
    lift[:, 2, 2] = lift[:, 3, 3] = 1.0
    P = np.matmul(lift, view)
    return P, np.linalg.inv(P)
