"""Raw (compressed) video members -> frame tensors, on OpenCV's decoder.

``decode_frames(blob, indices)`` returns ``uint8 [len(indices), H, W, 3]`` RGB frames of an MP4 / MKV / WebM byte
string at the given source-frame indices (monotone, as ``data.sampling.frame_offsets`` produces them).  The container
is parsed from a private temporary file (OpenCV's capture API takes paths); frames are read sequentially with a seek
only when the next wanted index is far ahead, so fps-resampled offsets cost one pass over the span.  ``probe`` gives
frame count, fps and geometry.  ``load_clip`` dispatches on the member name: ``.npy`` arrays pass through, anything
else goes to the decoder (the reference decodes with decord: solar/backends/wan22/runtime/data.py raw readers;
decord is not in this image, OpenCV is).
"""
from __future__ import annotations

import io
import os
import tempfile
from typing import Optional, Sequence, Tuple

import numpy as np

from ..errors import DataContractError

_SEEK_AHEAD = 48          # frames; nearer targets are reached by decoding through


def _capture(path: str):
    import cv2

    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise DataContractError("the video member could not be opened by the decoder")
    return cap, cv2


def _with_tempfile(blob: bytes, suffix: str, fn):
    fd, path = tempfile.mkstemp(prefix="solar-raw-", suffix=suffix)
    try:
        with os.fdopen(fd, "wb") as fh:
            fh.write(blob)
        return fn(path)
    finally:
        try:
            os.unlink(path)
        except FileNotFoundError:
            pass


def probe(blob: bytes, suffix: str = ".mp4") -> dict:
    def run(path):
        cap, cv2 = _capture(path)
        try:
            return {"frames": int(cap.get(cv2.CAP_PROP_FRAME_COUNT)), "fps": float(cap.get(cv2.CAP_PROP_FPS)),
                    "width": int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), "height": int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT))}
        finally:
            cap.release()

    return _with_tempfile(blob, suffix, run)


def decode_frames(blob: bytes, indices: Sequence[int], *, size: Optional[Tuple[int, int]] = None, suffix: str = ".mp4") -> np.ndarray:
    """``size`` = (height, width) resizes with area / bilinear interpolation as the frames are read."""
    idx = [int(i) for i in indices]
    if not idx or any(b < a for a, b in zip(idx, idx[1:])) or idx[0] < 0:
        raise DataContractError("frame indices must be a non-empty non-decreasing sequence of non-negative integers")

    def run(path):
        cap, cv2 = _capture(path)
        try:
            out, pos, last = [], 0, None
            for want in idx:
                if last is not None and want == pos - 1:
                    out.append(last)                      # repeated index (up-sampled fps)
                    continue
                if want - pos > _SEEK_AHEAD:
                    cap.set(cv2.CAP_PROP_POS_FRAMES, want)
                    pos = want
                frame = None
                while pos <= want:
                    ok, frame = cap.read()
                    if not ok:
                        raise DataContractError(f"the video ends before frame {want}")
                    pos += 1
                rgb = cv2.cvtColor(frame, cv2.COLOR_BGR2RGB)
                if size is not None and rgb.shape[:2] != tuple(size):
                    shrink = rgb.shape[0] > size[0]
                    rgb = cv2.resize(rgb, (size[1], size[0]), interpolation=cv2.INTER_AREA if shrink else cv2.INTER_LINEAR)
                last = rgb
                out.append(rgb)
            return np.stack(out)
        finally:
            cap.release()

    return _with_tempfile(blob, suffix, run)


def load_clip(member_name: str, blob: bytes, frames: int, *, offsets: Optional[Sequence[int]] = None,
              size: Optional[Tuple[int, int]] = None) -> np.ndarray:
    """A raw dataset member -> ``uint8 [frames, H, W, 3]``: ``.npy`` arrays are sliced, containers are decoded."""
    take = list(range(frames)) if offsets is None else [int(o) for o in offsets]
    if member_name.endswith(".npy"):
        vid = np.load(io.BytesIO(blob), allow_pickle=False)
        if vid.ndim != 4 or vid.shape[-1] != 3 or vid.shape[0] <= take[-1]:
            raise DataContractError(f"{member_name}: video must be [T>{take[-1]}, H, W, 3] uint8")
        return vid[take]
    return decode_frames(blob, take, size=size, suffix=os.path.splitext(member_name)[1] or ".mp4")
