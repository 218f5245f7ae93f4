"""Headless frame sink: decoded frames -> RGB8 (device kernel or the C++ host routine) -> an ffmpeg
pipe when the binary exists, else raw ``.rgb`` / ``.npy`` files; a fragment store for previews
(reference: deploy/solar_wm/shared/media/{pixels.py,encoder.py,pipeline.py,store.py})."""
from __future__ import annotations

import shutil
import subprocess
import threading
from pathlib import Path
from typing import List, Optional

import numpy as np
import torch

from .. import ops


SIGNED_UNIT = ((0.5, 0.5, 0.5), (0.5, 0.5, 0.5))      # (mean, std) that maps decoder output in [-1, 1] to [0, 1]


def frame_to_rgb8(frame_chw: torch.Tensor, normalization=None) -> np.ndarray:
    """bf16 [3, H, W] -> uint8 [H, W, 3]; conversion happens on the tensor's device, only the 8-bit
    pixels cross PCIe.  ``normalization`` = (mean, std) of the pixel = x * std + mean step (default: the conversion
    kernel's own constants; ``SIGNED_UNIT`` for frames in [-1, 1]).  Raises on non-finite pixels."""
    kw = {} if normalization is None else {"mean": tuple(normalization[0]), "std": tuple(normalization[1])}
    rgb, flag = ops.rgb8(frame_chw.to(torch.bfloat16), **kw)
    if flag is not None and int(flag.item()) != 0:
        raise FloatingPointError("nonfinite RGB pixel")
    return rgb.cpu().numpy()


class FrameSink:
    def __init__(self, out_dir, width: int, height: int, fps: float = 16.0, use_ffmpeg: Optional[bool] = None,
                 normalization=None):
        self.normalization = normalization
        self.dir = Path(out_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.width, self.height, self.fps = width, height, fps
        self.frames = 0
        self.proc = None
        ffmpeg = shutil.which("ffmpeg")
        if (use_ffmpeg if use_ffmpeg is not None else bool(ffmpeg)) and ffmpeg:
            self.proc = subprocess.Popen(
                [ffmpeg, "-loglevel", "error", "-y", "-f", "rawvideo", "-pix_fmt", "rgb24", "-s", f"{width}x{height}",
                 "-r", str(fps), "-i", "-", "-an", "-c:v", "libx264", "-pix_fmt", "yuv420p", "-movflags",
                 "frag_keyframe+empty_moov", str(self.dir / "video.mp4")], stdin=subprocess.PIPE)
        else:
            self.raw = (self.dir / "video.rgb").open("wb")

    def push(self, frame_chw: torch.Tensor) -> None:
        rgb = frame_to_rgb8(frame_chw, self.normalization)
        if rgb.shape[:2] != (self.height, self.width):
            raise ValueError(f"frame is {rgb.shape[:2]}, sink expects {(self.height, self.width)}")
        (self.proc.stdin if self.proc else self.raw).write(rgb.tobytes())
        self.frames += 1

    def close(self) -> dict:
        if self.proc:
            self.proc.stdin.close()
            self.proc.wait(timeout=60)
        else:
            self.raw.close()
        return {"frames": self.frames, "container": "mp4" if self.proc else "raw-rgb24", "dir": str(self.dir)}


class FragmentStore:
    """Thread-safe ring of the most recent encoded fragments, polled by preview clients."""

    def __init__(self, keep: int = 64):
        self.keep, self.items, self.next_index = keep, [], 0
        self.lock = threading.Lock()

    def add(self, blob: bytes) -> int:
        with self.lock:
            self.items.append((self.next_index, blob))
            self.items = self.items[-self.keep:]
            self.next_index += 1
            return self.next_index - 1

    def since(self, index: int) -> List[tuple]:
        with self.lock:
            return [it for it in self.items if it[0] >= index]
