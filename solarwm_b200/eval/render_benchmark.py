"""Render a benchmark's cases with a method, resumably: ``<renders>/<split>/<id>.mp4`` per case.

``render_fn(case) -> RGB8 frames [T, H, W, 3]`` is the method under test (the renderer service with its codecs, a baseline,
a test stub).  A case whose video is already there is skipped; a video is written under a temporary name and renamed, so
an interrupted pass never leaves half a file where ``run_metrics`` would read it; workers split the cases
``shard::shards``; every render appends one line (case, seconds, frames) to ``render-log.jsonl``.  A method that fails
on a case is recorded and the pass goes on, so one bad case does not cost the rest of the benchmark
(reference: eval/solar_renderer/render_benchmark.py).
"""
from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Callable, Mapping, Sequence

import numpy as np

from .benchmark import Case, load_cases


def write_video(path, frames: np.ndarray, fps: float = 24.0) -> None:
    import cv2

    if frames.ndim != 4 or frames.shape[-1] != 3 or frames.dtype != np.uint8 or len(frames) < 1:
        raise ValueError("a render is RGB8 [T, H, W, 3]")
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(f".{path.stem}.{os.getpid()}.tmp.mp4")
    writer = cv2.VideoWriter(str(tmp), cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (frames.shape[2], frames.shape[1]))
    if not writer.isOpened():
        raise RuntimeError("the video encoder could not be opened")
    try:
        for f in frames:
            writer.write(cv2.cvtColor(f, cv2.COLOR_RGB2BGR))
    finally:
        writer.release()
    os.replace(tmp, path)


def render_cases(root, renders, render_fn: Callable[[Case], np.ndarray], *, split: str = "all", shard: int = 0, shards: int = 1,
                 fps: float = 24.0) -> Mapping[str, object]:
    renders = Path(renders)
    renders.mkdir(parents=True, exist_ok=True)
    done, skipped, failed = [], [], []
    with (renders / f"render-log-{shard:04d}.jsonl").open("a") as log:
        for case in load_cases(root, split)[shard::shards]:
            target = case.render(renders)
            if target.is_file():
                skipped.append(case.key)
                continue
            t0 = time.perf_counter()
            try:
                frames = render_fn(case)
                write_video(target, frames, fps)
            except Exception as exc:  # noqa: BLE001 - recorded; the pass goes on
                failed.append({"case": case.key, "error": f"{type(exc).__name__}: {exc}"})
                log.write(json.dumps({"case": case.key, "error": failed[-1]["error"]}) + "\n")
                continue
            log.write(json.dumps({"case": case.key, "seconds": round(time.perf_counter() - t0, 3), "frames": int(len(frames))}) + "\n")
            log.flush()
            done.append(case.key)
    return {"rendered": done, "skipped": skipped, "failed": failed}
