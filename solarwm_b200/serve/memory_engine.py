"""Interactive sessions with long-range memory: the web engine of the Memory backend.

A session is ``start -> (advance_camera -> generate)* -> stop``:

  cameras     every chunk arrives as a packet of key sets, one per generated latent (4 for the first chunk, whose first
              latent is the anchor's camera; 5 afterwards).  A latent's camera is the pose after 1, 4, 4, 4, 4 (repeating)
              steps of the keyboard camera.  Poses are kept ABSOLUTE in the first camera's frame for the whole session --
              retrieval compares cameras that may be thousands of frames apart, so the recent-window re-basing of the
              plain streaming engine must not run here.  The device buffers of view matrices and intrinsics grow by
              doubling.  Retrieval sees the fp64 inverse of the fp32 view matrices the model sees, not a separate
              higher-precision trajectory.
  memory      before a chunk is generated the latents outside the recent window are scored against the chunk's last
              camera (``serve.memory``), the best ``top_k`` are gathered from the bf16 latent bank and installed as memory
              rows with their own cameras; the Memory adapter bank is active exactly while rows are installed.  Every
              chunk's selection is recorded and checked: count = min(top_k, eligible), unique, strictly older than the
              recent window, and the recent KV never exceeds the window.
  noise       one seeded generator per session; ``noise_window`` reproduces the released schedule of refills (a 50-latent
              buffer walked in 5-latent steps, refilled every 10 chunks once the first 58 chunks have used their own).
  failure     a non-finite chunk or a failed invariant marks the engine failed; it refuses further work until a new
              engine is built.  ``stop`` writes the session report (create-only) and clears every per-session buffer.

Reference: MemoryEngine (deploy/solar_wm/backends/memory/runtime/memory_engine.py:17-200), memory_window.py,
memory_namespace.py.
"""
from __future__ import annotations

import hashlib
import json
import time
from pathlib import Path
from typing import Any, List, Mapping, Optional, Sequence

import numpy as np
import torch

from .camera_control import KeyboardCameraConfig, KeyboardCameraState
from .h3_stream import H3StreamConfig, H3StreamingGenerator
from .memory import LatentMemoryBank, select_memory

CADENCE = (1, 4, 4, 4, 4)


def noise_window(index: int):
    """(offset into the 10-chunk noise buffer, whether the buffer is refilled before this chunk)."""
    if type(index) is not int or index < 0:
        raise ValueError("a non-negative chunk index is required")
    offset = index if index < 58 else (index - 58) % 10
    return offset, index >= 58 and offset == 0


def check_selection(record: Mapping[str, Any], *, chunk_latents: int = 5, top_k: int = 5, recent_chunks: int = 5) -> None:
    j, ids = record["chunk"], record["memory_latent_indices"]
    stop = max(0, j - recent_chunks) * chunk_latents
    if len(ids) != min(top_k, stop) or len(set(ids)) != len(ids):
        raise RuntimeError("retrieval count or uniqueness differs")
    if any(type(i) is not int or not 0 <= i < stop for i in ids):
        raise RuntimeError("retrieved a recent, future or invalid latent")
    if record["cached_chunks"] > recent_chunks:
        raise RuntimeError("the recent KV window exceeded its size")


def cache_key(*, sources_sha256: str, runtime: Mapping[str, Any], inference: Mapping[str, Any]) -> str:
    """The namespace of prepared scenes: what was encoded, with which runtime, for which inference settings."""
    doc = json.dumps({"sources": sources_sha256, "runtime": dict(runtime), "inference": dict(inference)}, sort_keys=True,
                     separators=(",", ":"))
    return hashlib.sha256(doc.encode()).hexdigest()[:24]


def _invert_rigid(m: np.ndarray) -> np.ndarray:
    out = np.tile(np.eye(4, dtype=m.dtype), (m.shape[0], 1, 1))
    R = np.transpose(m[:, :3, :3], (0, 2, 1))
    out[:, :3, :3] = R
    out[:, :3, 3] = -np.einsum("nij,nj->ni", R, m[:, :3, 3])
    return out


class MemorySessionEngine:
    def __init__(self, model, cfg: H3StreamConfig, *, run_dir, rank: int = 0, sp=None, top_k: int = 5,
                 camera: Optional[KeyboardCameraConfig] = None, intrinsics: Optional[np.ndarray] = None, identity: Optional[Mapping] = None):
        if cfg.memory_latents < top_k:
            raise ValueError("the stream configuration must reserve memory rows for top_k latents")
        self.model, self.cfg, self.sp, self.rank, self.top_k = model, cfg, sp, int(rank), int(top_k)
        self.run = Path(run_dir)
        self.run.mkdir(parents=True, exist_ok=True)
        self.camera_cfg = camera or KeyboardCameraConfig(frames_per_second=24.0)
        self.K = np.asarray(intrinsics if intrinsics is not None else [[cfg.fx, 0, 0.5], [0, cfg.fy, 0.5], [0, 0, 1.0]], dtype=np.float64)
        self.identity = dict(identity or {})
        self.condition: Optional[Mapping[str, torch.Tensor]] = None
        self.failed = False
        self.session_count = 0
        self._clear()

    def _clear(self) -> None:
        self.gen = self.bank = self.camera = None
        self.views = self.K_rows = None            # device buffers [capacity, 4, 4] / [capacity, 3, 3]
        self.poses: List[np.ndarray] = []
        self.records: List[dict] = []
        self.session_times: List[float] = []
        self.index = 0
        self.active = False
        self._packet_ready = False

    # -- scene ------------------------------------------------------------------------------------------------------------
    def set_condition(self, *, text: torch.Tensor, anchor_latent: torch.Tensor, scene_id: str) -> None:
        if self.active:
            raise RuntimeError("stop the active session before changing the scene")
        self.condition = {"text": text, "anchor_latent": anchor_latent, "scene_id": str(scene_id)}

    # -- lifecycle --------------------------------------------------------------------------------------------------------
    def start(self, *, seed: int = 42) -> None:
        if self.failed or self.condition is None or self.active:
            raise RuntimeError("an inactive healthy engine with a scene is required")
        self.session_count += 1
        cfg = self.cfg.__class__(**{**self.cfg.__dict__, "seed": int(seed)})
        self.gen = H3StreamingGenerator(self.model, cfg, sp=self.sp)
        self.gen.start(self.condition["text"], self.condition["anchor_latent"], torch.eye(4))
        self.bank = LatentMemoryBank(chunk_latents=cfg.chunk_latents)
        self.camera = KeyboardCameraState(self.camera_cfg)
        dev = self.gen.device
        self.views = torch.eye(4, device=dev).repeat(16, 1, 1)
        self.K_rows = torch.as_tensor(self.K, device=dev, dtype=torch.float32).repeat(16, 1, 1)
        self.active, self.started = True, time.perf_counter()

    def advance_camera(self, actions: Sequence[Sequence[str]]) -> None:
        """One key set per NEW latent of the chunk about to be generated."""
        k = self.cfg.chunk_latents
        expected = k - 1 if self.index == 0 else k
        if not self.active or self._packet_ready or len(actions) != expected:
            raise ValueError("the camera packet differs from the active chunk")
        if self.index == 0:
            self.poses.append(self.camera.c2w.copy())                # the first latent sits at the anchor's camera
        for keys in actions:
            done = len(self.poses) - 1
            for _ in range(CADENCE[done % len(CADENCE)]):
                self.camera.step([key for key in keys if key not in "qe"])
            self.poses.append(self.camera.c2w.copy())
        if len(self.poses) != (self.index + 1) * k:
            raise RuntimeError("camera sampling or order changed")
        needed = len(self.poses)
        if needed > self.views.shape[0]:
            capacity = max(needed, 2 * self.views.shape[0])
            grown = torch.eye(4, device=self.views.device).repeat(capacity, 1, 1)
            grown[:self.views.shape[0]].copy_(self.views)
            grown_K = self.K_rows[-1:].repeat(capacity, 1, 1)
            grown_K[:self.K_rows.shape[0]].copy_(self.K_rows)
            self.views, self.K_rows = grown, grown_K
        start = self.index * k
        fresh = _invert_rigid(np.asarray(self.poses[start:], dtype=np.float64)).astype(np.float32)
        self.views[start:needed].copy_(torch.from_numpy(fresh))
        self._packet_ready = True

    def _retrieval_cameras(self, needed: int):
        view = self.views[:needed].cpu().numpy().astype(np.float64)
        return _invert_rigid(view), self.K_rows[:needed].cpu().numpy().astype(np.float64)

    def generate(self):
        """-> (latent chunk [C, chunk_latents, H, W], milliseconds)."""
        if self.failed or not self.active or not self._packet_ready:
            raise RuntimeError("a healthy active session with a camera packet is required")
        k, index = self.cfg.chunk_latents, self.index
        lo, hi = index * k, (index + 1) * k
        t0 = time.perf_counter()
        try:
            c2w, K = self._retrieval_cameras(hi)
            ids, scores = select_memory(c2w, K, index, chunk_latents=k, top_k=self.top_k, recent_chunks=self.cfg.window_chunks)
            ids = [int(i) for i in ids]
            if ids:
                mem = self.bank.gather(ids, self.condition["anchor_latent"].unsqueeze(0))[0]
                self.gen.set_memory(mem, self.views[ids])
            else:
                self.gen.set_memory(None)
            chunk = self.gen.next_chunk(self.views[lo:hi])
            if not bool(torch.isfinite(chunk.float()).all()):
                raise FloatingPointError("non-finite memory chunk")
            self.bank.commit(chunk.unsqueeze(0), index)
            elapsed = (time.perf_counter() - t0) * 1e3
            record = {"chunk": index, "memory_latent_indices": ids, "scores": [float(s) for s in scores],
                      "cached_chunks": int(min(self.gen.hist_chunks, self.cfg.window_chunks)),
                      "noise_window": list(noise_window(index))}
            check_selection(record, chunk_latents=k, top_k=self.top_k, recent_chunks=self.cfg.window_chunks)
            self.records.append(record)
            self.session_times.append(elapsed)
            self.index += 1
            self._packet_ready = False
            return chunk, elapsed
        except BaseException:
            self.failed = True
            raise

    def stop(self) -> Mapping[str, Any]:
        if not self.active:
            raise RuntimeError("no active memory session")
        report = {"schema": "solarwm.memory-session.v1", "session": self.session_count, "chunks": self.index,
                  "dit_ms": [round(t, 3) for t in self.session_times], "scene_id": self.condition["scene_id"],
                  "memory": self.identity, "retrieval": self.records, "top_k": self.top_k,
                  "camera_policy": "absolute first-camera coordinates; no local rebase"}
        with (self.run / f"memory-session-{self.session_count}-rank{self.rank}.json").open("x") as fh:
            json.dump(report, fh)
        self._clear()
        return report

    def close(self) -> None:
        self._clear()
