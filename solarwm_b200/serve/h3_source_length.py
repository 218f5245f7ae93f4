"""Source-length H3 evaluation: a plan of clips of arbitrary length, prepared once and generated resumably.

  geometry   a source clip of ``F >= 22`` frames maps to ``n = ceil((F - 5) / 17)`` codec groups: ``17 n + 5`` decoded
             frames from ``5 n + 2`` latents, generated as whole 5-latent chunks.  Generated latent ``i`` takes the
             camera of source frame ``0, 1, 5, 9, 13, 17, 18, 22, ...`` (steps 1, 4, 4, 4, 4 repeating); indices past
             the clip repeat the last camera (``tail_camera_rows`` counts them).  Only the first ``F`` decoded frames
             are exported, at the source's frame rate or the model's 24.
  plan       a JSON array of rows ``{key, dataset, num_frames, fps, caption, ...}``; keys are unique single path
             components; clips above 960 frames need streaming decode.
  prepare    per case: first-frame-relative world-to-camera matrices at the geometry's camera indices, normalised
             intrinsics, the encoded prompt and anchor -> ``condition.safetensors`` + ``READY.json`` (digests, geometry,
             identity of what produced it).  A case whose receipt matches is skipped; a receipt that differs is an
             error, never silently redone.
  generate   rows ``rank::world``; per case the chunked rollout (optionally with memory retrieval) streams through the
             decoder into the writer; the result manifest carries an identity over condition, checkpoint, seed and
             options, so a finished case is verified and skipped on re-run and a changed setup is refused.

Reference: solar/backends/minimax_h3/full_length.py:7-45, full_inference.py:31-645.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import time
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable, Mapping, Optional, Sequence

import torch

from ..errors import BackendContractError

CADENCE = (1, 4, 4, 4, 4)
MODEL_FPS = 24.0
CONDITION_SCHEMA = "solarwm.h3-full-condition.v1"
RESULT_SCHEMA = "solarwm.h3-full-result.v1"


@dataclass(frozen=True)
class FullLengthGeometry:
    source_frames: int
    decoded_frames: int
    decode_latents: int
    rollout_latents: int
    camera_indices: tuple
    tail_camera_rows: int


def full_length_geometry(source_frames: int, chunk_latents: int = 5) -> FullLengthGeometry:
    if type(source_frames) is not int or source_frames < 22:
        raise ValueError("source-length evaluation needs at least 22 consecutive source frames")
    groups = -(-(source_frames - 5) // 17)
    decode = 5 * groups + 2
    rollout = -(-decode // chunk_latents) * chunk_latents
    cams, frame, tail = [0], 0, 0
    for i in range(rollout - 1):
        frame += CADENCE[i % len(CADENCE)]
        if frame < source_frames:
            cams.append(frame)
        else:
            cams.append(cams[-1])
            tail += 1
    return FullLengthGeometry(source_frames, 17 * groups + 5, decode, rollout, tuple(cams), tail)


def exported_fps(source_fps: float, policy: str) -> float:
    if not math.isfinite(source_fps) or source_fps <= 0:
        raise ValueError("the source frame rate must be finite and positive")
    if policy not in ("source", "h3"):
        raise ValueError("the frame-rate policy is 'source' or 'h3'")
    return float(source_fps) if policy == "source" else MODEL_FPS


def storyboard_indices(source_frames: int) -> list:
    """The frames a contact sheet shows: start, 10 %, quartiles, 90 %, end."""
    return sorted({round((source_frames - 1) * p) for p in (0, 0.1, 0.25, 0.5, 0.75, 0.9, 1)})


def _component(value, what: str) -> str:
    if not isinstance(value, str) or not value or "/" in value or "\\" in value or value in (".", "..") or "\0" in value:
        raise BackendContractError(f"{what} must be one path component, got {value!r}")
    return value


def load_plan(path, *, stream_decode: bool = False, fps_policy: str = "source") -> list:
    rows = json.loads(Path(path).read_text())
    if not isinstance(rows, list) or not rows:
        raise BackendContractError("a source-length plan is a non-empty JSON array of rows")
    seen = set()
    for row in rows:
        if not isinstance(row, dict):
            raise BackendContractError("plan rows are JSON objects")
        key = _component(row.get("key"), "case key")
        _component(row.get("dataset"), "dataset")
        if key in seen:
            raise BackendContractError(f"duplicate case key {key!r} in the plan")
        seen.add(key)
        frames = row.get("num_frames")
        if type(frames) is not int:
            raise BackendContractError(f"{key}: num_frames must be an integer")
        if frames > 960 and not stream_decode:
            raise BackendContractError(f"{key}: clips above 960 frames need inference.stream_decode")
        full_length_geometry(frames)
        exported_fps(float(row.get("fps", 0)), fps_policy)
    return rows


def relative_views(c2w: torch.Tensor) -> torch.Tensor:
    """[F, 4, 4] camera-to-world -> world-to-camera relative to the first frame (the first is exactly the identity)."""
    c2w = c2w.double()
    if c2w.ndim != 3 or tuple(c2w.shape[1:]) != (4, 4) or not bool(torch.isfinite(c2w).all()):
        raise BackendContractError("a camera trajectory is finite [F, 4, 4]")
    bottom = torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=torch.float64)
    if not torch.allclose(c2w[:, 3], bottom.expand(c2w.shape[0], 4), atol=1e-5):
        raise BackendContractError("camera matrices must end in the row 0 0 0 1")
    rel = torch.linalg.inv(c2w[0]) @ c2w
    rel[0] = torch.eye(4, dtype=torch.float64)
    return torch.linalg.inv(rel).float().contiguous()


def _sha(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


def _digest(value) -> str:
    return hashlib.sha256(json.dumps(value, sort_keys=True, separators=(",", ":"), default=str).encode()).hexdigest()


def _atomic_json(path: Path, value) -> None:
    tmp = path.with_name("." + path.name + ".tmp")
    tmp.write_text(json.dumps(value, sort_keys=True, indent=1))
    os.replace(tmp, path)


def prepare_case(work_dir, row: Mapping, *, c2w: torch.Tensor, intrinsics: torch.Tensor,
                 encode_prompt: Callable[[str], torch.Tensor], encode_anchor: Callable[[], torch.Tensor],
                 identity: Mapping) -> Mapping:
    """``c2w`` [F, 4, 4] and normalised ``intrinsics`` [F, 3, 3] for every source frame.  Returns the receipt."""
    from safetensors.torch import save_file

    case = Path(work_dir) / "cases" / _component(row["key"], "case key")
    frames = int(row["num_frames"])
    want = _digest({"row": dict(row), "identity": dict(identity)})
    receipt_path = case / "READY.json"
    if receipt_path.is_file():
        receipt = json.loads(receipt_path.read_text())
        if receipt.get("preparation_identity") != want:
            raise BackendContractError(f"{row['key']}: prepared under another plan row or setup; remove {case} to redo it")
        if _sha(case / "condition.safetensors") != receipt.get("condition_sha256"):
            raise BackendContractError(f"{row['key']}: condition file differs from its receipt")
        return receipt
    started = time.perf_counter()
    if c2w.shape[0] != frames or intrinsics.shape != (frames, 3, 3) or not bool(torch.isfinite(intrinsics).all()):
        raise BackendContractError(f"{row['key']}: cameras do not cover the clip's {frames} frames")
    geometry = full_length_geometry(frames)
    views = relative_views(c2w)
    idx = torch.tensor(geometry.camera_indices)
    values = {"prompt_embeds": encode_prompt(str(row.get("caption", ""))).detach().cpu().contiguous(),
              "anchor_latents": encode_anchor().detach().cpu().contiguous(),
              "viewmats": views[idx].contiguous(), "K": intrinsics.float()[idx].contiguous()}
    if not all(bool(torch.isfinite(t.float()).all()) for t in values.values()):
        raise FloatingPointError(f"{row['key']}: non-finite encoded condition")
    case.mkdir(parents=True, exist_ok=True)
    tmp = case / ".condition.tmp"
    save_file(values, str(tmp))
    os.replace(tmp, case / "condition.safetensors")
    receipt = {"schema": CONDITION_SCHEMA, "row": dict(row), "preparation_identity": want, "geometry": asdict(geometry),
               "condition_sha256": _sha(case / "condition.safetensors"),
               "preparation_seconds": round(time.perf_counter() - started, 4),
               "full_camera_max_relative_translation": float(views[:, :3, 3].norm(dim=-1).max()),
               "camera_convention": "relative_w2c+normalized_K", "source_frame_policy": "all_consecutive_no_resampling",
               "model_fps": MODEL_FPS}
    _atomic_json(receipt_path, receipt)
    return json.loads(receipt_path.read_text())


def run_plan(model, rows: Sequence[Mapping], *, work_dir, out_dir, stream_cfg, identity: Mapping, rank: int = 0, world: int = 1,
             noise_seed: int = 0, decoder_factory: Optional[Callable[[], object]] = None,
             writer_factory: Optional[Callable[[Path, float], object]] = None, use_memory: bool = False, top_k: int = 5,
             fps_policy: str = "source", sp=None, save_latents: bool = False) -> Mapping:
    """Generate this rank's share of the plan.  ``decoder_factory()`` gives a fresh streaming decoder per case,
    ``writer_factory(path, fps)`` an object with ``push(frames [3, F, H, W])`` and ``close()``.  Returns a summary."""
    from safetensors.torch import load_file

    from .h3_full_inference import generate_full_length

    done, skipped = [], []
    for row in list(rows)[rank::world]:
        key = row["key"]
        case = Path(work_dir) / "cases" / key
        if not (case / "READY.json").is_file():
            raise BackendContractError(f"{key}: not prepared (no READY.json under {case})")
        receipt = json.loads((case / "READY.json").read_text())
        seed = int(row.get("validation_noise_seed", row.get("validation_seed", noise_seed)))
        want = _digest({"condition": receipt["condition_sha256"], "identity": dict(identity), "seed": seed,
                        "memory": {"enabled": bool(use_memory), "top_k": int(top_k)}, "fps_policy": fps_policy})
        dest = Path(out_dir) / row["dataset"]
        manifest_path = dest / f"{key}.json"
        if manifest_path.is_file():
            old = json.loads(manifest_path.read_text())
            if old.get("result_identity") != want:
                raise BackendContractError(f"{key}: a result made under another setup is in the way ({manifest_path})")
            if save_latents and not (dest / f"{key}.latents.pt").is_file():
                raise BackendContractError(f"{key}: the finished result holds no latents")
            skipped.append(key)
            continue
        values = load_file(str(case / "condition.safetensors"))
        if _sha(case / "condition.safetensors") != receipt["condition_sha256"]:
            raise BackendContractError(f"{key}: condition file differs from its receipt")
        geometry = full_length_geometry(int(row["num_frames"]), stream_cfg.chunk_latents)
        views, K = values["viewmats"], values["K"]
        if views.shape[0] != geometry.rollout_latents:
            raise BackendContractError(f"{key}: {views.shape[0]} prepared cameras for {geometry.rollout_latents} latents")
        # the generator takes camera-to-world with the anchor first; the anchor sees through the first camera
        c2w = torch.linalg.inv(torch.cat([views[:1], views]).double()).float()
        fps = exported_fps(float(row["fps"]), fps_policy)
        dest.mkdir(parents=True, exist_ok=True)
        video = dest / f"{key}.mp4"
        part = dest / f".{key}.tmp.mp4"
        writer = writer_factory(part, fps) if writer_factory is not None else None
        cfg = stream_cfg.__class__(**{**stream_cfg.__dict__, "seed": seed})
        started = time.perf_counter()
        try:
            result = generate_full_length(
                model, text=values["prompt_embeds"], anchor_latent=values["anchor_latents"], c2w=c2w,
                intrinsics=torch.cat([K[:1], K]), stream_cfg=cfg, sp=sp,
                decoder=decoder_factory() if decoder_factory is not None else None,
                frame_sink=None if writer is None else writer.push, use_memory=use_memory, top_k=top_k,
                decode_latents=geometry.decode_latents, max_frames=geometry.source_frames, keep_latents=save_latents)
        finally:
            if writer is not None:
                writer.close()
        result = dict(result)
        latents = result.pop("latents_tensor", None)
        if writer is not None and part.exists():
            os.replace(part, video)
        if save_latents:
            torch.save(latents, dest / f"{key}.latents.pt")
        _atomic_json(manifest_path, {"schema": RESULT_SCHEMA, "key": key, "dataset": row["dataset"], "result_identity": want,
                                     "geometry": asdict(geometry), "noise_seed": seed, "fps": fps,
                                     "storyboard_frames": storyboard_indices(geometry.source_frames),
                                     "seconds": round(time.perf_counter() - started, 4), "generation": result})
        done.append(key)
    return {"generated": done, "skipped": skipped, "rank": rank, "world": world}
