"""Generated-versus-source comparison views.

``side_by_side`` pads two clips to a common height, trims both to the shorter length and
concatenates them on the width axis with a separator band; ``write_comparison`` encodes the view
through ``serve.media.FrameSink`` (an ffmpeg pipe when the binary exists, a raw RGB8 ``.npy``
stack otherwise) and records a small JSON manifest next to it
(reference: solar/inference/comparison.py:38-276).

``publish_comparison_view`` turns one published validation partition (``slot-NNNNNN/`` folders with a ``compare.mp4``
each) into the flat comparison directory people browse: ``compare/rankSSS_roundRR_dpDDD_<key>_startFFFFFF.mp4`` (hard
links, so nothing is copied) and ``manifests/rank_SSS.json`` (one summary per slot, create-only), and
``seal_comparison_view`` writes its ``COMPLETE.json`` once every partition of a step has been merged.  Several
partitions (one per node or replica) may be merged into the same destination; a slot that is already there is an error.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping, Optional, Sequence

import torch


def _fit_height(clip: torch.Tensor, height: int) -> torch.Tensor:
    """clip [T, 3, H, W] in [-1, 1] -> centred on a canvas of the given height (black bars)."""
    T, C, H, W = clip.shape
    if H == height:
        return clip
    canvas = torch.full((T, C, height, W), -1.0, dtype=clip.dtype, device=clip.device)
    top = (height - H) // 2
    canvas[:, :, top:top + H] = clip
    return canvas


def side_by_side(generated: torch.Tensor, source: torch.Tensor, separator: int = 8) -> torch.Tensor:
    """[T, 3, H, W] x 2 -> [T', 3, max(H), Wg + separator + Ws] (T' = shorter clip)."""
    if generated.dim() != 4 or source.dim() != 4 or generated.shape[1] != 3 or source.shape[1] != 3:
        raise ValueError("comparison clips are [T, 3, H, W]")
    T = min(generated.shape[0], source.shape[0])
    H = max(generated.shape[2], source.shape[2])
    g, s = _fit_height(generated[:T].float(), H), _fit_height(source[:T].float().to(generated.device), H)
    band = torch.ones(T, 3, H, separator, device=g.device)
    return torch.cat([g, band, s], dim=3)


def write_comparison(out_dir, generated: torch.Tensor, source: torch.Tensor, *, fps: float = 16.0,
                     meta: Optional[Mapping[str, object]] = None, use_ffmpeg: Optional[bool] = None) -> Mapping[str, object]:
    from ..serve.media import FrameSink

    view = side_by_side(generated, source)
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    sink = FrameSink(out, width=view.shape[3], height=view.shape[2], fps=fps, use_ffmpeg=use_ffmpeg)
    for frame in view:
        sink.push(frame)
    info = dict(sink.close())
    info.update({"schema": "solarwm.comparison.v1", "frames": int(view.shape[0]), "layout": "generated|source",
                 **dict(meta or {})})
    (out / "comparison.json").write_text(json.dumps(info, sort_keys=True, default=str))
    return info


VIEW_SCHEMA = "solarwm.validation-comparison.v1"


@dataclass(frozen=True)
class ComparisonRecord:
    slot: int
    video: Path
    manifest: Path


def _slug(text: str) -> str:
    return re.sub(r"[^A-Za-z0-9._-]+", "-", str(text)).strip("-")[:80] or "sample"


def _create_only(path: Path, data: bytes) -> None:
    fd = os.open(path, os.O_CREAT | os.O_EXCL | os.O_WRONLY | getattr(os, "O_NOFOLLOW", 0), 0o444)
    try:
        with os.fdopen(fd, "wb") as fh:
            fh.write(data)
            fh.flush()
            os.fsync(fh.fileno())
    except BaseException:
        path.unlink(missing_ok=True)
        raise


def publish_comparison_view(source, destination, *, step: int, pass_name: str, cases: int, dp_world_size: int,
                            sp_size: int, run_root, cases_per_round: Optional[int] = None,
                            video_name: str = "compare.mp4") -> Sequence[ComparisonRecord]:
    """Merge the slots of ``source`` (a sealed inference publication) into ``destination``.  ``cases`` is the global
    number of validation cases of the step; they must form whole rounds of ``cases_per_round`` (default: one round)."""
    from ..errors import BackendContractError

    source, destination, run_root = Path(source), Path(destination), Path(run_root)
    per_round = int(cases) if cases_per_round is None else int(cases_per_round)
    if int(cases) < 1 or per_round < 1 or int(cases) % per_round:
        raise BackendContractError("comparison cases must form complete rounds")
    (destination / "compare").mkdir(parents=True, exist_ok=True)
    (destination / "manifests").mkdir(parents=True, exist_ok=True)
    records = []
    for folder in sorted(source.glob("slot-*")):
        manifest = json.loads((folder / "manifest.json").read_text())
        case = manifest["case"]
        slot, start = int(case["slot"]), int(case.get("start_frame", 0))
        if not 0 <= slot < int(cases):
            raise BackendContractError(f"slot {slot} is outside the {cases} validation cases")
        video = folder / video_name
        if not video.is_file():
            raise BackendContractError(f"validation slot {slot} holds no {video_name}")
        name = f"rank{slot:03d}_round{slot // per_round:02d}_dp{slot % int(dp_world_size):03d}_{_slug(case['sample_id'])}_start{start:06d}.mp4"
        link, summary_path = destination / "compare" / name, destination / "manifests" / f"rank_{slot:03d}.json"
        try:
            os.link(video, link)
        except FileExistsError as exc:
            raise BackendContractError(f"comparison view already holds {link.name}") from exc
        summary = {"schema": VIEW_SCHEMA, "step": int(step), "pass": pass_name, "slot": slot,
                   "round": slot // per_round, "rounds": int(cases) // per_round, "dp_rank": slot % int(dp_world_size),
                   "dp_world_size": int(dp_world_size), "sp_size": int(sp_size), "sample_id": case["sample_id"],
                   "start_frame": start, "noise_seed": int(case["noise_seed"]), "prompt": case.get("prompt"),
                   "compare_mp4": link.relative_to(run_root).as_posix() if run_root in link.parents else str(link),
                   "metrics": manifest.get("metrics", {}), "provenance": manifest.get("provenance", {}),
                   "weights_id": manifest.get("weights_id"), "shape": manifest.get("shape")}
        try:
            _create_only(summary_path, (json.dumps(summary, indent=2, sort_keys=True) + "\n").encode())
        except BaseException:
            link.unlink(missing_ok=True)
            raise
        records.append(ComparisonRecord(slot, link, summary_path))
    if not records:
        raise BackendContractError(f"no validation slots under {source}")
    return tuple(records)


def seal_comparison_view(destination, *, step: int, pass_name: str, cases: int) -> Mapping[str, object]:
    """Write ``COMPLETE.json`` once every slot ``0 .. cases - 1`` has its video and its summary (create-only)."""
    from ..errors import BackendContractError

    destination = Path(destination)
    have = sorted(int(p.stem.split("_")[1]) for p in (destination / "manifests").glob("rank_*.json"))
    if have != list(range(int(cases))):
        missing = sorted(set(range(int(cases))) - set(have))
        raise BackendContractError(f"comparison view is incomplete: slots {missing[:8]} are missing")
    videos = sorted(p.name for p in (destination / "compare").glob("*.mp4"))
    if len(videos) != int(cases):
        raise BackendContractError(f"comparison view holds {len(videos)} videos for {cases} cases")
    seal = {"schema": VIEW_SCHEMA, "step": int(step), "pass": pass_name, "slots": int(cases), "videos": videos}
    _create_only(destination / "COMPLETE.json", (json.dumps(seal, sort_keys=True) + "\n").encode())
    return seal
