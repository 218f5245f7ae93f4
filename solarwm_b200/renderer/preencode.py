"""Pre-encoding of the renderer's training corpus: media rows -> omni members + a shard index.

Every row of the input JSON lines is

    {"id": "...", "target": "clip.mp4", "text": "...", "source": "dataset",
     "observations": [{"media": "x.mp4" | "x.png", "frames": "all" | [0, 5] | null, "degree": 0.999, "box": [x0, y0, x1, y1]?}, ...],
     "known_mask": "mask.mp4" | null}

``frames`` says how an observation relates to the clip: ``"all"`` or a list of target latent frames for an aligned one,
``null`` for a free-floating one; no field names a task.  For each row the worker

  1. reads the target, resamples it onto the model's 24 frames-per-second grid (nearest source frame), keeps the longest
     prefix of ``17 n + 5`` frames (``5 n + 2`` latents) and fits it onto the canvas (cover-resize + centre crop);
  2. does the same for every observation (a still image becomes a held clip of 13 frames; a ``box`` crops first);
  3. pools a known-mask video down to one known degree per packed target row;
  4. encodes pixels and text through the configured codecs and writes ONE member file under a temporary name, then
     publishes it by rename (a reader never sees half a member), and appends its index row.

Workers split the rows ``shard::shards``; a member that is already published is skipped, a row whose media cannot be
fetched is reported as pending instead of failing the shard (it may simply not be there yet), a refused write is fatal.
The shard's index is rewritten (atomically) after every member, the corpus index is the union of the shard indexes.

Reference: solar/renderer/preencode.py:73-902 (Sink, fetch / prepare helpers, encode, main).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import DataContractError
from .data import write_member

MODEL_FPS = 24.0
STILL_FRAMES = 13
IMAGE_SUFFIXES = (".png", ".jpg", ".jpeg", ".webp", ".bmp")


class FetchFailed(RuntimeError):
    """A row's media could not be read -- most often because it is not there yet."""


class WriteRefused(RuntimeError):
    """The destination would not take a member this worker had already encoded."""


# ---------------------------------------------------------------------------------------------------------------------
# frames
# ---------------------------------------------------------------------------------------------------------------------
def usable_frames(available: int) -> int:
    """The longest ``17 n + 5`` that fits (0 when even the shortest clip does not)."""
    return 0 if available < 22 else 17 * ((available - 5) // 17) + 5


def latent_frames(pixel_frames: int) -> int:
    if pixel_frames < 22 or (pixel_frames - 5) % 17:
        raise DataContractError(f"{pixel_frames} pixel frames are not 17 n + 5")
    return 5 * ((pixel_frames - 5) // 17) + 2


def on_grid(frames: np.ndarray, fps: float) -> np.ndarray:
    """[T, H, W, 3] at ``fps`` -> the frames nearest to the model's 24 fps sampling instants."""
    if fps <= 0 or not np.isfinite(fps):
        raise DataContractError("the source frame rate must be finite and positive")
    if abs(fps - MODEL_FPS) < 1e-3:
        return frames
    count = int(np.floor((len(frames) - 1) / fps * MODEL_FPS)) + 1
    index = np.minimum(np.rint(np.arange(count) / MODEL_FPS * fps).astype(np.int64), len(frames) - 1)
    return frames[index]


def fit(frames: np.ndarray, canvas: Tuple[int, int]) -> np.ndarray:
    """Cover-resize (aspect kept, the canvas fully covered) and centre crop to ``canvas`` = (height, width)."""
    import cv2

    H, W = canvas
    h, w = frames.shape[1:3]
    scale = max(H / h, W / w)
    nh, nw = max(H, int(round(h * scale))), max(W, int(round(w * scale)))
    top, left = (nh - H) // 2, (nw - W) // 2
    interp = cv2.INTER_AREA if scale < 1 else cv2.INTER_LANCZOS4
    return np.stack([cv2.resize(f, (nw, nh), interpolation=interp)[top:top + H, left:left + W] for f in frames])


def region(frames: np.ndarray, box: Optional[Sequence[float]]) -> np.ndarray:
    """Crop a normalised ``[x0, y0, x1, y1]`` box (None: the whole frame)."""
    if box is None:
        return frames
    x0, y0, x1, y1 = (float(v) for v in box)
    if not (0 <= x0 < x1 <= 1 and 0 <= y0 < y1 <= 1):
        raise DataContractError("an observation box is normalised x0 < x1, y0 < y1 inside [0, 1]")
    h, w = frames.shape[1:3]
    return frames[:, int(y0 * h):max(int(y0 * h) + 2, int(round(y1 * h))), int(x0 * w):max(int(x0 * w) + 2, int(round(x1 * w)))]


def read_media(path) -> Tuple[np.ndarray, float]:
    """A video or a still image as RGB8 frames [T, H, W, 3] and its frame rate (stills: one frame at 24)."""
    import cv2

    p = str(path)
    if not os.path.isfile(p):
        raise FetchFailed(p)
    if p.lower().endswith(IMAGE_SUFFIXES):
        image = cv2.imread(p, cv2.IMREAD_COLOR)
        if image is None:
            raise FetchFailed(p)
        return cv2.cvtColor(image, cv2.COLOR_BGR2RGB)[None], MODEL_FPS
    cap = cv2.VideoCapture(p)
    try:
        if not cap.isOpened():
            raise FetchFailed(p)
        fps = float(cap.get(cv2.CAP_PROP_FPS)) or MODEL_FPS
        frames = []
        while True:
            ok, frame = cap.read()
            if not ok:
                break
            frames.append(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB))
    finally:
        cap.release()
    if not frames:
        raise FetchFailed(p)
    return np.stack(frames), fps


def known_degrees(mask_frames: np.ndarray, latents: int, grid: Tuple[int, int]) -> torch.Tensor:
    """A mask clip (white = known) on the target's pixel grid -> one degree in [0, 1] per packed target row
    ``[latents * h * w]``: the mean over the pixels and the pixel frames a token covers."""
    h, w = grid
    m = torch.from_numpy(mask_frames.astype(np.float32).mean(axis=-1) / 255.0)           # [T, H, W]
    T = m.shape[0]
    # latent 0 covers frame 0; afterwards 4 frames per latent except where the 17 n + 5 cadence inserts a single frame
    edges = np.unique(np.clip(np.rint(np.linspace(0, T, latents + 1)).astype(np.int64), 0, T))
    if len(edges) != latents + 1:
        raise DataContractError("the known mask is shorter than the clip's latent frames")
    per_latent = torch.stack([m[a:b].mean(dim=0) for a, b in zip(edges[:-1], edges[1:])])
    pooled = torch.nn.functional.adaptive_avg_pool2d(per_latent.unsqueeze(1), (h, w)).squeeze(1)
    return pooled.reshape(-1).clamp_(0, 1)


# ---------------------------------------------------------------------------------------------------------------------
# encoding one row
# ---------------------------------------------------------------------------------------------------------------------
@dataclass
class Codecs:
    """``video(frames uint8 [T, H, W, 3]) -> latents [C, F, 2h, 2w]`` and ``text(str) -> (embeds [L, D], tags [L])``."""
    video: Callable[[np.ndarray], torch.Tensor]
    text: Callable[[str], Tuple[torch.Tensor, torch.Tensor]]
    canvas: Tuple[int, int] = (768, 1344)


def _clip(path, canvas, box=None, limit: Optional[int] = None) -> np.ndarray:
    frames, fps = read_media(path)
    if len(frames) == 1:
        frames = np.repeat(frames, STILL_FRAMES, axis=0)          # a still is a held clip
    else:
        frames = on_grid(frames, fps)
    frames = fit(region(frames, box), canvas)
    return frames if limit is None else frames[:limit]


def encode_row(row: Mapping[str, Any], codecs: Codecs, media_root) -> Tuple[Dict[str, torch.Tensor], List[dict], dict]:
    """-> (tensors, observation descriptions, index fields) of one member."""
    root = Path(media_root)
    target = _clip(root / row["target"], codecs.canvas)
    keep = usable_frames(len(target))
    if not keep:
        raise DataContractError(f"{row['id']}: the target holds {len(target)} frames on the 24 fps grid; 22 are needed")
    latents = codecs.video(target[:keep])
    n_lat = latent_frames(keep)
    if latents.ndim != 4 or latents.shape[1] != n_lat or not bool(torch.isfinite(latents.float()).all()):
        raise DataContractError(f"{row['id']}: the video codec returned {tuple(latents.shape)} for {n_lat} latent frames")
    embeds, tags = codecs.text(str(row.get("text", "")))
    tensors: Dict[str, torch.Tensor] = {"target_latents": latents, "prompt_embeds": embeds, "text_token_tags": tags.to(torch.int64)}
    described = []
    for i, obs in enumerate(row.get("observations") or ()):
        frames = obs.get("frames")
        aligned_all = frames == "all"
        pixels = _clip(root / obs["media"], codecs.canvas, obs.get("box"), keep if aligned_all else None)
        usable = usable_frames(len(pixels))
        lat = codecs.video(pixels[:usable] if usable else np.repeat(pixels[:1], 22, axis=0))
        if not usable:
            lat = lat[:, :1]                                       # a still or a very short clip: one latent frame
        if aligned_all:
            at = list(range(min(lat.shape[1], n_lat)))
            lat = lat[:, :len(at)]
        elif frames is None:
            at = None
        else:
            at = [int(f) for f in frames]
            if len(at) > lat.shape[1] or any(not 0 <= f < n_lat for f in at):
                raise DataContractError(f"{row['id']}: observation {i} names latent frames outside the clip")
            lat = lat[:, :len(at)]
        tensors[f"observation_{i}_latents"] = lat
        item = {"frames": at, "degree": float(obs.get("degree", 0.999))}
        if obs.get("box") is not None:
            item["boxes"] = [[float(v) for v in obs["box"]]]
        described.append(item)
    if row.get("known_mask"):
        mask = _clip(root / row["known_mask"], codecs.canvas, limit=keep)
        if len(mask) < keep:
            raise DataContractError(f"{row['id']}: the known mask is shorter than the target")
        tensors["known_degrees"] = known_degrees(mask, n_lat, (latents.shape[2] // 2, latents.shape[3] // 2))
    return tensors, described, {"latent_frames": n_lat, "observations": len(described), "pixel_frames": keep}


# ---------------------------------------------------------------------------------------------------------------------
# the shard loop
# ---------------------------------------------------------------------------------------------------------------------
def member_name(sample_id: str) -> str:
    import hashlib
    import re

    safe = re.sub(r"[^A-Za-z0-9._-]+", "_", sample_id).strip("._") or "sample"
    return f"{safe[:80]}-{hashlib.sha256(sample_id.encode()).hexdigest()[:12]}.safetensors"


def run_shard(rows: Sequence[Mapping[str, Any]], *, out, media_root, codecs: Codecs, shard: int = 0, shards: int = 1) -> Mapping[str, Any]:
    out = Path(out)
    members = out / "members"
    members.mkdir(parents=True, exist_ok=True)
    index_path = out / f"index-{shard:04d}.jsonl"
    index: Dict[str, dict] = {}
    if index_path.is_file():
        index = {r["id"]: r for r in (json.loads(l) for l in index_path.read_text().splitlines() if l.strip())}
    ids = [r["id"] for r in rows]
    if len(set(ids)) != len(ids):
        raise DataContractError("the input holds duplicate sample ids")

    def publish_index():
        tmp = index_path.with_name("." + index_path.name + ".tmp")
        tmp.write_text("".join(json.dumps(index[k], sort_keys=True) + "\n" for k in sorted(index)))
        os.replace(tmp, index_path)

    done, skipped, pending = [], [], []
    for row in list(rows)[shard::shards]:
        name = member_name(row["id"])
        final = members / name
        if final.is_file() and row["id"] in index:
            skipped.append(row["id"])
            continue
        try:
            tensors, described, fields = encode_row(row, codecs, media_root)
        except FetchFailed as exc:
            pending.append({"id": row["id"], "missing": str(exc)})
            continue
        tmp = members / f".{name}.{os.getpid()}.tmp"
        try:
            write_member(tmp, tensors, observations=described, source=str(row.get("source", "")))
            os.replace(tmp, final)
        except OSError as exc:
            tmp.unlink(missing_ok=True)
            raise WriteRefused(f"{final}: {exc}") from exc
        index[row["id"]] = {"id": row["id"], "member": f"members/{name}", "source": str(row.get("source", "")), **fields}
        publish_index()
        done.append(row["id"])
    return {"shard": shard, "shards": shards, "encoded": done, "skipped": skipped, "pending": pending, "index": str(index_path)}


def merge_indexes(out) -> int:
    """The corpus index = the union of the shard indexes (written last, atomically)."""
    out = Path(out)
    rows: Dict[str, dict] = {}
    for part in sorted(out.glob("index-*.jsonl")):
        for line in part.read_text().splitlines():
            if line.strip():
                r = json.loads(line)
                if r["id"] in rows:
                    raise DataContractError(f"sample {r['id']!r} was encoded by two shards")
                rows[r["id"]] = r
    tmp = out / ".index.jsonl.tmp"
    tmp.write_text("".join(json.dumps(rows[k], sort_keys=True) + "\n" for k in sorted(rows)))
    os.replace(tmp, out / "index.jsonl")
    return len(rows)
