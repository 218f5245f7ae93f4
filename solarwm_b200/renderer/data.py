"""Reader of the renderer's encoded training corpus ("omni" members) with a resumable, rank-aware plan.

  member   one safetensors file per clip: ``target_latents`` [C, 5n + 2, H, W], ``prompt_embeds`` [L, D],
           ``text_token_tags`` [L] (modality ids 0..2), optionally ``anchor_latents`` [C, 1, H, W], ``structure_latents``
           (the target's shape), ``camera_c2w`` [F, 4, 4] absolute with ``camera_K`` [F, 3, 3] or [3, 3] normalised,
           ``known_degrees`` (one value in [0, 1] per packed target row), and ``observation_<i>_latents`` described by the
           file's ``omni`` metadata (``frames``, ``degree``, ``boxes``).  Everything is validated on read; cameras become
           world-to-camera matrices relative to the clip's first camera (guarded in magnitude).
  index    JSON lines ``{id, member, latent_frames?, observations?, first_frame?, ...}``; ids unique; rows sorted by id.
  plan     per epoch a seeded permutation, cut to a multiple of the data-parallel size; reader ``r`` takes every
           ``world``-th row from ``r``.  With ``length_buckets`` the rows are grouped by (clip length, observation count),
           each group is shuffled and cut into runs of ``world`` rows, and the runs are shuffled: at every step all readers
           hold clips of one length, so no rank waits on a longer sequence.  A group's last partial run sits the epoch out.
  resume   ``state_dict()`` = (epoch, cursor, plan fingerprint); a failed read leaves the cursor where it was; a plan
           whose fingerprint changed refuses the state.

Reference: H3OmniReader / H3OmniStream (solar/renderer/data.py:89-396).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import DataContractError

PLAN_SCHEMA = "solarwm.renderer-data-plan.v1"
CAMERA_GUARD = 20.0


@dataclass(frozen=True)
class MemberContract:
    """What a member must look like.  The released geometry is the default; tests and small models pass their own."""
    latent_channels: int = 24
    text_dim: int = 5120
    grids: Tuple[Tuple[int, int], ...] = ((48, 84), (84, 48))
    frames_period: int = 5
    frames_offset: int = 2


@dataclass(frozen=True)
class VisualObservation:
    latents: torch.Tensor                       # [C, F, 2h, 2w]
    frames: Optional[Tuple[int, ...]]           # target latent each frame is pinned to; None: free-floating
    degree: float = 0.999
    boxes: Optional[Tuple[Tuple[float, ...], ...]] = None


@dataclass
class OmniSample:
    sample_id: str
    target_latents: torch.Tensor
    prompt_embeds: torch.Tensor
    text_token_tags: torch.Tensor
    anchor_latents: Optional[torch.Tensor] = None
    structure_latents: Optional[torch.Tensor] = None
    camera_w2c: Optional[torch.Tensor] = None    # [1 + F, 4, 4]: the anchor's camera (the first) in front
    camera_K: Optional[torch.Tensor] = None
    known_degree: Optional[torch.Tensor] = None
    observations: Tuple[VisualObservation, ...] = ()
    source: str = ""
    plan_fingerprint: str = "render"

    def as_training_sample(self) -> Dict[str, Any]:
        """The mapping ``renderer.core.OmniFlowTrainer`` consumes."""
        lat = self.target_latents
        out = {"target_latents": lat, "prompt_embeds": self.prompt_embeds, "shape": tuple(lat.shape),
               "anchor_latents": self.anchor_latents if self.anchor_latents is not None else torch.zeros_like(lat[:, :1])}
        for key in ("structure_latents", "camera_w2c", "known_degree"):
            if getattr(self, key) is not None:
                out[key] = getattr(self, key)
        return out


def views_from_c2w(c2w: torch.Tensor) -> torch.Tensor:
    """Absolute camera-to-world [F, 4, 4] -> world-to-camera relative to the first camera (fp64 inside)."""
    m = c2w.double()
    rel = torch.linalg.inv(m[0]) @ m
    rel[0] = torch.eye(4, dtype=torch.float64)
    return torch.linalg.inv(rel).float().contiguous()


def _finite(t: torch.Tensor) -> bool:
    return bool(torch.isfinite(t.float()).all())


def _camera(tensors: Mapping[str, torch.Tensor], frames: int):
    c2w, K = tensors.get("camera_c2w"), tensors.get("camera_K")
    if c2w is None and K is None:
        return None, None
    if c2w is None or K is None:
        raise DataContractError("an omni camera needs both the poses and the intrinsics")
    if tuple(c2w.shape) != (frames, 4, 4):
        raise DataContractError(f"omni camera holds {tuple(c2w.shape)}, not [{frames}, 4, 4]")
    if tuple(K.shape) == (3, 3):
        K = K.unsqueeze(0).expand(frames, -1, -1).clone()
    if tuple(K.shape) != (frames, 3, 3):
        raise DataContractError(f"omni intrinsics hold {tuple(K.shape)}, not [{frames}, 3, 3]")
    c2w, K = c2w.float(), K.float()
    if not _finite(c2w) or not _finite(K):
        raise DataContractError("omni camera holds non-finite values")
    bottom = torch.tensor([0.0, 0.0, 0.0, 1.0])
    rot = c2w[:, :3, :3]
    if not torch.allclose(c2w[:, 3], bottom.expand(frames, 4), atol=1e-4) or \
            not torch.allclose(rot @ rot.transpose(1, 2), torch.eye(3).expand(frames, 3, 3), atol=1e-3):
        raise DataContractError("omni camera poses must be rigid camera-to-world matrices")
    if bool((K[:, 0, 0] <= 0).any() or (K[:, 1, 1] <= 0).any() or (K[:, :2, 2] < 0).any() or (K[:, :2, 2] > 1).any()):
        raise DataContractError("omni intrinsics must be normalised (positive focal lengths, principal point in [0, 1])")
    views = views_from_c2w(c2w)
    if float(views.abs().max()) > CAMERA_GUARD:
        raise DataContractError("omni camera exceeds the magnitude guard")
    return torch.cat([views[:1], views]), K.contiguous()


def read_member(path, row: Mapping[str, Any], contract: MemberContract = MemberContract(), plan_fingerprint: str = "render") -> OmniSample:
    from safetensors import safe_open

    with safe_open(str(path), framework="pt") as handle:
        meta = json.loads((handle.metadata() or {}).get("omni", "{}"))
        tensors = {key: handle.get_tensor(key) for key in handle.keys()}
    for need in ("target_latents", "prompt_embeds", "text_token_tags"):
        if need not in tensors:
            raise DataContractError(f"omni member holds no {need}")
    target, prompt, tags = tensors["target_latents"], tensors["prompt_embeds"], tensors["text_token_tags"]
    c = contract
    if target.ndim != 4 or target.shape[0] != c.latent_channels or (target.shape[1] - c.frames_offset) % c.frames_period \
            or target.shape[1] < c.frames_offset:
        raise DataContractError(f"omni target latents {tuple(target.shape)} are not [{c.latent_channels}, "
                                f"{c.frames_period}n + {c.frames_offset}, h, w]")
    if tuple(target.shape[2:]) not in c.grids:
        raise DataContractError(f"omni target grid {tuple(target.shape[2:])} is not one of {list(c.grids)}")
    if prompt.ndim != 2 or prompt.shape[1] != c.text_dim or tags.shape != prompt.shape[:1]:
        raise DataContractError("omni prompt embeddings and token tags do not fit the text contract")
    if tags.dtype not in (torch.int32, torch.int64) or not bool(((tags >= 0) & (tags <= 2)).all()):
        raise DataContractError("omni token tags must be integer modality ids in [0, 2]")
    if not _finite(target) or not _finite(prompt):
        raise DataContractError("omni member holds non-finite values")
    frames = int(target.shape[1])
    for name, shape in (("anchor_latents", (c.latent_channels, 1, *target.shape[2:])), ("structure_latents", tuple(target.shape))):
        if name in tensors and (tuple(tensors[name].shape) != shape or not _finite(tensors[name])):
            raise DataContractError(f"omni {name} must be finite {list(shape)}")
    observations: List[VisualObservation] = []
    for i, item in enumerate(meta.get("observations", ())):
        lat = tensors.get(f"observation_{i}_latents")
        if lat is None or lat.ndim != 4 or lat.shape[0] != c.latent_channels or min(lat.shape[1:]) < 1 \
                or any(s % 2 for s in lat.shape[2:]) or not _finite(lat):
            raise DataContractError("visual observations must be finite [C, F, 2h, 2w] tensors")
        at = item.get("frames")
        if at is not None and (len(at) != lat.shape[1] or any(type(f) is not int or not 0 <= f < frames for f in at)):
            raise DataContractError("observation frames must align with the target latent range")
        degree = float(item.get("degree", 0.999))
        if not 0 < degree <= 1:
            raise DataContractError("observation degree must lie in (0, 1]")
        boxes = item.get("boxes")
        observations.append(VisualObservation(lat.contiguous(), None if at is None else tuple(at), degree,
                                              None if not boxes else tuple(tuple(float(v) for v in b) for b in boxes)))
    if row.get("free_observations"):
        observations = [VisualObservation(o.latents, None, o.degree, o.boxes) if o.frames is not None and len(o.frames) > 1 else o
                        for o in observations]
    known = tensors.get("known_degrees")
    rows = frames * target.shape[2] * target.shape[3] // 4
    if known is not None and (known.numel() != rows or not _finite(known) or not bool(((known >= 0) & (known <= 1)).all())):
        raise DataContractError("known_degrees must cover each target row with a value in [0, 1]")
    views, K = _camera(tensors, frames)
    return OmniSample(sample_id=str(row["id"]), target_latents=target.contiguous(), prompt_embeds=prompt.contiguous(),
                      text_token_tags=tags.contiguous(), anchor_latents=tensors.get("anchor_latents"),
                      structure_latents=tensors.get("structure_latents"), camera_w2c=views, camera_K=K,
                      known_degree=None if known is None else known.reshape(-1).float(), observations=tuple(observations),
                      source=str(meta.get("source", row.get("source", ""))), plan_fingerprint=plan_fingerprint)


def write_member(path, tensors: Mapping[str, torch.Tensor], *, observations: Sequence[Mapping[str, Any]] = (), source: str = "") -> None:
    """Write one member (what the renderer's preencode step produces); ``observations[i]`` describes
    ``tensors['observation_<i>_latents']``."""
    from safetensors.torch import save_file

    meta = {"omni": json.dumps({"observations": list(observations), "source": source}, sort_keys=True)}
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path), metadata=meta)


class OmniStream:
    def __init__(self, *, root, index, dp_rank: int, dp_size: int, seed: int, shuffle: bool = True, length_buckets: bool = False,
                 contract: MemberContract = MemberContract()):
        self.root, self.contract = Path(root).resolve(), contract
        rows = [json.loads(line) for line in Path(index).read_text().splitlines() if line.strip()]
        if not rows:
            raise DataContractError(f"omni index {index} is empty")
        if any(not isinstance(r.get("id"), str) or not r["id"] for r in rows):
            raise DataContractError("omni index ids must be non-empty strings")
        self.rows = sorted(rows, key=lambda r: r["id"])
        if len({r["id"] for r in self.rows}) != len(self.rows):
            raise DataContractError("omni index contains duplicate sample ids")
        self.rank, self.world = int(dp_rank), int(dp_size)
        if self.world < 1 or not 0 <= self.rank < self.world:
            raise DataContractError("invalid data-parallel rank or size")
        if len(self.rows) < self.world:
            raise DataContractError("omni index holds fewer samples than data-parallel readers")
        self.seed, self.shuffle, self.length_buckets = int(seed), bool(shuffle), bool(length_buckets)
        self.epoch = self.cursor = 0
        self._order_of: Optional[Tuple[int, np.ndarray]] = None
        identity = {"schema": PLAN_SCHEMA, "root": str(self.root), "rows": self.rows, "seed": self.seed, "shuffle": self.shuffle,
                    "length_buckets": self.length_buckets, "world_size": self.world}
        self.plan_fingerprint = hashlib.sha256(json.dumps(identity, sort_keys=True, separators=(",", ":"), allow_nan=False).encode()).hexdigest()

    # -- the epoch's order ------------------------------------------------------------------------------------------------
    def _bucketed(self, rng) -> np.ndarray:
        groups: Dict[Tuple[int, int], List[int]] = {}
        for i, row in enumerate(self.rows):
            groups.setdefault((int(row.get("latent_frames") or 47), int(row.get("observations") or 0)), []).append(i)
        runs = []
        for key in sorted(groups):
            members = np.asarray(groups[key], dtype=np.int64)
            rng.shuffle(members)
            whole = len(members) - len(members) % self.world
            runs.extend(members[:whole].reshape(-1, self.world))
        if not runs:
            return np.zeros(0, dtype=np.int64)
        runs = np.stack(runs)
        rng.shuffle(runs)
        return runs.reshape(-1)

    def global_order(self, epoch: int) -> np.ndarray:
        rng = np.random.default_rng([self.seed, epoch])
        if self.length_buckets and self.shuffle:
            order = self._bucketed(rng)
            if len(order):
                return order
            rng = np.random.default_rng([self.seed, epoch])
        order = np.arange(len(self.rows))
        if self.shuffle:
            rng.shuffle(order)
        return order[:len(order) - len(order) % self.world]

    def _mine(self) -> np.ndarray:
        if self._order_of is None or self._order_of[0] != self.epoch:
            self._order_of = (self.epoch, self.global_order(self.epoch)[self.rank::self.world])
        return self._order_of[1]

    # -- iteration ----------------------------------------------------------------------------------------------------------
    def next(self) -> OmniSample:
        before = (self.epoch, self.cursor)
        order = self._mine()
        if self.cursor == len(order):
            self.epoch, self.cursor = self.epoch + 1, 0
            order = self._mine()
        row = self.rows[int(order[self.cursor])]
        try:
            member = Path(row["member"])
            sample = read_member(member if member.is_absolute() else self.root / member, row, self.contract, self.plan_fingerprint)
        except Exception as exc:  # noqa: BLE001 - the cursor must not move past a sample that was not delivered
            self.epoch, self.cursor = before
            raise DataContractError(f"cannot read renderer sample {row['id']!r}: {exc}") from exc
        self.cursor += 1
        return sample

    def __iter__(self):
        while True:
            yield self.next()

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "cursor": self.cursor, "plan_fingerprint": self.plan_fingerprint}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        if state.get("plan_fingerprint") != self.plan_fingerprint:
            raise DataContractError("renderer data plan fingerprint changed since the checkpoint")
        epoch, cursor = state.get("epoch"), state.get("cursor")
        if any(type(v) is not int or v < 0 for v in (epoch, cursor)):
            raise DataContractError("renderer data epoch and cursor must be non-negative integers")
        before = (self.epoch, self.cursor)
        self.epoch, self.cursor = epoch, cursor
        if cursor > len(self._mine()):
            self.epoch, self.cursor = before
            raise DataContractError("renderer data cursor exceeds the epoch length")

    def close(self) -> None:
        return None
