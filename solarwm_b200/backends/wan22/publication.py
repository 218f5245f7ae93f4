"""Dataset-triplet publication of a camera-length generation run.

A finished generation transaction holds, per case, ``slot-NNNNNN/{video.mp4, compare.mp4, camera.npy, manifest.json}``.
Consumers of a generated DATASET want three parallel trees instead -- ``generate/<dataset>/<stem>.mp4``,
``compare/<dataset>/<stem>.mp4``, ``camera/<dataset>/<stem>.npy`` -- that look like the source corpus.  Publication:

  plan        every case names its ``physical_dataset`` and ``publish_stem`` (portable path components), the number of
              published pixel frames and that its cameras are authoritative absolute camera-to-world matrices;
              duplicate slots or destinations are refused;
  preflight   BEFORE any generation starts: none of the public names exists, no provenance of an earlier publication;
  publish     the source transaction must be sealed; every artifact is re-read and must still have the size and digest
              its slot manifest recorded; ``camera.npy`` must be finite float64 ``[frames, 4, 4]``; files are published
              as create-only hard links (nothing is copied), each case gets a receipt, then the ordered manifest, and
              ``publication/COMPLETE.json`` LAST: a reader that sees it sees everything.

Reference: preflight_camera_publication / publish_camera_triplets (solar/backends/wan22/runtime/publication.py:60-340).
"""
from __future__ import annotations

import hashlib
import json
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping, Sequence

import numpy as np

from ...config.loader import canonical_json
from ...engine.inference_engine import InferenceCase
from ...errors import BackendContractError
from ...runtime.create_only import link_file_create_only, write_file_create_only
from ...runtime.output_layout import DATASET_TRIPLET, dataset_triplet_dirs

SAMPLE_SCHEMA = "solarwm.wan22-camera-publication-sample.v1"
COMPLETE_SCHEMA = "solarwm.wan22-camera-publication-complete.v1"
ARTIFACT_TREE = {"video.mp4": "generate", "compare.mp4": "compare", "camera.npy": "camera"}


def _component(value, what: str) -> str:
    text = str(value or "")
    if not re.fullmatch(r"[A-Za-z0-9][A-Za-z0-9._-]{0,200}", text) or text in (".", ".."):
        raise BackendContractError(f"{what} must be one portable path component, got {value!r}")
    return text


@dataclass(frozen=True)
class Target:
    case: InferenceCase
    dataset: str
    stem: str
    frames: int
    destinations: Mapping[str, Path]


@dataclass(frozen=True)
class TripletPlan:
    root: Path
    run_id: str
    targets: tuple

    @property
    def provenance_dir(self) -> Path:
        return dataset_triplet_dirs(self.root, self.run_id)["run"] / "publication"


def plan_triplets(root, run_id: str, cases: Sequence[InferenceCase]) -> TripletPlan:
    dirs = dataset_triplet_dirs(root, run_id)
    targets, slots, paths = [], set(), set()
    for case in cases:
        if case.slot in slots:
            raise BackendContractError(f"publication holds slot {case.slot} twice")
        slots.add(case.slot)
        meta = case.metadata
        dataset = _component(meta.get("physical_dataset"), f"slot {case.slot} physical_dataset")
        stem = _component(meta.get("publish_stem"), f"slot {case.slot} publish_stem")
        try:
            frames = int(meta["publication_pixel_frames"])
        except (KeyError, TypeError, ValueError) as exc:
            raise BackendContractError(f"slot {case.slot} lacks publication_pixel_frames") from exc
        if frames < 1:
            raise BackendContractError(f"slot {case.slot} publishes {frames} frames")
        if str(meta.get("camera_publication_convention", "")) != "authoritative_absolute_c2w":
            raise BackendContractError(f"slot {case.slot} does not carry authoritative absolute camera-to-world matrices")
        dest = {name: dirs[tree] / dataset / f"{stem}{Path(name).suffix}" for name, tree in ARTIFACT_TREE.items()}
        for d in dest.values():
            if d in paths:
                raise BackendContractError(f"two cases publish to {d}")
            paths.add(d)
        targets.append(Target(case, dataset, stem, frames, dest))
    if not targets:
        raise BackendContractError("a publication needs at least one case")
    return TripletPlan(Path(root), run_id, tuple(targets))


def preflight(plan: TripletPlan) -> None:
    """Refuse occupied public names and earlier provenance before anything is generated."""
    taken = [str(d) for t in plan.targets for d in t.destinations.values() if d.exists() or d.is_symlink()]
    if taken:
        raise BackendContractError(f"publication targets already exist (first: {taken[:4]})")
    if plan.provenance_dir.exists() or plan.provenance_dir.is_symlink():
        raise BackendContractError(f"publication provenance already exists: {plan.provenance_dir}")


def _identity(path: Path):
    h, size = hashlib.blake2s(), 0
    try:
        with path.open("rb") as fh:
            for chunk in iter(lambda: fh.read(1 << 20), b""):
                size += len(chunk)
                h.update(chunk)
    except OSError as exc:
        raise BackendContractError(f"cannot read {path}: {exc}") from exc
    return size, h.hexdigest()


def _verified_artifacts(folder: Path, manifest: Mapping[str, Any], frames: int) -> dict:
    listed = manifest.get("artifacts")
    if not isinstance(listed, list):
        raise BackendContractError(f"{folder.name}: the slot manifest lists no artifacts")
    found = {}
    for rec in listed:
        path = str(rec.get("path", "")) if isinstance(rec, Mapping) else ""
        if not path.startswith(folder.name + "/"):
            raise BackendContractError(f"{folder.name}: artifact path {path!r} is outside its slot")
        name = path[len(folder.name) + 1:]
        if name not in ARTIFACT_TREE:
            continue
        if name in found:
            raise BackendContractError(f"{folder.name}: {name} is listed twice")
        size, digest = _identity(folder / name)
        if (size, digest) != (int(rec.get("bytes", -1)), str(rec.get("digest", ""))):
            raise BackendContractError(f"{folder / name} changed since its manifest was written")
        found[name] = (folder / name, size, digest)
    missing = sorted(set(ARTIFACT_TREE) - set(found))
    if missing:
        raise BackendContractError(f"{folder.name} lacks {missing}")
    try:
        c2w = np.load(found["camera.npy"][0], allow_pickle=False)
    except (OSError, ValueError) as exc:
        raise BackendContractError(f"{found['camera.npy'][0]} is not a valid array file") from exc
    if c2w.shape != (frames, 4, 4) or c2w.dtype != np.float64 or not np.isfinite(c2w).all():
        raise BackendContractError(f"{folder.name}/camera.npy must be finite float64 [{frames}, 4, 4]")
    return found


def publish_triplets(generation_dir, plan: TripletPlan, *, family: str, weights_id: str) -> Mapping[str, Any]:
    generation_dir = Path(generation_dir)
    preflight(plan)
    seal_path = generation_dir / "COMPLETE.json"
    if not seal_path.is_file():
        raise BackendContractError("the generation transaction is not sealed")
    seal = json.loads(seal_path.read_text())
    if seal.get("family") != family or seal.get("weights_id") != weights_id:
        raise BackendContractError("the generation transaction belongs to another family or other weights")
    prepared = []
    for t in plan.targets:                               # verify everything before the first public name appears
        folder = generation_dir / f"slot-{t.case.slot:06d}"
        try:
            manifest = json.loads((folder / "manifest.json").read_text())
        except (OSError, ValueError) as exc:
            raise BackendContractError(f"{folder}/manifest.json is unreadable: {exc}") from exc
        case = manifest.get("case", {})
        if int(case.get("slot", -1)) != t.case.slot or case.get("sample_id") != t.case.sample_id \
                or manifest.get("family") != family or manifest.get("weights_id") != weights_id:
            raise BackendContractError(f"slot {t.case.slot} is not the case that was planned")
        prepared.append((t, manifest, _verified_artifacts(folder, manifest, t.frames)))
    records = []
    for t, manifest, artifacts in prepared:
        public = {}
        for name in ARTIFACT_TREE:
            src, size, digest = artifacts[name]
            try:
                link_file_create_only(src, t.destinations[name])
            except FileExistsError as exc:
                raise BackendContractError(f"{t.destinations[name]} appeared during publication") from exc
            public[name] = {"path": t.destinations[name].relative_to(plan.root).as_posix(), "bytes": size, "digest": digest}
        record = {"schema": SAMPLE_SCHEMA, "slot": t.case.slot, "sample_id": t.case.sample_id, "physical_dataset": t.dataset,
                  "stem": t.stem, "published_pixel_frames": t.frames,
                  "source_manifest_digest": hashlib.blake2s(canonical_json(manifest)).hexdigest(), "artifacts": public}
        write_file_create_only(plan.provenance_dir / "samples" / f"slot-{t.case.slot:06d}.json", canonical_json(record))
        records.append(record)
    ordered = b"".join(canonical_json(r) for r in records)
    digest = hashlib.blake2s(ordered).hexdigest()
    write_file_create_only(plan.provenance_dir / "ordered-manifest.jsonl", ordered)
    complete = {"schema": COMPLETE_SCHEMA, "layout": DATASET_TRIPLET, "run_id": plan.run_id, "family": family,
                "weights_id": weights_id, "generation_complete_digest": seal.get("ordered_manifest_digest"),
                "cases": len(records), "ordered_manifest_digest": digest}
    write_file_create_only(plan.provenance_dir / "COMPLETE.json", canonical_json(complete))      # the visibility gate
    return complete
