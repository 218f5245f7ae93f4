"""Checkpoint transactions.

On-disk layout (kept byte-compatible with the reference so either side can verify the other's
checkpoints; reference: solar/checkpoint/store.py:21-285):

    <parent>/.<name>.<uuid>.partial/        private staging directory
        <component files ...>               e.g. model.pt, critic.pt, adapter.pt, optimizer.pt ...
        checkpoint-manifest.json            schema solarwm.checkpoint.v2: step, contract, required
                                            components, every file with its byte size, metadata
        COMPLETE.json                       schema solarwm.checkpoint-complete.v2: step + blake2s of
                                            the manifest bytes
    -> one os.replace onto <parent>/<name> and an fsync of the parent directory.

A directory without COMPLETE.json is never a checkpoint; an aborted transaction leaves its
``.partial`` directory behind for diagnosis.  Verification reads only the two small JSON files
and ``stat``s the payload (no re-hash of multi-GB tensors).
"""
from __future__ import annotations

import hashlib
import json
import os
import uuid
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Mapping, Sequence

from ..config.loader import canonical_json
from ..errors import CheckpointError

MANIFEST_NAME = "checkpoint-manifest.json"
COMPLETE_NAME = "COMPLETE.json"
MANIFEST_SCHEMA = "solarwm.checkpoint.v2"
COMPLETE_SCHEMA = "solarwm.checkpoint-complete.v2"

_REQUIRED_TEXT = ("family", "stage", "causal_mode", "objective", "camera_translation_transform",
                  "parameterization", "data_generation")


@dataclass(frozen=True)
class CheckpointContract:
    """Every algorithm-bearing setting that must be identical for an exact resume."""

    family: str
    stage: str
    causal_mode: str
    objective: str
    objective_variant: str
    camera_translation_transform: str
    parameterization: str
    sp_size: int
    data_generation: str
    extras: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        for name in _REQUIRED_TEXT:
            if not str(getattr(self, name)).strip():
                raise CheckpointError(f"checkpoint contract {name} must be non-empty")
        if int(self.sp_size) < 1:
            raise CheckpointError("checkpoint contract sp_size must be positive")

    def as_dict(self) -> dict:
        return asdict(self)

    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> "CheckpointContract":
        try:
            return cls(family=str(value["family"]), stage=str(value["stage"]),
                       causal_mode=str(value["causal_mode"]), objective=str(value["objective"]),
                       objective_variant=str(value.get("objective_variant", "")),
                       camera_translation_transform=str(value["camera_translation_transform"]),
                       parameterization=str(value["parameterization"]), sp_size=int(value["sp_size"]),
                       data_generation=str(value["data_generation"]), extras=dict(value.get("extras", {})))
        except (KeyError, TypeError, ValueError) as exc:
            raise CheckpointError("invalid checkpoint contract") from exc


@dataclass(frozen=True)
class ComponentFile:
    path: str
    size: int

    def __post_init__(self):
        if not isinstance(self.path, str) or not self.path:
            raise CheckpointError("checkpoint component path must be non-empty")
        if type(self.size) is not int or self.size < 1:
            raise CheckpointError(f"checkpoint component size must be positive: {self.path!r}")


@dataclass(frozen=True)
class VerifiedCheckpoint:
    path: Path
    step: int
    contract: CheckpointContract
    files: tuple
    metadata: Mapping[str, Any]
    manifest_digest: str


def _write_durably(path: Path, data: bytes) -> None:
    tmp = path.with_name(f".{path.name}.{os.getpid()}.tmp")
    with tmp.open("wb") as handle:
        handle.write(data)
        handle.flush()
        os.fsync(handle.fileno())
    os.replace(tmp, path)


def _inventory(root: Path, required: Sequence[str]) -> tuple:
    names = list(required)
    if not names or "" in names:
        raise CheckpointError("required checkpoint components must be non-empty")
    if len(set(names)) != len(names):
        raise CheckpointError("required checkpoint components contain duplicates")
    records = []
    for name in sorted(names):
        if "/" in name or name in (".", "..", MANIFEST_NAME, COMPLETE_NAME):
            raise CheckpointError(f"invalid checkpoint component {name!r}")
        target = root / name
        if not target.exists():
            raise CheckpointError(f"checkpoint component is missing: {name}")
        if target.is_symlink():
            raise CheckpointError(f"checkpoint component may not be a symlink: {name}")
    for name in sorted(names):
        target = root / name
        for item in ((target,) if target.is_file() else sorted(target.rglob("*"))):
            if item.is_symlink():
                raise CheckpointError(f"checkpoint contents may not be symlinks: {item.relative_to(root)}")
            if item.is_file():
                records.append(ComponentFile(item.relative_to(root).as_posix(), item.stat().st_size))
    if not records:
        raise CheckpointError("checkpoint contains no component files")
    return tuple(records)


class CheckpointTransaction:
    """``with CheckpointTransaction(dir) as tx: write files under tx.path; tx.commit(...)``."""

    def __init__(self, target):
        self.target = Path(target).resolve()
        self.path = self.target.with_name(f".{self.target.name}.{uuid.uuid4().hex}.partial")
        self._done = False

    def __enter__(self):
        if self.target.exists():
            raise CheckpointError(f"checkpoint target already exists: {self.target}")
        self.target.parent.mkdir(parents=True, exist_ok=True)
        self.path.mkdir(mode=0o755)
        return self

    def __exit__(self, *_):
        return None  # an uncommitted .partial directory stays for diagnosis

    def commit(self, *, step: int, contract: CheckpointContract, required_components: Sequence[str],
               metadata: Mapping[str, Any]) -> VerifiedCheckpoint:
        if self._done:
            raise CheckpointError("checkpoint transaction was already committed")
        if step < 0:
            raise CheckpointError("checkpoint step must be non-negative")
        files = _inventory(self.path, required_components)
        manifest = canonical_json({
            "schema": MANIFEST_SCHEMA, "step": int(step), "contract": contract.as_dict(),
            "required_components": sorted(required_components),
            "files": [{"path": f.path, "size": f.size} for f in files], "metadata": dict(metadata)})
        digest = hashlib.blake2s(manifest).hexdigest()
        _write_durably(self.path / MANIFEST_NAME, manifest)
        _write_durably(self.path / COMPLETE_NAME, canonical_json(
            {"schema": COMPLETE_SCHEMA, "step": int(step), "manifest_digest": digest}))
        if self.target.exists():
            raise CheckpointError(f"checkpoint target appeared during commit: {self.target}")
        os.replace(self.path, self.target)
        fd = os.open(self.target.parent, os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)
        self._done = True
        return verify_checkpoint(self.target)


def verify_checkpoint(path) -> VerifiedCheckpoint:
    root = Path(path).resolve()
    complete_path, manifest_path = root / COMPLETE_NAME, root / MANIFEST_NAME
    if not complete_path.is_file() or not manifest_path.is_file():
        raise CheckpointError(f"checkpoint is not complete: {root}")
    try:
        complete = json.loads(complete_path.read_bytes())
        manifest_bytes = manifest_path.read_bytes()
        manifest = json.loads(manifest_bytes)
    except (OSError, json.JSONDecodeError) as exc:
        raise CheckpointError(f"checkpoint metadata is invalid: {root}") from exc
    if complete.get("schema") != COMPLETE_SCHEMA or manifest.get("schema") != MANIFEST_SCHEMA:
        raise CheckpointError("unknown or mismatched checkpoint schemas")
    digest = hashlib.blake2s(manifest_bytes).hexdigest()
    if complete.get("manifest_digest") != digest:
        raise CheckpointError("checkpoint manifest identity differs from COMPLETE")
    if complete.get("step") != manifest.get("step"):
        raise CheckpointError("checkpoint step differs between manifest and COMPLETE")
    try:
        files = tuple(ComponentFile(**entry) for entry in manifest["files"])
        contract = CheckpointContract.from_dict(manifest["contract"])
        metadata = dict(manifest["metadata"])
        step = int(manifest["step"])
    except (KeyError, TypeError, ValueError) as exc:
        raise CheckpointError("checkpoint manifest fields are invalid") from exc
    if not files:
        raise CheckpointError("checkpoint manifest has no files")
    if len({f.path for f in files}) != len(files):
        raise CheckpointError("checkpoint manifest has duplicate file paths")
    for f in files:
        rel = Path(f.path)
        if rel.is_absolute() or ".." in rel.parts:
            raise CheckpointError(f"checkpoint manifest has unsafe path {f.path!r}")
        target = root / rel
        if not target.is_file() or target.is_symlink():
            raise CheckpointError(f"checkpoint file is missing: {f.path}")
        if target.stat().st_size != f.size:
            raise CheckpointError(f"checkpoint file size differs: {f.path}")
    return VerifiedCheckpoint(root, step, contract, files, metadata, digest)


def assert_resume_compatible(expected: CheckpointContract, actual: CheckpointContract) -> None:
    want, got = expected.as_dict(), actual.as_dict()
    if want == got:
        return
    diff = {k: {"expected": want[k], "actual": got[k]} for k in want if want[k] != got[k]}
    raise CheckpointError(f"exact-resume contract mismatch: {diff}")
