"""Checkpoint directories that are either whole or absent.

Layout on disk (a shared contract: the reference's verifier accepts directories written here and this verifier
accepts the reference's, which ``tests/test_reference_contracts.py`` checks; contract: solar/checkpoint/store.py:21-285):

    <parent>/.<name>.<32 hex>.partial/      staging directory, private to one writer
        model.pt, optimizer.pt, adapter/...  the components, written by the caller
        checkpoint-manifest.json             ``solarwm.checkpoint.v2``: step, resume contract, the required component
                                             names, every payload file with its size in bytes, caller metadata
        COMPLETE.json                        ``solarwm.checkpoint-complete.v2``: step and the blake2s of the manifest's
                                             bytes; written last
    one rename onto <parent>/<name>, then an fsync of <parent>

The pieces, each usable on its own:

  ``CheckpointContract``   the settings an exact resume must find unchanged
  ``Manifest``             the manifest as a value: built from a staging directory's ``payload_files``, turned into
                           canonical bytes, parsed back; its digest is the checkpoint's identity
  ``CheckpointTransaction`` the staging directory, the two durable writes and the rename
  ``verify_checkpoint``    reads the two small JSON files and ``stat``s the payload -- multi-GB tensors are never
                           re-hashed -- through an ordered list of named checks

A directory without ``COMPLETE.json`` is never a checkpoint, and a transaction that does not commit leaves its
``.partial`` directory in place for inspection.
"""
from __future__ import annotations

import hashlib
import json
import os
import stat as stat_mod
import uuid
from dataclasses import dataclass, field, fields
from pathlib import Path, PurePosixPath
from typing import Any, Dict, Iterator, List, Mapping, Sequence, Tuple

from ..config.loader import canonical_json
from ..errors import CheckpointError

MANIFEST_NAME = "checkpoint-manifest.json"
COMPLETE_NAME = "COMPLETE.json"
MANIFEST_SCHEMA = "solarwm.checkpoint.v2"
COMPLETE_SCHEMA = "solarwm.checkpoint-complete.v2"
_RESERVED = frozenset({".", "..", MANIFEST_NAME, COMPLETE_NAME})


# ---------------------------------------------------------------------------------------------------------------------
# resume contract
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CheckpointContract:
    """What must be identical between the run that saved and the run that resumes."""

    family: str
    stage: str
    causal_mode: str
    objective: str
    objective_variant: str                  # may be empty
    camera_translation_transform: str
    parameterization: str
    sp_size: int
    data_generation: str
    extras: Mapping[str, Any] = field(default_factory=dict)

    _MAY_BE_EMPTY = ("objective_variant",)

    def __post_init__(self):
        for f in fields(self):
            if f.type in ("str", str) and f.name not in self._MAY_BE_EMPTY and not str(getattr(self, f.name)).strip():
                raise CheckpointError(f"checkpoint contract {f.name} must be non-empty")
        if int(self.sp_size) < 1:
            raise CheckpointError("checkpoint contract sp_size must be positive")

    def as_dict(self) -> Dict[str, Any]:
        out = {f.name: getattr(self, f.name) for f in fields(self)}
        out["extras"] = dict(self.extras)
        return out

    @classmethod
    def from_dict(cls, value: Mapping[str, Any]) -> "CheckpointContract":
        try:
            text = {f.name: str(value[f.name]) for f in fields(cls)
                    if f.type in ("str", str) and f.name not in cls._MAY_BE_EMPTY}
            return cls(**text, objective_variant=str(value.get("objective_variant", "")), sp_size=int(value["sp_size"]),
                       extras=dict(value.get("extras", {})))
        except (KeyError, TypeError, ValueError) as exc:
            raise CheckpointError("invalid checkpoint contract") from exc


def assert_resume_compatible(expected: CheckpointContract, actual: CheckpointContract) -> None:
    want, got = expected.as_dict(), actual.as_dict()
    changed = {name: {"expected": want[name], "actual": got[name]} for name in want if want[name] != got[name]}
    if changed:
        raise CheckpointError(f"exact-resume contract mismatch: {changed}")


# ---------------------------------------------------------------------------------------------------------------------
# payload inventory and manifest
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class ComponentFile:
    path: str          # POSIX, relative to the checkpoint directory
    size: int          # bytes; empty files are refused (a zero-length tensor file is always a failed write)

    def __post_init__(self):
        if not (isinstance(self.path, str) and self.path):
            raise CheckpointError("checkpoint component path must be non-empty")
        if type(self.size) is not int or self.size <= 0:
            raise CheckpointError(f"checkpoint component size must be positive: {self.path!r}")


def _regular_files(top: Path) -> Iterator[Path]:
    """Every regular file at or under ``top`` in sorted order; a symbolic link anywhere is an error."""
    if top.is_symlink():
        raise CheckpointError(f"checkpoint contents may not be symlinks: {top.name}")
    if top.is_file():
        yield top
        return
    for child in sorted(top.iterdir()):
        yield from _regular_files(child)


def payload_files(root: Path, required: Sequence[str]) -> Tuple[ComponentFile, ...]:
    """The files that make up the named components of a staging directory, sorted by component name."""
    names = sorted(required)
    if not names or any(not n for n in names):
        raise CheckpointError("required checkpoint components must be non-empty")
    if len(set(names)) < len(names):
        raise CheckpointError("required checkpoint components contain duplicates")
    for name in names:
        if "/" in name or name in _RESERVED:
            raise CheckpointError(f"invalid checkpoint component {name!r}")
        if not os.path.lexists(root / name):
            raise CheckpointError(f"required component {name!r} was not written")
    found: List[ComponentFile] = []
    for name in names:
        for f in _regular_files(root / name):
            found.append(ComponentFile(f.relative_to(root).as_posix(), f.stat().st_size))
    if not found:
        raise CheckpointError("checkpoint contains no component files")
    return tuple(found)


@dataclass(frozen=True)
class Manifest:
    step: int
    contract: CheckpointContract
    required_components: Tuple[str, ...]
    files: Tuple[ComponentFile, ...]
    metadata: Mapping[str, Any]

    def to_bytes(self) -> bytes:
        return canonical_json({"schema": MANIFEST_SCHEMA, "step": int(self.step), "contract": self.contract.as_dict(),
                               "required_components": sorted(self.required_components),
                               "files": [{"path": f.path, "size": f.size} for f in self.files],
                               "metadata": dict(self.metadata)})

    @classmethod
    def from_bytes(cls, raw: bytes) -> "Manifest":
        try:
            doc = json.loads(raw)
            if doc.get("schema") != MANIFEST_SCHEMA:
                raise CheckpointError("unknown checkpoint manifest schema")
            return cls(step=int(doc["step"]), contract=CheckpointContract.from_dict(doc["contract"]),
                       required_components=tuple(doc.get("required_components", ())),
                       files=tuple(ComponentFile(**entry) for entry in doc["files"]), metadata=dict(doc["metadata"]))
        except CheckpointError:
            raise
        except (AttributeError, KeyError, TypeError, ValueError) as exc:
            raise CheckpointError("checkpoint manifest fields are invalid") from exc

    @staticmethod
    def digest_of(raw: bytes) -> str:
        return hashlib.blake2s(raw).hexdigest()


@dataclass(frozen=True)
class VerifiedCheckpoint:
    path: Path
    step: int
    contract: CheckpointContract
    files: tuple
    metadata: Mapping[str, Any]
    manifest_digest: str


# ---------------------------------------------------------------------------------------------------------------------
# writing
# ---------------------------------------------------------------------------------------------------------------------
def _durable_write(path: Path, data: bytes) -> None:
    """Create ``path`` with ``data`` and force it to disk (the staging directory is private: no rename needed)."""
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o644)
    try:
        view = memoryview(data)
        while view:
            view = view[os.write(fd, view):]
        os.fsync(fd)
    finally:
        os.close(fd)


def _sync_directory(path: Path) -> None:
    fd = os.open(path, os.O_RDONLY | getattr(os, "O_DIRECTORY", 0))
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


class CheckpointTransaction:
    """``with CheckpointTransaction(directory) as tx:`` write the components under ``tx.path``, then ``tx.commit(...)``."""

    def __init__(self, target):
        self.target = Path(target).resolve()
        self.path = self.target.parent / f".{self.target.name}.{uuid.uuid4().hex}.partial"
        self._committed = False

    def __enter__(self) -> "CheckpointTransaction":
        if os.path.lexists(self.target):
            raise CheckpointError(f"checkpoint target already exists: {self.target}")
        self.target.parent.mkdir(parents=True, exist_ok=True)
        self.path.mkdir(mode=0o755)
        return self

    def __exit__(self, *exc_info) -> None:
        # nothing to undo: an uncommitted staging directory is evidence, not a checkpoint
        return None

    def commit(self, *, step: int, contract: CheckpointContract, required_components: Sequence[str],
               metadata: Mapping[str, Any]) -> VerifiedCheckpoint:
        if self._committed:
            raise CheckpointError("checkpoint transaction was already committed")
        if int(step) < 0:
            raise CheckpointError("checkpoint step must be non-negative")
        manifest = Manifest(int(step), contract, tuple(required_components),
                            payload_files(self.path, required_components), dict(metadata))
        raw = manifest.to_bytes()
        _durable_write(self.path / MANIFEST_NAME, raw)
        _durable_write(self.path / COMPLETE_NAME, canonical_json(
            {"schema": COMPLETE_SCHEMA, "step": int(step), "manifest_digest": Manifest.digest_of(raw)}))
        _sync_directory(self.path)
        if os.path.lexists(self.target):
            raise CheckpointError(f"checkpoint target already exists (it appeared during the commit): {self.target}")
        os.rename(self.path, self.target)
        _sync_directory(self.target.parent)
        self._committed = True
        return verify_checkpoint(self.target)


# ---------------------------------------------------------------------------------------------------------------------
# verification
# ---------------------------------------------------------------------------------------------------------------------
def _check_identity(root: Path, raw: bytes, complete: Mapping[str, Any], manifest: Manifest) -> None:
    if complete.get("schema") != COMPLETE_SCHEMA:
        raise CheckpointError("unknown or mismatched checkpoint schemas")
    if complete.get("manifest_digest") != Manifest.digest_of(raw):
        raise CheckpointError("the manifest is not the one COMPLETE.json was written for")
    if complete.get("step") != manifest.step:
        raise CheckpointError("checkpoint step differs between manifest and COMPLETE")


def _check_listing(root: Path, raw: bytes, complete: Mapping[str, Any], manifest: Manifest) -> None:
    if not manifest.files:
        raise CheckpointError("checkpoint manifest has no files")
    paths = [f.path for f in manifest.files]
    if len(set(paths)) < len(paths):
        raise CheckpointError("checkpoint manifest has duplicate file paths")
    for p in paths:
        pure = PurePosixPath(p)
        if pure.is_absolute() or ".." in pure.parts:
            raise CheckpointError(f"checkpoint manifest has unsafe path {p!r}")


def _check_payload(root: Path, raw: bytes, complete: Mapping[str, Any], manifest: Manifest) -> None:
    for f in manifest.files:
        try:
            st = os.lstat(root / f.path)
        except OSError:
            raise CheckpointError(f"checkpoint file is missing: {f.path}") from None
        if not stat_mod.S_ISREG(st.st_mode):
            raise CheckpointError(f"checkpoint file is missing: {f.path} (not a regular file)")
        if st.st_size != f.size:
            raise CheckpointError(f"checkpoint file size differs: {f.path} has {st.st_size} bytes, manifest says {f.size}")


_CHECKS = (_check_identity, _check_listing, _check_payload)


def verify_checkpoint(path) -> VerifiedCheckpoint:
    root = Path(path).resolve()
    marker, listing = root / COMPLETE_NAME, root / MANIFEST_NAME
    if not (marker.is_file() and listing.is_file()):
        raise CheckpointError(f"checkpoint is not complete: {root}")
    try:
        raw = listing.read_bytes()
        complete = json.loads(marker.read_bytes())
    except (OSError, json.JSONDecodeError) as exc:
        raise CheckpointError(f"checkpoint metadata is invalid: {root}") from exc
    if not isinstance(complete, Mapping):
        raise CheckpointError(f"checkpoint metadata is invalid: {root}")
    try:
        manifest = Manifest.from_bytes(raw)
    except json.JSONDecodeError as exc:
        raise CheckpointError(f"checkpoint metadata is invalid: {root}") from exc
    for check in _CHECKS:
        check(root, raw, complete, manifest)
    return VerifiedCheckpoint(root, manifest.step, manifest.contract, manifest.files, manifest.metadata,
                              Manifest.digest_of(raw))
