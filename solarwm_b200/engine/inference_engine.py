"""Fixed-plan generation with atomic, create-only publication.

Every case is generated into a private ``.<name>.<uuid>.partial`` directory as
``slot-%06d/<artifact>`` + ``slot-%06d/manifest.json`` (schema ``solarwm.inference-sample.v1``);
then ``ordered-manifest.jsonl`` and ``COMPLETE.json`` are written and the directory is renamed to
its public name with RENAME_NOREPLACE -- a published result is never replaced, a concurrent
publisher loses with an error.  With ``collective_error`` set, ranks exchange their error text
after output setup, after every case wave and after the commit, so all ranks fail together
(ranks with fewer cases still take part in ``collective_case_waves`` exchanges).

Reference: solar/inference/engine.py:43-295.
"""
from __future__ import annotations

import hashlib
import stat
import uuid
from dataclasses import asdict, dataclass, field
from pathlib import Path, PurePosixPath
from typing import Any, Callable, Mapping, Optional, Protocol, Sequence, Union

from ..config.loader import canonical_json
from ..errors import BackendContractError
from ..runtime.create_only import link_file_create_only, publish_directory_no_replace, write_file_create_only

SAMPLE_SCHEMA = "solarwm.inference-sample.v1"
COMPLETE_SCHEMA = "solarwm.inference-complete.v1"


def _artifact_path(name: str) -> PurePosixPath:
    p = PurePosixPath(str(name))
    if not str(name) or p.is_absolute() or any(part in ("", ".", "..") for part in p.parts) or \
            p.name in ("manifest.json",):
        raise BackendContractError(f"invalid generated artifact name {name!r}")
    return p


@dataclass(frozen=True)
class InferenceCase:
    slot: int
    sample_id: str
    prompt: str
    start_frame: int
    noise_seed: int
    camera_fingerprint: str
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.slot < 0 or self.start_frame < 0 or self.noise_seed < 0:
            raise BackendContractError("inference slot/start/noise values must be non-negative")
        if not self.sample_id or not self.camera_fingerprint:
            raise BackendContractError("inference case lacks sample/camera identity")


@dataclass(frozen=True)
class GeneratedFile:
    """An artifact that already sits on the output filesystem (large videos are never held in memory);
    it is published with a hard link and the private name is then removed."""

    path: Path
    delete_after_publish: bool = True

    def __post_init__(self):
        p = Path(self.path).expanduser()
        try:
            mode = p.lstat().st_mode
        except OSError as exc:
            raise BackendContractError(f"generated file is not readable: {p}: {exc}") from exc
        if not stat.S_ISREG(mode) or p.is_symlink():
            raise BackendContractError(f"generated file must be a regular non-symlink file: {p}")
        object.__setattr__(self, "path", p.resolve())


@dataclass(frozen=True)
class GeneratedSample:
    artifacts: Mapping[str, Union[bytes, GeneratedFile]]
    shape: tuple
    dtype: str
    metrics: Mapping[str, float] = field(default_factory=dict)
    provenance: Mapping[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if not self.artifacts or not self.shape or not self.dtype:
            raise BackendContractError("generated sample lacks artifacts/shape/dtype")
        seen = []
        for name, value in self.artifacts.items():
            p = _artifact_path(name)
            if not isinstance(value, (bytes, GeneratedFile)):
                raise BackendContractError(f"invalid generated artifact {name!r}")
            if any(p == q or p in q.parents or q in p.parents for q in seen):
                raise BackendContractError(f"generated artifact paths collide: {name!r}")
            seen.append(p)


class InferenceAdapter(Protocol):
    family: str

    def generate(self, case: InferenceCase, *, weights_id: str) -> GeneratedSample: ...


@dataclass(frozen=True)
class InferenceSummary:
    output_dir: Path
    weights_id: str
    cases: int
    ordered_manifest_digest: str


def _digest_file(path: Path):
    h, size = hashlib.blake2s(), 0
    try:
        with path.open("rb") as f:
            for chunk in iter(lambda: f.read(1 << 20), b""):
                size += len(chunk)
                h.update(chunk)
    except OSError as exc:
        raise BackendContractError(f"cannot read generated file {path}: {exc}") from exc
    return size, h.hexdigest()


def _create(path: Path, data: bytes) -> None:
    try:
        write_file_create_only(path, data)
    except OSError as exc:
        raise BackendContractError(f"inference output file {path.name}: {exc}") from exc


def _publish_artifact(dest: Path, name: str, value: Union[bytes, GeneratedFile]):
    """Put one artifact at ``dest`` (bytes are written create-only, files are hard-linked); returns (size, digest)."""
    if isinstance(value, GeneratedFile):
        size, digest = _digest_file(value.path)
        try:
            link_file_create_only(value.path, dest)
        except OSError as exc:
            raise BackendContractError(f"inference generated file {name}: {exc}") from exc
        return size, digest
    _create(dest, value)
    return len(value), hashlib.blake2s(value).hexdigest()


class _Together:
    """Runs the phases of a publication so that every rank learns of any rank's failure before the next phase: the
    phase body runs (or is skipped on ranks that have nothing to do in it), its error text -- or None -- goes through
    the ``exchange`` callable, which raises on every rank when any rank failed, and a local failure is raised here."""

    def __init__(self, exchange: Optional[Callable[[Optional[str], str], None]]):
        self.exchange = exchange or (lambda err, phase: None)

    def phase(self, label: str, body: Callable[[], Any], *, active: bool = True):
        result, error = None, None
        if active:
            try:
                result = body()
            except Exception as exc:  # noqa: BLE001 - only the text crosses ranks
                error = f"{type(exc).__name__}: {exc}"
        self.exchange(error, label)
        if error is not None:
            raise BackendContractError(f"inference {label} failed: {error}")
        return result


class InferenceEngine:
    def __init__(self, adapter: InferenceAdapter):
        self.adapter = adapter

    # -- one case -------------------------------------------------------------------------------------------------
    def _emit_case(self, staging: Path, case: InferenceCase, weights_id: str) -> dict:
        sample = self.adapter.generate(case, weights_id=weights_id)
        try:
            slot = f"slot-{case.slot:06d}"
            folder = staging / slot
            folder.mkdir()
            listing = []
            for name in sorted(sample.artifacts):
                size, digest = _publish_artifact(folder / name, name, sample.artifacts[name])
                listing.append({"path": f"{slot}/{name}", "bytes": size, "digest": digest})
            manifest = {"schema": SAMPLE_SCHEMA, "family": self.adapter.family, "weights_id": weights_id,
                        "case": asdict(case), "shape": list(sample.shape), "dtype": sample.dtype,
                        "metrics": dict(sample.metrics), "provenance": dict(sample.provenance), "artifacts": listing}
            _create(folder / "manifest.json", canonical_json(manifest))
            return manifest
        finally:
            for value in sample.artifacts.values():            # private names of linked files go away either way
                if isinstance(value, GeneratedFile) and value.delete_after_publish:
                    value.path.unlink(missing_ok=True)

    # -- the plan -------------------------------------------------------------------------------------------------
    @staticmethod
    def _check_plan(cases: Sequence[InferenceCase], weights_id: str, collective_case_waves: Optional[int]) -> int:
        if not weights_id:
            raise BackendContractError("inference requires a stable weights_id")
        if not cases and collective_case_waves is None:
            raise BackendContractError("inference requires cases")
        if len({c.slot for c in cases}) != len(cases):
            raise BackendContractError("inference case slots are duplicated")
        waves = len(cases) if collective_case_waves is None else int(collective_case_waves)
        if waves < 1:
            raise BackendContractError("inference collective case waves must be positive")
        if waves < len(cases):
            raise BackendContractError("inference collective case waves are shorter than local cases")
        return waves

    @staticmethod
    def _open_staging(target: Path) -> Path:
        if target.exists():
            raise BackendContractError(f"inference output already exists: {target}")
        target.parent.mkdir(parents=True, exist_ok=True)
        staging = target.with_name(f".{target.name}.{uuid.uuid4().hex}.partial")
        staging.mkdir()
        return staging

    def _seal(self, staging: Path, target: Path, manifests: Sequence[dict], weights_id: str) -> str:
        ordered = b"".join(canonical_json(m) for m in manifests)
        digest = hashlib.blake2s(ordered).hexdigest()
        _create(staging / "ordered-manifest.jsonl", ordered)
        _create(staging / "COMPLETE.json", canonical_json({
            "schema": COMPLETE_SCHEMA, "family": self.adapter.family, "weights_id": weights_id,
            "cases": len(manifests), "ordered_manifest_digest": digest}))
        publish_directory_no_replace(staging, target)
        return digest

    def run(self, cases: Sequence[InferenceCase], *, weights_id: str, output_dir,
            collective_error: Optional[Callable[[Optional[str], str], None]] = None,
            collective_case_waves: Optional[int] = None) -> InferenceSummary:
        """Generate ``cases`` in order and publish them as one directory.  With ``collective_error`` every rank takes
        part in ``collective_case_waves`` exchanges (ranks with fewer cases idle through the extra waves)."""
        waves = self._check_plan(cases, weights_id, collective_case_waves)
        together = _Together(collective_error)
        target = Path(output_dir).resolve()
        staging = together.phase("output setup", lambda: self._open_staging(target))
        manifests = []
        for wave in range(waves):
            mine = wave < len(cases)
            manifest = together.phase(f"case wave {wave}", lambda: self._emit_case(staging, cases[wave], weights_id),
                                      active=mine)
            if mine:
                manifests.append(manifest)
        digest = together.phase("partition commit", lambda: self._seal(staging, target, manifests, weights_id))
        return InferenceSummary(target, weights_id, len(cases), digest)


def run_validation(adapter: InferenceAdapter, cases, *, weights_id: str, output_dir) -> InferenceSummary:
    """Training-time validation is inference under another name."""
    return InferenceEngine(adapter).run(cases, weights_id=weights_id, output_dir=output_dir)
