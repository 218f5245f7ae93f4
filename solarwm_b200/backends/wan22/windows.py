"""Fixed training windows of the Wan corpora: start-frame rules and the 153-frame window index.

Two things live here.

*Start-frame rules* (pure arithmetic, part of the data contract -- a pre-encoded latent is only valid for the
window these rules give; reference: solar/backends/wan22/windows.py:55-107):

  81 frames   a clip of ``n`` frames carries ``max(1, (n - 1 + 40) // 80)`` windows, evenly spaced with both ends
              included (a single window is centred);
  153 frames  clips of the three long-form datasets carry six evenly spaced windows; every other clip carries one
              window whose start is a keyed hash of its identity modulo the number of admissible starts.

*The window index* (``write_window_index``, ``solar data materialize-wan153f``): the released "authority" indexes name
every window (``<source id>/latent-153f-wNN`` with its 153 contiguous frame indices); the raw indexes describe the
clips.  Joining them gives one gzip JSONL row per window that carries the raw row's fields plus the window geometry,
which is what ``solar preencode`` reads.  The join is strict: roles must agree, every clip must receive exactly its
expected window ordinals, long-form starts must equal the rule above, nothing may already be materialised, and the
output is created exactly once (hard-link commit).  The implementation holds the raw rows in a dictionary keyed by
sample id and marks ordinals in a per-clip bit set; output bytes are canonical JSON in authority order, gzip level 9
with a zero time stamp, so equal inputs give equal files.
"""
from __future__ import annotations

import gzip
import hashlib
import json
import os
import re
import uuid
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterable, Mapping, Tuple

from ...data.index import IndexRow, iter_index
from ...errors import DataContractError

FRAMES_81, FRAMES_153 = 81, 153
HASH_NAMESPACE_153 = "solarwm-latent-153f-v1"
LONG_FORM_DATASETS = frozenset({"abot", "miradata", "sekai_game"})
_WINDOW_ID = re.compile(r"^(?P<source>.+)/latent-153f-w(?P<ordinal>[0-9]{2})$")
_WINDOW_FIELDS = ("source_sample_id", "source_dataset", "window_index", "window_count", "start_frame",
                  "source_frame_indices")


# ---------------------------------------------------------------------------------------------------------------------
# start-frame rules
# ---------------------------------------------------------------------------------------------------------------------
def _ordinal_and_count(meta: Mapping[str, Any], what: str) -> Tuple[int, int]:
    try:
        return int(meta["window_index"]), int(meta["window_count"])
    except (KeyError, TypeError, ValueError) as exc:
        raise DataContractError(f"{what} preencoding window metadata is incomplete") from exc


def window_count_81f(num_frames: int) -> int:
    if num_frames < FRAMES_81:
        raise DataContractError("81f preencoding source is shorter than 81 frames")
    return max(1, (int(num_frames) + 39) // 80)


def window_start_81f(meta: Mapping[str, Any], num_frames: int) -> int:
    ordinal, count = _ordinal_and_count(meta, "81f")
    want = window_count_81f(num_frames)
    if count != want or not 0 <= ordinal < count:
        raise DataContractError(f"81f source requires {want} window ordinals, got index={ordinal} count={count}")
    room = int(num_frames) - FRAMES_81
    if count == 1:
        return room // 2
    # round(ordinal * room / (count - 1)) with halves rounded up, in integers
    return (2 * ordinal * room + (count - 1)) // (2 * (count - 1))


def windows_per_clip_153f(dataset: str) -> int:
    return 6 if dataset in LONG_FORM_DATASETS else 1


def window_start_153f(meta: Mapping[str, Any], num_frames: int) -> int:
    try:
        source, dataset = str(meta["source_sample_id"]), str(meta["source_dataset"])
    except KeyError as exc:
        raise DataContractError("153f preencoding window metadata is incomplete") from exc
    ordinal, count = _ordinal_and_count(meta, "153f")
    if num_frames < FRAMES_153:
        raise DataContractError("153f preencoding source is shorter than 153 frames")
    room = int(num_frames) - FRAMES_153
    if dataset in LONG_FORM_DATASETS:
        if count != 6 or not 0 <= ordinal < 6:
            raise DataContractError("long-form 153f source must carry six valid window ordinals")
        return (ordinal * room + 2) // 5
    if (ordinal, count) != (0, 1):
        raise DataContractError("ordinary 153f source must carry exactly one window")
    namespace = str(meta.get("window_hash_namespace", HASH_NAMESPACE_153))
    digest = hashlib.blake2b(f"{namespace}\0{source}".encode(), digest_size=8).digest()
    return int.from_bytes(digest, "little") % (room + 1)


# ---------------------------------------------------------------------------------------------------------------------
# the join
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class WindowIndexSummary:
    output: Path
    train_sources: int
    test_sources: int
    train_windows: int
    test_windows: int
    decompressed_sha256: str
    compressed_sha256: str

    def as_dict(self) -> Dict[str, Any]:
        return {"schema": "solarwm.wan22-153f-window-index.v1", "output": str(self.output),
                "train_sources": self.train_sources, "test_sources": self.test_sources,
                "train_windows": self.train_windows, "test_windows": self.test_windows,
                "total_windows": self.train_windows + self.test_windows, "window_hash_namespace": HASH_NAMESPACE_153,
                "decompressed_sha256": self.decompressed_sha256, "compressed_sha256": self.compressed_sha256}


@dataclass
class _Clip:
    role: str
    row: IndexRow
    dataset: str
    num_frames: int
    expected: int                  # bit set of the ordinals this clip must receive
    seen: int = 0


def _declared_role(row: IndexRow) -> set:
    found = set()
    for name in ("split", "role", "recipe_role"):
        value = row.values.get(name)
        if value in (None, ""):
            continue
        if not isinstance(value, str):
            raise DataContractError(f"source row {row.sample_id!r} field {name!r} must be a string")
        found.add(value.strip().lower())
    return found


def _clip_from_raw(row: IndexRow, role: str) -> _Clip:
    if _declared_role(row) != {role}:
        raise DataContractError(f"source row {row.sample_id!r} must declare only role {role!r}, got "
                                f"{sorted(_declared_role(row))}")
    if row.sample_id.rsplit("/", 1)[-1].startswith("latent-153f-w") or any(f in row.values for f in _WINDOW_FIELDS):
        raise DataContractError(f"source row {row.sample_id!r} is already window-materialized")
    dataset = str(row.values.get("dataset") or "").strip().lower()
    if not dataset:
        raise DataContractError(f"source row {row.sample_id!r} lacks dataset")
    if dataset not in row.sample_id.split("/")[:2]:
        raise DataContractError(f"source row {row.sample_id!r} does not contain dataset {dataset!r} in its identity")
    manifest = row.values.get("manifest")
    video = manifest.get("video", {}) if isinstance(manifest, Mapping) else {}
    try:
        frames = int(row.values.get("num_frames") or video["num_frames"])
    except (KeyError, TypeError, ValueError) as exc:
        raise DataContractError(f"source row {row.sample_id!r} lacks num_frames") from exc
    if frames < FRAMES_153:
        raise DataContractError(f"source row {row.sample_id!r} has {frames} frames, needs at least 153")
    return _Clip(role, row, dataset, frames, (1 << windows_per_clip_153f(dataset)) - 1)


def _shard_identity(row: IndexRow):
    return tuple(row.values.get(k) for k in ("shard_size", "shard_sha256", "shard_generation"))


@dataclass
class WindowJoin:
    """Raw clips by sample id; ``window_row`` turns one authority row into its materialised row."""

    clips: Dict[str, _Clip] = field(default_factory=dict)
    _shards: Dict[str, Any] = field(default_factory=dict)
    _windows: set = field(default_factory=set)

    def add_sources(self, rows: Iterable[IndexRow], role: str) -> int:
        n = 0
        for row in rows:
            if row.sample_id in self.clips:
                raise DataContractError(f"duplicate or train/test-overlapping source sample_id: {row.sample_id!r}")
            ident = _shard_identity(row)
            if self._shards.setdefault(row.shard, ident) != ident:
                raise DataContractError(f"shard identity drift inside source indexes: {row.shard}")
            self.clips[row.sample_id] = _clip_from_raw(row, role)
            n += 1
        if n == 0:
            raise DataContractError(f"empty {role} index")
        return n

    def window_row(self, authority: IndexRow, role: str) -> Dict[str, Any]:
        if authority.sample_id in self._windows:
            raise DataContractError(f"duplicate window authority sample_id: {authority.sample_id!r}")
        self._windows.add(authority.sample_id)
        m = _WINDOW_ID.fullmatch(authority.sample_id)
        if m is None:
            raise DataContractError(f"window authority sample_id must end in /latent-153f-wNN: {authority.sample_id!r}")
        source, ordinal = m.group("source"), int(m.group("ordinal"))
        try:
            start = int(authority.values["start_frame"])
            frames = [int(v) for v in authority.values["source_frame_indices"]]
        except (KeyError, TypeError, ValueError) as exc:
            raise DataContractError(f"window authority row {authority.sample_id!r} lacks fixed frame geometry") from exc
        if frames != list(range(start, start + FRAMES_153)):
            raise DataContractError(f"window authority row {authority.sample_id!r} is not one contiguous 153f window")
        clip = self.clips.get(source)
        if clip is None:
            raise DataContractError(f"window authority source is absent from raw indexes: {source!r}")
        if clip.role != role:
            raise DataContractError(f"window authority role {role!r} differs from raw role {clip.role!r} for {source!r}")
        count = windows_per_clip_153f(clip.dataset)
        if not 0 <= ordinal < count:
            raise DataContractError(f"window authority row {authority.sample_id!r} has an invalid ordinal")
        if start < 0 or start + FRAMES_153 > clip.num_frames:
            raise DataContractError(f"window authority row {authority.sample_id!r} lies outside {clip.num_frames} frames")
        want_key = f"{clip.row.key}__latent153f_w{ordinal:02d}"
        if authority.key != want_key:
            raise DataContractError(f"window authority key {authority.key!r} != expected {want_key!r}")
        geometry = {"source_sample_id": source, "source_dataset": clip.dataset, "window_index": ordinal,
                    "window_count": count}
        if clip.dataset in LONG_FORM_DATASETS:
            rule = window_start_153f(geometry, clip.num_frames)
            if start != rule:
                raise DataContractError(f"long-form authority start {start} != expected {rule} for {authority.sample_id!r}")
        bit = 1 << ordinal
        if clip.seen & bit:
            raise DataContractError(f"duplicate window ordinal {ordinal} for source {source!r}")
        clip.seen |= bit
        out = dict(clip.row.values)
        out.update(geometry, sample_id=authority.sample_id, key=authority.key, epoch_repeats=1, split=role,
                   window_hash_namespace=HASH_NAMESPACE_153, start_frame=start, source_frame_indices=frames)
        return out

    def first_incomplete(self):
        return next((sid for sid, c in self.clips.items() if c.seen != c.expected), None)


def write_window_index(train_index, test_index, train_window_index, test_window_index, output) -> WindowIndexSummary:
    """Join the released window authority to the raw clip rows; create ``output`` (``.jsonl.gz``) exactly once."""
    target = Path(output).expanduser().resolve()
    if target.exists():
        raise DataContractError(f"window index output already exists: {target}")
    target.parent.mkdir(parents=True, exist_ok=True)
    staging = target.with_name(f".{target.name}.{uuid.uuid4().hex}.partial")
    join = WindowJoin()
    sources = {"train": join.add_sources(iter_index(train_index), "train"),
               "test": join.add_sources(iter_index(test_index), "test")}
    windows = {"train": 0, "test": 0}
    plain = hashlib.sha256()
    try:
        with staging.open("xb") as raw:
            with gzip.GzipFile(filename="", mode="wb", fileobj=raw, compresslevel=9, mtime=0) as gz:
                for path, role in ((train_window_index, "train"), (test_window_index, "test")):
                    for authority in iter_index(path):
                        line = (json.dumps(join.window_row(authority, role), allow_nan=False, ensure_ascii=False,
                                           separators=(",", ":"), sort_keys=True) + "\n").encode("utf-8")
                        plain.update(line)
                        gz.write(line)
                        windows[role] += 1
                    if windows[role] == 0:
                        raise DataContractError(f"empty {role} window authority index: {Path(path)}")
            missing = join.first_incomplete()
            if missing is not None:
                raise DataContractError(f"raw source lacks complete window authority: {missing!r}")
            raw.flush()
            os.fsync(raw.fileno())
        packed = hashlib.sha256()
        with staging.open("rb") as handle:
            for block in iter(lambda: handle.read(8 << 20), b""):
                packed.update(block)
        try:
            os.link(staging, target)                   # create-only commit: fails if the name appeared meanwhile
        except FileExistsError as exc:
            raise DataContractError(f"window index output already exists: {target}") from exc
        return WindowIndexSummary(target, sources["train"], sources["test"], windows["train"], windows["test"],
                                  plain.hexdigest(), packed.hexdigest())
    finally:
        staging.unlink(missing_ok=True)
