"""JSONL / JSONL.GZ dataset index.

One object per line with non-empty ``sample_id`` and ``key``, a relative POSIX ``shard`` path, an
integer ``epoch_repeats >= 1`` and free-form extra fields (``num_frames``, ``fps``, member names,
caption ...).  ``inventory`` gives the digests used to prove two runs read the same index
(reference: solar/data/index.py:77-313).
"""
from __future__ import annotations

import gzip
import hashlib
import json
from dataclasses import dataclass
from pathlib import Path, PurePosixPath
from typing import Any, Iterable, Iterator, Mapping, Sequence

from ..errors import DataContractError


def validate_relative_key(value) -> str:
    if not isinstance(value, str) or not value:
        raise DataContractError("shard must be a non-empty relative POSIX path")
    p = PurePosixPath(value)
    if p.is_absolute() or any(part in ("", ".", "..") for part in p.parts) or "\\" in value:
        raise DataContractError(f"shard path {value!r} is not a clean relative POSIX path")
    return value


@dataclass(frozen=True)
class IndexRow:
    ordinal: int
    sample_id: str
    key: str
    shard: str
    epoch_repeats: int
    values: Mapping[str, Any]

    @classmethod
    def from_mapping(cls, ordinal: int, values: Mapping[str, Any]) -> "IndexRow":
        if not isinstance(values, Mapping):
            raise DataContractError(f"index row {ordinal} is not an object")
        for name in ("sample_id", "key"):
            v = values.get(name)
            if not isinstance(v, str) or not v:
                raise DataContractError(f"index row {ordinal} {name} must be a non-empty string")
        reps = values.get("epoch_repeats", 1)
        if type(reps) is not int:
            raise DataContractError(f"index row {ordinal} epoch_repeats must be an integer")
        if reps < 1:
            raise DataContractError(f"index row {ordinal} epoch_repeats must be >= 1")
        return cls(ordinal, values["sample_id"], values["key"], validate_relative_key(values.get("shard")),
                   reps, dict(values))


@dataclass(frozen=True)
class IndexInventory:
    rows: int
    virtual_occurrences: int
    ordered_sample_id_digest: str
    ordered_row_digest: str
    decompressed_digest: str


def _open_text(path: Path):
    return gzip.open(path, "rb") if path.suffix == ".gz" else path.open("rb")


def iter_index(path) -> Iterator[IndexRow]:
    path = Path(path)
    ordinal = 0
    with _open_text(path) as handle:
        for line_no, raw in enumerate(handle, 1):
            if not raw.strip():
                continue
            try:
                obj = json.loads(raw)
            except json.JSONDecodeError as exc:
                raise DataContractError(f"{path}:{line_no}: invalid JSON: {exc}") from exc
            yield IndexRow.from_mapping(ordinal, obj)
            ordinal += 1


def read_index(path) -> tuple:
    rows = tuple(iter_index(path))
    if not rows:
        raise DataContractError(f"index {path} has no rows")
    seen = set()
    for r in rows:
        if r.sample_id in seen:
            raise DataContractError(f"duplicate sample_id {r.sample_id!r} in {path}")
        seen.add(r.sample_id)
    return rows


def inventory(path) -> IndexInventory:
    path = Path(path)
    ids, rows_h, raw_h = hashlib.blake2s(), hashlib.blake2s(), hashlib.blake2s()
    with _open_text(path) as handle:
        for chunk in iter(lambda: handle.read(1 << 20), b""):
            raw_h.update(chunk)
    n = occ = 0
    for row in iter_index(path):
        ids.update(row.sample_id.encode() + b"\n")
        rows_h.update(json.dumps(row.values, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode() + b"\n")
        n += 1
        occ += row.epoch_repeats
    return IndexInventory(n, occ, ids.hexdigest(), rows_h.hexdigest(), raw_h.hexdigest())


def assert_disjoint(a: Sequence[IndexRow], b: Sequence[IndexRow], what: str = "train/validation") -> None:
    overlap = {r.sample_id for r in a} & {r.sample_id for r in b}
    if overlap:
        raise DataContractError(f"{what} indexes share {len(overlap)} sample ids, e.g. {sorted(overlap)[:3]}")


def write_index(path, rows: Iterable[Mapping[str, Any]]) -> int:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    opener = gzip.open if path.suffix == ".gz" else open
    n = 0
    with opener(path, "wb") as handle:
        for i, row in enumerate(rows):
            IndexRow.from_mapping(i, row)
            handle.write(json.dumps(row, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode() + b"\n")
            n += 1
    return n
