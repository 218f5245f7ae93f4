"""Tar shard reader with an LRU of open shards (reference: solar/data/archive.py:21-150)."""
from __future__ import annotations

import tarfile
from collections import OrderedDict
from dataclasses import dataclass
from pathlib import Path
from typing import Mapping

from ..errors import DataContractError


@dataclass(frozen=True)
class RawSample:
    sample_id: str
    members: Mapping[str, bytes]


class TarShardReader:
    def __init__(self, max_open: int = 8):
        if max_open < 1:
            raise DataContractError("max_open must be positive")
        self.max_open = max_open
        self._open: "OrderedDict[str, tuple]" = OrderedDict()

    def _shard(self, path: Path):
        key = str(path)
        if key in self._open:
            self._open.move_to_end(key)
            return self._open[key]
        try:
            tf = tarfile.open(path, "r:*")
        except (OSError, tarfile.TarError) as exc:
            raise DataContractError(f"cannot open shard {path}: {exc}") from exc
        table = {m.name: m for m in tf.getmembers() if m.isfile()}
        self._open[key] = (tf, table)
        while len(self._open) > self.max_open:
            _, (old, _t) = self._open.popitem(last=False)
            old.close()
        return self._open[key]

    def read_members(self, shard_path, names) -> dict:
        tf, table = self._shard(Path(shard_path))
        out = {}
        for name in names:
            if name not in table:
                raise DataContractError(f"shard {shard_path} lacks member {name!r}")
            out[name] = tf.extractfile(table[name]).read()
        return out

    def read_sample(self, shard_path, sample_id: str, member_names: Mapping[str, str]) -> RawSample:
        blobs = self.read_members(shard_path, list(member_names.values()))
        return RawSample(sample_id, {k: blobs[v] for k, v in member_names.items()})

    def close(self) -> None:
        for tf, _ in self._open.values():
            tf.close()
        self._open.clear()
