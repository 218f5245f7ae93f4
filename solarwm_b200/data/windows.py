"""Window index over long clips: every fixed-length training window of every clip, queryable by rank.

A pre-encoded clip of ``F`` latent frames yields windows ``[start, start + window)`` at a fixed stride;
the index is one SQLite file (``windows`` table: clip id, shard, start, length, ordinal) written inside a
transaction and published by rename, so readers never see a partial index.  ``WindowIndex.slice(rank,
world)`` gives the deterministic ``ordinal % world == rank`` share (reference: 153-frame window index,
solar/backends/wan22/runtime/windows.py:388).
"""
from __future__ import annotations

import os
import sqlite3
from pathlib import Path
from typing import Iterable, Iterator, Mapping, NamedTuple

from ..errors import DataContractError


class Window(NamedTuple):
    ordinal: int
    clip_id: str
    shard: str
    start: int
    length: int


def enumerate_windows(clip_frames: int, window: int, stride: int) -> Iterator[int]:
    if window < 1 or stride < 1:
        raise DataContractError("window and stride must be positive")
    start = 0
    while start + window <= clip_frames:
        yield start
        start += stride


def build_index(path, clips: Iterable[Mapping[str, object]], *, window: int, stride: int) -> int:
    """clips: rows with ``sample_id``, ``shard`` and ``num_frames``.  Returns the number of windows written."""
    path = Path(path)
    if path.exists():
        raise DataContractError(f"window index already exists: {path}")
    tmp = path.with_name(f".{path.name}.{os.getpid()}.partial")
    con = sqlite3.connect(tmp)
    n = 0
    try:
        with con:
            con.execute("CREATE TABLE meta (key TEXT PRIMARY KEY, value TEXT)")
            con.execute("CREATE TABLE windows (ordinal INTEGER PRIMARY KEY, clip_id TEXT NOT NULL, shard TEXT NOT NULL, "
                        "start INTEGER NOT NULL, length INTEGER NOT NULL)")
            seen = set()
            for clip in clips:
                cid = str(clip["sample_id"])
                if cid in seen:
                    raise DataContractError(f"duplicate clip id {cid!r}")
                seen.add(cid)
                for start in enumerate_windows(int(clip["num_frames"]), window, stride):
                    con.execute("INSERT INTO windows VALUES (?, ?, ?, ?, ?)", (n, cid, str(clip["shard"]), start, window))
                    n += 1
            con.executemany("INSERT INTO meta VALUES (?, ?)", [("window", str(window)), ("stride", str(stride)),
                                                               ("count", str(n)), ("schema", "solarwm.window-index.v1")])
    finally:
        con.close()
    if n == 0:
        tmp.unlink()
        raise DataContractError("no clip is long enough for one window")
    os.replace(tmp, path)
    return n


class WindowIndex:
    def __init__(self, path):
        self.con = sqlite3.connect(f"file:{Path(path)}?mode=ro", uri=True)
        meta = dict(self.con.execute("SELECT key, value FROM meta"))
        if meta.get("schema") != "solarwm.window-index.v1":
            raise DataContractError("not a window index of this framework")
        self.window, self.stride, self.count = int(meta["window"]), int(meta["stride"]), int(meta["count"])

    def __len__(self) -> int:
        return self.count

    def __getitem__(self, ordinal: int) -> Window:
        row = self.con.execute("SELECT * FROM windows WHERE ordinal = ?", (int(ordinal),)).fetchone()
        if row is None:
            raise IndexError(ordinal)
        return Window(*row)

    def slice(self, rank: int, world: int) -> Iterator[Window]:
        for row in self.con.execute("SELECT * FROM windows WHERE ordinal % ? = ? ORDER BY ordinal", (world, rank)):
            yield Window(*row)

    def close(self) -> None:
        self.con.close()
