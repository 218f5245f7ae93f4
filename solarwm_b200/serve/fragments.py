"""Fragmented-MP4 preview delivery: split an encoder's byte stream into complete fragments, record them in an
append-only delivery trace, and serve them to clients that resume by cursor.

An encoder that writes fragmented MP4 to a pipe (``-movflags frag_keyframe+empty_moov+default_base_moof``) emits one
initialisation segment (``ftyp`` + ``moov``) followed by ``moof`` + ``mdat`` pairs.  The pipe delivers arbitrary byte
chunks, a browser's media source wants WHOLE fragments:

  ``FragmentSplitter``   incremental box parser: feed it chunks, it returns the complete segments they finished, each
                         fragment with the number of video samples its ``trun`` boxes declare;
  ``DeliveryTrace``      the producer's JSON-lines record next to the growing ``.part.mp4``: one row per fragment
                         (serial, byte offset, first frame, frame count, length) and one ``finish`` row;
  ``TraceIndex``         the consumer's view of that file: reads only what was appended since the last call, checks
                         that serials, offsets and frame numbers continue without a gap, keeps a bounded window in
                         memory and falls back to scanning the file for older cursors;
  ``MediaStore``         ``fragments(scene, sequence, cursor, limit)`` -> the rows and their bytes, from the part file
                         while the stream is live and from the final file afterwards; names are validated and symlinks
                         refused because the arguments come from HTTP clients.

Reference: deploy/solar_wm/shared/media/encoder.py:14-170 (splitting and tracing inside the preview writer),
deploy/solar_wm/shared/media/store.py:6-110 (trace index and store).
"""
from __future__ import annotations

import collections
import json
import re
import struct
import threading
from pathlib import Path
from typing import Iterator, List, Optional, Tuple

MAX_FRAGMENT_BYTES = 32 << 20
MAX_FRAGMENT_SAMPLES = 128


def iter_boxes(data: bytes) -> Iterator[Tuple[bytes, bytes]]:
    """(type, body) of every box in ``data``, which must hold whole boxes only."""
    pos = 0
    while pos < len(data):
        if len(data) - pos < 8:
            raise ValueError("truncated MP4 box header")
        size, kind = struct.unpack_from(">I4s", data, pos)
        if size < 8 or pos + size > len(data):
            raise ValueError("invalid MP4 box size")
        yield kind, data[pos + 8:pos + size]
        pos += size


def fragment_sample_count(moof: bytes) -> int:
    """Video samples declared by the ``trun`` boxes of one ``moof`` box (header included in ``moof``)."""
    count = 0
    for kind, body in iter_boxes(moof[8:]):
        if kind == b"traf":
            for k, b in iter_boxes(body):
                if k == b"trun":
                    count += struct.unpack_from(">I", b, 4)[0]          # version / flags, then sample_count
    if not 1 <= count <= MAX_FRAGMENT_SAMPLES:
        raise ValueError(f"unsupported fragment sample count {count}")
    return count


class FragmentSplitter:
    """``feed(chunk)`` -> list of ``("init", bytes, 0)`` / ``("fragment", bytes, samples)`` completed by the chunk."""

    def __init__(self):
        self.buffer = bytearray()
        self.init_done = False
        self._pending: List[bytes] = []            # boxes of the segment being assembled

    def feed(self, chunk: bytes) -> list:
        self.buffer += chunk
        out = []
        while len(self.buffer) >= 8:
            size, kind = struct.unpack_from(">I4s", self.buffer, 0)
            if size < 8 or size > MAX_FRAGMENT_BYTES:
                raise ValueError(f"invalid MP4 box size {size} for {kind!r}")
            if len(self.buffer) < size:
                break
            box = bytes(self.buffer[:size])
            del self.buffer[:size]
            self._pending.append(box)
            if not self.init_done:
                if kind == b"moov":
                    out.append(("init", b"".join(self._pending), 0))
                    self._pending, self.init_done = [], True
                elif kind not in (b"ftyp", b"free", b"styp"):
                    raise ValueError(f"unexpected {kind!r} box before the initialisation segment ended")
            elif kind == b"mdat":
                moofs = [b for b in self._pending if b[4:8] == b"moof"]
                if len(moofs) != 1:
                    raise ValueError("a media fragment needs exactly one moof before its mdat")
                out.append(("fragment", b"".join(self._pending), fragment_sample_count(moofs[0])))
                self._pending = []
            elif kind not in (b"moof", b"styp", b"free", b"sidx", b"mfra"):
                raise ValueError(f"unexpected {kind!r} box inside the fragment stream")
        return out

    def finish(self) -> None:
        if self.buffer or any(b[4:8] == b"moof" for b in self._pending):
            raise ValueError("the stream ended inside a fragment")


class DeliveryTrace:
    """Append-only record of what the producer wrote to the part file; one flushed line per event."""

    def __init__(self, path):
        self.path = Path(path)
        self.file = self.path.open("x", buffering=1)
        self.serial = self.offset = self.frames = 0
        self.lock = threading.Lock()

    def _row(self, **row) -> None:
        self.file.write(json.dumps(row, sort_keys=True) + "\n")

    def init(self, length: int) -> None:
        with self.lock:
            self._row(event="init", length=int(length))
            self.offset += int(length)

    def fragment(self, length: int, count: int) -> dict:
        with self.lock:
            row = dict(event="fragment", serial=self.serial, offset=self.offset, first=self.frames, count=int(count),
                       length=int(length))
            self._row(**row)
            self.serial += 1
            self.offset += int(length)
            self.frames += int(count)
            return row

    def finish(self, rc: int = 0, error: Optional[str] = None) -> None:
        with self.lock:
            self._row(event="finish", rc=int(rc), error=error, output_frames=self.frames)
            self.file.close()


class TraceIndex:
    def __init__(self, path, capacity: int = 8192):
        self.path, self.position = Path(path), 0
        self.rows = collections.deque(maxlen=capacity)
        self.serial = self.offset = self.frames = 0
        self.init_length = 0
        self.done = False
        self.lock = threading.Lock()

    def _check(self, row) -> None:
        if row["serial"] != self.serial or row["offset"] != self.offset or row["first"] != self.frames \
                or not 0 <= row["count"] <= MAX_FRAGMENT_SAMPLES or not 0 < row["length"] <= MAX_FRAGMENT_BYTES:
            raise ValueError("the delivery trace does not continue where it left off")

    def update(self) -> None:
        with self.path.open("rb") as src:
            src.seek(self.position)
            while True:
                line = src.readline(65537)
                if not line or not line.endswith(b"\n"):            # nothing new, or a row still being written
                    if len(line) > 65536:
                        raise ValueError("oversized trace row")
                    break
                row = json.loads(line)
                if row.get("event") == "init":
                    self.init_length = int(row["length"])
                    self.offset += self.init_length
                elif row.get("event") == "fragment":
                    self._check(row)
                    self.rows.append(row)
                    self.serial += 1
                    self.offset += row["length"]
                    self.frames += row["count"]
                elif row.get("event") == "finish":
                    if row.get("rc") != 0 or row.get("error") or row.get("output_frames") != self.frames:
                        raise ValueError("the encoder did not finish cleanly")
                    self.done = True
                self.position = src.tell()

    def batch(self, cursor: int, limit: int):
        """Rows ``cursor .. cursor + limit`` that exist so far, the number produced, and whether the stream is over."""
        with self.lock:
            self.update()
            if cursor > self.serial:
                raise ValueError("cursor beyond the produced fragments")
            if self.rows and cursor < self.rows[0]["serial"]:       # older than the window: scan the file
                rows = []
                with self.path.open("rb") as src:
                    for line in src:
                        if not line.endswith(b"\n"):
                            break
                        row = json.loads(line)
                        if row.get("event") == "fragment" and row["serial"] >= cursor:
                            rows.append(row)
                            if len(rows) == limit:
                                break
            else:
                rows = [r for r in self.rows if r["serial"] >= cursor][:limit]
            if rows and rows[0]["serial"] != cursor:
                raise ValueError("the requested fragment is missing from the trace")
            return rows, self.serial, self.done


class MediaStore:
    """Fragments of the live previews under ``root``; file stem ``<scene>-session-<sequence>-live``."""

    def __init__(self, root, keep_indices: int = 2):
        self.root = Path(root).resolve()
        self.indices: "collections.OrderedDict[str, TraceIndex]" = collections.OrderedDict()
        self.keep, self.lock = int(keep_indices), threading.Lock()

    @staticmethod
    def stem(scene: str, sequence: int) -> str:
        if not re.fullmatch(r"[A-Za-z0-9_-]{1,80}", scene):
            raise ValueError("invalid scene name")
        if not 1 <= int(sequence) <= 10 ** 9:
            raise ValueError("invalid sequence number")
        return f"{scene}-session-{int(sequence)}-live"

    def paths(self, scene: str, sequence: int):
        stem = self.stem(scene, sequence)
        return (self.root / f".{stem}.part.mp4", self.root / f"{stem}.mp4", self.root / f"{stem}.delivery.jsonl")

    def fragments(self, scene: str, sequence: int, cursor: int, limit: int = 16) -> dict:
        if not 0 <= int(cursor) <= 10 ** 12 or not 1 <= int(limit) <= 64:
            raise ValueError("invalid cursor or batch size")
        part, final, trace = self.paths(scene, sequence)
        if trace.is_symlink() or part.is_symlink() or final.is_symlink():
            raise ValueError("symlinked media files are refused")
        stem = self.stem(scene, sequence)
        with self.lock:
            index = self.indices.get(stem)
            if index is None:
                index = self.indices[stem] = TraceIndex(trace)
            self.indices.move_to_end(stem)
            while len(self.indices) > self.keep:
                self.indices.popitem(last=False)
        rows, produced, done = index.batch(int(cursor), int(limit))
        source = part if part.exists() else final
        blobs = []
        with source.open("rb") as fh:
            for row in rows:
                fh.seek(row["offset"])
                data = fh.read(row["length"])
                if len(data) != row["length"]:
                    raise ValueError("the media file is shorter than its trace")
                blobs.append(data)
        init = None
        if int(cursor) == 0 and index.init_length:
            with source.open("rb") as fh:
                init = fh.read(index.init_length)
        return {"rows": rows, "data": blobs, "init": init, "produced": produced, "done": done,
                "next_cursor": int(cursor) + len(rows)}


class FragmentedPreviewWriter:
    """Owns one live preview: bytes from the encoder go in through ``write`` (any chunking), whole segments land in
    the part file and in the trace; ``finish`` renames the part file to its final name."""

    def __init__(self, store: MediaStore, scene: str, sequence: int):
        self.part, self.final, trace = store.paths(scene, sequence)
        for p in (self.part, self.final, trace):
            if p.exists() or p.is_symlink():
                raise FileExistsError(p)
        self.part.parent.mkdir(parents=True, exist_ok=True)
        self.file = self.part.open("xb", buffering=0)
        self.trace, self.splitter = DeliveryTrace(trace), FragmentSplitter()

    def write(self, chunk: bytes) -> int:
        """Returns the number of fragments this chunk completed."""
        done = 0
        for kind, data, count in self.splitter.feed(chunk):
            self.file.write(data)
            if kind == "init":
                self.trace.init(len(data))
            else:
                self.trace.fragment(len(data), count)
                done += 1
        return done

    def finish(self, rc: int = 0, error: Optional[str] = None) -> None:
        try:
            if rc == 0 and error is None:
                self.splitter.finish()
        except ValueError as exc:
            rc, error = 1, str(exc)
        self.file.close()
        self.trace.finish(rc, error)
        if rc == 0 and error is None:
            self.part.rename(self.final)
