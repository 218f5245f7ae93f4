"""Shard transport: ``LocalResolver`` maps a shard key to a file under an absolute root;
``CachedRemoteResolver`` stages remote objects (``gs://`` through an injected downloader) into a
local cache with per-object flock, size receipts and LRU eviction, so concurrent readers on a node
download each shard once.  ``resolver_from_config`` picks one from ``data.transport``
(reference: solar/data/transport.py:47-623; the network downloader itself is injected because
this package makes no outbound connections on its own)."""
from __future__ import annotations

import fcntl
import json
import os
import time
from pathlib import Path
from typing import Callable, Mapping, Optional

from ..errors import DataContractError
from .index import validate_relative_key


class LocalResolver:
    def __init__(self, root):
        self.root = Path(str(root)).expanduser()
        if not self.root.is_absolute():
            raise DataContractError("local data.transport.root must be absolute")

    def resolve(self, shard_key: str, expected_size: Optional[int] = None) -> Path:
        path = self.root / validate_relative_key(shard_key)
        if not path.is_file():
            raise DataContractError(f"shard is missing: {path}")
        if expected_size is not None and path.stat().st_size != int(expected_size):
            raise DataContractError(f"shard size differs from the index: {path}")
        return path


class CachedRemoteResolver:
    def __init__(self, base_uri: str, cache_dir, downloader: Callable[[str, Path], None], max_cache_bytes: int = 0):
        self.base_uri = base_uri.rstrip("/")
        self.cache = Path(cache_dir)
        self.cache.mkdir(parents=True, exist_ok=True)
        self.downloader = downloader
        self.max_cache_bytes = int(max_cache_bytes)

    def _receipt(self, path: Path) -> Path:
        return path.with_name(path.name + ".receipt.json")

    def resolve(self, shard_key: str, expected_size: Optional[int] = None) -> Path:
        key = validate_relative_key(shard_key)
        dest = self.cache / key
        dest.parent.mkdir(parents=True, exist_ok=True)
        lock = os.open(dest.with_name(dest.name + ".lock"), os.O_CREAT | os.O_RDWR, 0o644)
        try:
            fcntl.flock(lock, fcntl.LOCK_EX)
            rec = self._receipt(dest)
            if dest.is_file() and rec.is_file():
                info = json.loads(rec.read_text())
                if info.get("size") == dest.stat().st_size and (expected_size is None or info["size"] == int(expected_size)):
                    os.utime(dest)
                    return dest
            tmp = dest.with_name(dest.name + f".{os.getpid()}.part")
            try:
                self.downloader(f"{self.base_uri}/{key}", tmp)
                size = tmp.stat().st_size
                if expected_size is not None and size != int(expected_size):
                    raise DataContractError(f"downloaded shard {key} has {size} bytes, index says {expected_size}")
                os.replace(tmp, dest)
            finally:
                tmp.unlink(missing_ok=True)
            rec.write_text(json.dumps({"size": size, "uri": f"{self.base_uri}/{key}", "time": time.time()}))
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
            os.close(lock)
        self._evict(keep=dest)
        return dest

    def _evict(self, keep: Path) -> None:
        if self.max_cache_bytes <= 0:
            return
        files = [p for p in self.cache.rglob("*") if p.is_file() and not p.name.endswith((".lock", ".receipt.json", ".part"))]
        total = sum(p.stat().st_size for p in files)
        for p in sorted(files, key=lambda q: q.stat().st_mtime):
            if total <= self.max_cache_bytes:
                break
            if p == keep:
                continue
            total -= p.stat().st_size
            p.unlink(missing_ok=True)
            self._receipt(p).unlink(missing_ok=True)

    def reap_orphans(self, older_than_s: float = 3600.0) -> int:
        n, now = 0, time.time()
        for p in self.cache.rglob("*.part"):
            if now - p.stat().st_mtime > older_than_s:
                p.unlink(missing_ok=True)
                n += 1
        return n


def resolver_from_config(data_config: Mapping, downloader: Optional[Callable[[str, Path], None]] = None):
    transport = data_config.get("transport")
    if not isinstance(transport, Mapping):
        raise DataContractError("data.transport must be a mapping")
    kind = str(transport.get("kind") or "").strip().lower()
    root = str(transport.get("root") or "")
    if kind == "local" or (not kind and root.startswith("/")):
        return LocalResolver(root)
    if root.startswith("gs://") or kind in ("gcs", "bucket"):
        if downloader is None:
            raise DataContractError("bucket transport needs a downloader (no network access from this package)")
        cache = data_config.get("cache_dir")
        if not cache:
            raise DataContractError("bucket transport requires data.cache_dir")
        return CachedRemoteResolver(root, cache, downloader, int(transport.get("max_cache_bytes", 0)))
    raise DataContractError(f"unknown data.transport kind {kind!r}")
