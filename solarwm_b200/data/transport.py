"""Shard transport: ``LocalResolver`` maps a shard key to a file under an absolute root;
``CachedRemoteResolver`` stages remote objects (``gs://`` through an injected downloader) into a
local cache with per-object flock, size receipts and LRU eviction, so concurrent readers on a node
download each shard once.  ``resolver_from_config`` picks one from ``data.transport``
(reference: solar/data/transport.py:47-623).  ``GCSRestDownloader`` is the stdlib downloader for ``gs://`` objects
(JSON API ``alt=media``, bearer token from ``TokenProvider``: a token file, ``GOOGLE_OAUTH_ACCESS_TOKEN`` or the
metadata server): bounded by a deadline, retries transient failures with capped exponential back-off, gives
authorisation failures a longer budget (tokens rotate) and never retries other 4xx answers.  Its URL opener, clock
and sleep are injectable, which is how it is tested without a network."""
from __future__ import annotations

import fcntl
import json
import os
import time
from pathlib import Path
from typing import Callable, Mapping, Optional

from ..errors import DataContractError
from .index import validate_relative_key


class DownloadTimeout(DataContractError):
    """A transfer did not finish inside its time budget (transient: the caller may try again later)."""


def parse_gs_uri(uri: str):
    if not uri.startswith("gs://"):
        raise DataContractError(f"not a gs:// uri: {uri!r}")
    bucket, _, name = uri[5:].partition("/")
    if not bucket or not name:
        raise DataContractError(f"gs:// uri needs a bucket and an object name: {uri!r}")
    return bucket, name


def is_transient(exc: Optional[BaseException]) -> bool:
    """Worth retrying: time-outs, connection failures, short reads, 408 / 429 / 5xx; never other 4xx answers."""
    import http.client
    import urllib.error

    while exc is not None:
        if isinstance(exc, urllib.error.HTTPError):
            return exc.code in (408, 429) or exc.code >= 500
        if isinstance(exc, (TimeoutError, ConnectionError, http.client.IncompleteRead, urllib.error.URLError, OSError)):
            return True
        exc = exc.__cause__
    return False


class TokenProvider:
    """Bearer token for bucket reads: ``token_file`` if it holds one, else ``GOOGLE_OAUTH_ACCESS_TOKEN``, else the
    instance metadata server (reference: GoogleTokenProvider, solar/data/transport.py:134-163)."""

    METADATA_URL = "http://metadata.google.internal/computeMetadata/v1/instance/service-accounts/default/token"

    def __init__(self, token_file=None, opener=None, environ=None):
        self.token_file = None if token_file is None else Path(token_file)
        self.opener, self.environ = opener, os.environ if environ is None else environ

    def __call__(self) -> str:
        import urllib.request

        if self.token_file is not None and self.token_file.is_file():
            text = self.token_file.read_text().strip()
            if text:
                return text
        text = str(self.environ.get("GOOGLE_OAUTH_ACCESS_TOKEN", "")).strip()
        if text:
            return text
        request = urllib.request.Request(self.METADATA_URL, headers={"Metadata-Flavor": "Google"})
        try:
            with (self.opener or urllib.request.urlopen)(request, timeout=10) as response:
                token = str(json.load(response).get("access_token") or "")
        except (OSError, ValueError) as exc:
            raise DataContractError("no access token: give a token file, GOOGLE_OAUTH_ACCESS_TOKEN or run where the "
                                    "metadata server answers") from exc
        if not token:
            raise DataContractError("the metadata server returned an empty access token")
        return token


class GCSRestDownloader:
    """``downloader(uri, path)`` for ``CachedRemoteResolver`` (reference: GCSRestDownloader,
    solar/data/transport.py:166-265)."""

    def __init__(self, token: Optional[Callable[[], str]] = None, *, socket_timeout_s: float = 120.0,
                 time_budget_s: float = 300.0, attempts: int = 12, auth_attempts: int = 72,
                 chunk_bytes: int = 16 << 20, opener=None, sleep=time.sleep, clock=time.monotonic):
        if min(socket_timeout_s, time_budget_s) <= 0 or min(attempts, auth_attempts, chunk_bytes) < 1:
            raise DataContractError("downloader limits must be positive")
        self.token = token or TokenProvider()
        self.socket_timeout_s, self.time_budget_s = float(socket_timeout_s), float(time_budget_s)
        self.attempts, self.auth_attempts, self.chunk_bytes = int(attempts), int(auth_attempts), int(chunk_bytes)
        self.opener, self.sleep, self.clock = opener, sleep, clock

    @staticmethod
    def media_url(uri: str) -> str:
        import urllib.parse

        bucket, name = parse_gs_uri(uri)
        return (f"https://storage.googleapis.com/download/storage/v1/b/{urllib.parse.quote(bucket, safe='')}/o/"
                f"{urllib.parse.quote(name, safe='')}?alt=media")

    def __call__(self, uri: str, path, deadline: Optional[float] = None) -> int:
        import urllib.error
        import urllib.request

        url, start = self.media_url(uri), self.clock()
        deadline = start + self.time_budget_s if deadline is None else min(float(deadline), start + self.time_budget_s)
        opener = self.opener or urllib.request.urlopen
        last, auth_seen = None, False
        for attempt in range(max(self.attempts, self.auth_attempts)):
            left = deadline - self.clock()
            if left <= 0:
                raise DownloadTimeout(f"{uri}: time budget used up after {attempt} attempt(s)") from last
            try:
                request = urllib.request.Request(url, headers={"Authorization": f"Bearer {self.token()}"})
                size = 0
                with opener(request, timeout=max(1e-3, min(self.socket_timeout_s, left))) as response, open(path, "wb") as out:
                    read = getattr(response, "read1", response.read)
                    while True:
                        if self.clock() >= deadline:
                            raise DownloadTimeout(f"{uri}: time budget used up after {size} bytes")
                        chunk = read(self.chunk_bytes)
                        if not chunk:
                            break
                        out.write(chunk)
                        size += len(chunk)
                return size
            except DownloadTimeout:
                raise
            except Exception as exc:  # noqa: BLE001 - urllib raises environment-specific types; classified below
                last = exc
                auth = isinstance(exc, urllib.error.HTTPError) and exc.code in (401, 403)
                auth_seen = auth_seen or auth
                if not auth and not is_transient(exc):
                    break                                             # a permanent answer (404, 400 ...)
                if attempt + 1 >= (self.auth_attempts if auth_seen else self.attempts):
                    break
                self.sleep(max(0.0, min(10.0, 0.5 * 2 ** min(attempt, 5), deadline - self.clock())))
        if is_transient(last):
            raise DownloadTimeout(f"{uri}: retries used up: {last}") from last
        raise DataContractError(f"download of {uri} failed: {last}") from last


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
            downloader = GCSRestDownloader(TokenProvider(transport.get("token_file")),
                                           time_budget_s=float(transport.get("download_seconds", 300.0)))
        cache = data_config.get("cache_dir")
        if not cache:
            raise DataContractError("bucket transport requires data.cache_dir")
        return CachedRemoteResolver(root, cache, downloader, int(transport.get("max_cache_bytes", 0)))
    raise DataContractError(f"unknown data.transport kind {kind!r}")
