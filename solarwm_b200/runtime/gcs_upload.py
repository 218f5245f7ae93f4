"""Object-store upload over the JSON/REST API (no SDK), plus a file:// twin for tests and on-prem.

``Uploader.upload(path, key)`` sends one object with ``ifGenerationMatch=0`` (create-only: an
existing object is a conflict, never an overwrite), retries transient statuses with exponential
backoff and returns a receipt ``{key, size, crc32c-less blake2s, generation}``.  The token comes
from a caller-supplied provider so no credential is read or stored here
(reference: solar/runtime/gcs_upload.py:87).
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
import urllib.error
import urllib.parse
import urllib.request
from pathlib import Path
from typing import Callable, Mapping, Optional

from ..errors import SolarWMError

_TRANSIENT = (408, 429, 500, 502, 503, 504)


class UploadError(SolarWMError):
    pass


def file_digest(path) -> str:
    h = hashlib.blake2s()
    with open(path, "rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


class FileUploader:
    """``file:///root`` destination: hard create-only copy (``O_EXCL``) with fsync."""

    def __init__(self, root):
        self.root = Path(root)

    def upload(self, path, key: str) -> Mapping[str, object]:
        dst = self.root / key
        dst.parent.mkdir(parents=True, exist_ok=True)
        try:
            fd = os.open(dst, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
        except FileExistsError as exc:
            raise UploadError(f"destination object already exists: {dst}") from exc
        with os.fdopen(fd, "wb") as out, open(path, "rb") as src:
            shutil.copyfileobj(src, out, 1 << 20)
            out.flush()
            os.fsync(out.fileno())
        return {"key": key, "size": dst.stat().st_size, "blake2s": file_digest(dst), "generation": "file"}


class GCSUploader:
    def __init__(self, bucket: str, token_provider: Callable[[], str], *, prefix: str = "", retries: int = 5,
                 opener=urllib.request.urlopen, sleep=time.sleep):
        self.bucket, self.prefix = bucket, prefix.strip("/")
        self.token_provider, self.retries, self.opener, self.sleep = token_provider, retries, opener, sleep

    def upload(self, path, key: str) -> Mapping[str, object]:
        name = f"{self.prefix}/{key}" if self.prefix else key
        url = ("https://storage.googleapis.com/upload/storage/v1/b/" + urllib.parse.quote(self.bucket, safe="") +
               "/o?uploadType=media&ifGenerationMatch=0&name=" + urllib.parse.quote(name, safe=""))
        data = Path(path).read_bytes()
        last: Optional[Exception] = None
        for attempt in range(self.retries):
            req = urllib.request.Request(url, data=data, method="POST", headers={
                "Authorization": f"Bearer {self.token_provider()}", "Content-Type": "application/octet-stream"})
            try:
                with self.opener(req) as resp:
                    body = json.loads(resp.read().decode() or "{}")
                return {"key": name, "size": len(data), "blake2s": hashlib.blake2s(data).hexdigest(),
                        "generation": str(body.get("generation", ""))}
            except urllib.error.HTTPError as exc:
                if exc.code == 412:
                    raise UploadError(f"destination object already exists: gs://{self.bucket}/{name}") from exc
                if exc.code not in _TRANSIENT:
                    raise UploadError(f"upload of {name} failed with HTTP {exc.code}") from exc
                last = exc
            except urllib.error.URLError as exc:
                last = exc
            self.sleep(min(2.0 ** attempt, 30.0))
        raise UploadError(f"upload of {name} failed after {self.retries} attempts: {last}")


def uploader_for(destination: str, token_provider: Optional[Callable[[], str]] = None):
    if destination.startswith("gs://"):
        bucket, _, prefix = destination[5:].partition("/")
        if token_provider is None:
            raise UploadError("a token provider is required for gs:// destinations")
        return GCSUploader(bucket, token_provider, prefix=prefix)
    if destination.startswith("file://"):
        return FileUploader(destination[7:])
    return FileUploader(destination)
