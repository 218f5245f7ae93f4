"""A bucket as a no-overwrite object store with resumable uploads, over the JSON API and the standard library.

``GCSStore("gs://bucket/run-prefix")`` keeps every key under its prefix.  An object is identified by ``(size, md5)``:

  put        if the object exists with the same identity the call is a no-op (re-running a publication is safe); with
             another identity it is a CONFLICT, never an overwrite (``ifGenerationMatch=0`` guards the race).  Data goes
             through a resumable session in 8 MiB chunks; after a transport failure the session is asked how much it
             has (``Content-Range: bytes */N`` -> 308 + ``Range``) and the upload continues from there; a session that
             acknowledges nothing new several times in a row is reported as stalled.  Files are streamed, never read
             whole.
  metadata / read / list (paginated)   what the multi-node publication protocol needs to see other nodes' receipts.

The HTTP layer is one callable ``transport(method, path, body, headers) -> (status, headers, payload)``; the default
opens an HTTPS connection per request, tests pass a fake that plays the server.  Transient statuses and transport
failures are retried with capped back-off; authentication comes from ``data.transport.TokenProvider`` unless a token
callable is given.

Reference: GCSStore (solar/runtime/gcs_upload.py:36-282).
"""
from __future__ import annotations

import base64
import hashlib
import io
import json
import mimetypes
import re
import time
from dataclasses import dataclass
from pathlib import Path
from typing import BinaryIO, Callable, Dict, Optional, Tuple
from urllib.parse import quote, urlencode, urlsplit

from ..errors import SolarWMError

HOST = "storage.googleapis.com"
CHUNK = 8 << 20
RETRYABLE = (408, 429, 500, 502, 503, 504)


class StoreError(SolarWMError):
    def __init__(self, code: str, *, retryable: bool = False):
        super().__init__(code)
        self.code, self.retryable = code, retryable


@dataclass(frozen=True)
class ObjectInfo:
    size: int
    md5: str                    # base64, as the API reports it

    @classmethod
    def of_bytes(cls, data: bytes) -> "ObjectInfo":
        return cls(len(data), base64.b64encode(hashlib.md5(data).digest()).decode())

    @classmethod
    def of_file(cls, path) -> "ObjectInfo":
        h, size = hashlib.md5(), 0
        with open(path, "rb") as fh:
            for block in iter(lambda: fh.read(1 << 20), b""):
                h.update(block)
                size += len(block)
        return cls(size, base64.b64encode(h.digest()).decode())


def relative_key(key: str) -> str:
    parts = key.split("/")
    if not key or key.startswith("/") or any(p in ("", ".", "..") for p in parts) or "\\" in key or "\0" in key:
        raise StoreError("invalid_object_key")
    return key


def _https_transport(timeout: float):
    import http.client

    def send(method, path, body, headers):
        conn = http.client.HTTPSConnection(HOST, timeout=timeout)
        try:
            conn.request(method, path, body=body, headers=headers)
            resp = conn.getresponse()
            payload = resp.read(16 * (1 << 20) + 1)
            return resp.status, {k.lower(): v for k, v in resp.getheaders()}, payload
        finally:
            conn.close()

    return send


class GCSStore:
    def __init__(self, destination: str, *, token: Optional[Callable[[], str]] = None, transport=None, timeout: float = 60.0,
                 attempts: int = 4, sleep=time.sleep, chunk: int = CHUNK):
        uri = urlsplit(destination)
        if uri.scheme != "gs" or not re.fullmatch(r"[a-z0-9][a-z0-9._-]*", uri.netloc) or uri.query or uri.fragment \
                or not uri.path.startswith("/"):
            raise StoreError("invalid_destination")
        self.bucket, self.prefix = uri.netloc, relative_key(uri.path[1:].rstrip("/")) + "/"
        if token is None:
            from ..data.transport import TokenProvider

            token = TokenProvider()
        self.token, self.transport = token, transport or _https_transport(timeout)
        self.attempts, self.sleep, self.chunk = int(attempts), sleep, int(chunk)

    # -- one request with retries -------------------------------------------------------------------------------------
    def _request(self, method: str, path: str, *, body: bytes = b"", headers=None, accepted=(200,), retry: bool = True):
        tries = self.attempts if retry else 1
        for attempt in range(tries):
            try:
                credential = self.token()
                if not credential or "\r" in credential or "\n" in credential:
                    raise ValueError
            except Exception:  # noqa: BLE001 - whatever the provider raised, the caller sees one code
                raise StoreError("storage_authentication_failed") from None
            try:
                status, rh, payload = self.transport(method, path, body, {"Authorization": "Bearer " + credential, **(headers or {})})
                if len(payload) > 16 * (1 << 20):
                    raise StoreError("storage_response_too_large")
                if status in accepted:
                    return status, rh, payload
                error = StoreError(f"storage_http_{status}", retryable=status in RETRYABLE)
            except OSError:
                error = StoreError("storage_transport_failed", retryable=True)
            if not error.retryable or attempt + 1 == tries:
                raise error
            self.sleep(min(2 ** attempt, 8))
        raise StoreError("storage_retry_exhausted")

    def _object_path(self, key: str) -> str:
        return f"/storage/v1/b/{self.bucket}/o/" + quote(self.prefix + relative_key(key), safe="")

    @staticmethod
    def _info(value: dict) -> ObjectInfo:
        try:
            return ObjectInfo(int(value["size"]), str(value["md5Hash"]))
        except (KeyError, TypeError, ValueError):
            raise StoreError("storage_metadata_invalid") from None

    @staticmethod
    def _json(payload: bytes) -> dict:
        try:
            value = json.loads(payload.decode() or "{}")
        except (UnicodeDecodeError, ValueError):
            raise StoreError("storage_response_invalid") from None
        if not isinstance(value, dict):
            raise StoreError("storage_response_invalid")
        return value

    # -- reads ----------------------------------------------------------------------------------------------------------
    def metadata(self, key: str) -> Optional[ObjectInfo]:
        status, _, payload = self._request("GET", self._object_path(key) + "?fields=size,md5Hash", accepted=(200, 404))
        return None if status == 404 else self._info(self._json(payload))

    def read(self, key: str) -> bytes:
        return self._request("GET", self._object_path(key) + "?alt=media")[2]

    def list(self, prefix: str) -> Dict[str, ObjectInfo]:
        prefix = relative_key(prefix.rstrip("/")) + "/"
        found, page = {}, ""
        while True:
            query = {"prefix": self.prefix + prefix, "fields": "items(name,size,md5Hash),nextPageToken", "maxResults": "1000"}
            if page:
                query["pageToken"] = page
            payload = self._json(self._request("GET", f"/storage/v1/b/{self.bucket}/o?" + urlencode(query))[2])
            for item in payload.get("items", []):
                name = str(item.get("name", ""))
                if not name.startswith(self.prefix + prefix):
                    raise StoreError("storage_prefix_mismatch")
                found[name[len(self.prefix):]] = self._info(item)
            page = payload.get("nextPageToken", "")
            if not page:
                return found

    # -- writes ---------------------------------------------------------------------------------------------------------
    def put_bytes(self, key: str, data: bytes) -> bool:
        return self._put(key, io.BytesIO(data), ObjectInfo.of_bytes(data))

    def put_file(self, key: str, path, expected: Optional[ObjectInfo] = None) -> bool:
        expected = expected or ObjectInfo.of_file(path)
        with open(path, "rb") as fh:
            return self._put(key, fh, expected)

    def _present(self, key: str, expected: ObjectInfo) -> bool:
        have = self.metadata(key)
        if have is not None and have != expected:
            raise StoreError("object_content_conflict")
        return have is not None

    def _put(self, key: str, stream: BinaryIO, expected: ObjectInfo) -> bool:
        """True when bytes were sent, False when the identical object was already there."""
        if expected.size <= 0:
            raise StoreError("empty_object")
        if self._present(key, expected):
            return False
        ctype = mimetypes.guess_type(key)[0] or "application/octet-stream"
        status, headers, _ = self._request(
            "POST", f"/upload/storage/v1/b/{self.bucket}/o?" + urlencode({"uploadType": "resumable", "ifGenerationMatch": "0"}),
            body=json.dumps({"name": self.prefix + relative_key(key), "md5Hash": expected.md5, "contentType": ctype}).encode(),
            headers={"Content-Type": "application/json", "X-Upload-Content-Type": ctype,
                     "X-Upload-Content-Length": str(expected.size)}, accepted=(200, 201, 412))
        if status != 412:                           # 412: somebody created it meanwhile; verified below
            session = urlsplit(headers.get("location", ""))
            if session.scheme != "https" or session.netloc != HOST or not session.path.startswith("/upload/") or session.fragment:
                raise StoreError("invalid_upload_session")
            spath = session.path + "?" + session.query
            offset = stalls = 0
            while offset < expected.size:
                want = min(self.chunk, expected.size - offset)
                stream.seek(offset)
                chunk = stream.read(want)
                if len(chunk) != want:
                    raise StoreError("local_file_changed")
                try:
                    status, headers, _ = self._request(
                        "PUT", spath, body=chunk, retry=False, accepted=(200, 201, 308, 412),
                        headers={"Content-Range": f"bytes {offset}-{offset + want - 1}/{expected.size}"})
                except StoreError as exc:
                    if not exc.retryable:
                        raise
                    # ask the session what it holds and continue from there
                    status, headers, _ = self._request("PUT", spath, accepted=(200, 201, 308, 412),
                                                       headers={"Content-Range": f"bytes */{expected.size}"})
                if status != 308:
                    break
                got = headers.get("range", "")
                m = re.fullmatch(r"bytes=0-(\d+)", got)
                if got and m is None:
                    raise StoreError("invalid_upload_offset")
                nxt = int(m[1]) + 1 if m else 0
                if nxt < offset or nxt > offset + want:
                    raise StoreError("invalid_upload_offset")
                stalls = stalls + 1 if nxt == offset else 0
                if stalls >= self.attempts:
                    raise StoreError("upload_stalled", retryable=True)
                offset = nxt
        if not self._present(key, expected):
            raise StoreError("upload_not_committed", retryable=True)
        return True


class DirectoryStore:
    """The same protocol over a local directory (``file://`` destinations, tests, on-prem exports)."""

    def __init__(self, root):
        self.root = Path(root)

    def _path(self, key: str) -> Path:
        return self.root / relative_key(key)

    def metadata(self, key: str) -> Optional[ObjectInfo]:
        p = self._path(key)
        return ObjectInfo.of_file(p) if p.is_file() else None

    def read(self, key: str) -> bytes:
        return self._path(key).read_bytes()

    def list(self, prefix: str) -> Dict[str, ObjectInfo]:
        base = self._path(prefix.rstrip("/"))
        return {p.relative_to(self.root).as_posix(): ObjectInfo.of_file(p) for p in sorted(base.rglob("*")) if p.is_file()} \
            if base.is_dir() else {}

    def put_bytes(self, key: str, data: bytes) -> bool:
        return self._put(key, data, ObjectInfo.of_bytes(data))

    def put_file(self, key: str, path, expected: Optional[ObjectInfo] = None) -> bool:
        return self._put(key, Path(path).read_bytes(), expected or ObjectInfo.of_file(path))

    def _put(self, key: str, data: bytes, expected: ObjectInfo) -> bool:
        from .create_only import write_file_create_only

        have = self.metadata(key)
        if have is not None:
            if have != expected:
                raise StoreError("object_content_conflict")
            return False
        write_file_create_only(self._path(key), data)
        return True


def store_for(destination: str, **kw):
    if destination.startswith("gs://"):
        return GCSStore(destination, **kw)
    return DirectoryStore(destination[7:] if destination.startswith("file://") else destination)
