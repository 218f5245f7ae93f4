"""Scene uploads and isolated, cancellable conditioning preparation for the realtime host.

* ``store_upload``: accepts bytes only (never a server path or a URL): a prompt of 1-4000 characters and one
  base64 PNG / JPEG / WebP image of at most 8 MiB and 16 megapixels; the image is re-encoded to a normalised PNG,
  the scene identity is a digest of (image, prompt), and the scene manifest is updated under a file lock with
  create-only image files.
* ``prepare_isolated``: the conditioning encoders (text encoder, VAE) run in a short-lived child process that is
  started in its own session with the launcher's rank variables removed -- it never joins a collective and never
  shares the serving process's device memory -- and can be cancelled or timed out; its only channel back is an
  atomically written ``result.json``.  Results are cached by a digest of the request.

Reference behaviour: deploy/solar_wm/shared/scene_inputs.py:16-200.
"""
from __future__ import annotations

import base64
import fcntl
import hashlib
import importlib
import io
import json
import os
import signal
import subprocess
import sys
import tempfile
import time
import warnings
from pathlib import Path
from typing import Callable, Mapping

MAX_IMAGE_BYTES = 8 * 1024 * 1024
MAX_PIXELS = 16_000_000
_LAUNCHER_VARS = {"RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "ROLE_RANK", "ROLE_WORLD_SIZE",
                  "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID", "TORCHELASTIC_ERROR_FILE"}


class PreparationCancelled(Exception):
    pass


def write_json(path, value) -> None:
    """Atomic JSON write: temporary file in the same directory, fsync, replace."""
    path = Path(path)
    with tempfile.NamedTemporaryFile(mode="w", dir=path.parent, delete=False) as fh:
        tmp = Path(fh.name)
        try:
            json.dump(value, fh, ensure_ascii=False, indent=2)
            fh.flush()
            os.fsync(fh.fileno())
            os.replace(tmp, path)
        finally:
            tmp.unlink(missing_ok=True)


def _load_scenes(manifest: Path) -> dict:
    if not manifest.exists():
        return {}
    return {row["scene_id"]: row for row in json.loads(manifest.read_text())}


def store_upload(state_directory, body: Mapping) -> dict:
    from PIL import Image, ImageOps

    prompt, encoded = body.get("prompt"), body.get("image")
    if not isinstance(prompt, str) or not 1 <= len(prompt.strip()) <= 4000:
        raise ValueError("enter a prompt (1-4000 characters)")
    if not isinstance(encoded, str) or len(encoded) > (MAX_IMAGE_BYTES + 2) // 3 * 4:
        raise ValueError("image must be at most 8 MiB")
    try:
        data = base64.b64decode(encoded, validate=True)
    except (ValueError, TypeError) as exc:
        raise ValueError("invalid image encoding") from exc
    if not 0 < len(data) <= MAX_IMAGE_BYTES:
        raise ValueError("image must be at most 8 MiB")
    try:
        with warnings.catch_warnings():
            warnings.simplefilter("error", Image.DecompressionBombWarning)
            with Image.open(io.BytesIO(data)) as src:
                if src.format not in ("PNG", "JPEG", "WEBP") or getattr(src, "n_frames", 1) != 1:
                    raise ValueError("use a single PNG, JPEG or WebP image")
                if src.width * src.height > MAX_PIXELS:
                    raise ValueError("image must be at most 16 megapixels")
                image = ImageOps.exif_transpose(src).convert("RGB")
            out = io.BytesIO()
            image.save(out, format="PNG")
    except (OSError, Image.DecompressionBombWarning, Image.DecompressionBombError) as exc:
        raise ValueError("invalid or oversized image") from exc
    image_bytes, prompt = out.getvalue(), prompt.strip()
    identity = "upload-" + hashlib.sha256(image_bytes + b"\0" + prompt.encode()).hexdigest()[:24]
    root = Path(state_directory)
    root.mkdir(parents=True, exist_ok=True)
    manifest = root / "scenes.json"
    with (root / "scenes.lock").open("a") as lock:            # host I/O only under this lock
        fcntl.flock(lock, fcntl.LOCK_EX)
        scenes = _load_scenes(manifest)
        if identity in scenes:
            return scenes[identity]
        uploads = root / "uploads"
        uploads.mkdir(exist_ok=True)
        target = uploads / (identity + ".png")
        if target.exists():                                    # an interrupted registration already saved these bytes
            if target.read_bytes() != image_bytes:
                raise ValueError("stored upload differs")
        else:
            with target.open("xb") as fh:
                fh.write(image_bytes)
                fh.flush()
                os.fsync(fh.fileno())
        row = dict(scene_id=identity, title="My scene " + identity[-6:], first=str(target), prompt=prompt)
        scenes[identity] = row
        write_json(manifest, list(scenes.values()))
        return row


def request_digest(request: Mapping) -> str:
    return hashlib.sha256(json.dumps(request, sort_keys=True).encode()).hexdigest()


def prepare_isolated(state_directory, request: Mapping, *, cancelled: Callable[[], bool] = lambda: False,
                     progress: Callable[[str], None] = lambda _: None, timeout_s: float = 1800.0,
                     poll_s: float = 0.05) -> dict:
    """Run ``request = {"callable": "package.module:function", "args": [...], "kwargs": {...}}`` in a child
    process and return its JSON result (cached by the request digest).  Raises ``PreparationCancelled`` when
    ``cancelled()`` turns true (the child's process group is terminated), ``TimeoutError`` after ``timeout_s``,
    ``RuntimeError`` with the child's error line otherwise."""
    if cancelled():
        raise PreparationCancelled()
    root = Path(state_directory)
    cache = root / "scene-features" / (request_digest(request) + ".json")
    if cache.exists():
        return json.loads(cache.read_text())
    progress("encoding")
    jobs = root / "scene-jobs"
    jobs.mkdir(parents=True, exist_ok=True)
    job = Path(tempfile.mkdtemp(prefix="request-", dir=jobs))
    write_json(job / "request.json", dict(request))
    env = {k: v for k, v in os.environ.items() if k not in _LAUNCHER_VARS}
    env.update(PYTHONDONTWRITEBYTECODE="1", OMP_NUM_THREADS="2")
    with (job / "encoder.log").open("wb") as log:
        child = subprocess.Popen([sys.executable, "-B", "-m", __name__, "--job", str(job / "request.json")], env=env,
                                 stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
        started = time.monotonic()
        try:
            while child.poll() is None:
                if cancelled():
                    raise PreparationCancelled()
                if time.monotonic() - started > timeout_s:
                    raise TimeoutError(f"conditioning preparation exceeded {timeout_s:.0f} s")
                time.sleep(poll_s)
        finally:
            if child.poll() is None:                           # ours alone: the session we started for it
                try:
                    os.killpg(child.pid, signal.SIGTERM)
                except ProcessLookupError:
                    pass
                try:
                    child.wait(timeout=5)
                except subprocess.TimeoutExpired:
                    os.killpg(child.pid, signal.SIGKILL)
                    child.wait()
    result_path = job / "result.json"
    if not result_path.exists():
        raise RuntimeError(f"the encoder process left no result (exit {child.returncode}); see {job / 'encoder.log'}")
    result = json.loads(result_path.read_text())
    if "error" in result:
        raise RuntimeError(result["error"])
    cache.parent.mkdir(parents=True, exist_ok=True)
    write_json(cache, result["value"])
    progress("encoded")
    return result["value"]


def _run_job(path: str) -> int:
    job = Path(path)
    request = json.loads(job.read_text())
    try:
        module, _, name = request["callable"].partition(":")
        fn = getattr(importlib.import_module(module), name)
        value = fn(*request.get("args", []), **request.get("kwargs", {}))
        write_json(job.parent / "result.json", dict(value=value))
        return 0
    except Exception as exc:  # noqa: BLE001 - the parent reports the line
        write_json(job.parent / "result.json", dict(error=f"{type(exc).__name__}: {exc}"))
        return 1


def image_statistics(path: str) -> dict:
    """A dependency-free conditioning function (per-channel mean / std of the stored image): the stand-in the host
    uses when no encoder weights are installed, and the function the isolation tests run in the child."""
    import numpy as np
    from PIL import Image

    with Image.open(path) as im:
        a = np.asarray(im.convert("RGB"), dtype=np.float64) / 255.0
    return {"mean": a.mean((0, 1)).round(6).tolist(), "std": a.std((0, 1)).round(6).tolist(), "pid": os.getpid()}


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--job", required=True)
    raise SystemExit(_run_job(ap.parse_args().job))
