"""Launch provenance: git identity, inline-secret rejection, the ``solarwm.launch.v2`` manifest
(reference: solar/runtime/provenance.py:48-142)."""
from __future__ import annotations

import os
import re
import socket
import subprocess
import sys
import time
from pathlib import Path
from typing import Any, Mapping

from ..errors import ConfigurationError

_SECRET_KEY = re.compile(r"(password|passwd|secret|token|api[_-]?key|credential|private[_-]?key)", re.I)
_SECRET_VALUE = re.compile(r"(AKIA[0-9A-Z]{16}|-----BEGIN [A-Z ]*PRIVATE KEY-----|ya29\.[0-9A-Za-z_-]{20,}|"
                           r"gh[pousr]_[0-9A-Za-z]{30,}|hf_[0-9A-Za-z]{30,})")


def git_identity(repo=None) -> dict:
    repo = Path(repo or Path(__file__).resolve().parents[2])

    def run(*args):
        try:
            out = subprocess.run(["git", "-C", str(repo), *args], capture_output=True, text=True, timeout=10)
            return out.stdout.strip() if out.returncode == 0 else None
        except (OSError, subprocess.SubprocessError):
            return None

    commit = run("rev-parse", "HEAD")
    dirty = run("status", "--porcelain")
    return {"commit": commit, "dirty": None if dirty is None else bool(dirty), "branch": run("rev-parse", "--abbrev-ref", "HEAD")}


def reject_inline_secrets(config: Mapping[str, Any], path: tuple = ()) -> None:
    """Configs are published with every run; credentials must come from the environment or files."""
    for key, value in config.items():
        here = (*path, str(key))
        if isinstance(value, Mapping):
            reject_inline_secrets(value, here)
            continue
        items = value if isinstance(value, list) else [value]
        for item in items:
            if isinstance(item, Mapping):
                reject_inline_secrets(item, here)
            elif isinstance(item, str) and item:
                if _SECRET_VALUE.search(item):
                    raise ConfigurationError(f"inline secret value at {'.'.join(here)}")
                if _SECRET_KEY.search(str(key)) and not item.startswith(("/", "~", "file:", "env:")):
                    raise ConfigurationError(f"inline secret at {'.'.join(here)}; reference a file or environment variable")


def build_launch_manifest(*, resolved, route, command: str, topology=None, extra=None) -> dict:
    return {
        "schema": "solarwm.launch.v2",
        "created_unix": time.time(),
        "command": command,
        "argv": list(sys.argv),
        "config_path": str(resolved.path),
        "source_digest": resolved.source_digest,
        "resolved_digest": resolved.resolved_digest,
        "route": route.key,
        "name": resolved.values.get("name"),
        "git": git_identity(),
        "host": socket.gethostname(),
        "pid": os.getpid(),
        "python": sys.version.split()[0],
        "world_size": None if topology is None else topology.raw_world_size,
        "sequence_parallel_size": None if topology is None else topology.sp_size,
        "extra": dict(extra or {}),
    }
