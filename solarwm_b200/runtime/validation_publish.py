"""Publication of finished validation passes.

A validation pass directory is publishable once it holds ``COMPLETE.json``.  Every file of the pass
is uploaded under ``<destination>/<run>/<pass>/...``; files are partitioned over nodes by a stable
hash of their relative path so each node uploads only what it owns; after the last file the node
writes a receipt ``.published/<node>.json`` (create-only) listing key, size and digest of what it
sent.  A pass with a receipt for this node is skipped, which makes the publisher re-runnable
(reference: solar/runtime/validation_publish.py:226-284).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Callable, Mapping, Optional

from ..errors import SolarWMError
from .create_only import write_file_create_only
from .gcs_upload import uploader_for

COMPLETE = "COMPLETE.json"


def owner_node(relative: str, nodes: int) -> int:
    return int.from_bytes(hashlib.sha256(relative.encode()).digest()[:8], "big") % max(int(nodes), 1)


def publishable_passes(source) -> list:
    root = Path(source)
    if (root / COMPLETE).is_file():
        return [root]
    return sorted(p for p in root.iterdir() if p.is_dir() and (p / COMPLETE).is_file())


def publish_validation(source, destination: str, *, node: int = 0, nodes: int = 1,
                       token_provider: Optional[Callable[[], str]] = None, uploader=None) -> Mapping[str, object]:
    if not 0 <= node < nodes:
        raise SolarWMError("node must lie in [0, nodes)")
    up = uploader or uploader_for(destination, token_provider)
    passes = publishable_passes(source)
    if not passes:
        raise SolarWMError(f"no complete validation pass under {source}")
    sent, skipped = 0, 0
    for vp in passes:
        receipt = vp / ".published" / f"node-{node:04d}.json"
        if receipt.exists():
            skipped += 1
            continue
        files = sorted(p for p in vp.rglob("*") if p.is_file() and ".published" not in p.parts)
        mine = [p for p in files if owner_node(p.relative_to(vp).as_posix(), nodes) == node]
        # COMPLETE.json goes last so a reader of the destination never sees a half-published pass as complete
        mine.sort(key=lambda p: (p.name == COMPLETE, p.as_posix()))
        receipts = [dict(up.upload(p, f"{vp.name}/{p.relative_to(vp).as_posix()}")) for p in mine]
        receipt.parent.mkdir(exist_ok=True)
        write_file_create_only(receipt, json.dumps({"schema": "solarwm.validation-receipt.v1", "node": node,
                                                    "nodes": nodes, "destination": destination,
                                                    "objects": receipts}, sort_keys=True).encode())
        sent += len(receipts)
    return {"passes": len(passes), "skipped_passes": skipped, "objects_sent": sent}
