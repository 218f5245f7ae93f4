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
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Mapping, Optional

from ..errors import SolarWMError
from .create_only import write_file_create_only
from .gcs_upload import uploader_for
from .object_store import ObjectInfo, StoreError

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


# ---------------------------------------------------------------------------------------------------------------------
# Multi-node publication of comparison views into one object store
# ---------------------------------------------------------------------------------------------------------------------
# Each node holds the comparison-view slots its ranks produced (``compare/rankSSS_*.mp4``, ``manifests/rank_SSS.json``,
# ``errors/rank_SSS.json`` for slots that failed).  ``publish_partition`` checks the local inventory, uploads it and then
# uploads the node's receipt; ``finalize`` (any node may call it, node 0 does) writes the destination's ``COMPLETE.json``
# only when every node's receipt is there, the receipts cover every slot exactly once, and the objects in the store are
# exactly the files the receipts name with the identities they name.  Until then it returns ``None``.  All writes are
# no-overwrite, so every step may be repeated after a crash (reference: solar/runtime/validation_publish.py:113-284).

RECEIPT_SCHEMA = "solarwm.validation-node-receipt.v1"
STORE_COMPLETE_SCHEMA = "solarwm.store-validation-complete.v1"
_PASS_DIR = re.compile(r"step_(\d{6,})_([A-Za-z0-9][A-Za-z0-9_.-]*)")
_SLOT_FILE = {"compare": re.compile(r"rank(\d+)_[A-Za-z0-9_.-]+\.mp4"), "manifests": re.compile(r"rank_(\d+)\.json"),
              "errors": re.compile(r"rank_(\d+)\.json")}
_SECRET_KEYS = ("authorization", "private_key", "client_secret", "session_url", "signed_url", "access_token")


def _canonical(value) -> bytes:
    return (json.dumps(value, sort_keys=True, separators=(",", ":"), allow_nan=False) + "\n").encode()


def _load_object(raw: bytes) -> dict:
    try:
        value = json.loads(raw)
    except (ValueError, UnicodeError):
        value = None
    if not isinstance(value, dict):
        raise StoreError("invalid_publication_json")
    return value


def _no_credentials(value) -> None:
    if isinstance(value, dict):
        for k, v in value.items():
            if str(k).lower() in _SECRET_KEYS and v:
                raise StoreError("credential_in_publication_json")
            _no_credentials(v)
    elif isinstance(value, (list, tuple)):
        for v in value:
            _no_credentials(v)
    elif isinstance(value, str) and ("-----BEGIN" in value or re.match(r"(?i)bearer\s+\S{16,}", value)):
        raise StoreError("credential_in_publication_json")


def _nat(value, least: int = 0) -> int:
    if type(value) is not int or value < least:
        raise StoreError("invalid_publication_integer")
    return value


def _plain(path: Path, root: Path) -> Path:
    """``path`` lies under ``root`` with no symlink on the way."""
    node = path
    while node != root:
        if root not in node.parents or node.is_symlink():
            raise StoreError("unsafe_publication_path")
        node = node.parent
    return path


def _slot_files(folder: Path, group: str, root: Path) -> dict:
    """slot -> file for the files of ``group`` whose names follow the pattern; anything else next to them is ignored,
    never uploaded."""
    base = folder / group
    if not base.exists() and not base.is_symlink():
        return {}
    if not _plain(base, root).is_dir():
        raise StoreError("missing_publication_file")
    found = {}
    for p in sorted(base.iterdir()):
        m = _SLOT_FILE[group].fullmatch(p.name)
        if m is None:
            continue
        if not _plain(p, root).is_file():
            raise StoreError("missing_publication_file")
        if int(m[1]) in found:
            raise StoreError("duplicate_local_slot")
        found[int(m[1])] = p
    return found


@dataclass(frozen=True)
class NodePartition:
    prefix: str                                   # key prefix of the pass in the store
    receipt: dict
    uploads: tuple = field(default_factory=tuple)   # (key, path, ObjectInfo)


def read_partition(run_root, directory, *, node: int, nodes: int) -> NodePartition:
    """Validate one node-local pass directory (``<run_root>/validation/step_NNNNNN_<pass>``) and describe its upload."""
    root, directory = Path(run_root), Path(directory)
    m = _PASS_DIR.fullmatch(directory.name)
    if m is None:
        raise StoreError("invalid_validation_directory")
    step, pass_name = int(m[1]), m[2]
    marker = _load_object(_plain(directory / COMPLETE, root).read_bytes())
    if marker.get("step") != step or marker.get("pass") != pass_name:
        raise StoreError("local_marker_mismatch")
    total = _nat(marker.get("global_slots", marker.get("slots")), 1)
    groups = {g: _slot_files(directory, g, root) for g in _SLOT_FILE}
    ok, failed = groups["compare"], groups["errors"]
    if ok.keys() != groups["manifests"].keys() or ok.keys() & failed.keys() or any(s >= total for s in (*ok, *failed)):
        raise StoreError("local_slot_inventory_mismatch")
    for kind, wants_error in (("manifests", False), ("errors", True)):
        for slot, p in groups[kind].items():
            doc = _load_object(p.read_bytes())
            _no_credentials(doc)
            if doc.get("slot", doc.get("logical_validation_rank")) != slot or doc.get("step") != step or doc.get("pass") != pass_name:
                raise StoreError("sample_identity_mismatch")
            if bool(doc.get("error")) != wants_error:
                raise StoreError("invalid_failure_sample" if wants_error else "invalid_successful_sample")
    prefix = directory.relative_to(root).as_posix()
    uploads, identities = [], {}
    for g, files in groups.items():
        for p in files.values():
            info = ObjectInfo.of_file(p)
            if info.size == 0:
                raise StoreError("empty_publication_object")
            key = f"{g}/{p.name}"
            identities[key] = {"size": info.size, "md5": info.md5}
            uploads.append((f"{prefix}/{key}", p, info))
    receipt = {"schema": RECEIPT_SCHEMA, "node": node, "nodes": nodes, "step": step, "pass": pass_name, "global_slots": total,
               "ok_slots": sorted(ok), "failed_slots": sorted(failed), "files": identities}
    return NodePartition(prefix, receipt, tuple(uploads))


def receipt_key(prefix: str, node: int) -> str:
    return f"{prefix}/receipts/node_{node:03d}.json"


def publish_partition(store, part: NodePartition) -> int:
    """Upload the partition's files, then its receipt (last, so a receipt implies its files).  Returns objects sent."""
    sent = sum(bool(store.put_file(key, path, info)) for key, path, info in part.uploads)
    store.put_bytes(receipt_key(part.prefix, part.receipt["node"]), _canonical(part.receipt))
    return sent


def _check_receipt(doc: dict, like: dict, node: int) -> None:
    for k in ("schema", "nodes", "step", "pass", "global_slots"):
        if type(doc.get(k)) is not type(like[k]) or doc[k] != like[k]:
            raise StoreError("node_receipt_identity_mismatch")
    if doc.get("node") != node:
        raise StoreError("node_receipt_identity_mismatch")
    ok, failed, files = doc.get("ok_slots"), doc.get("failed_slots"), doc.get("files")
    if not isinstance(ok, list) or not isinstance(failed, list) or not isinstance(files, dict):
        raise StoreError("invalid_node_receipt")
    slots = [_nat(s) for s in ok + failed]
    if len(set(slots)) != len(slots) or any(s >= like["global_slots"] for s in slots):
        raise StoreError("invalid_node_receipt")
    seen = {g: [] for g in _SLOT_FILE}
    for key, ident in files.items():
        g, _, name = key.partition("/")
        m = _SLOT_FILE[g].fullmatch(name) if g in _SLOT_FILE else None
        if m is None or not isinstance(ident, dict) or not isinstance(ident.get("md5"), str):
            raise StoreError("invalid_node_receipt")
        _nat(ident.get("size"), 1)
        seen[g].append(int(m[1]))
    if sorted(seen["compare"]) != sorted(ok) or sorted(seen["manifests"]) != sorted(ok) or sorted(seen["errors"]) != sorted(failed):
        raise StoreError("node_receipt_slot_files_mismatch")


def finalize(store, prefix: str, like: dict) -> Optional[str]:
    """``"complete"``/``"partial"`` once the destination marker is written (or was), ``None`` while receipts are missing."""
    have = store.list(prefix)
    wanted = {receipt_key(prefix, n) for n in range(like["nodes"])}
    if {k for k in have if k.startswith(prefix + "/receipts/")} - wanted:
        raise StoreError("unexpected_node_receipt")
    if not wanted <= have.keys():
        if f"{prefix}/{COMPLETE}" in have:
            raise StoreError("global_marker_without_receipts")
        return None
    ok, failed, named = [], [], {}
    for n in range(like["nodes"]):
        raw = store.read(receipt_key(prefix, n))
        if ObjectInfo.of_bytes(raw) != have[receipt_key(prefix, n)]:
            raise StoreError("node_receipt_changed")
        doc = _load_object(raw)
        _check_receipt(doc, like, n)
        ok += doc["ok_slots"]
        failed += doc["failed_slots"]
        for rel, ident in doc["files"].items():
            if f"{prefix}/{rel}" in named:
                raise StoreError("duplicate_global_slot")
            named[f"{prefix}/{rel}"] = ObjectInfo(ident["size"], ident["md5"])
    if sorted(ok + failed) != list(range(like["global_slots"])):
        raise StoreError("global_slot_inventory_mismatch")
    stored = {k: v for k, v in have.items() if k[len(prefix) + 1:].split("/")[0] in _SLOT_FILE}
    if stored != named:
        raise StoreError("global_object_inventory_mismatch")
    status = "partial" if failed else "complete"
    store.put_bytes(f"{prefix}/{COMPLETE}", _canonical({
        "schema": STORE_COMPLETE_SCHEMA, "step": like["step"], "pass": like["pass"], "global_slots": like["global_slots"],
        "ok_slots": len(ok), "failed_slots": sorted(failed), "status": status, "nodes": like["nodes"]}))
    return status


class ValidationPublisher:
    """One per node, polled while training runs: ``scan()`` publishes every sealed pass under ``<run>/validation`` that
    this node has not published yet and, on node 0, finalizes the passes whose receipts are all in.  A pass whose local
    marker changes after publication is an error (sealed means immutable)."""

    def __init__(self, run_dir, store, *, node: int, nodes: int):
        if type(nodes) is not int or type(node) is not int or not 0 <= node < nodes:
            raise StoreError("invalid_publisher_arguments")
        self.root, self.store, self.node, self.nodes = Path(run_dir).resolve(), store, node, nodes
        self._sent, self._final = {}, {}

    def scan(self) -> dict:
        out = {"node": self.node, "passes": [], "errors": 0, "pending": 0, "partial": 0}
        base = self.root / "validation"
        if not base.is_dir():
            out["pending"] = 1
            return out
        for d in sorted(base.iterdir()):
            if not _PASS_DIR.fullmatch(d.name):
                continue
            row = {"pass": d.name, "status": "pending"}
            try:
                if not (d / COMPLETE).exists():
                    out["pending"] += 1
                elif d.name in self._final:
                    row["status"] = self._final[d.name]
                else:
                    marker = _plain(d / COMPLETE, self.root).read_bytes()
                    if d.name in self._sent and self._sent[d.name][0] != marker:
                        raise StoreError("sealed_pass_changed")
                    if d.name not in self._sent:
                        part = read_partition(self.root, d, node=self.node, nodes=self.nodes)
                        row["objects_sent"] = publish_partition(self.store, part)
                        self._sent[d.name] = (marker, part)
                    part = self._sent[d.name][1]
                    row["status"] = "published"
                    if self.node == 0:
                        status = finalize(self.store, part.prefix, part.receipt)
                        if status is None:
                            out["pending"] += 1
                        else:
                            row["status"] = self._final[d.name] = status
                            out["partial"] += status == "partial"
            except StoreError as exc:
                row.update(status="error", code=exc.code, retryable=exc.retryable)
                out["errors"] += 1
            out["passes"].append(row)
        return out
