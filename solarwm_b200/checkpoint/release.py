"""Release manifests: which weights a published checkpoint package serves by default.

A released package is a checkpoint transaction directory plus ``release-manifest.json`` beside it:

    {"schema": "solarwm.public-weight-manifest.v1",
     "identity": {"model": {"family": ..., "stage": ..., "weight_role": "live+ema"}},
     "load": {"format": "solarwm_checkpoint_transaction_v2", "entrypoint": ".", "default_weights": "ema"}}

``resolve_default_weights(source)`` reads it (from the package directory or next to a file inside it) and returns the
role inference should load -- the release decides, there is no command-line choice -- refusing a manifest whose
contract differs, whose default role is not one of the roles the package holds, or that cannot be read.
``write_release_manifest`` produces one (create-only) when a run publishes its weights
(reference behaviour: solar/backends/wan22/runtime/stage2.py:1163-1192).
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping, Sequence

from ..errors import BackendContractError

SCHEMA = "solarwm.public-weight-manifest.v1"
FORMAT = "solarwm_checkpoint_transaction_v2"
NAME = "release-manifest.json"


def write_release_manifest(package_dir, *, family: str, stage: str, weight_roles: Sequence[str], default_weights: str,
                           extra: Mapping = None) -> Path:
    roles = [str(r).strip().lower() for r in weight_roles]
    if not roles or any(r not in ("live", "ema") for r in roles) or default_weights not in roles:
        raise BackendContractError("release roles must be among live / ema and include the default")
    path = Path(package_dir) / NAME
    manifest = {"schema": SCHEMA,
                "identity": {"model": {"family": family, "stage": stage, "weight_role": "+".join(roles)}},
                "load": {"format": FORMAT, "entrypoint": ".", "default_weights": default_weights}}
    if extra:
        manifest["metadata"] = dict(extra)
    with open(path, "x", encoding="utf-8") as fh:              # create-only: a published manifest is never rewritten
        json.dump(manifest, fh, indent=1, sort_keys=True)
    return path


def resolve_default_weights(source) -> str:
    requested = Path(source).expanduser().resolve()
    root = requested if requested.is_dir() else requested.parent
    try:
        manifest = json.loads((root / NAME).read_text(encoding="utf-8"))
    except Exception as exc:  # noqa: BLE001 - any unreadable manifest is the same contract error
        raise BackendContractError(f"the released checkpoint lacks a readable release manifest: {exc}") from exc
    if not isinstance(manifest, Mapping):
        raise BackendContractError("the release manifest must be a mapping")
    load, identity = manifest.get("load"), manifest.get("identity")
    model = identity.get("model") if isinstance(identity, Mapping) else None
    if (manifest.get("schema") != SCHEMA or not isinstance(load, Mapping) or load.get("format") != FORMAT
            or load.get("entrypoint") != "." or not isinstance(model, Mapping)):
        raise BackendContractError("the release manifest contract differs")
    role = str(load.get("default_weights", "")).strip().lower()
    available = str(model.get("weight_role", "")).strip().lower().split("+")
    if role not in ("live", "ema") or role not in available:
        raise BackendContractError("the release's default weight role is invalid")
    return role
