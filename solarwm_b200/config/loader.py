"""Strict run-config loader (schema ``solarwm.run.v1``).

Pipeline: parse YAML (or JSON, so a resolved config can be fed back for resume) with duplicate
and non-string keys rejected -> expand ``${ENV}`` references -> apply ``--set a.b=YAML``
overrides -> check the fixed top-level sections -> check every value is JSON-compatible and
finite -> validate the (family, stage, causal mode, objective) route -> blake2s digests of the
raw source and of the canonical JSON form.  No torch import; no constructor is ever executed.

Behavioural contract: solar/config/loader.py:22-248 of the reference.
"""
from __future__ import annotations

import copy
import hashlib
import json
import math
import os
import re
import tempfile
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, MutableMapping, Optional, Sequence

import yaml

from ..errors import ConfigurationError

SCHEMA = "solarwm.run.v1"
ACTIONS = ("train", "infer", "preencode")
TOP_LEVEL_SECTIONS = ("schema", "action", "name", "model", "data", "distributed", "train", "validation",
                      "checkpoint", "preencode", "inference", "runtime", "metadata")
_ENV_REF = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)\}")


class _StrictLoader(yaml.SafeLoader):
    pass


def _strict_mapping(loader: _StrictLoader, node: yaml.nodes.MappingNode, deep: bool = False):
    loader.flatten_mapping(node)
    out: dict = {}
    for key_node, value_node in node.value:
        key = loader.construct_object(key_node, deep=deep)
        line = key_node.start_mark.line + 1
        if not isinstance(key, str):
            raise ConfigurationError(f"YAML mapping keys must be strings at line {line}")
        if key in out:
            raise ConfigurationError(f"duplicate YAML key {key!r} at line {line}")
        out[key] = loader.construct_object(value_node, deep=deep)
    return out


_StrictLoader.add_constructor(yaml.resolver.BaseResolver.DEFAULT_MAPPING_TAG, _strict_mapping)


def _json_pairs(pairs):
    out: dict = {}
    for key, value in pairs:
        if key in out:
            raise ConfigurationError(f"duplicate JSON key {key!r}")
        out[key] = value
    return out


def expand_env(value: Any) -> Any:
    if isinstance(value, dict):
        return {k: expand_env(v) for k, v in value.items()}
    if isinstance(value, list):
        return [expand_env(v) for v in value]
    if isinstance(value, str):
        def sub(match):
            name = match.group(1)
            if name not in os.environ:
                raise ConfigurationError(f"environment variable {name!r} is not set")
            return os.environ[name]

        return _ENV_REF.sub(sub, value)
    return value


def apply_override(config: MutableMapping[str, Any], raw: str) -> None:
    """``a.b.c=VALUE`` with VALUE parsed as YAML; intermediate mappings are created on demand."""
    if "=" not in raw:
        raise ConfigurationError(f"override must be KEY=VALUE, got {raw!r}")
    dotted, text = raw.split("=", 1)
    keys = [k for k in dotted.split(".") if k]
    if not keys:
        raise ConfigurationError(f"override has an empty key: {raw!r}")
    try:
        value = yaml.load(text, Loader=_StrictLoader)
    except (yaml.YAMLError, ConfigurationError) as exc:
        raise ConfigurationError(f"invalid override {raw!r}: {exc}") from exc
    node = config
    for key in keys[:-1]:
        child = node.get(key)
        if child is None:
            child = node[key] = {}
        if not isinstance(child, MutableMapping):
            raise ConfigurationError(f"override {raw!r} crosses non-mapping key {key!r}")
        node = child
    node[keys[-1]] = value


def canonical_json(config: Mapping[str, Any]) -> bytes:
    """Stable byte form used for digests, manifests and checkpoint provenance."""
    text = json.dumps(config, allow_nan=False, sort_keys=True, separators=(",", ":"), ensure_ascii=False)
    return (text + "\n").encode("utf-8")


def _check_json_compatible(value: Any, path: tuple = ()) -> None:
    where = ".".join(path) or "<root>"
    if value is None or isinstance(value, (str, bool, int)):
        return
    if isinstance(value, float):
        if not math.isfinite(value):
            raise ConfigurationError(f"non-finite number at {where}")
        return
    if isinstance(value, list):
        for i, child in enumerate(value):
            _check_json_compatible(child, (*path, str(i)))
        return
    if isinstance(value, dict):
        for key, child in value.items():
            if not isinstance(key, str):
                raise ConfigurationError(f"non-string mapping key at {where}")
            _check_json_compatible(child, (*path, key))
        return
    raise ConfigurationError(f"unsupported YAML value {type(value).__name__} at {where}; "
                             "configs must be canonical JSON-compatible values")


def _check_top_level(config: Mapping[str, Any]) -> None:
    unknown = sorted(set(config) - set(TOP_LEVEL_SECTIONS))
    if unknown:
        raise ConfigurationError(f"unknown top-level config keys: {unknown}")
    if config.get("schema") != SCHEMA:
        raise ConfigurationError(f"schema must be exactly {SCHEMA!r}")
    if str(config.get("action", "")).strip().lower() not in ACTIONS:
        raise ConfigurationError("action must be one of: train, infer, preencode")
    if not str(config.get("name", "")).strip():
        raise ConfigurationError("name must be a non-empty run identifier")
    for section in ("model", "data", "runtime"):
        if not isinstance(config.get(section), Mapping):
            raise ConfigurationError(f"{section} must be a mapping")


@dataclass(frozen=True)
class ResolvedConfig:
    path: Path
    source_digest: str
    resolved_digest: str
    values: Mapping[str, Any]

    def mutable_copy(self) -> dict:
        return copy.deepcopy(dict(self.values))

    def write_json(self, path) -> None:
        """Atomic write of the canonical JSON form (temp file + fsync + rename)."""
        target = Path(path)
        target.parent.mkdir(parents=True, exist_ok=True)
        fd, tmp = tempfile.mkstemp(dir=target.parent, prefix=f".{target.name}.", suffix=".tmp")
        try:
            with os.fdopen(fd, "wb") as handle:
                handle.write(canonical_json(self.values))
                handle.flush()
                os.fsync(handle.fileno())
            os.replace(tmp, target)
            tmp = None
        finally:
            if tmp is not None:
                Path(tmp).unlink(missing_ok=True)


def load_config(path, overrides: Sequence[str] = (), *,
                route_validator: Optional[Callable[[Mapping[str, Any]], Any]] = None) -> ResolvedConfig:
    source = Path(path).resolve()
    raw = source.read_bytes()
    try:
        if source.suffix.lower() == ".json":
            loaded = json.loads(raw, object_pairs_hook=_json_pairs)
        else:
            loaded = yaml.load(raw, Loader=_StrictLoader)
    except (json.JSONDecodeError, UnicodeDecodeError, yaml.YAMLError, ConfigurationError) as exc:
        raise ConfigurationError(f"cannot parse {source}: {exc}") from exc
    if not isinstance(loaded, dict):
        raise ConfigurationError(f"{source} must contain a YAML mapping")
    values = expand_env(loaded)
    for item in overrides:
        apply_override(values, item)
    _check_top_level(values)
    _check_json_compatible(values)
    from .routes import validate_route

    (route_validator or validate_route)(values)
    return ResolvedConfig(path=source, source_digest=hashlib.blake2s(raw).hexdigest(),
                          resolved_digest=hashlib.blake2s(canonical_json(values)).hexdigest(), values=values)
