"""Strict run-config loader (schema ``solarwm.run.v1``).

A config file goes through a fixed sequence of stages, each a small object with one job, driven by one table:

    parse      YAML (or JSON, so that a resolved config can be fed back for a resume) into plain containers; a
               mapping with a repeated or a non-string key is an error, and no YAML tag can construct an object
    normalise  ONE walk over the tree that substitutes ``${NAME}`` environment references in strings and refuses
               anything that has no canonical JSON form (non-finite numbers, non-string keys, foreign types)
    override   ``--set a.b.c=VALUE`` items (VALUE parsed by the same strict YAML reader), re-normalised
    sections   the ``SECTIONS`` table below: which top-level keys exist, which are required, what each must look like
    route      the (family, stage, causal mode, objective) combination must be one the framework implements
    identity   blake2s of the file's bytes and of the canonical JSON of the resolved tree

The loader imports neither torch nor any backend.  What it shares with the reference is the CONTRACT -- accepted
files, resolved values, canonical JSON bytes and both digests are identical for the same input, which
``tests/test_reference_contracts.py`` checks against the reference package -- not its code
(contract: solar/config/loader.py:22-248 of the reference).
"""
from __future__ import annotations

import copy
import hashlib
import json
import math
import os
import re
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Dict, List, Mapping, MutableMapping, Optional, Sequence, Tuple

import yaml

from ..errors import ConfigurationError

SCHEMA = "solarwm.run.v1"
ACTIONS = ("train", "infer", "preencode")


# ---------------------------------------------------------------------------------------------------------------------
# the section table
# ---------------------------------------------------------------------------------------------------------------------
def _is_schema(v) -> Optional[str]:
    return None if v == SCHEMA else f"schema must be exactly {SCHEMA!r}"


def _is_action(v) -> Optional[str]:
    return None if str(v if v is not None else "").strip().lower() in ACTIONS else \
        "action must be one of: " + ", ".join(ACTIONS)


def _is_name(v) -> Optional[str]:
    return None if str(v if v is not None else "").strip() else "name must be a non-empty run identifier"


def _is_mapping(section: str) -> Callable[[Any], Optional[str]]:
    return lambda v: None if isinstance(v, Mapping) else f"{section} must be a mapping"


@dataclass(frozen=True)
class Section:
    name: str
    required: bool = False
    rule: Optional[Callable[[Any], Optional[str]]] = None      # returns a complaint, or None when satisfied


SECTIONS: Tuple[Section, ...] = (
    Section("schema", True, _is_schema),
    Section("action", True, _is_action),
    Section("name", True, _is_name),
    Section("model", True, _is_mapping("model")),
    Section("data", True, _is_mapping("data")),
    Section("runtime", True, _is_mapping("runtime")),
    Section("distributed"), Section("train"), Section("validation"), Section("checkpoint"), Section("preencode"),
    Section("inference"), Section("metadata"),
)
TOP_LEVEL_SECTIONS = tuple(s.name for s in SECTIONS)


def check_sections(tree: Mapping[str, Any]) -> None:
    stray = sorted(k for k in tree if k not in TOP_LEVEL_SECTIONS)
    if stray:
        raise ConfigurationError(f"unknown top-level config keys: {stray}")
    for section in SECTIONS:
        if section.rule is None or not (section.required or section.name in tree):
            continue
        complaint = section.rule(tree.get(section.name))
        if complaint:
            raise ConfigurationError(complaint)


# ---------------------------------------------------------------------------------------------------------------------
# parse
# ---------------------------------------------------------------------------------------------------------------------
class _PlainYAML(yaml.SafeLoader):
    """Safe loader whose mappings refuse repeated and non-string keys (both are silent data loss otherwise)."""

    def construct_mapping(self, node, deep=False):                    # noqa: D401 - yaml API
        self.flatten_mapping(node)
        built: Dict[str, Any] = {}
        for key_node, value_node in node.value:
            key = self.construct_object(key_node, deep=True)
            at = f"line {key_node.start_mark.line + 1}"
            if not isinstance(key, str):
                raise ConfigurationError(f"YAML mapping keys must be strings at {at}")
            if key in built:
                raise ConfigurationError(f"duplicate YAML key {key!r} at {at}")
            built[key] = self.construct_object(value_node, deep=True)
        return built


_PlainYAML.add_constructor(yaml.resolver.BaseResolver.DEFAULT_MAPPING_TAG,
                           lambda loader, node: loader.construct_mapping(node, deep=True))


def _unique_pairs(pairs: List[Tuple[str, Any]]) -> Dict[str, Any]:
    built: Dict[str, Any] = {}
    for key, value in pairs:
        if key in built:
            raise ConfigurationError(f"duplicate JSON key {key!r}")
        built[key] = value
    return built


def parse_text(raw: bytes, *, as_json: bool, origin: str = "<config>") -> Any:
    try:
        if as_json:
            return json.loads(raw, object_pairs_hook=_unique_pairs)
        return yaml.load(raw, Loader=_PlainYAML)
    except (json.JSONDecodeError, UnicodeDecodeError, yaml.YAMLError, ConfigurationError) as exc:
        raise ConfigurationError(f"cannot parse {origin}: {exc}") from exc


# ---------------------------------------------------------------------------------------------------------------------
# normalise: environment references + canonical-JSON compatibility in one walk
# ---------------------------------------------------------------------------------------------------------------------
_ENV_REFERENCE = re.compile(r"\$\{([A-Za-z_][A-Za-z0-9_]*)\}")


def _substitute(text: str, environ: Mapping[str, str]) -> str:
    def lookup(match: "re.Match[str]") -> str:
        name = match.group(1)
        try:
            return environ[name]
        except KeyError:
            raise ConfigurationError(f"environment variable {name!r} is not set") from None

    return _ENV_REFERENCE.sub(lookup, text)


def normalise(value: Any, *, environ: Optional[Mapping[str, str]] = None, expand: bool = True, _at: str = "") -> Any:
    """A fresh tree of dict / list / str / bool / int / finite float / None, with ``${NAME}`` substituted in strings
    when ``expand`` is set; anything else is refused with the dotted position of the offender."""
    environ = os.environ if environ is None else environ
    here = _at or "<root>"
    if value is None or isinstance(value, (bool, int)):
        return value
    if isinstance(value, str):
        return _substitute(value, environ) if expand else value
    if isinstance(value, float):
        if not math.isfinite(value):
            raise ConfigurationError(f"non-finite number at {here}")
        return value
    if isinstance(value, list):
        return [normalise(v, environ=environ, expand=expand, _at=f"{_at}.{i}" if _at else str(i)) for i, v in enumerate(value)]
    if isinstance(value, dict):
        out = {}
        for key, child in value.items():
            if not isinstance(key, str):
                raise ConfigurationError(f"non-string mapping key at {here}")
            out[key] = normalise(child, environ=environ, expand=expand, _at=f"{_at}.{key}" if _at else key)
        return out
    raise ConfigurationError(f"unsupported YAML value {type(value).__name__} at {here}; "
                             "configs must be canonical JSON-compatible values")


def expand_env(value: Any) -> Any:
    """Environment substitution alone (kept for callers that resolve fragments, e.g. serving manifests)."""
    return normalise(value, expand=True)


# ---------------------------------------------------------------------------------------------------------------------
# overrides
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Override:
    path: Tuple[str, ...]
    value: Any
    text: str

    @classmethod
    def parse(cls, text: str) -> "Override":
        dotted, sep, literal = text.partition("=")
        if not sep:
            raise ConfigurationError(f"override must be KEY=VALUE, got {text!r}")
        path = tuple(part for part in dotted.split(".") if part)
        if not path:
            raise ConfigurationError(f"override has an empty key: {text!r}")
        try:
            value = yaml.load(literal, Loader=_PlainYAML)
        except (yaml.YAMLError, ConfigurationError) as exc:
            raise ConfigurationError(f"invalid override {text!r}: {exc}") from exc
        return cls(path, value, text)

    def apply(self, tree: MutableMapping[str, Any]) -> None:
        cursor = tree
        for step in self.path[:-1]:
            if cursor.get(step) is None:
                cursor[step] = {}
            cursor = cursor[step]
            if not isinstance(cursor, MutableMapping):
                raise ConfigurationError(f"override {self.text!r} crosses non-mapping key {step!r}")
        cursor[self.path[-1]] = self.value


def apply_override(config: MutableMapping[str, Any], raw: str) -> None:
    Override.parse(raw).apply(config)


# ---------------------------------------------------------------------------------------------------------------------
# identity
# ---------------------------------------------------------------------------------------------------------------------
def canonical_json(config: Mapping[str, Any]) -> bytes:
    """The one byte form of a config: sorted keys, no spaces, UTF-8 kept, a final newline.  Digests, manifests and
    checkpoint provenance are all computed over these bytes."""
    return json.dumps(config, sort_keys=True, separators=(",", ":"), ensure_ascii=False, allow_nan=False).encode("utf-8") + b"\n"


def _digest(data: bytes) -> str:
    return hashlib.blake2s(data).hexdigest()


@dataclass(frozen=True)
class ResolvedConfig:
    path: Path
    source_digest: str
    resolved_digest: str
    values: Mapping[str, Any]

    def mutable_copy(self) -> dict:
        return copy.deepcopy(dict(self.values))

    def write_json(self, path) -> None:
        """Publish the canonical JSON form: written beside the target, flushed to disk, then renamed over it."""
        target = Path(path)
        target.parent.mkdir(parents=True, exist_ok=True)
        scratch = target.with_name(f".{target.name}.{os.getpid()}.{id(self):x}.tmp")
        try:
            with open(scratch, "xb") as handle:
                handle.write(canonical_json(self.values))
                handle.flush()
                os.fsync(handle.fileno())
            os.replace(scratch, target)
        finally:
            scratch.unlink(missing_ok=True)


def load_config(path, overrides: Sequence[str] = (), *,
                route_validator: Optional[Callable[[Mapping[str, Any]], Any]] = None) -> ResolvedConfig:
    source = Path(path).resolve()
    raw = source.read_bytes()
    tree = parse_text(raw, as_json=source.suffix.lower() == ".json", origin=str(source))
    if not isinstance(tree, dict):
        raise ConfigurationError(f"{source} must contain a YAML mapping")
    tree = normalise(tree, expand=True)
    for item in overrides:
        Override.parse(item).apply(tree)
    check_sections(tree)
    tree = normalise(tree, expand=False)          # override values get the same canonical-form check
    if route_validator is None:
        from .routes import validate_route as route_validator     # late: the route table imports nothing heavy either
    route_validator(tree)
    return ResolvedConfig(source, _digest(raw), _digest(canonical_json(tree)), tree)
