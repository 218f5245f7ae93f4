"""Lazy backend registry: a family name resolves to a module that exports
``create_backend(family=...)``; nothing heavy is imported until a backend is asked for
(reference: solar/backends/registry.py:13-61)."""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Mapping, Protocol, runtime_checkable

from .errors import BackendContractError


@dataclass(frozen=True)
class BackendSpec:
    family: str
    module: str
    factory: str = "create_backend"


@runtime_checkable
class Backend(Protocol):
    family: str

    def validate_config(self, config: Mapping[str, Any]) -> None: ...

    def train(self, config: Mapping[str, Any]) -> Mapping[str, Any]: ...

    def infer(self, config: Mapping[str, Any]) -> Mapping[str, Any]: ...

    def preencode(self, config: Mapping[str, Any]) -> Mapping[str, Any]: ...


_BUILTINS = {
    "wan22_ti2v_5b": BackendSpec("wan22_ti2v_5b", "solarwm_b200.backends.wan22"),
    "wan22_i2v_a14b": BackendSpec("wan22_i2v_a14b", "solarwm_b200.backends.wan22"),
    "ltx25_video": BackendSpec("ltx25_video", "solarwm_b200.backends.ltx25"),
    "minimax_h3": BackendSpec("minimax_h3", "solarwm_b200.backends.minimax_h3"),
}
_extra: dict[str, BackendSpec] = {}


def register_backend(spec: BackendSpec) -> None:
    _extra[spec.family] = spec


def backend_specs() -> tuple:
    return tuple({**_BUILTINS, **_extra}.values())


def load_backend(family: str) -> Backend:
    spec = {**_BUILTINS, **_extra}.get(family)
    if spec is None:
        raise BackendContractError(f"unknown backend family {family!r}")
    try:
        module = importlib.import_module(spec.module)
    except ImportError as exc:
        raise BackendContractError(f"backend {family!r} cannot be imported: {exc}") from exc
    factory = getattr(module, spec.factory, None)
    if factory is None:
        raise BackendContractError(f"{spec.module} does not export {spec.factory}")
    backend = factory(family=family)
    if getattr(backend, "family", None) != family:
        raise BackendContractError(f"{spec.module} returned a backend for {getattr(backend, 'family', None)!r}")
    return backend
