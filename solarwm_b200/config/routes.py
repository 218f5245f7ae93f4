"""Supported (family, stage, causal mode, objective, variant) routes and their data gates.

Same public table as the reference (solar/config/routes.py:11-122): nine training routes over four
families, pixel-frame gates per family/stage, and the camera translation transform check.  Unlike
the reference's backend contracts, sequence-parallel sizes are NOT pinned per family here: any SP
size that divides the head count is accepted.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..errors import ConfigurationError

FAMILY_ALIASES = {
    "wan22_ti2v_5b": "wan22_ti2v_5b", "wan2.2-ti2v-5b": "wan22_ti2v_5b",
    "wan22_i2v_a14b": "wan22_i2v_a14b", "wan2.2-i2v-a14b": "wan22_i2v_a14b",
    "ltx25_video": "ltx25_video", "ltx-2.5": "ltx25_video",
    "minimax_h3": "minimax_h3", "minimax-h3": "minimax_h3",
}


@dataclass(frozen=True, order=True)
class Route:
    family: str
    stage: str
    causal_mode: str
    objective: str
    variant: str = ""

    @property
    def key(self) -> str:
        tail = f":{self.variant}" if self.variant else ""
        return f"{self.family}:{self.stage}:{self.causal_mode}:{self.objective}{tail}"


_TABLE = frozenset({
    Route("wan22_ti2v_5b", "stage0p5", "bidirectional", "flow_matching"),
    Route("wan22_ti2v_5b", "stage1", "teacher_forcing", "flow_matching"),
    Route("wan22_ti2v_5b", "stage1", "teacher_forcing", "anyflow_forward_map", "v1_5"),
    Route("wan22_ti2v_5b", "stage2", "self_gradient_forcing", "flow_matching"),
    Route("wan22_i2v_a14b", "stage0p5", "bidirectional", "flow_matching"),
    Route("ltx25_video", "stage0p5", "bidirectional", "native_rectified_flow"),
    Route("minimax_h3", "stage0p5", "bidirectional", "flow_matching"),
    Route("minimax_h3", "stage1", "teacher_forcing", "anyflow_forward_map", "v1_5"),
    Route("minimax_h3", "stage2", "self_gradient_forcing", "flow_matching"),
})

_FRAME_GATES = {
    "wan22_ti2v_5b": lambda stage: {81, 153} if stage == "stage0p5" else {81},
    "wan22_i2v_a14b": lambda stage: {81, 153} if stage == "stage0p5" else {81},
    "ltx25_video": lambda stage: {153},
    "minimax_h3": lambda stage: {158},
}


def _section(config: Mapping[str, Any], key: str) -> Mapping[str, Any]:
    value = config.get(key, {})
    if not isinstance(value, Mapping):
        raise ConfigurationError(f"{key} must be a mapping")
    return value


def _family(config: Mapping[str, Any]) -> str:
    raw = str(_section(config, "model").get("family", "")).strip().lower()
    if raw not in FAMILY_ALIASES:
        raise ConfigurationError(f"unsupported model.family {raw!r}")
    return FAMILY_ALIASES[raw]


def resolve_route(config: Mapping[str, Any]) -> Route:
    model, train = _section(config, "model"), _section(config, "train")
    family = _family(config)
    stage = str(train.get("stage", model.get("stage", ""))).strip().lower()
    causal = str(train.get("causal_mode", "")).strip().lower()
    objective = str(train.get("objective", "")).strip().lower()
    variant = str(train.get("objective_variant", "")).strip().lower()
    if objective == "anyflow_forward_map" and not variant:
        variant = "v1_5"
    if family == "ltx25_video" and objective == "flow_matching":
        objective = "native_rectified_flow"
    return Route(family, stage, causal, objective, variant)


def validate_route(config: Mapping[str, Any]) -> Route:
    if str(config.get("action", "")).lower() == "preencode":
        return Route(_family(config), "preencode", "none", "none")
    route = resolve_route(config)
    if route not in _TABLE:
        allowed = sorted(r.key for r in _TABLE if r.family == route.family)
        raise ConfigurationError(f"unsupported route {route.key!r}; allowed for {route.family}: {allowed}")
    frames = int(_section(config, "data").get("pixel_frames", 0))
    allowed_frames = _FRAME_GATES[route.family](route.stage)
    if frames not in allowed_frames:
        raise ConfigurationError(f"{route.family} {route.stage} requires pixel_frames in "
                                 f"{sorted(allowed_frames)}, got {frames}")
    transform = str(_section(config, "model").get("camera_translation_transform", "linear")).lower()
    if transform not in ("linear", "logd4"):
        raise ConfigurationError("camera_translation_transform must be linear or logd4")
    if route.family == "minimax_h3" and transform != "logd4":
        raise ConfigurationError("MiniMax-H3 requires logd4")
    return route


def supported_routes():
    return tuple(sorted(_TABLE))
