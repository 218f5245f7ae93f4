"""Backend boundary of the Wan2.2 families: route -> runtime dispatch
(reference: Wan22Backend, solar/backends/wan22/backend.py:38-191)."""
from __future__ import annotations

from typing import Any, Mapping

from ...config.routes import validate_route
from ...errors import BackendContractError
from .contracts import PROFILES, validate_wan_config


class Wan22Backend:
    def __init__(self, family: str):
        if family not in PROFILES:
            raise BackendContractError(f"not a Wan family: {family!r}")
        self.family = family

    def validate_config(self, config: Mapping[str, Any]) -> None:
        """Structural validation always; ``metadata.contract: release`` additionally holds the config to the pinned
        release recipe of the family (geometry, optimizer, EMA, sharding, initialisation)."""
        validate_wan_config(config, self.family)
        if str((config.get("metadata") or {}).get("contract", "structural")).lower() == "release":
            from .contracts import validate_release_recipe

            validate_release_recipe(config, self.family)

    def readiness(self, config: Mapping[str, Any], *, require_cuda: bool = False):
        """Dependencies, assets, architecture, weights, indexes, inference controls and the device in one report."""
        self.validate_config(config)
        from .readiness import probe_runtime

        return probe_runtime(config, family=self.family, require_cuda=require_cuda)

    def train(self, config: Mapping[str, Any]) -> Mapping[str, Any]:
        route = validate_route(config)
        from .readiness import require_training_runtime

        require_training_runtime(config, family=self.family)
        if route.stage == "stage0p5":
            from .runtime import run_training

            return run_training(config)
        if route.stage == "stage1":
            from .stage1 import run_stage1_training

            return run_stage1_training(config)
        if route.stage == "stage2":
            from .stage2 import run_stage2_training

            return run_stage2_training(config)
        raise BackendContractError(f"no Wan training runtime for route {route.key}")

    def infer(self, config: Mapping[str, Any]) -> Mapping[str, Any]:
        from .inference import run_inference

        return run_inference(config, self.family)

    def preencode(self, config: Mapping[str, Any]) -> Mapping[str, Any]:
        from .preencode import run_preencode

        return run_preencode(config, self.family)
