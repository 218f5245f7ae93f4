"""Wan checkpoints: one ``model.pt`` inside a checkpoint transaction with the keys
``generator`` (live weights), ``generator_ema``, ``optimizer``, ``scheduler``, ``global_step``,
``config``, ``ema_num_updates`` and ``rank_runtime_state`` (per raw rank RNG + reader cursor) --
the reference layout (solar/backends/wan22/runtime/checkpoint.py:986-1060).  Modes: ``weights_only``
restores the generator (optionally from EMA), ``full_resume`` restores everything and checks the
exact-resume contract.  Every load passes ``weights_only=True``."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from ...checkpoint.store import (CheckpointContract, CheckpointTransaction, assert_resume_compatible,
                                 verify_checkpoint)
from ...errors import CheckpointError
from ...runtime.output_layout import checkpoint_model_dir


def build_contract(config: Mapping[str, Any], route, sp_size: int) -> CheckpointContract:
    model, data = config.get("model", {}), config.get("data", {})
    return CheckpointContract(
        family=route.family, stage=route.stage, causal_mode=route.causal_mode, objective=route.objective,
        objective_variant=route.variant, camera_translation_transform=str(model.get("camera_translation_transform", "linear")),
        parameterization=str(config.get("train", {}).get("parameterization", "full")), sp_size=int(sp_size),
        data_generation=str(data.get("generation", data.get("source", "index"))),
        extras={"timestep_shift": float(model.get("timestep_shift", 5.0))})


def save_checkpoint(root, step: int, *, model, scheduler, contract: CheckpointContract, config,
                    ema_state: Optional[Mapping[str, Any]], ema_num_updates: int, rank_states, is_main: bool,
                    barrier=None, optimizer=None, optimizer_state=None, weights=None) -> str:
    """``optimizer_state``: the un-sharded ``optimizer.state_dict()`` gathered by the caller on every rank (a sharded
    optimizer's ``state_dict`` is a collective, so it cannot be called from the main rank alone); ``optimizer`` is
    accepted for single-rank callers and read here.  ``weights``: the full name -> tensor mapping when the model's
    parameters are sharded (``ShardedParameters.materialize``); default ``model.state_dict()``."""
    if optimizer_state is None and is_main:
        if optimizer is None:
            raise CheckpointError("save_checkpoint needs optimizer_state (or an unsharded optimizer)")
        if getattr(optimizer, "shard_world", 1) != 1:
            raise CheckpointError("a sharded optimizer's state must be gathered by every rank before saving")
        optimizer_state = optimizer.state_dict()
    target = checkpoint_model_dir(root, step)
    ident = ""
    if is_main:
        with CheckpointTransaction(target) as tx:
            payload = {
                "generator": {k: v.detach().cpu() for k, v in (weights if weights is not None else model.state_dict()).items()},
                "generator_ema": None if ema_state is None else {k: v.detach().cpu() for k, v in ema_state.items()},
                "optimizer": optimizer_state,
                "scheduler": scheduler.state_dict(),
                "global_step": int(step),
                "config": dict(config),
                "ema_num_updates": int(ema_num_updates),
                "rank_runtime_state": list(rank_states),
            }
            torch.save(payload, tx.path / "model.pt")
            done = tx.commit(step=step, contract=contract, required_components=["model.pt"],
                             metadata={"ema_num_updates": int(ema_num_updates)})
            ident = done.manifest_digest
    if barrier is not None:
        ident = barrier(ident)
    return ident or verify_checkpoint(target).manifest_digest


def load_checkpoint(path, *, model, optimizer=None, scheduler=None, mode: str = "weights_only",
                    expected: Optional[CheckpointContract] = None, weight_source: str = "live", map_location="cpu"):
    verified = verify_checkpoint(path)
    if mode == "full_resume":
        if expected is None:
            raise CheckpointError("full_resume needs the expected checkpoint contract")
        assert_resume_compatible(expected, verified.contract)
    payload = torch.load(Path(path) / "model.pt", map_location=map_location, weights_only=True)
    weights = payload["generator_ema"] if (weight_source == "ema" and payload.get("generator_ema")) else payload["generator"]
    provider = getattr(model, "param_provider", None)
    if provider is not None:
        try:
            provider.load_state(model, weights)               # sharded parameters: every rank keeps its own slice
        except (KeyError, ValueError) as exc:
            raise CheckpointError(str(exc)) from exc
    else:
        missing = model.load_state_dict(weights, strict=True)
        if missing.missing_keys or missing.unexpected_keys:
            raise CheckpointError(f"checkpoint weights do not match the model: {missing}")
    if mode == "full_resume":
        if optimizer is not None:
            optimizer.load_state_dict(payload["optimizer"])
        if scheduler is not None:
            scheduler.load_state_dict(payload["scheduler"])
    return verified, payload
