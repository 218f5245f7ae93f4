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


_WRAPPER_SEGMENTS = ("_fsdp_wrapped_module", "_checkpoint_wrapped_module", "_orig_mod")


def normalize_weight_names(state: Mapping[str, Any], field: str = "generator") -> dict:
    """Parameter names as this package spells them: an optional root ``model.`` namespace is removed (it must be on
    every key or on none), wrapper segments that sharding / checkpointing / compilation wrappers insert are dropped,
    and the result may not collide (reference: normalize_model_state, _strip_parameter_wrapper_segments,
    solar/backends/wan22/runtime/checkpoint.py:126-228)."""
    if not isinstance(state, Mapping) or not state:
        raise CheckpointError(f"checkpoint field {field} must be a non-empty mapping")
    rooted = [isinstance(k, str) and k.startswith("model.") for k in state]
    if any(rooted) and not all(rooted):
        raise CheckpointError(f"checkpoint field {field} mixes model-prefixed and plain parameter names")
    out = {}
    for key, value in state.items():
        if not isinstance(key, str) or not key:
            raise CheckpointError(f"checkpoint field {field} has a non-string key")
        name = key[len("model."):] if rooted[0] else key
        name = ".".join(part for part in name.split(".") if part not in _WRAPPER_SEGMENTS)
        if name in out:
            raise CheckpointError(f"checkpoint field {field}: {key!r} collides with another key after normalisation")
        out[name] = value
    return out


def named_optimizer_moments(state: Mapping[str, Any]):
    """A ``torch.optim.AdamW``-style full state whose entries are keyed by parameter NAME
    (``{"state": {name: {"step", "exp_avg", "exp_avg_sq"}}, "param_groups": [{"params": [names], ...}]}``, the
    reference's checkpoint form) -> (``{name: {"exp_avg", "exp_avg_sq"}}``, step) with the names normalised like the
    weights.  The slot names and the group names must agree and every entry must be at the same step."""
    slots, groups = state.get("state"), state.get("param_groups")
    if not isinstance(slots, Mapping) or not isinstance(groups, (list, tuple)):
        raise CheckpointError("optimizer state is incomplete (state / param_groups)")
    if not all(isinstance(k, str) for k in slots):
        raise CheckpointError("optimizer state must name its parameters")
    named = normalize_weight_names(slots, "optimizer.state")
    listed = normalize_weight_names({n: None for g in groups for n in g.get("params", ())}, "optimizer.param_groups")
    if set(named) != set(listed):
        odd = sorted(set(named) ^ set(listed))
        raise CheckpointError(f"optimizer slot and group names differ after normalisation (e.g. {odd[:4]})")
    steps = {int(v["step"]) for v in named.values()}
    if len(steps) != 1:
        raise CheckpointError(f"optimizer entries are at different steps: {sorted(steps)[:4]}")
    return {n: {"exp_avg": v["exp_avg"], "exp_avg_sq": v["exp_avg_sq"]} for n, v in named.items()}, steps.pop()


def upgrade_flow_matching_to_anyflow(weights: Mapping[str, Any], model) -> tuple:
    """Flow-matching weights into a model with the AnyFlow ``delta_embedding``: the ONLY tensors the source may lack
    are the four ``delta_embedding.*`` ones, each of which starts as a copy of its ``time_embedding.*`` counterpart;
    anything else must match exactly.  Returns (upgraded mapping, names that were initialised) (reference:
    _load_stage0p5_state_into_anyflow, solar/backends/wan22/runtime/checkpoint.py:419-452)."""
    wanted = {n for n, _ in model.named_parameters()}
    delta = sorted(n for n in wanted if n.startswith("delta_embedding."))
    time_keys = sorted(n for n in weights if n.startswith("time_embedding."))
    if len(delta) != 4 or len(time_keys) != 4 or any(n in weights for n in delta):
        raise CheckpointError("flow-matching -> AnyFlow initialisation permits exactly four missing delta_embedding "
                              "tensors and no delta state in the source")
    out = dict(weights)
    for t in time_keys:
        out[t.replace("time_embedding.", "delta_embedding.", 1)] = weights[t].detach().clone()
    if set(out) != wanted:
        odd = sorted(set(out) ^ wanted)
        raise CheckpointError(f"flow-matching -> AnyFlow initialisation: other names differ too (e.g. {odd[:4]})")
    return out, tuple(delta)


def load_checkpoint(path, *, model, optimizer=None, scheduler=None, mode: str = "weights_only",
                    expected: Optional[CheckpointContract] = None, weight_source: str = "live", map_location="cpu",
                    ema_source: Optional[str] = None):
    """``mode``: "weights_only" (the weights named by ``weight_source``: "live" or "ema"; optimizer moments and step
    start fresh, its master copies and EMA shadow are re-based on the loaded weights; ``ema_source`` = "ema" seeds the
    shadow from the checkpoint's averaged weights instead: the LIVE + EMA start of a fine-tune) or "full_resume".
    A flow-matching checkpoint loads into an AnyFlow model through ``upgrade_flow_matching_to_anyflow``."""
    verified = verify_checkpoint(path)
    if mode == "full_resume":
        if expected is None:
            raise CheckpointError("full_resume needs the expected checkpoint contract")
        assert_resume_compatible(expected, verified.contract)
    payload = torch.load(Path(path) / "model.pt", map_location=map_location, weights_only=True)
    if int(payload.get("global_step", verified.step)) != verified.step:
        raise CheckpointError("the payload's step differs from its manifest")
    weights = payload["generator_ema"] if (weight_source == "ema" and payload.get("generator_ema")) else payload["generator"]
    weights = normalize_weight_names(weights, "generator_ema" if weight_source == "ema" else "generator")
    initialised = ()
    wanted = {n for n, _ in model.named_parameters()}
    if mode == "weights_only" and any(n.startswith("delta_embedding.") for n in wanted - set(weights)):
        weights, initialised = upgrade_flow_matching_to_anyflow(weights, model)
    payload["initialised_from_time_embedding"] = initialised
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
            saved = payload["optimizer"]
            if "units" in saved:
                optimizer.load_state_dict(saved)
            else:                                  # a name-keyed AdamW state (the reference's checkpoints)
                moments, step = named_optimizer_moments(saved)
                optimizer.adopt_live_weights(reset_ema=False)
                optimizer.load_named_moments(model, moments, step)
                if payload.get("generator_ema") and getattr(optimizer, "ema_decay", None) is not None:
                    optimizer.load_named_ema(model, normalize_weight_names(payload["generator_ema"], "generator_ema"))
        if scheduler is not None:
            scheduler.load_state_dict(payload["scheduler"])
    elif optimizer is not None and hasattr(optimizer, "adopt_live_weights"):
        optimizer.adopt_live_weights(reset_ema=True)
        if ema_source == "ema":
            if not payload.get("generator_ema"):
                raise CheckpointError("the checkpoint holds no averaged weights to seed the EMA from")
            optimizer.load_named_ema(model, normalize_weight_names(payload["generator_ema"], "generator_ema"))
    return verified, payload
