"""Allocation-free validation of every Wan config section, run before any process group or model
exists (reference: solar/backends/wan22/contracts.py:21-746).  Differences from the reference are
deliberate: the sequence-parallel size is NOT pinned per family (any divisor of the head count and
of the world size is accepted) and ``data.source: synthetic`` is a first-class input mode."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ...errors import ConfigurationError
from ...models.wan import WanConfig, wan_preset


@dataclass(frozen=True)
class FamilyProfile:
    family: str
    preset: str
    latent_channels: int
    vae_stride: tuple          # (temporal, height, width)
    default_shift: float


PROFILES = {
    "wan22_ti2v_5b": FamilyProfile("wan22_ti2v_5b", "ti2v_5b", 48, (4, 16, 16), 5.0),
    "wan22_i2v_a14b": FamilyProfile("wan22_i2v_a14b", "i2v_a14b", 16, (4, 8, 8), 5.0),
}
_STRATEGIES = ("FULL_SHARD", "HYBRID_SHARD", "SHARD_GRAD_OP", "NO_SHARD")


def _map(cfg, key, required=True) -> Mapping[str, Any]:
    v = cfg.get(key)
    if v is None and not required:
        return {}
    if not isinstance(v, Mapping):
        raise ConfigurationError(f"{key} must be a mapping")
    return v


def _pos_int(section, key, default=None, minimum=1) -> int:
    v = section.get(key, default)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigurationError(f"{key} must be an integer >= {minimum}, got {v!r}")
    return v


def architecture(config: Mapping[str, Any]) -> WanConfig:
    model = _map(config, "model")
    family = str(model.get("family"))
    arch = model.get("architecture")
    if arch is None or isinstance(arch, str):
        base = wan_preset(arch or PROFILES[family].preset)
    elif isinstance(arch, Mapping):
        base = WanConfig(**{**wan_preset(PROFILES[family].preset).to_dict(), **dict(arch),
                            "patch_size": tuple(arch.get("patch_size", (1, 2, 2)))})
    else:
        raise ConfigurationError("model.architecture must be a preset name or a mapping")
    if str(_map(config, "train", required=False).get("objective", "")) == "anyflow_forward_map":
        base.flow_objective = "anyflow_forward_map"
    return base


def latent_frames(pixel_frames: int, temporal_stride: int) -> int:
    return (pixel_frames - 1) // temporal_stride + 1


def validate_wan_config(config: Mapping[str, Any], family: str) -> None:
    if family not in PROFILES:
        raise ConfigurationError(f"not a Wan family: {family!r}")
    model, data = _map(config, "model"), _map(config, "data")
    dist_cfg = _map(config, "distributed", required=False)
    arch = architecture(config)
    sp = _pos_int(dist_cfg, "sequence_parallel_size", 1)
    world = _pos_int(dist_cfg, "world_size", sp)
    if world % sp != 0:
        raise ConfigurationError("distributed.world_size must be a multiple of sequence_parallel_size")
    if arch.num_heads % sp != 0:
        raise ConfigurationError(f"sequence_parallel_size {sp} must divide num_heads {arch.num_heads}")
    if dist_cfg.get("sp_peers_share_sample", True) is not True or dist_cfg.get("sp_peers_share_rng", True) is not True:
        raise ConfigurationError("SP peers must share samples and RNG")
    shift = float(model.get("timestep_shift", PROFILES[family].default_shift))
    if not shift > 0:
        raise ConfigurationError("model.timestep_shift must be positive")
    source = str(data.get("source", "index"))
    if source not in ("synthetic", "index"):
        raise ConfigurationError("data.source must be 'synthetic' or 'index'")
    if source == "index" and not data.get("index"):
        raise ConfigurationError("data.index is required unless data.source is synthetic")
    _pos_int(data, "pixel_frames")
    if str(config.get("action")) == "train":
        train = _map(config, "train")
        micro = _pos_int(train, "micro_batch_size", 1)
        accum = _pos_int(train, "grad_accum", train.get("gradient_accumulation_steps", 1))
        gbs = train.get("global_batch_size")
        if gbs is not None and int(gbs) != (world // sp) * micro * accum:
            raise ConfigurationError(f"train.global_batch_size must equal DP*micro*accum = {(world // sp) * micro * accum}")
        _pos_int(train, "max_steps")
        _pos_int(train, "warmup_steps", 0, minimum=0)
        opt = _map(train, "optimizer", required=False)
        if opt and not float(opt.get("lr", 1e-4)) > 0:
            raise ConfigurationError("train.optimizer.lr must be positive")
        fsdp = _map(train, "fsdp", required=False)
        if fsdp and str(fsdp.get("strategy", fsdp.get("sharding_strategy", "FULL_SHARD"))) not in _STRATEGIES:
            raise ConfigurationError(f"train.fsdp.strategy must be one of {_STRATEGIES}")
        ckpt = _map(config, "checkpoint", required=False)
        if ckpt and str(ckpt.get("mode", "none")) not in ("none", "weights_only", "full_resume"):
            raise ConfigurationError("checkpoint.mode must be none, weights_only or full_resume")
    if not _map(config, "runtime").get("output_dir"):
        raise ConfigurationError("runtime.output_dir is required")
