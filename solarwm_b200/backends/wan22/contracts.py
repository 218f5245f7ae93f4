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
    mode = model.get("camera_attention_mode")
    if mode is not None:                       # the reference spells the parallel branch's default by name
        if mode not in ("none", "fused_prope", "parallel"):
            raise ConfigurationError(f"model.camera_attention_mode must be none, fused_prope or parallel, not {mode!r}")
        base.camera_attention_mode = str(mode)
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


# =====================================================================================================================
# Release recipes: the pinned form of a Wan config
# =====================================================================================================================
# ``validate_wan_config`` above is structural: it accepts any architecture, shape and parallel layout that the runtime
# can execute (tests, benchmarks, synthetic data).  A *release recipe* is narrower: the published Wan camera models
# were trained with fixed geometry, optimizer, EMA, sharding and initialisation settings, and a config that claims to
# reproduce one (``metadata.contract: release``) is held to those values one by one, before any device or model
# exists.  The pins are data -- the tables below -- evaluated by one small engine; each entry names the dotted path,
# what it must equal (a value, or a function of the context) and, optionally, when it applies.  What the pins say comes
# from the reference's recipe contract (solar/backends/wan22/contracts.py:21-76, 294-343, 427-560, 562-706); one
# deliberate difference: ``distributed.sequence_parallel_size`` may be any divisor of the head count when
# ``distributed.allow_sequence_parallel_override`` is true (the reference pins 1 for the 5B family and 2 for A14B),
# and the expected whole-frame splits are then computed for that size.
import math as _math
from pathlib import PurePosixPath as _PurePosixPath
from typing import Callable, Optional, Sequence, Tuple

from ...errors import BackendContractError


@dataclass(frozen=True)
class ReleaseProfile:
    family: str
    model_name: str
    timestep_shift: float
    latent_channels: int
    height: int
    width: int
    latent_height: int
    latent_width: int
    frame_sequence_length: int          # tokens per latent frame after the 1 x 2 x 2 patch
    sequence_parallel_size: int
    fsdp_strategy: str
    num_heads: int


RELEASE_PROFILES = {
    "wan22_ti2v_5b": ReleaseProfile("wan22_ti2v_5b", "Wan2.2-TI2V-5B-Camera", 5.0, 48, 480, 864, 30, 54, 405, 1,
                                    "HYBRID_SHARD", 24),
    "wan22_i2v_a14b": ReleaseProfile("wan22_i2v_a14b", "Wan2.2-I2V-A14B-High-Camera", 3.0, 16, 480, 832, 60, 104, 1560, 2,
                                     "FULL_SHARD", 40),
}
TI2V_720P_153F_SCHEMA = "solarwm.wan22_ti2v_5b.720p.153f.v1"
TI2V_720P_153F_PROFILE = ReleaseProfile("wan22_ti2v_5b", "Wan2.2-TI2V-5B-Camera", 5.0, 48, 704, 1280, 44, 80, 880, 1,
                                        "HYBRID_SHARD", 24)
_MISSING = object()


def release_profile(config: Mapping[str, Any], family: str) -> ReleaseProfile:
    data = config.get("data") or {}
    if family == "wan22_ti2v_5b" and str(data.get("encoding", "")).lower() == "preencoded" \
            and str(data.get("preencode_schema", "")) == TI2V_720P_153F_SCHEMA:
        return TI2V_720P_153F_PROFILE
    return RELEASE_PROFILES[family]


def pixel_to_latent_frames(pixel_frames) -> int:
    if isinstance(pixel_frames, bool) or not isinstance(pixel_frames, int) or pixel_frames < 1 or (pixel_frames - 1) % 4:
        raise BackendContractError("Wan pixel frames must satisfy pixel_frames = 1 + 4*(latent_frames-1)")
    return 1 + (pixel_frames - 1) // 4


def whole_frame_splits(latent_frame_count: int, sp: int) -> Tuple[int, ...]:
    """Frames per SP rank under whole-frame sharding (the first ``F mod sp`` ranks hold one more)."""
    base, extra = divmod(int(latent_frame_count), int(sp))
    return tuple(base + (1 if r < extra else 0) for r in range(sp))


class _Ctx:
    """What the pin tables can see: the config, its route and profile, and a few derived quantities."""

    def __init__(self, config, route, profile: ReleaseProfile):
        self.config, self.route, self.profile = config, route, profile
        self.action = str(config.get("action", "")).strip().lower()
        data = config.get("data") or {}
        self.pixel_frames = data.get("pixel_frames")
        self.latent_frames = pixel_to_latent_frames(self.pixel_frames)
        self.encoding = str(data.get("encoding", "")).strip().lower()
        inference = config.get("inference") or {}
        self.camera_length = self.action == "infer" and str(inference.get("length", "fixed")).strip().lower() == "camera"
        dist_cfg = config.get("distributed") or {}
        self.sp = dist_cfg.get("sequence_parallel_size")
        self.sp_override = bool(dist_cfg.get("allow_sequence_parallel_override", False))
        self.checkpoint_mode = str((config.get("checkpoint") or {}).get("mode", "")).strip().lower()

    def get(self, dotted: str):
        node = self.config
        for part in dotted.split("."):
            if not isinstance(node, Mapping) or part not in node:
                return _MISSING
            node = node[part]
        return node


@dataclass(frozen=True)
class Pin:
    path: str
    expect: Any                                            # a value, or callable(ctx) -> value
    when: Optional[Callable[["_Ctx"], bool]] = None
    test: Optional[Callable[[Any, Any], bool]] = None      # default: typed equality (an int pin refuses True / "3")
    note: str = ""

    def check(self, ctx: "_Ctx") -> Optional[str]:
        if self.when is not None and not self.when(ctx):
            return None
        want = self.expect(ctx) if callable(self.expect) else self.expect
        got = ctx.get(self.path)
        ok = self.test(got, want) if self.test is not None else _same(got, want)
        if ok:
            return None
        shown = "<missing>" if got is _MISSING else repr(got)
        return f"{self.path} must be {want!r}{' (' + self.note + ')' if self.note else ''}, got {shown}"


def _same(got, want) -> bool:
    if got is _MISSING:
        return False
    if isinstance(want, bool):
        return got is want
    if isinstance(want, int):
        return isinstance(got, int) and not isinstance(got, bool) and got == want
    if isinstance(want, float):
        return isinstance(got, (int, float)) and not isinstance(got, bool) and _math.isfinite(float(got)) and float(got) == want
    if isinstance(want, (list, tuple)):
        return isinstance(got, (list, tuple)) and list(got) == list(want)
    return got == want


def _one_of(*allowed):
    return lambda got, _want: got is not _MISSING and got in allowed


def _absolute(got, _want) -> bool:
    return isinstance(got, str) and got.startswith("/")


def _relative_posix(got, _want) -> bool:
    if not isinstance(got, str) or not got or got.startswith("/") or "://" in got or "\\" in got:
        return False
    return all(part not in ("", ".", "..") for part in _PurePosixPath(got).parts)


def _positive_int(got, _want) -> bool:
    return isinstance(got, int) and not isinstance(got, bool) and got > 0


_stage = lambda *names: (lambda c: c.route.stage in names)                      # noqa: E731
_training = lambda c: c.action == "train"                                       # noqa: E731
_a14b = lambda c: c.profile.family == "wan22_i2v_a14b"                          # noqa: E731
_anyflow = lambda c: c.route.stage == "stage1" and c.route.objective == "anyflow_forward_map"   # noqa: E731
_init_from_checkpoint = lambda c: c.checkpoint_mode in ("weights_only", "full_resume")          # noqa: E731

MODEL_PINS: Sequence[Pin] = (
    Pin("model.family", lambda c: c.profile.family),
    Pin("model.name", lambda c: c.profile.model_name),
    Pin("model.timestep_shift", lambda c: c.profile.timestep_shift),
    Pin("model.latent_channels", lambda c: c.profile.latent_channels),
    Pin("model.frame_sequence_length", lambda c: c.profile.frame_sequence_length),
    Pin("model.camera_attention_mode", "fused_prope"),
    Pin("model.camera_translation_transform", "linear or logd4", test=_one_of("linear", "logd4")),
    Pin("model.causal", lambda c: c.route.stage in ("stage1", "stage2"), note="causal exactly for stage1 / stage2"),
    Pin("model.base_path", "an absolute path", test=_absolute),
    Pin("model.num_output_frames", lambda c: c.latent_frames, note="data.latent_frames"),
    Pin("model.num_frame_per_block", 3),
    Pin("model.local_attn_size", lambda c: c.latent_frames if _a14b(c) else 21, when=_stage("stage0p5", "stage1")),
    Pin("model.use_echorope", False, when=_stage("stage1")),
    Pin("model.max_prior_clean_chunks", 5, when=_stage("stage1"), note="six-chunk context"),
)
DATA_PINS: Sequence[Pin] = (
    Pin("data.encoding", "online or preencoded", test=_one_of("online", "preencoded")),
    Pin("data.latent_frames", lambda c: c.latent_frames, note="1 + (pixel_frames - 1) / 4"),
    Pin("data.height", lambda c: c.profile.height),
    Pin("data.width", lambda c: c.profile.width),
    Pin("data.max_rel_translation", 20.0),
    Pin("data.max_camera_abs", 20.0),
    Pin("data.streaming_index", True),
    Pin("data.random_start", lambda c: c.pixel_frames == 81 and c.encoding == "online" and not c.camera_length,
        note="random starts only for online 81-frame training"),
    Pin("data.train_index", "a relative POSIX path", test=_relative_posix),
    Pin("data.test_index", "a relative POSIX path", test=_relative_posix),
    Pin("data.partition_mode", "node_shard"),
    Pin("data.num_workers", "a positive integer", test=_positive_int),
    Pin("data.camera_array_key", "c2w", when=lambda c: c.encoding == "online"),
    Pin("data.pixel_frames", 81, when=_stage("stage1", "stage2"), note="stage1 / stage2 train on 81 frames"),
    Pin("data.transport.kind", "local or gcs", test=_one_of("local", "gcs")),
)
DISTRIBUTED_PINS: Sequence[Pin] = (
    Pin("distributed.world_size", "a positive integer", test=_positive_int),
    Pin("distributed.sequence_parallel_size", lambda c: c.profile.sequence_parallel_size,
        when=lambda c: not c.sp_override, note="set distributed.allow_sequence_parallel_override to lift"),
    Pin("distributed.sample_sharding", "logical_dp"),
    Pin("distributed.rng_scope", "logical_dp", note="SP peers share randomness"),
    Pin("distributed.sequence_layout", "whole_frame_uneven", when=_a14b),
    Pin("distributed.sp_frame_splits", lambda c: list(whole_frame_splits(c.latent_frames, c.sp)), when=_a14b),
    Pin("distributed.sp_token_splits",
        lambda c: [n * c.profile.frame_sequence_length for n in whole_frame_splits(c.latent_frames, c.sp)], when=_a14b),
)
TRAIN_PINS: Sequence[Pin] = (
    Pin("train.timestep_mode", lambda c: "uniform_per_video" if c.route.stage == "stage0p5" else "per_block"),
    Pin("train.num_train_timesteps", 1000),
    Pin("train.i2v_image_condition_dropout", lambda c: 0.0 if c.route.stage == "stage2" else 0.1),
    Pin("train.optimizer.lr", lambda c: 2.0e-6 if c.route.stage == "stage2" else 5.0e-5),
    Pin("train.optimizer.betas", lambda c: [0.0, 0.999] if c.route.stage == "stage2" else [0.9, 0.95]),
    Pin("train.fsdp.strategy", lambda c: c.profile.fsdp_strategy),
    Pin("train.fsdp.param_dtype", "bfloat16"),
    Pin("train.fsdp.reduce_dtype", "float32"),
    Pin("train.noise_augmentation_max_timestep", 0, when=_stage("stage1"), note="clean context"),
    Pin("train.ema.enabled", True),
    Pin("train.ema.device", "cuda"),
    Pin("train.ema.dtype", "float32"),
    Pin("train.ema.sharded", True),
    Pin("train.ema.decay", 0.99, when=_stage("stage2")),
    Pin("train.ema.start_step", 39, when=_stage("stage2"), note="after student update 39"),
    Pin("train.ema.decay", 0.999, when=_anyflow),
    Pin("train.ema.warmup_steps", 1000, when=_anyflow),
    Pin("train.ema.decay", "0.999 or 0.9999", when=_stage("stage0p5"), test=_one_of(0.999, 0.9999)),
    Pin("train.ema.warmup_steps", 500, when=lambda c: c.route.stage == "stage0p5" and c.get("train.ema.decay") == 0.999),
    Pin("train.ema.decay", 0.9999, when=lambda c: c.route.stage == "stage1" and not _anyflow(c)),
    Pin("train.ema.start_step", 0, when=_stage("stage0p5", "stage1")),
)
CHECKPOINT_PINS: Sequence[Pin] = (
    Pin("checkpoint.mode", "none, weights_only, full_resume or stage2_roles", when=_training,
        test=_one_of("none", "weights_only", "full_resume", "stage2_roles")),
    Pin("checkpoint.mode", "weights_only or full_resume", when=lambda c: _training(c) and c.route.stage == "stage1",
        test=_one_of("weights_only", "full_resume"), note="stage1 starts from stage0.5 weights or resumes"),
    Pin("checkpoint.mode", "stage2_roles", when=lambda c: _training(c) and c.route.stage == "stage2"),
    Pin("checkpoint.mode", "weights_only or full_resume", test=_one_of("weights_only", "full_resume"),
        when=lambda c: _training(c) and c.route.stage == "stage0p5" and c.pixel_frames == 153,
        note="153-frame training continues an 81-frame model"),
    Pin("checkpoint.path", "an absolute path", test=_absolute, when=lambda c: _training(c) and _init_from_checkpoint(c)),
    Pin("checkpoint.path", "an absolute path", test=_absolute, when=lambda c: c.action == "infer"),
    Pin("checkpoint.source_contract.stage", lambda c: c.route.stage if c.checkpoint_mode == "full_resume" else "stage0p5",
        when=lambda c: _training(c) and _init_from_checkpoint(c)),
    Pin("checkpoint.source_contract.objective",
        lambda c: str(c.get("train.objective")) if c.checkpoint_mode == "full_resume" else "flow_matching",
        when=lambda c: _training(c) and _init_from_checkpoint(c)),
    Pin("checkpoint.resume_step", "a positive integer", test=_positive_int,
        when=lambda c: _training(c) and c.checkpoint_mode == "full_resume"),
    Pin("checkpoint.weights", "ema", when=lambda c: _training(c) and c.checkpoint_mode == "weights_only" and c.route.stage == "stage1"),
    Pin("checkpoint.source_step", "a positive integer", test=_positive_int,
        when=lambda c: _training(c) and c.checkpoint_mode == "weights_only"),
    Pin("checkpoint.weights", "[live, ema] or [ema, ema]",
        test=lambda got, _w: got is not _MISSING and list(got) in (["live", "ema"], ["ema", "ema"]) if not isinstance(got, str) else False,
        when=lambda c: _training(c) and c.checkpoint_mode == "weights_only" and c.route.stage == "stage0p5"),
    Pin("checkpoint.weights", "live or ema", test=_one_of("live", "ema"),
        when=lambda c: c.action == "infer" and not c.camera_length),
)
RELEASE_PIN_TABLES = (("model", MODEL_PINS), ("data", DATA_PINS), ("distributed", DISTRIBUTED_PINS),
                      ("train", TRAIN_PINS), ("checkpoint", CHECKPOINT_PINS))
_ASSET_NAMES = ("text_encoder", "tokenizer", "transformer_config", "transformer_weights", "vae")


def _cross_field_problems(ctx: "_Ctx") -> list:
    """Constraints that tie several fields together (not expressible as one pinned path)."""
    out = []
    cfg = ctx.config
    dist_cfg, train = cfg.get("distributed") or {}, cfg.get("train") or {}
    world, sp = dist_cfg.get("world_size"), ctx.sp
    if _positive_int(world, None) and _positive_int(sp, None):
        if world % sp:
            out.append("distributed.world_size must divide evenly by sequence_parallel_size")
        elif ctx.profile.num_heads % sp:
            out.append(f"sequence_parallel_size {sp} must divide the {ctx.profile.num_heads} attention heads")
        elif ctx.action == "train":
            micro, accum = train.get("micro_batch_size"), train.get("grad_accum")
            if _positive_int(micro, None) and _positive_int(accum, None):
                want = world // sp * micro * accum
                if train.get("global_batch_size") != want:
                    out.append(f"train.global_batch_size must equal DP*micro*grad_accum={want}")
            else:
                out.append("train.micro_batch_size and train.grad_accum must be positive integers")
    assets = (cfg.get("model") or {}).get("assets")
    if not isinstance(assets, Mapping) or sorted(assets) != sorted(_ASSET_NAMES):
        out.append(f"model.assets fields must be exactly {sorted(_ASSET_NAMES)}")
    else:
        for name in _ASSET_NAMES:
            value = str(assets[name]).strip()
            if name == "transformer_config" and value == "builtin":
                continue
            parts = [p for p in _PurePosixPath(value).parts if p != "/"]
            if not value or "://" in value or "\\" in value or any(p in ("", ".", "..") for p in parts):
                out.append(f"model.assets.{name} must be an absolute or base-relative POSIX path")
    transport = (cfg.get("data") or {}).get("transport") or {}
    kind, root = str(transport.get("kind", "")).lower(), str(transport.get("root", ""))
    if kind == "local" and not root.startswith("/"):
        out.append("local data.transport.root must be absolute")
    if kind == "gcs":
        if not root.startswith("gs://"):
            out.append("gcs data.transport.root must be a gs:// URI")
        if not str(transport.get("cache_dir", "")).startswith("/"):
            out.append("gcs data.transport.cache_dir must be absolute")
        if not _positive_int(transport.get("cache_max_gib"), None):
            out.append("data.transport.cache_max_gib must be positive")
    runtime = cfg.get("runtime") or {}
    overrides = [runtime.get(k) for k in ("data_cache_dir", "data_cache_max_gib", "validation_cache_dir", "validation_cache_max_gib")]
    if kind != "gcs" and any(v is not None for v in overrides):
        out.append("runtime cache overrides are valid only for gcs data transport")
    if (runtime.get("validation_cache_dir") is None) != (runtime.get("validation_cache_max_gib") is None):
        out.append("runtime validation cache directory and size must be configured together")
    source = (cfg.get("checkpoint") or {}).get("source_contract")
    if isinstance(source, Mapping):
        now = str((cfg.get("model") or {}).get("camera_translation_transform", "linear"))
        before = str(source.get("camera_translation_transform", "linear"))
        if now != before and not (ctx.checkpoint_mode == "weights_only"
                                  and bool(train.get("allow_camera_translation_transform_change_on_init", False))):
            out.append("camera translation transform mismatch is allowed only for an explicit weights-only ablation")
    return out


def release_recipe_problems(config: Mapping[str, Any], family: str) -> list:
    """Every way in which ``config`` departs from the release recipe of ``family`` (empty list: it conforms)."""
    from ...config.routes import validate_route

    if family not in RELEASE_PROFILES:
        raise BackendContractError(f"unknown Wan family {family!r}")
    action = str(config.get("action", "")).strip().lower()
    if action not in ("train", "infer"):
        return ["a Wan recipe is a train or an infer config"]
    try:
        route = validate_route(config)
    except ConfigurationError as exc:
        return [str(exc)]
    if route.family != family:
        return [f"backend {family} cannot execute route {route.family}"]
    try:
        ctx = _Ctx(config, route, release_profile(config, family))
    except BackendContractError as exc:
        return [str(exc)]
    problems = []
    for section, table in RELEASE_PIN_TABLES:
        if section in ("train",) and action != "train":
            continue
        for pin in table:
            complaint = pin.check(ctx)
            if complaint:
                problems.append(complaint)
    if family == "wan22_i2v_a14b" and route.stage != "stage0p5":
        problems.append("A14B supports stage0p5 only")
    problems.extend(_cross_field_problems(ctx))
    return problems


def validate_release_recipe(config: Mapping[str, Any], family: str):
    """Raise ``BackendContractError`` naming every departure from the release recipe; returns the route."""
    from ...config.routes import validate_route

    problems = release_recipe_problems(config, family)
    if problems:
        raise BackendContractError(f"{family} release recipe: " + "; ".join(problems))
    return validate_route(config)
