"""Header-only authority over LTX checkpoints, and the identity a full resume has to match.

  header     a safetensors file starts with an 8-byte little-endian length and a JSON header.  ``read_header`` reads only
             that (bounded), refuses repeated JSON keys, unknown dtypes, shapes that do not multiply out to the byte range,
             and ranges that overlap, leave gaps or stop short of the file's end: everything a later mmap would trust.
  inventory  the published audio-video checkpoint holds four tensor families under ``model.diffusion_model.``: the video
             core (what the video-only runtime keeps), the text-embedding connector of the video stream (kept), the audio
             stream and the audio-video cross attention (both dropped).  ``classify`` names a tensor's family from the
             key alone; ``inspect_base_checkpoint`` counts tensors and parameters per family, checks them against the
             expected ``Inventory`` (the published numbers by default), checks the dtype policy (bf16 everywhere except
             the fp32 scale-shift tables, one per model and two per block), and digests the retained layout -- before a
             single weight byte is read.
  resume     ``runtime_fingerprint`` collects what must be identical between the run that wrote a checkpoint and the run
             that continues it (geometry, data generation, camera transform, adapter and averaging recipe);
             ``validate_full_resume`` names the fields that differ.

Reference: solar/backends/ltx25/checkpoint.py:90-763.
"""
from __future__ import annotations

import hashlib
import json
import struct
from collections import Counter
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Mapping, Optional, Sequence, Tuple

from ...errors import BackendContractError

PREFIX = "model.diffusion_model."
MAX_HEADER_BYTES = 64 << 20
DTYPE_BYTES = {"BOOL": 1, "I8": 1, "U8": 1, "F8_E4M3": 1, "F8_E4M3FN": 1, "F8_E5M2": 1, "F8_E8M0": 1, "I16": 2, "U16": 2, "F16": 2,
               "BF16": 2, "I32": 4, "U32": 4, "F32": 4, "C64": 8, "I64": 8, "U64": 8, "F64": 8, "C128": 16}

# family -> (top-level prefixes, top-level exact names, block sub-modules, block-level exact names)
FAMILIES = {
    "video_core": (("patchify_proj.", "adaln_single.", "prompt_adaln_single.", "proj_out."),
                   ("keyframes_abs_pos_embedding", "scale_shift_table"), ("attn1", "attn2", "ff"),
                   ("scale_shift_table", "prompt_scale_shift_table")),
    "audio": (("audio_patchify_proj.", "audio_proj_out.", "audio_adaln_single.", "audio_prompt_adaln_single.", "audio_embeddings_connector."),
              ("audio_scale_shift_table",), ("audio_attn1", "audio_attn2", "audio_ff"),
              ("audio_scale_shift_table", "audio_prompt_scale_shift_table")),
    "av_cross": (("av_ca_video_scale_shift_adaln_single.", "av_ca_audio_scale_shift_adaln_single.", "av_ca_a2v_gate_adaln_single.",
                  "av_ca_v2a_gate_adaln_single."), (), ("audio_to_video_attn", "video_to_audio_attn"),
                 ("scale_shift_table_a2v_ca_audio", "scale_shift_table_a2v_ca_video")),
}
CONNECTOR = "video_embeddings_connector."


@dataclass(frozen=True)
class Inventory:
    """What a base checkpoint must hold.  The defaults are the published LTX-2.5 audio-video checkpoint."""
    blocks: int = 48
    tensors: Mapping[str, int] = field(default_factory=lambda: {"video_core": 1362, "video_connector": 129, "audio": 1586, "av_cross": 1272})
    parameters: Mapping[str, int] = field(default_factory=lambda: {"video_core": 13_123_337_344, "video_connector": 1_612_546_304,
                                                                  "audio": 3_690_028_416, "av_cross": 2_578_113_536})
    model_version: Optional[str] = "2.5.0"
    transformer: Mapping[str, Any] = field(default_factory=lambda: {
        "_class_name": "AVTransformer3DModel", "num_layers": 48, "num_attention_heads": 32, "attention_head_dim": 128, "in_channels": 128,
        "out_channels": 128, "cross_attention_dim": 4096, "caption_channels": 3840, "connector_num_layers": 8,
        "connector_num_attention_heads": 32, "connector_attention_head_dim": 128, "use_audio_video_cross_attention": True,
        "use_embeddings_connector": True})
    scheduler: Mapping[str, Any] = field(default_factory=lambda: {"_class_name": "RectifiedFlowScheduler", "num_train_timesteps": 1000,
                                                                "sampler": "LinearQuadratic"})

    @property
    def fp32_tables(self) -> int:
        return 1 + 2 * self.blocks


PUBLISHED = Inventory()
LORA_R384_TRAINABLE = 1_962_934_272


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str
    shape: Tuple[int, ...]
    begin: int
    end: int

    @property
    def numel(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n


@dataclass(frozen=True)
class Header:
    metadata: Mapping[str, str]
    tensors: Tuple[TensorEntry, ...]
    header_size: int
    file_size: int
    digest: str


def _unique_object(pairs):
    out: Dict[str, Any] = {}
    for k, v in pairs:
        if k in out:
            raise BackendContractError(f"repeated JSON key {k!r}")
        out[k] = v
    return out


def _natural(value, what: str) -> int:
    if type(value) is not int or value < 0:
        raise BackendContractError(f"{what} must be a non-negative integer")
    return value


def read_header(path, *, max_header_bytes: int = MAX_HEADER_BYTES) -> Header:
    src = Path(path)
    if type(max_header_bytes) is not int or max_header_bytes < 2:
        raise BackendContractError("max_header_bytes must be an integer >= 2")
    try:
        size = src.stat().st_size
        with src.open("rb") as fh:
            lead = fh.read(8)
            if len(lead) != 8:
                raise BackendContractError("the safetensors length prefix is truncated")
            n = struct.unpack("<Q", lead)[0]
            if not 2 <= n <= max_header_bytes:
                raise BackendContractError(f"safetensors header size {n} is outside the accepted range")
            raw = fh.read(n)
    except OSError as exc:
        raise BackendContractError(f"cannot read checkpoint header {src}: {exc}") from exc
    if len(raw) != n or 8 + n > size:
        raise BackendContractError("the safetensors JSON header is truncated")
    try:
        doc = json.loads(raw.decode("utf-8").rstrip(" "), object_pairs_hook=_unique_object)
    except (UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise BackendContractError(f"invalid safetensors JSON header in {src}") from exc
    if not isinstance(doc, dict):
        raise BackendContractError("a safetensors header is a JSON object")
    meta = doc.pop("__metadata__", {})
    if not isinstance(meta, dict) or any(not isinstance(k, str) or not isinstance(v, str) for k, v in meta.items()):
        raise BackendContractError("safetensors metadata holds strings only")
    entries = []
    for name, item in doc.items():
        if not isinstance(item, dict) or set(item) != {"dtype", "shape", "data_offsets"}:
            raise BackendContractError(f"tensor {name!r} has a malformed header entry")
        dtype, shape, span = item["dtype"], item["shape"], item["data_offsets"]
        if dtype not in DTYPE_BYTES or not isinstance(shape, list) or not isinstance(span, list) or len(span) != 2:
            raise BackendContractError(f"tensor {name!r} has an unknown dtype or malformed shape / offsets")
        entry = TensorEntry(name, dtype, tuple(_natural(d, f"{name} shape") for d in shape), _natural(span[0], f"{name} offset"),
                            _natural(span[1], f"{name} offset"))
        if entry.end - entry.begin != entry.numel * DTYPE_BYTES[dtype]:
            raise BackendContractError(f"tensor {name!r}: byte range does not match shape x dtype")
        entries.append(entry)
    at = 0
    for e in sorted(entries, key=lambda e: (e.begin, e.end, e.name)):
        if e.begin != at:
            raise BackendContractError(f"safetensors data is not contiguous before {e.name!r}")
        at = e.end
    if at != size - 8 - n:
        raise BackendContractError("safetensors data ranges do not cover the file")
    return Header(dict(meta), tuple(entries), n, size, hashlib.blake2s(lead + raw).hexdigest())


def classify(name: str, blocks: int = 48) -> Tuple[str, Optional[str]]:
    """(family, name the video-only runtime keeps it under | None when the tensor is dropped)."""
    if not name.startswith(PREFIX):
        return "unknown", None
    rest = name[len(PREFIX):]
    if rest.startswith(CONNECTOR):
        return "video_connector", "video_connector." + rest[len(CONNECTOR):]
    for family, (prefixes, exact, _, _) in FAMILIES.items():
        if rest in exact or (prefixes and rest.startswith(prefixes)):
            return family, rest if family == "video_core" else None
    parts = rest.split(".")
    if len(parts) < 3 or parts[0] != "transformer_blocks" or not parts[1].isdigit() or (len(parts[1]) > 1 and parts[1][0] == "0") \
            or not 0 <= int(parts[1]) < blocks:
        return "unknown", None
    module, tail = parts[2], parts[3:]
    for family, (_, _, modules, exact) in FAMILIES.items():
        if (module in modules and tail) or (module in exact and not tail):
            return family, rest if family == "video_core" else None
    return "unknown", None


@dataclass(frozen=True)
class BaseInspection:
    path: str
    file_size: int
    header_size: int
    header_digest: str
    retained_layout_digest: str
    tensors: Mapping[str, int]
    parameters: Mapping[str, int]
    fp32_scale_tables: int
    retained: Tuple[Tuple[str, str], ...]          # (name in the runtime, name in the file), sorted

    def as_dict(self) -> dict:
        d = asdict(self)
        d["retained"] = len(self.retained)
        return d


def _metadata_object(meta: Mapping[str, str], key: str) -> Mapping[str, Any]:
    try:
        value = json.loads(meta[key], object_pairs_hook=_unique_object)
    except (KeyError, json.JSONDecodeError) as exc:
        raise BackendContractError(f"checkpoint metadata {key!r} is missing or invalid") from exc
    if not isinstance(value, dict):
        raise BackendContractError(f"checkpoint metadata {key!r} is not an object")
    return value


def inspect_base_checkpoint(path, expect: Inventory = PUBLISHED) -> BaseInspection:
    """Fail closed on any drift of header, keys, dtypes or layout."""
    header = read_header(path)
    if expect.model_version is not None:
        if header.metadata.get("model_version") != expect.model_version:
            raise BackendContractError(f"checkpoint model_version must be {expect.model_version}")
        config = _metadata_object(header.metadata, "config")
        for section, want in (("transformer", expect.transformer), ("scheduler", expect.scheduler)):
            have = config.get(section)
            if not isinstance(have, Mapping):
                raise BackendContractError(f"checkpoint metadata lacks the {section} description")
            for k, v in want.items():
                if have.get(k) != v:
                    raise BackendContractError(f"checkpoint {section}.{k} differs from the required model layout")
    groups: Dict[str, list] = {k: [] for k in ("video_core", "video_connector", "audio", "av_cross")}
    kept, strangers = [], []
    for t in header.tensors:
        family, target = classify(t.name, expect.blocks)
        if family == "unknown":
            strangers.append(t.name)
            continue
        groups[family].append(t)
        if target is not None:
            kept.append((target, t))
    if strangers:
        raise BackendContractError(f"unknown checkpoint keys: {strangers[:8]!r}")
    tensors = {k: len(v) for k, v in groups.items()}
    parameters = {k: sum(t.numel for t in v) for k, v in groups.items()}
    if tensors != dict(expect.tensors) or parameters != dict(expect.parameters):
        raise BackendContractError(f"checkpoint inventory differs: tensors {tensors}, parameters {parameters}")
    fp32 = {target for target, t in kept if t.dtype == "F32"}
    want_fp32 = {"scale_shift_table"} | {f"transformer_blocks.{i}.{n}" for i in range(expect.blocks)
                                         for n in ("scale_shift_table", "prompt_scale_shift_table")}
    if fp32 != want_fp32:
        raise BackendContractError("the fp32 scale-table inventory differs")
    others = Counter(t.dtype for target, t in kept if target not in want_fp32)
    if set(others) - {"BF16"}:
        raise BackendContractError(f"retained tensors must be bf16 apart from the scale tables, found {dict(others)}")
    if len({target for target, _ in kept}) != len(kept):
        raise BackendContractError("retained target names are not unique")
    layout = hashlib.blake2s()
    for target, t in sorted(kept, key=lambda p: p[0]):
        layout.update(json.dumps({"dtype": t.dtype, "shape": list(t.shape), "source": t.name, "target": target}, sort_keys=True,
                                 separators=(",", ":")).encode() + b"\n")
    return BaseInspection(str(Path(path).resolve()), header.file_size, header.header_size, header.digest, layout.hexdigest(), tensors,
                          parameters, len(fp32), tuple(sorted((target, t.name) for target, t in kept)))


# ---------------------------------------------------------------------------------------------------------------------
# resume identity
# ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LoRARecipe:
    rank: int = 384
    alpha: int = 384
    dropout: float = 0.0
    target_count: int = 480
    trainable_parameters: int = LORA_R384_TRAINABLE
    base_scale_tables_trainable: bool = False


@dataclass(frozen=True)
class EMARecipe:
    enabled: bool = True
    start_step: int = 0
    update_every_steps: int = 1
    decay: float = 0.999
    dtype: str = "float32"
    trainable_only: bool = True


def runtime_fingerprint(*, camera_translation_transform: str, data_generation: str, lora: LoRARecipe = LoRARecipe(),
                        ema: EMARecipe = EMARecipe(), inventory: Inventory = PUBLISHED) -> Dict[str, Any]:
    from .geometry import STABLE

    if camera_translation_transform not in ("linear", "logd4"):
        raise BackendContractError("the camera translation transform is linear or logd4")
    if not str(data_generation).strip():
        raise BackendContractError("data_generation must be non-empty")
    return {"schema": "solarwm.ltx25.checkpoint.v1", "family": "ltx25_video", "stage": "stage0p5", "objective": "native_rectified_flow",
            "geometry": asdict(STABLE), "data_generation": str(data_generation), "camera_translation_transform": camera_translation_transform,
            "base_checkpoint": {"tensors": {k: inventory.tensors[k] for k in ("video_core", "video_connector")},
                                "parameters": {k: inventory.parameters[k] for k in ("video_core", "video_connector")},
                                "fp32_scale_tables": inventory.fp32_tables, "dropped_streams": ["audio", "audio_video_cross_attention"],
                                "strict_load": True},
            "lora": asdict(lora), "ema": asdict(ema)}


def fingerprint_digest(value: Mapping[str, Any]) -> str:
    return hashlib.blake2s(json.dumps(value, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


@dataclass(frozen=True)
class TrainingCheckpointManifest:
    """What a same-stage full resume needs to find."""
    global_step: int
    runtime_fingerprint: Mapping[str, Any]
    adapter_targets: Sequence[str]
    ema_targets: Sequence[str]
    optimizer_present: bool
    scheduler_present: bool

    def validate(self, expected_targets: Sequence[str]) -> None:
        if type(self.global_step) is not int or self.global_step < 0:
            raise BackendContractError("global_step must be a non-negative integer")
        if tuple(self.adapter_targets) != tuple(expected_targets):
            raise BackendContractError("the checkpoint's adapter target inventory is not exact")
        if tuple(self.ema_targets) != tuple(expected_targets):
            raise BackendContractError("the average must hold exactly the trainable adapter targets")
        if not (self.optimizer_present and self.scheduler_present):
            raise BackendContractError("a full resume needs optimizer and scheduler state")
        if self.runtime_fingerprint.get("schema") != "solarwm.ltx25.checkpoint.v1":
            raise BackendContractError("the checkpoint's runtime fingerprint has no known schema")


def validate_full_resume(saved: TrainingCheckpointManifest, current: Mapping[str, Any], expected_targets: Sequence[str]) -> None:
    saved.validate(expected_targets)
    if dict(saved.runtime_fingerprint) != dict(current):
        differing = sorted(k for k in set(saved.runtime_fingerprint) | set(current) if saved.runtime_fingerprint.get(k) != current.get(k))
        raise BackendContractError(f"a full resume needs identical runtime semantics; differing: {differing}")
