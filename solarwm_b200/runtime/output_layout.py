"""Names of everything a run writes under ``runtime.output_dir``
(reference: solar/runtime/output_layout.py:15-211).

  checkpoint_model_{step:06d}/                  checkpoint transaction directories
  validation/step_{step:06d}_{pass}/            published validation passes
  validation/.staging/                          private staging for the above
  events/rank-{rank:05d}.jsonl                  per-rank training events
  resolved-config.json, launch-manifest.json, run-result.json
  camera-length inference, layout ``dataset_triplet_v1``:  generate/  compare/  camera/  runs/<run_id>/
  everything else, layout ``transaction_v1``:   one create-only directory per run
"""
from __future__ import annotations

import re
from pathlib import Path

from ..errors import ConfigurationError

DATASET_TRIPLET = "dataset_triplet_v1"
TRANSACTION = "transaction_v1"
_SAFE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9._-]*$")


def _safe(name: str, what: str) -> str:
    if not _SAFE.match(str(name)):
        raise ConfigurationError(f"{what} {name!r} is not a safe path component")
    return str(name)


def output_root(config) -> Path:
    runtime = config.get("runtime", {})
    root = runtime.get("output_dir")
    if not root:
        raise ConfigurationError("runtime.output_dir is required")
    return Path(str(root))


def checkpoint_model_dir(root, step: int, width: int = 6) -> Path:
    if step < 0:
        raise ConfigurationError("checkpoint step must be non-negative")
    return Path(root) / f"checkpoint_model_{int(step):0{width}d}"


def parse_checkpoint_step(path) -> int:
    m = re.fullmatch(r"checkpoint_model_(\d{6,8})", Path(path).name)
    if not m:
        raise ConfigurationError(f"not a checkpoint directory name: {Path(path).name!r}")
    return int(m.group(1))


def latest_checkpoint(root):
    best = None
    for item in Path(root).glob("checkpoint_model_*"):
        try:
            step = parse_checkpoint_step(item)
        except ConfigurationError:
            continue
        if (item / "COMPLETE.json").is_file() and (best is None or step > best[0]):
            best = (step, item)
    return None if best is None else best[1]


def public_validation_dir(root, step: int, pass_name: str) -> Path:
    return Path(root) / "validation" / f"step_{int(step):06d}_{_safe(pass_name, 'validation pass')}"


def validation_staging_dir(root) -> Path:
    return Path(root) / "validation" / ".staging"


def events_path(root, rank: int) -> Path:
    return Path(root) / "events" / f"rank-{int(rank):05d}.jsonl"


def inference_layout(config) -> str:
    inference = config.get("inference", {}) or {}
    return DATASET_TRIPLET if str(inference.get("length_policy", "")) == "camera" else TRANSACTION


def dataset_triplet_dirs(root, run_id: str) -> dict:
    root = Path(root)
    return {"generate": root / "generate", "compare": root / "compare", "camera": root / "camera",
            "run": root / "runs" / _safe(run_id, "run id")}


def slot_dir(parent, slot: int) -> Path:
    return Path(parent) / f"slot-{int(slot):06d}"
