"""One report of everything a Wan job needs before it allocates a model: dependencies, asset files, the transformer
architecture, the weight inventory, corpus indexes, inference controls and the device.

Every check appends to ONE list of issues (``code``, ``message``, ``severity``, ``path``) instead of raising at the
first problem, so a user fixes a broken set-up in one pass; ``Report.require_ready`` raises with all errors rendered.
Which checks apply depends on the action: pre-encoding needs the codecs but no transformer; training from a
pre-encoded corpus needs the transformer but no codecs; a ``full_resume`` takes its weights from the checkpoint, not
from ``model.base_path``; synthetic runs (``data.source: synthetic``, no ``model.base_path``) need no files at all.

Asset layout (``model.base_path`` absolute; ``model.assets.<name>`` overrides, relative names resolve under the base):
``transformer_config`` (``config.json`` or ``builtin``), ``transformer_weights`` (a directory of safetensors shards),
``text_encoder``, ``tokenizer``, ``vae``.  Paths that still start with ``/path/to`` are documentation placeholders
and are reported as such.

Reference: WanAssetLayout (solar/backends/wan22/runtime/assets.py:14-99), probe_runtime / require_training_runtime
(solar/backends/wan22/runtime/readiness.py:25-505).
"""
from __future__ import annotations

import importlib
import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, List, Mapping, Optional

from ...errors import BackendContractError

SCHEMA = "solarwm.wan22-readiness.v1"
_DEFAULTS = {"text_encoder": "models_t5_umt5-xxl-enc-bf16.pth", "tokenizer": "google/umt5-xxl", "vae": "Wan2.2_VAE.pth"}


@dataclass(frozen=True)
class Issue:
    code: str
    message: str
    severity: str = "error"            # "error" | "warning" | "info"
    path: Optional[str] = None


@dataclass(frozen=True)
class AssetLayout:
    base: Optional[Path]
    transformer_config: Optional[Path]      # None: the built-in architecture of the family
    transformer_weights: Optional[Path]
    text_encoder: Optional[Path]
    tokenizer: Optional[Path]
    vae: Optional[Path]

    @classmethod
    def from_config(cls, config: Mapping[str, Any]) -> "AssetLayout":
        model = config.get("model", {}) or {}
        raw = str(model.get("base_path", "") or "").strip()
        assets = model.get("assets", {}) or {}
        if not isinstance(assets, Mapping):
            raise BackendContractError("model.assets must be a mapping")
        if not raw:
            if assets:
                raise BackendContractError("model.assets needs model.base_path")
            return cls(None, None, None, None, None, None)
        if not raw.startswith("/"):
            raise BackendContractError("model.base_path must be an absolute path")
        base = Path(raw)

        def resolve(name, default):
            value = str(assets.get(name, "") or "").strip()
            if not value:
                return default
            path = Path(value)
            return path if path.is_absolute() else base / path

        arch = str(assets.get("transformer_config", "") or "").strip()
        return cls(base, None if arch == "builtin" else resolve("transformer_config", base / "config.json"),
                   resolve("transformer_weights", base), resolve("text_encoder", base / _DEFAULTS["text_encoder"]),
                   resolve("tokenizer", base / _DEFAULTS["tokenizer"]), resolve("vae", base / _DEFAULTS["vae"]))

    def as_dict(self) -> dict:
        return {k: (None if v is None else str(v)) for k, v in asdict(self).items()}


@dataclass(frozen=True)
class Report:
    family: str
    ready: bool
    assets: Mapping[str, Any]
    dependencies: Mapping[str, Any]
    weight_inventory: Mapping[str, Any]
    index_inventories: Mapping[str, Any]
    issues: tuple = field(default_factory=tuple)

    def as_dict(self) -> dict:
        return {"schema": SCHEMA, "family": self.family, "ready": self.ready, "assets": dict(self.assets),
                "dependencies": dict(self.dependencies), "weight_inventory": dict(self.weight_inventory),
                "index_inventories": {k: dict(v) for k, v in self.index_inventories.items()},
                "issues": [asdict(i) for i in self.issues]}

    def require_ready(self) -> None:
        errors = [i for i in self.issues if i.severity == "error"]
        if errors:
            text = "; ".join(f"{i.code}: {i.message}" + (f" [{i.path}]" if i.path else "") for i in errors)
            raise BackendContractError(f"the Wan runtime is not ready: {text}")


def is_placeholder(path: Path) -> bool:
    return str(path).startswith("/path/to")


# ---------------------------------------------------------------------------------------------------------------------
# checks
# ---------------------------------------------------------------------------------------------------------------------
def _dependencies(issues: List[Issue], *, decode: bool) -> dict:
    found = {}
    for name, needed in (("torch", True), ("numpy", True), ("cv2", decode), ("yaml", False)):
        try:
            found[name] = getattr(importlib.import_module(name), "__version__", "present")
        except ImportError:
            found[name] = None
            if needed:
                issues.append(Issue("dependency_missing", f"python module {name!r} cannot be imported"))
    try:
        from ...ops import _lib

        found["native_library"] = bool(_lib.available())
    except Exception as exc:  # noqa: BLE001 - reported, not raised
        found["native_library"] = False
        issues.append(Issue("native_library", f"the native kernel library cannot be inspected: {exc}", "warning"))
    return found


def _file(issues: List[Issue], code: str, path: Optional[Path], *, what: str, directory: bool = False) -> bool:
    if path is None:
        issues.append(Issue(code, f"{what} is not configured (set model.base_path)"))
        return False
    if is_placeholder(path):
        issues.append(Issue(code, f"{what} still names a documentation placeholder", path=str(path)))
        return False
    if path.is_symlink() and not path.exists():
        issues.append(Issue(code, f"{what} is a dangling symlink", path=str(path)))
        return False
    ok = path.is_dir() if directory else path.is_file()
    if not ok:
        issues.append(Issue(code, f"{what} is missing" + (" (a directory is expected)" if directory else ""), path=str(path)))
    return ok


def _architecture(issues: List[Issue], layout: AssetLayout, config: Mapping[str, Any], family: str) -> None:
    from .contracts import architecture

    try:
        arch = architecture(config)
    except Exception as exc:  # noqa: BLE001
        issues.append(Issue("architecture", f"model.architecture does not resolve: {exc}"))
        return
    if layout.transformer_config is None:
        return
    if not _file(issues, "transformer_config", layout.transformer_config, what="the transformer configuration"):
        return
    try:
        declared = json.loads(layout.transformer_config.read_text())
    except (OSError, ValueError) as exc:
        issues.append(Issue("transformer_config", f"unreadable: {exc}", path=str(layout.transformer_config)))
        return
    for theirs, ours in (("dim", arch.dim), ("ffn_dim", arch.ffn_dim), ("num_heads", arch.num_heads),
                         ("num_layers", arch.num_layers), ("in_dim", arch.in_dim), ("out_dim", arch.out_dim)):
        if theirs in declared and int(declared[theirs]) != int(ours):
            issues.append(Issue("transformer_config", f"{theirs} is {declared[theirs]} in the file, {ours} for {family}",
                                path=str(layout.transformer_config)))


def _weights(issues: List[Issue], layout: AssetLayout) -> dict:
    from .loader import inventory

    if not _file(issues, "transformer_weights", layout.transformer_weights, what="the transformer weights", directory=True):
        return {}
    try:
        entries = inventory(layout.transformer_weights)
    except BackendContractError as exc:
        issues.append(Issue("transformer_weights", str(exc), path=str(layout.transformer_weights)))
        return {}
    shards = sorted({e.shard for e in entries.values()})
    numel = 0
    for e in entries.values():
        n = 1
        for d in e.shape:
            n *= d
        numel += n
    return {"tensors": len(entries), "shards": len(shards), "parameters": numel, "dtypes": sorted({e.dtype for e in entries.values()})}


def _indexes(issues: List[Issue], config: Mapping[str, Any], *, contents: bool) -> dict:
    data = config.get("data", {}) or {}
    if str(data.get("source", "synthetic")) != "index":
        return {}
    out = {}
    for key in ("index", "validation_index", "test_index"):
        raw = data.get(key) or (config.get("validation", {}) or {}).get(key) if key != "index" else data.get(key)
        if not raw:
            if key == "index":
                issues.append(Issue("index", "data.source is index but data.index is not set"))
            continue
        path = Path(str(raw))
        if not _file(issues, "index", path, what=f"data.{key}"):
            continue
        if contents:
            from ...data.index import inventory as index_inventory
            from ...errors import DataContractError

            try:
                inv = index_inventory(path)
                out[key] = {"rows": inv.rows, "virtual_occurrences": inv.virtual_occurrences, "digest": inv.ordered_row_digest}
            except (DataContractError, OSError, ValueError) as exc:
                issues.append(Issue("index", f"data.{key} cannot be read: {exc}", path=str(path)))
    return out


def _inference_controls(issues: List[Issue], config: Mapping[str, Any]) -> None:
    inf = config.get("inference", {}) or {}
    if not inf:
        return
    steps = inf.get("steps", 50)
    if isinstance(steps, bool) or not isinstance(steps, int) or steps < 1:
        issues.append(Issue("inference", f"inference.steps must be a positive integer, got {steps!r}"))
    if str(inf.get("solver", "unipc")) not in ("unipc", "euler"):
        issues.append(Issue("inference", f"inference.solver must be unipc or euler, got {inf.get('solver')!r}"))
    if inf.get("compare_source") and not inf.get("vae"):
        issues.append(Issue("inference", "inference.compare_source needs inference.vae (both clips are decoded)"))
    if int(inf.get("sequence_parallel_size", 1)) < 1:
        issues.append(Issue("inference", "inference.sequence_parallel_size must be positive"))


def _cuda(issues: List[Issue], *, required: bool) -> None:
    import torch

    if torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability(0)
        if (major, minor) != (10, 0):
            issues.append(Issue("device", f"the native kernels are built for sm_100a; device 0 is sm_{major}{minor}",
                                "error" if required else "warning"))
    elif required:
        issues.append(Issue("device", "no CUDA device is visible"))


def probe_runtime(config: Mapping[str, Any], *, family: str, require_cuda: bool = False, require_transformer_weights: bool = True,
                  validate_index_contents: bool = True) -> Report:
    action = str(config.get("action", ""))
    data = config.get("data", {}) or {}
    synthetic = str(data.get("source", "synthetic")) == "synthetic" and not (config.get("model", {}) or {}).get("base_path")
    online = action in ("infer", "preencode") or str(data.get("encoding", "preencoded")) == "online"
    transformer = action != "preencode"
    issues: List[Issue] = []
    layout = AssetLayout.from_config(config)
    deps = _dependencies(issues, decode=bool((config.get("inference", {}) or {}).get("vae")))
    weights: dict = {}
    if transformer:
        _architecture(issues, layout, config, family)
    if synthetic:
        issues.append(Issue("assets", "synthetic run: no asset files are required", "info"))
    elif layout.base is None:
        # no released package is named: the transformer starts from its seeded initialisation and the codecs, where an
        # action needs them, come from its own section (``preencode.codecs``, ``inference.vae`` / ``text_encoder``)
        issues.append(Issue("assets", "no model.base_path: seeded random initialisation, codecs from the action's own section", "info"))
        resume = (config.get("checkpoint", {}) or {})
        if str(resume.get("mode", "none")) in ("full_resume", "weights_only") and resume.get("resume_from"):
            weights = {"source": "checkpoint"}
            _file(issues, "checkpoint", Path(str(resume["resume_from"])), what="checkpoint.resume_from", directory=True)
    else:
        if online:
            for name, what in (("text_encoder", "the text encoder weights"), ("vae", "the VAE weights")):
                _file(issues, name, getattr(layout, name), what=what)
            _file(issues, "tokenizer", layout.tokenizer, what="the tokenizer directory", directory=True)
        resume = (config.get("checkpoint", {}) or {})
        from_checkpoint = str(resume.get("mode", "none")) in ("full_resume", "weights_only") and resume.get("resume_from")
        if transformer and require_transformer_weights and not from_checkpoint:
            weights = _weights(issues, layout)
        elif from_checkpoint:
            weights = {"source": "checkpoint"}
            _file(issues, "checkpoint", Path(str(resume["resume_from"])), what="checkpoint.resume_from", directory=True)
    inventories = _indexes(issues, config, contents=validate_index_contents)
    _inference_controls(issues, config)
    _cuda(issues, required=require_cuda)
    return Report(family, not any(i.severity == "error" for i in issues), layout.as_dict(), deps, weights, inventories, tuple(issues))


def require_training_runtime(config: Mapping[str, Any], *, family: str, require_cuda: bool = False) -> Report:
    report = probe_runtime(config, family=family, require_cuda=require_cuda, validate_index_contents=False)
    report.require_ready()
    return report
