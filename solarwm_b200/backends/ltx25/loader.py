"""Strict load of a released LTX transformer checkpoint's VIDEO CORE into ``LTXDiT``.

The released file names its tensors ``model.diffusion_model.<module path>`` in the layout of the publisher's own
classes.  This loader does not instantiate those classes and swap them afterwards: it maps names straight onto the
parameters of this package's model with a rule table, checks EVERYTHING first (every destination filled exactly once,
shapes after the stated reshape, floating dtypes, finite fp32 tables) and only then copies, tensor by tensor, out of
the memory-mapped file into the parameters (which are views of the model's resident buffers).

  rules       per block: ``attn1`` -> self attention, ``attn2`` -> text cross attention (``to_q / to_k / to_v /
              to_out.0 / q_norm / k_norm / to_gate_logits``), ``ff.net.0.proj`` / ``ff.net.2`` -> the feed-forward pair,
              ``scale_shift_table [6, dim]`` -> the block's modulation ``[1, 6, dim]``.  Top level: ``patchify_proj``
              (a linear map; the model holds it as a 1 x 1 x 1 convolution), ``adaln_single`` (timestep embedder and
              the 6-way projection), ``caption_projection``, the head's ``scale_shift_table [2, dim]`` and
              ``proj_out``.
  families    audio, audio-video cross attention and the embeddings connector are dropped (the video-only runtime
              never evaluates them); they are counted, not read.
  unplaced    a video-core tensor with no destination (the prompt-conditioned adaLN tables of the 2.5 release,
              ``prompt_adaln_single`` / ``prompt_scale_shift_table``) is an error unless ``allow_unplaced`` names its
              pattern: a model loaded without them is NOT the published model, and the report says so.
  missing     likewise a parameter of the model that the file does not hold (``text_embedding.*`` against a release
              whose text path is the embeddings connector) is an error unless ``allow_missing`` names it.

Reference: the video-only load of the official audio-video checkpoint (solar/backends/ltx25/torch_model.py:400-560,
checkpoint.py:240-400).
"""
from __future__ import annotations

import fnmatch
import re
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ...errors import BackendContractError
from .checkpoint import PREFIX, classify, read_header

_ATTN = {"to_q": "q", "to_k": "k", "to_v": "v", "to_out.0": "o", "q_norm": "norm_q", "k_norm": "norm_k", "to_gate_logits": "to_gate_logits"}
_TOP = {"patchify_proj": "patch_embedding", "adaln_single.emb.timestep_embedder.linear_1": "time_embedding.0",
        "adaln_single.emb.timestep_embedder.linear_2": "time_embedding.2", "adaln_single.linear": "time_projection.1",
        "caption_projection.linear_1": "text_embedding.0", "caption_projection.linear_2": "text_embedding.2", "proj_out": "head.head"}
_BLOCK = re.compile(r"^transformer_blocks\.(\d+)\.(.+)$")
_FLOATS = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16}


def destination(name: str) -> Optional[str]:
    """Released video-core name (prefix stripped) -> the model's parameter name, or None when there is none."""
    if name == "scale_shift_table":
        return "head.modulation"
    for src, dst in _TOP.items():
        if name in (src + ".weight", src + ".bias"):
            return dst + name[len(src):]
    m = _BLOCK.match(name)
    if not m:
        return None
    i, rest = m.group(1), m.group(2)
    if rest == "scale_shift_table":
        return f"blocks.{i}.modulation"
    for released, ours in (("attn1.", "self_attn."), ("attn2.", "cross_attn.")):
        if rest.startswith(released):
            module, _, leaf = rest[len(released):].rpartition(".")
            return f"blocks.{i}.{ours}{_ATTN[module]}.{leaf}" if module in _ATTN and leaf in ("weight", "bias") else None
    for released, ours in (("ff.net.0.proj.", "ffn.0."), ("ff.net.2.", "ffn.2.")):
        if rest.startswith(released) and rest[len(released):] in ("weight", "bias"):
            return f"blocks.{i}.{ours}{rest[len(released):]}"
    return None


def _fits(src: Tuple[int, ...], dst: Tuple[int, ...]) -> bool:
    """Equal, or equal once the destination's unit axes are dropped / added (tables ``[n, d]`` <-> ``[1, n, d]``, the
    patch projection ``[d, c]`` <-> ``[d, c, 1, 1, 1]``)."""
    strip = lambda s: tuple(x for x in s if x != 1)   # noqa: E731
    return src == dst or strip(src) == strip(dst)


@dataclass
class LoadReport:
    placed: int = 0
    parameters: int = 0
    dropped: Dict[str, int] = field(default_factory=dict)        # family -> tensors not read
    unplaced: List[str] = field(default_factory=list)            # video-core tensors the architecture has no place for
    missing: List[str] = field(default_factory=list)             # parameters the file does not hold (kept as initialised)
    header_digest: str = ""

    @property
    def published_model(self) -> bool:
        return not self.unplaced and not self.missing


def plan(model, path, *, allow_unplaced: Sequence[str] = (), allow_missing: Sequence[str] = ()) -> Tuple[Dict[str, str], LoadReport]:
    """Verify the whole file against the model; returns {released name: parameter name} and the report.  Nothing is read
    but the header."""
    header = read_header(path)
    params = dict(model.named_parameters())
    blocks = len(model.blocks)
    report = LoadReport(header_digest=header.digest)
    mapping: Dict[str, str] = {}
    problems: List[str] = []
    for entry in header.tensors:
        family, _ = classify(entry.name, blocks=max(blocks, 48))
        if family == "unknown" and entry.name.startswith(PREFIX + "caption_projection."):
            family = "video_core"                  # the text projection of the releases that have no embeddings connector
        if family == "unknown":
            problems.append(f"unknown tensor {entry.name}")
            continue
        if family != "video_core":
            report.dropped[family] = report.dropped.get(family, 0) + 1
            continue
        name = entry.name[len(PREFIX):]
        m = _BLOCK.match(name)
        if m and int(m.group(1)) >= blocks:
            problems.append(f"{name}: the model has {blocks} blocks")
            continue
        dst = destination(name)
        if dst is None or dst not in params:
            if any(fnmatch.fnmatchcase(name, pat) for pat in allow_unplaced):
                report.unplaced.append(name)
            else:
                problems.append(f"{name}: no destination in this architecture")
            continue
        if dst in mapping.values():
            problems.append(f"{name}: {dst} is filled twice")
        elif entry.dtype not in _FLOATS:
            problems.append(f"{name}: dtype {entry.dtype} is not a floating type")
        elif not _fits(tuple(entry.shape), tuple(params[dst].shape)):
            problems.append(f"{name}: shape {tuple(entry.shape)} does not fit {dst} {tuple(params[dst].shape)}")
        else:
            mapping[entry.name] = dst
            report.parameters += params[dst].numel()
    for name in sorted(set(params) - set(mapping.values())):
        if any(fnmatch.fnmatchcase(name, pat) for pat in allow_missing):
            report.missing.append(name)
        else:
            problems.append(f"parameter {name} is not in the file")
    if problems:
        raise BackendContractError("the LTX checkpoint does not fit the model: " + "; ".join(problems[:8])
                                   + (f" (+{len(problems) - 8} more)" if len(problems) > 8 else ""))
    report.placed = len(mapping)
    return mapping, report


def load_video_core(model, path, *, allow_unplaced: Sequence[str] = (), allow_missing: Sequence[str] = ()) -> LoadReport:
    """Verify, then copy.  ``model`` keeps its dtype: bf16 parameters take the file's values rounded once, fp32 tables
    (modulation) stay exact when the model holds them in fp32."""
    from safetensors import safe_open

    mapping, report = plan(model, path, allow_unplaced=allow_unplaced, allow_missing=allow_missing)
    params = dict(model.named_parameters())
    with safe_open(str(Path(path)), framework="pt", device="cpu") as fh, torch.no_grad():
        for released, dst in mapping.items():
            value = fh.get_tensor(released)
            if dst.endswith("modulation") and not bool(torch.isfinite(value.float()).all()):
                raise BackendContractError(f"{released}: non-finite modulation table")
            params[dst].copy_(value.reshape(params[dst].shape))
    return report


def export_released(model) -> Mapping[str, torch.Tensor]:
    """The model's parameters under the released names (the inverse of ``destination``): what a checkpoint written from
    this package holds so that the publisher's tools can read it."""
    out = {}
    inv_attn = {v: k for k, v in _ATTN.items()}
    inv_top = {v: k for k, v in _TOP.items()}
    for name, p in model.named_parameters():
        value = p.detach().cpu()
        if name == "head.modulation":
            out[PREFIX + "scale_shift_table"] = value.reshape(value.shape[-2:]).contiguous()
            continue
        stem, _, leaf = name.rpartition(".")
        if stem in inv_top:
            out[PREFIX + f"{inv_top[stem]}.{leaf}"] = value.reshape(value.shape[0], -1).contiguous() if stem == "patch_embedding" and leaf == "weight" else value.contiguous()
            continue
        m = re.match(r"^blocks\.(\d+)\.(.+)$", name)
        if not m:
            raise BackendContractError(f"{name} has no released name")
        i, rest = m.group(1), m.group(2)
        base = f"{PREFIX}transformer_blocks.{i}."
        if rest == "modulation":
            out[base + "scale_shift_table"] = value.reshape(value.shape[-2:]).contiguous()
        elif rest.startswith(("self_attn.", "cross_attn.")):
            side, module, leaf = rest.split(".", 2)
            out[base + f"{'attn1' if side == 'self_attn' else 'attn2'}.{inv_attn[module]}.{leaf}"] = value.contiguous()
        elif rest.startswith("ffn."):
            _, idx, leaf = rest.split(".")
            out[base + ("ff.net.0.proj." if idx == "0" else "ff.net.2.") + leaf] = value.contiguous()
        else:
            raise BackendContractError(f"{name} has no released name")
    return out
