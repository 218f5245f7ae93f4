"""Strict load of released H3-style transformer weights into ``models.h3.H3DiT``.

The released layout names tensors the way module trees do (``transformer_blocks.3.attn.to_q.weight``,
``...ffn.gate_proj.weight`` / ``...ffn.up_proj.weight`` as two matrices); ``H3DiT`` keeps flat names and ONE fused
gate|up matrix per block.  ``plan_load`` turns a shard inventory into a copy plan through an ordered table of
``(pattern, target)`` rules -- a target ending in ``#k`` is the k-th equal row block of a fused destination --
and refuses, before a byte is copied: checkpoint tensors no rule claims, model tensors nothing fills (adapter banks
excepted: they are trained, not released), shape mismatches, halves of a fused matrix filled twice or not at all,
and non-floating dtypes.  ``strict_load_mapped`` then streams shard by shard; norm gains and the adaLN table stay in
the model's own (fp32) dtype whatever the file holds (reference behaviour: solar/backends/minimax_h3/optional.py:
102-143 -- strict load with fp32 units -- and diffusers_compat.py).

The default table below is the naming this package assumes for a diffusers-style export; a deployment whose export
differs passes its own ``rules`` (``model.weight_rules`` in the run configuration).
"""
from __future__ import annotations

import re
from pathlib import Path
from typing import Dict, List, Mapping, NamedTuple, Optional, Sequence, Tuple

import torch

from ...errors import BackendContractError
from ..wan22.loader import TensorEntry, inventory

_FLOAT = {"F32", "F16", "BF16", "F64"}

_BLOCK = r"(transformer_blocks|token_refiner)\.(\d+)\."


def _tree(match_group: str) -> str:
    return "blocks" if match_group == "transformer_blocks" else "refiner"


DEFAULT_RULES: Sequence[Tuple[str, str]] = (
    (r"^" + _BLOCK + r"attn\.(to_q|to_k|to_v)\.weight$", r"{tree}.\2.\3.weight"),
    (r"^" + _BLOCK + r"attn\.to_out\.0\.weight$", r"{tree}.\2.to_out.weight"),
    (r"^" + _BLOCK + r"attn\.(norm_q|norm_k)\.weight$", r"{tree}.\2.\3"),
    (r"^" + _BLOCK + r"(norm1|norm2)\.weight$", r"{tree}.\2.\3"),
    (r"^" + _BLOCK + r"adaln_proj\.weight$", r"{tree}.\2.adaln_proj"),
    (r"^" + _BLOCK + r"ffn\.gate_proj\.weight$", r"{tree}.\2.ffn_gate_up.weight#0"),
    (r"^" + _BLOCK + r"ffn\.up_proj\.weight$", r"{tree}.\2.ffn_gate_up.weight#1"),
    (r"^" + _BLOCK + r"ffn\.down_proj\.weight$", r"{tree}.\2.ffn_down.weight"),
    (r"^proj_in\.weight$", "proj_in"), (r"^proj_out\.weight$", "proj_out"),
    (r"^audio_proj_in\.weight$", "audio_proj_in"), (r"^audio_proj_out\.weight$", "audio_proj_out"),
    (r"^context_embedder\.weight$", "context_embedder"),
    (r"^time_embed\.linear_1\.weight$", "time_in"), (r"^time_embed\.linear_2\.weight$", "time_out"),
    (r"^norm_out\.weight$", "norm_out"),
)


class Copy(NamedTuple):
    source: str                 # tensor name in the checkpoint
    shard: str
    target: str                 # parameter name in the model
    block: Optional[int]        # row block of a fused destination (None: the whole tensor)
    blocks: int                 # how many row blocks the destination has (1 unless fused)


def _apply(rules, name: str) -> Optional[str]:
    for pattern, target in rules:
        m = re.match(pattern, name)
        if m:
            if "{tree}" in target:
                target = target.replace("{tree}", _tree(m.group(1)))
            return m.expand(target)
    return None


def plan_load(entries: Mapping[str, TensorEntry], model: torch.nn.Module,
              rules: Sequence[Tuple[str, str]] = DEFAULT_RULES) -> List[Copy]:
    want = {k: tuple(v.shape) for k, v in model.state_dict().items() if "lora_" not in k}
    unclaimed, mapped = [], []
    for name, e in sorted(entries.items()):
        target = _apply(rules, name)
        if target is None:
            unclaimed.append(name)
            continue
        block = None
        if "#" in target:
            target, idx = target.rsplit("#", 1)
            block = int(idx)
        mapped.append((name, e, target, block))
    if unclaimed:
        raise BackendContractError(f"{len(unclaimed)} checkpoint tensors match no rule, e.g. {unclaimed[:5]}")
    fills: Dict[str, List[Optional[int]]] = {}
    for name, e, target, block in mapped:
        if target not in want:
            raise BackendContractError(f"{name} maps to {target!r}, which the model does not have")
        if e.dtype not in _FLOAT:
            raise BackendContractError(f"{name}: dtype {e.dtype} is not a floating type this loader accepts")
        fills.setdefault(target, []).append(block)
    missing = sorted(set(want) - set(fills))
    if missing:
        raise BackendContractError(f"{len(missing)} model tensors are not in the checkpoint, e.g. {missing[:5]}")
    plan = []
    for name, e, target, block in mapped:
        got = fills[target]
        if None in got:
            if len(got) != 1:
                raise BackendContractError(f"{target} is filled more than once")
            n_blocks = 1
        else:
            n_blocks = len(got)
            rows_given = sum(x[1].shape[0] for x in mapped if x[2] == target)
            if sorted(got) != list(range(n_blocks)) or rows_given != want[target][0]:
                raise BackendContractError(f"{target}: row blocks {sorted(got)} ({rows_given} rows) do not tile the fused "
                                           f"tensor of {want[target][0]} rows")
            if want[target][0] % n_blocks:
                raise BackendContractError(f"{target}: {want[target][0]} rows do not split into {n_blocks} blocks")
        expect = want[target] if block is None else (want[target][0] // n_blocks,) + want[target][1:]
        if tuple(e.shape) != tuple(expect):
            raise BackendContractError(f"{name}: shape {tuple(e.shape)} in the checkpoint, {tuple(expect)} expected for {target}")
        plan.append(Copy(name, e.shard, target, block, n_blocks))
    return plan


@torch.no_grad()
def strict_load_mapped(model: torch.nn.Module, directory, rules: Sequence[Tuple[str, str]] = DEFAULT_RULES) -> Mapping[str, int]:
    """Verify the whole plan, then copy shard by shard.  Returns ``{shard: tensors copied}``."""
    from safetensors import safe_open

    plan = plan_load(inventory(directory), model, rules)
    params = dict(model.state_dict(keep_vars=True))
    by_shard: Dict[str, List[Copy]] = {}
    for c in plan:
        by_shard.setdefault(c.shard, []).append(c)
    copied = {}
    for shard, items in sorted(by_shard.items()):
        with safe_open(str(Path(directory) / shard), framework="pt", device="cpu") as fh:
            for c in items:
                dst = params[c.target].data
                if c.block is not None:
                    rows = dst.shape[0] // c.blocks
                    dst = dst[c.block * rows:(c.block + 1) * rows]
                dst.copy_(fh.get_tensor(c.source).to(dst.dtype))
        copied[shard] = len(items)
    return copied


def export_released_layout(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    """The inverse naming (used by tests and by ``merge``-then-release flows): model tensors under the released names,
    the fused gate|up matrix split back into its two halves."""
    out: Dict[str, torch.Tensor] = {}
    top = {"proj_in": "proj_in.weight", "proj_out": "proj_out.weight", "audio_proj_in": "audio_proj_in.weight",
           "audio_proj_out": "audio_proj_out.weight", "context_embedder": "context_embedder.weight",
           "time_in": "time_embed.linear_1.weight", "time_out": "time_embed.linear_2.weight", "norm_out": "norm_out.weight"}
    for name, t in model.state_dict().items():
        if "lora_" in name:
            continue
        t = t.detach().cpu().contiguous()
        if name in top:
            out[top[name]] = t
            continue
        tree, idx, rest = name.split(".", 2)
        pre = ("transformer_blocks" if tree == "blocks" else "token_refiner") + f".{idx}."
        if rest in ("to_q.weight", "to_k.weight", "to_v.weight"):
            out[pre + "attn." + rest] = t
        elif rest == "to_out.weight":
            out[pre + "attn.to_out.0.weight"] = t
        elif rest in ("norm_q", "norm_k"):
            out[pre + f"attn.{rest}.weight"] = t
        elif rest in ("norm1", "norm2"):
            out[pre + f"{rest}.weight"] = t
        elif rest == "adaln_proj":
            out[pre + "adaln_proj.weight"] = t
        elif rest == "ffn_gate_up.weight":
            half = t.shape[0] // 2
            out[pre + "ffn.gate_proj.weight"], out[pre + "ffn.up_proj.weight"] = t[:half].contiguous(), t[half:].contiguous()
        elif rest == "ffn_down.weight":
            out[pre + "ffn.down_proj.weight"] = t
        else:
            raise BackendContractError(f"no released name for {name}")
    return out
