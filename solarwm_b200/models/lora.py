"""Low-rank adapters over the frozen linears of a ``WanDiT`` / ``LTXDiT``.

``inject_lora`` freezes every base parameter and gives each targeted linear of every block a pair ``lora_A`` [r, in]
(Kaiming-uniform) / ``lora_B`` [out, r] (zeros), so the adapted model starts as the base model.  The block routes its
targeted projections through ``ops.functional.lora_linear`` (adapter product accumulated into the base GEMM's output);
the fused q | k | v projection is issued per part while adapters are installed.  ``LoRARuntime`` is the adapter's
state: an ordered key -> parameter table under the key inventory of the released recipe
(``transformer_blocks.<i>.<module>.lora_A.weight`` ...), strict ``load_state_dict`` (same keys, shapes, dtypes),
``broadcast`` from rank 0 and the metadata record that travels with a checkpoint.  The adapters are replicated on every
rank and never sharded; their gradients are reduced by the trainer.

Reference: inject_lora / LoRARuntime (solar/backends/ltx25/torch_model.py:844-955), target set and rank
(solar/backends/ltx25/adapter.py:21-43: q / k / v / out of both attentions and both FFN linears, r = alpha = 384),
adapters ignored by the sharding wrap (solar/backends/ltx25/torch_training.py:82-138).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Mapping, Sequence

import torch
import torch.nn as nn

from ..errors import BackendContractError

METADATA_SCHEMA = "solarwm.ltx25.peft-lora.v1"

# this package's projection name -> the released recipe's module suffix
TARGET_SUFFIX = OrderedDict([
    ("self_attn.q", "attn1.to_q"), ("self_attn.k", "attn1.to_k"), ("self_attn.v", "attn1.to_v"), ("self_attn.o", "attn1.to_out.0"),
    ("cross_attn.q", "attn2.to_q"), ("cross_attn.k", "attn2.to_k"), ("cross_attn.v", "attn2.to_v"), ("cross_attn.o", "attn2.to_out.0"),
    ("ffn.0", "ff.net.0.proj"), ("ffn.2", "ff.net.2"),
])


class Adapter(nn.Module):
    def __init__(self, d_in: int, d_out: int, rank: int, scale: float, device, dtype, gen):
        super().__init__()
        bound = 1.0 / math.sqrt(d_in)                                   # Kaiming-uniform with a = sqrt(5)
        a = (torch.rand(rank, d_in, generator=gen) * 2 - 1) * bound
        self.lora_A = nn.Parameter(a.to(device, dtype))
        self.lora_B = nn.Parameter(torch.zeros(d_out, rank, device=device, dtype=dtype))
        self.scale = float(scale)


class LoRARuntime:
    def __init__(self, model, parameter_by_key: "OrderedDict[str, nn.Parameter]", rank: int, alpha: float, targets):
        self.model, self.parameter_by_key = model, parameter_by_key
        self.parameters = tuple(parameter_by_key.values())
        self.keys = tuple(parameter_by_key)
        self.rank, self.alpha, self.targets = int(rank), float(alpha), tuple(targets)

    def state_dict(self) -> "OrderedDict[str, torch.Tensor]":
        return OrderedDict((k, p.detach()) for k, p in self.parameter_by_key.items())

    def load_state_dict(self, values: Mapping[str, torch.Tensor], *, broadcast: bool = True) -> None:
        if set(values) != set(self.parameter_by_key):
            odd = sorted(set(values) ^ set(self.parameter_by_key))
            raise BackendContractError(f"adapter checkpoint key inventory differs (e.g. {odd[:4]})")
        for key, p in self.parameter_by_key.items():
            v = values[key]
            if tuple(v.shape) != tuple(p.shape) or v.dtype != p.dtype:
                raise BackendContractError(f"adapter checkpoint layout differs for {key}: {tuple(v.shape)} {v.dtype}")
        with torch.no_grad():
            for key, p in self.parameter_by_key.items():
                p.copy_(values[key].to(p.device))
        if broadcast:
            self.broadcast()

    def broadcast(self, group=None) -> None:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            for p in self.parameters:
                dist.broadcast(p.data, src=0 if group is None else dist.get_global_rank(group, 0), group=group)

    def metadata(self) -> dict:
        return {"schema": METADATA_SCHEMA, "runtime": "native", "rank": self.rank, "alpha": self.alpha,
                "targets": [f"transformer_blocks.{i}.{TARGET_SUFFIX[t]}" for i in range(len(self.model.blocks)) for t in self.targets],
                "state_keys": list(self.keys),
                "state_shapes": {k: list(p.shape) for k, p in self.parameter_by_key.items()},
                "state_dtypes": {k: str(p.dtype).replace("torch.", "") for k, p in self.parameter_by_key.items()}}

    @torch.no_grad()
    def merge_(self) -> None:
        """Fold every adapter into its base weight and zero it (export of merged weights)."""
        for block in self.model.blocks:
            for key, ad in block.lora.items():
                w = block._p(f"{key.replace('__', '.')}.weight")
                w.add_((ad.scale * (ad.lora_B.float() @ ad.lora_A.float())).to(w.dtype))
                ad.lora_B.zero_()


def adapter_parameter_count(cfg, rank: int = 384, targets: Sequence[str] = tuple(TARGET_SUFFIX)) -> int:
    """Trainable parameters ``inject_lora`` adds to a model of configuration ``cfg``."""
    d, f = cfg.dim, cfg.ffn_dim
    shapes = {"ffn.0": (f, d), "ffn.2": (d, f)}
    return cfg.num_layers * sum(rank * sum(shapes.get(t, (d, d))) for t in targets)


def inject_lora(model, rank: int = 384, alpha: float = None, targets: Sequence[str] = tuple(TARGET_SUFFIX), seed: int = 0) -> LoRARuntime:
    if rank < 1:
        raise BackendContractError("adapter rank must be positive")
    unknown = [t for t in targets if t not in TARGET_SUFFIX]
    if unknown:
        raise BackendContractError(f"unknown adapter targets {unknown}")
    if any(getattr(b, "lora", None) for b in model.blocks):
        raise BackendContractError("adapters are already installed")
    alpha = float(rank if alpha is None else alpha)
    for p in model.parameters():
        p.requires_grad_(False)
    gen = torch.Generator().manual_seed(int(seed))
    table: "OrderedDict[str, nn.Parameter]" = OrderedDict()
    for i, block in enumerate(model.blocks):
        block.lora = nn.ModuleDict()
        for t in targets:
            w = block._p(f"{t}.weight")
            ad = Adapter(w.shape[1], w.shape[0], rank, alpha / rank, w.device, w.dtype, gen)
            block.lora[t.replace(".", "__")] = ad
            base = f"transformer_blocks.{i}.{TARGET_SUFFIX[t]}"
            table[f"{base}.lora_A.weight"], table[f"{base}.lora_B.weight"] = ad.lora_A, ad.lora_B
    if len(table) != 2 * len(targets) * len(model.blocks):
        raise BackendContractError("realised adapter inventory drifted")
    return LoRARuntime(model, table, rank, alpha, targets)
