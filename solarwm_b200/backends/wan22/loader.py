"""Released-weight loading for the Wan families: safetensors shard inventory and strict load.

``inventory(dir)`` reads ``*.safetensors`` headers (or a ``*.index.json`` weight map) without touching
tensor data and reports, per tensor name, the shard, dtype and shape; ``strict_load(model, dir)``
refuses missing, unexpected, mis-shaped or non-floating tensors before a single byte is copied, then
streams shard by shard into the model's flat buffers (the parameters are views, so a load is a set of
``copy_`` calls into resident memory).  Built-in architecture descriptions of the two released
families live in ``ARCHITECTURES`` (reference: solar/backends/wan22/runtime/loader.py:122-256,
runtime/architectures/{ti2v_5b,i2v_a14b}.json).
"""
from __future__ import annotations

import json
import struct
from pathlib import Path
from typing import Dict, Mapping, NamedTuple, Optional

import torch

from ...errors import BackendContractError

ARCHITECTURES: Mapping[str, Mapping[str, object]] = {
    "ti2v_5b": {"model_type": "ti2v", "patch_size": [1, 2, 2], "in_dim": 48, "out_dim": 48, "dim": 3072, "ffn_dim": 14336,
                "num_heads": 24, "num_layers": 30, "text_dim": 4096, "text_len": 512, "freq_dim": 256, "eps": 1e-6},
    "i2v_a14b": {"model_type": "i2v", "patch_size": [1, 2, 2], "in_dim": 36, "out_dim": 16, "dim": 5120, "ffn_dim": 13824,
                 "num_heads": 40, "num_layers": 40, "text_dim": 4096, "text_len": 512, "freq_dim": 256, "eps": 1e-6},
}
_DTYPES = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64}


class TensorEntry(NamedTuple):
    shard: str
    dtype: str
    shape: tuple


def read_header(path) -> Dict[str, dict]:
    """The JSON header of one safetensors file (8-byte little-endian length, then JSON)."""
    with open(path, "rb") as fh:
        raw = fh.read(8)
        if len(raw) != 8:
            raise BackendContractError(f"{path}: not a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        if n <= 0 or n > 1 << 28:
            raise BackendContractError(f"{path}: implausible safetensors header length {n}")
        header = json.loads(fh.read(n).decode("utf-8"))
    header.pop("__metadata__", None)
    return header


def inventory(directory) -> Dict[str, TensorEntry]:
    root = Path(directory)
    shards = sorted(root.glob("*.safetensors"))
    if not shards:
        raise BackendContractError(f"no safetensors shards under {root}")
    index = next(iter(sorted(root.glob("*.index.json"))), None)
    wanted: Optional[Mapping[str, str]] = None
    if index is not None:
        wanted = json.loads(index.read_text())["weight_map"]
    out: Dict[str, TensorEntry] = {}
    for shard in shards:
        for name, meta in read_header(shard).items():
            if name in out:
                raise BackendContractError(f"tensor {name!r} appears in {out[name].shard} and {shard.name}")
            if wanted is not None and wanted.get(name) != shard.name:
                raise BackendContractError(f"tensor {name!r}: index points at {wanted.get(name)!r}, found in {shard.name}")
            out[name] = TensorEntry(shard.name, meta["dtype"], tuple(int(d) for d in meta["shape"]))
    if wanted is not None and set(wanted) - set(out):
        raise BackendContractError(f"index lists tensors that no shard holds: {sorted(set(wanted) - set(out))[:5]}")
    return out


def check_against(model: torch.nn.Module, entries: Mapping[str, TensorEntry], prefix: str = "") -> None:
    want = {prefix + k: tuple(v.shape) for k, v in model.state_dict().items()}
    missing = sorted(set(want) - set(entries))
    extra = sorted(set(entries) - set(want))
    if missing or extra:
        raise BackendContractError(f"checkpoint does not match the architecture: missing {missing[:5]} "
                                   f"({len(missing)}), unexpected {extra[:5]} ({len(extra)})")
    for name, shape in want.items():
        e = entries[name]
        if e.shape != shape:
            raise BackendContractError(f"{name}: shape {e.shape} in the checkpoint, {shape} in the model")
        if e.dtype not in _DTYPES:
            raise BackendContractError(f"{name}: dtype {e.dtype} is not a floating type this loader accepts")


@torch.no_grad()
def strict_load(model: torch.nn.Module, directory, prefix: str = "") -> Mapping[str, int]:
    """Verify first, copy after.  Returns {shard: tensors copied}."""
    from safetensors import safe_open

    entries = inventory(directory)
    check_against(model, entries, prefix)
    params = dict(model.state_dict(keep_vars=True))
    by_shard: Dict[str, list] = {}
    for name, e in entries.items():
        by_shard.setdefault(e.shard, []).append(name)
    copied = {}
    for shard, names in sorted(by_shard.items()):
        with safe_open(str(Path(directory) / shard), framework="pt", device="cpu") as fh:
            for name in names:
                dst = params[name[len(prefix):]]
                dst.data.copy_(fh.get_tensor(name).to(dst.dtype))
        copied[shard] = len(names)
    return copied
