"""Tar shards of pre-encoded samples and their JSONL index.

A sample is stored as ``<sample_id>.<tensor>.npy`` members (bf16 as uint16 views with a dtype tag
in the sidecar) plus ``<sample_id>.json`` (contract digest, dtypes, source identity).  A shard is
written under a temporary name, fsynced, and published create-only; the index is written last, so
an index row never points at a shard that is not complete (reference: solar/preencode/shards.py:55-128).
"""
from __future__ import annotations

import io
import json
import os
import tarfile
import time
from pathlib import Path
from typing import Any, Iterable, List, Mapping

import numpy as np

from ..data.index import write_index
from ..errors import DataContractError
from ..runtime.create_only import rename_noreplace
from .contracts import EncoderContract, validate_encoded_tensors


def _to_numpy(t):
    """-> (array, dtype tag).  bf16 torch tensors are stored as their uint16 bit pattern."""
    if isinstance(t, np.ndarray):
        return t, str(t.dtype)
    import torch

    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.uint16).numpy(), "bfloat16"
    return t.numpy(), str(t.dtype).replace("torch.", "")


def _from_numpy(arr: np.ndarray, tag: str):
    import torch

    if tag == "bfloat16":
        return torch.from_numpy(arr.copy()).view(torch.bfloat16)
    return torch.from_numpy(arr.copy())


class EncodedShardWriter:
    def __init__(self, root, contract: EncoderContract, samples_per_shard: int = 64, prefix: str = "encoded"):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        self.contract = contract
        self.per = int(samples_per_shard)
        self.prefix = prefix
        self.rows: List[dict] = []
        self._n_shards = 0
        self._tar = None
        self._tmp = None
        self._in_shard = 0
        self._pending: List[dict] = []

    def _open(self):
        name = f"{self.prefix}-{self._n_shards:06d}.tar"
        self._final = self.root / name
        if self._final.exists():
            raise DataContractError(f"encoded shard already exists: {self._final}")
        self._tmp = self.root / f".{name}.{os.getpid()}.partial"
        self._tar = tarfile.open(self._tmp, "w")
        self._in_shard = 0
        self._pending = []

    def _add(self, name: str, data: bytes):
        info = tarfile.TarInfo(name)
        info.size = len(data)
        info.mtime = int(time.time())
        self._tar.addfile(info, io.BytesIO(data))

    def add(self, sample_id: str, tensors: Mapping[str, Any], meta: Mapping[str, Any] = None) -> None:
        validate_encoded_tensors(self.contract, tensors)
        if self._tar is None:
            self._open()
        tags = {}
        for name, t in tensors.items():
            arr, tag = _to_numpy(t)
            tags[name] = tag
            buf = io.BytesIO()
            np.save(buf, arr, allow_pickle=False)
            self._add(f"{sample_id}.{name}.npy", buf.getvalue())
        side = {"sample_id": sample_id, "contract_digest": self.contract.digest, "dtypes": tags, **dict(meta or {})}
        self._add(f"{sample_id}.json", json.dumps(side, sort_keys=True).encode())
        self._pending.append({"sample_id": sample_id, "key": sample_id, "shard": self._final.name,
                              "epoch_repeats": 1, "contract_digest": self.contract.digest,
                              "members": {n: f"{sample_id}.{n}.npy" for n in tensors}, **dict(meta or {})})
        self._in_shard += 1
        if self._in_shard >= self.per:
            self._close_shard()

    def _close_shard(self):
        if self._tar is None:
            return
        self._tar.close()
        with open(self._tmp, "rb") as fh:
            os.fsync(fh.fileno())
        rename_noreplace(self._tmp, self._final)
        size = self._final.stat().st_size
        for row in self._pending:
            row["shard_size"] = size
        self.rows.extend(self._pending)
        self._tar, self._tmp, self._pending = None, None, []
        self._n_shards += 1

    def finish(self, index_name: str = "index.jsonl") -> Path:
        """Close the open shard, then write the contract and -- last -- the index."""
        self._close_shard()
        (self.root / "encoder-contract.json").write_text(json.dumps(self.contract.as_dict(), sort_keys=True, indent=1))
        path = self.root / index_name
        write_encoded_index(path, self.rows)
        return path


def write_encoded_index(path, rows: Iterable[Mapping[str, Any]]) -> int:
    return write_index(path, rows)


def read_encoded_sample(root, row: Mapping[str, Any], contract: EncoderContract = None) -> dict:
    """Load one sample's tensors (torch) from its shard; verifies the contract digest when given."""
    shard = Path(root) / row["shard"]
    out = {}
    with tarfile.open(shard, "r") as tar:
        side = json.loads(tar.extractfile(f"{row['sample_id']}.json").read())
        if contract is not None and side["contract_digest"] != contract.digest:
            raise DataContractError(f"sample {row['sample_id']} was encoded under a different contract")
        for name, member in row["members"].items():
            arr = np.load(io.BytesIO(tar.extractfile(member).read()), allow_pickle=False)
            out[name] = _from_numpy(arr, side["dtypes"][name])
    return out
