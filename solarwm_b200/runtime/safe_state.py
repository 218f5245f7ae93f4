"""RNG state <-> plain containers, so checkpoints stay loadable with ``torch.load(weights_only=True)``.

Python's ``random`` state is ``(version, tuple[625 ints], gauss_next)`` and NumPy's legacy
MT19937 state is ``('MT19937', uint32[624], pos, has_gauss, cached_gaussian)``; both are stored as
dicts of ints, floats and lists -- no pickled objects
(reference: solar/runtime/safe_state.py:43-195)."""
from __future__ import annotations

import random
from typing import Any, Mapping

from ..errors import CheckpointError

PY_SCHEMA = "solarwm.python-rng.v1"
NP_SCHEMA = "solarwm.numpy-rng.v1"


def encode_python_rng(state=None) -> dict:
    version, internal, gauss = random.getstate() if state is None else state
    return {"schema": PY_SCHEMA, "version": int(version), "internal": [int(v) for v in internal],
            "gauss_next": None if gauss is None else float(gauss)}


def decode_python_rng(value: Mapping[str, Any]):
    if value.get("schema") != PY_SCHEMA:
        raise CheckpointError("unknown python RNG state schema")
    internal = value["internal"]
    if not isinstance(internal, (list, tuple)) or len(internal) != 625:
        raise CheckpointError("python RNG state must hold 625 integers")
    gauss = value.get("gauss_next")
    return (int(value["version"]), tuple(int(v) for v in internal), None if gauss is None else float(gauss))


def restore_python_rng(value: Mapping[str, Any]) -> None:
    random.setstate(decode_python_rng(value))


def encode_numpy_rng(state=None) -> dict:
    import numpy as np

    name, keys, pos, has_gauss, cached = np.random.get_state() if state is None else state
    if name != "MT19937":
        raise CheckpointError(f"unsupported numpy bit generator {name!r}")
    return {"schema": NP_SCHEMA, "keys": [int(k) for k in keys], "pos": int(pos), "has_gauss": int(has_gauss),
            "cached_gaussian": float(cached)}


def decode_numpy_rng(value: Mapping[str, Any]):
    import numpy as np

    if value.get("schema") != NP_SCHEMA:
        raise CheckpointError("unknown numpy RNG state schema")
    keys = value["keys"]
    if not isinstance(keys, (list, tuple)) or len(keys) != 624:
        raise CheckpointError("numpy RNG state must hold 624 words")
    return ("MT19937", np.asarray(keys, dtype=np.uint32), int(value["pos"]), int(value["has_gauss"]),
            float(value["cached_gaussian"]))


def restore_numpy_rng(value: Mapping[str, Any]) -> None:
    import numpy as np

    np.random.set_state(decode_numpy_rng(value))


def capture_rank_state(device=None) -> dict:
    """Everything a rank needs for an exact resume of its random streams."""
    import torch

    out = {"python": encode_python_rng(), "numpy": encode_numpy_rng(), "torch_cpu": torch.get_rng_state()}
    if device is not None and torch.device(device).type == "cuda":
        out["torch_cuda"] = torch.cuda.get_rng_state(device)
    return out


def restore_rank_state(state: Mapping[str, Any], device=None) -> None:
    import torch

    restore_python_rng(state["python"])
    restore_numpy_rng(state["numpy"])
    torch.set_rng_state(state["torch_cpu"])
    if "torch_cuda" in state and device is not None:
        torch.cuda.set_rng_state(state["torch_cuda"], device)
