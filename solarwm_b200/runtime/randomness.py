"""Seed domains.  Model initialisation uses a per-family namespace; the objective stream is shared
by sequence-parallel peers (they must draw identical noise/timesteps) and differs across
data-parallel ranks: ``objective_seed = base * 100003 + dp_rank * 1024``
(reference: solar/runtime/randomness.py:16-97)."""
from __future__ import annotations

import hashlib
import random

_MODEL_INIT_NAMESPACE = {
    "wan22_ti2v_5b": 0x5B, "wan22_i2v_a14b": 0xA14B, "ltx25_video": 0x17C5, "minimax_h3": 0x33B,
}


def model_init_seed(family: str, base_seed: int) -> int:
    if family not in _MODEL_INIT_NAMESPACE:
        raise KeyError(f"no model-init namespace for family {family!r}")
    return (int(base_seed) * 1000003 + _MODEL_INIT_NAMESPACE[family]) % (2 ** 63)


def objective_seed(base_seed: int, dp_rank: int) -> int:
    return int(base_seed) * 100003 + int(dp_rank) * 1024


def stable_validation_seed(*parts) -> int:
    """Seed that depends only on its arguments (never on process hashing)."""
    h = hashlib.blake2b("\x1f".join(str(p) for p in parts).encode(), digest_size=8).digest()
    return int.from_bytes(h, "big") % (2 ** 63)


def seed_process(seed: int, *, cuda: bool = True) -> None:
    import numpy as np
    import torch

    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if cuda and torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
