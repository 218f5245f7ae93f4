"""Long-range memory for streaming generation: which past latents does the current view overlap?

The current chunk's last latent is the query camera.  Its frustum is sampled as an 8 x 8 grid of
pixel rays times four logarithmic depth bins (near 2, far 60 camera units; all lengths divided by 4);
every candidate camera outside the recent window is scored by

    overlap(fraction of those points it sees) - 0.2 * (translation distance + 4 * viewing-angle difference)

and the ``top_k`` best are returned in score order (ties keep index order).  ``LatentMemoryBank``
keeps committed chunks in bf16 and gathers single latents by absolute index; the gathered latents
enter the packed document as memory rows with their own cameras
(reference: solar/backends/minimax_h3/memory_retrieval.py:13-86).

All of this runs on the host in fp64 (a few hundred cameras); nothing here is on the device path.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import numpy as np

GRID = 8
DEPTH_BINS = 4
NEAR, FAR, UNIT = 2.0, 60.0, 4.0


def frustum_points(intrinsics, width: int, height: int) -> Tuple[np.ndarray, tuple]:
    """Camera-space sample points [3, GRID*GRID*DEPTH_BINS] and pixel intrinsics (fx, fy, cx, cy)."""
    K = np.asarray(intrinsics, dtype=np.float64)
    fx, fy, cx, cy = K[0, 0] * width, K[1, 1] * height, K[0, 2] * width, K[1, 2] * height
    u = (np.arange(GRID) + 0.5) / GRID * width
    v = (np.arange(GRID) + 0.5) / GRID * height
    uu, vv = np.meshgrid(u, v, indexing="ij")
    rays = np.stack([(uu.ravel() - cx) / fx, (vv.ravel() - cy) / fy, np.ones(GRID * GRID)])
    edges = np.linspace(np.log(NEAR / UNIT), np.log(FAR / UNIT), DEPTH_BINS + 1)
    depths = np.exp(0.5 * (edges[:-1] + edges[1:]))
    return (rays[:, :, None] * depths[None, None, :]).reshape(3, -1), (fx, fy, cx, cy)


def retrieval_scores(query_c2w, candidate_c2w, intrinsics, *, width: int = 1344, height: int = 768) -> np.ndarray:
    q = np.array(query_c2w, dtype=np.float64)
    c = np.array(candidate_c2w, dtype=np.float64).reshape(-1, 4, 4)
    if c.shape[0] == 0:
        return np.empty(0, dtype=np.float64)
    q[:3, 3] /= UNIT
    c[:, :3, 3] /= UNIT
    pts, (fx, fy, cx, cy) = frustum_points(intrinsics, width, height)
    world = q[:3, :3] @ pts + q[:3, 3:4]
    rt = np.transpose(c[:, :3, :3], (0, 2, 1))                       # world -> candidate camera
    pc = np.einsum("mij,jp->mip", rt, world) - np.einsum("mij,mj->mi", rt, c[:, :3, 3])[:, :, None]
    z = pc[:, 2]
    zs = np.clip(z, 1e-9, None)
    pu, pv = pc[:, 0] * fx / zs + cx, pc[:, 1] * fy / zs + cy
    seen = (z > 0.5) & (z < 15.0) & (pu >= 0) & (pu <= width) & (pv >= 0) & (pv <= height)
    overlap = seen.mean(axis=1)
    distance = np.linalg.norm(c[:, :3, 3] - q[:3, 3], axis=1)
    angle = np.arccos(np.clip(c[:, :3, 2] @ q[:3, 2], -1.0, 1.0))
    return overlap - 0.2 * (distance + 4.0 * angle)


def select_memory(c2w: Sequence, intrinsics: Sequence, chunk_index: int, *, chunk_latents: int = 5, top_k: int = 5,
                  recent_chunks: int = 5):
    """Indices (absolute latent numbers) and scores of the retrieved latents for ``chunk_index``."""
    poses = np.asarray(c2w, dtype=np.float64)
    stop = max(0, chunk_index - recent_chunks) * chunk_latents
    cand = np.arange(stop, dtype=np.int64)
    if cand.size == 0:
        return cand, np.empty(0)
    query = chunk_latents * chunk_index + chunk_latents - 1
    scores = retrieval_scores(poses[query], poses[cand], np.asarray(intrinsics)[query])
    order = np.argsort(-scores, kind="stable")[:top_k]
    return cand[order], scores[order]


@dataclass
class LatentMemoryBank:
    chunk_latents: int = 5
    chunks: List = field(default_factory=list)

    def commit(self, chunk, index: int) -> None:
        """chunk [B, C, chunk_latents, H, W]; chunks must arrive complete and in order."""
        import torch

        if index != len(self.chunks) or chunk.shape[2] != self.chunk_latents:
            raise ValueError("memory bank takes complete chunks in order")
        self.chunks.append(chunk.detach().to(torch.bfloat16).clone())

    def gather(self, indices, like):
        import torch

        if len(indices) == 0:
            return like[:, :, :0]
        n = self.chunk_latents
        return torch.cat([self.chunks[int(i) // n][:, :, int(i) % n:int(i) % n + 1] for i in indices], dim=2).float()


class RetrievalCameras:
    """Append-only host record of every generated latent's camera (what retrieval scores against)."""

    def __init__(self):
        self.c2w: List[np.ndarray] = []
        self.K: List[np.ndarray] = []

    def append(self, c2w, K) -> None:
        c2w, K = np.asarray(c2w, dtype=np.float64), np.asarray(K, dtype=np.float64)
        if c2w.shape != (4, 4) or K.shape != (3, 3):
            raise ValueError("cameras are 4x4 camera-to-world with 3x3 normalised intrinsics")
        self.c2w.append(c2w)
        self.K.append(K)

    def select(self, chunk_index: int, **kw):
        return select_memory(np.stack(self.c2w), np.stack(self.K), chunk_index, **kw)


def adapter_digest(state) -> str:
    """sha256 over names and bytes of an adapter state, in name order."""
    import hashlib

    import torch

    h = hashlib.sha256()
    for key in sorted(state):
        h.update(key.encode())
        h.update(state[key].detach().cpu().contiguous().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


def attach_memory_adapter(model, *, rank: int, memory_state=None, frozen_identity: str = "", seed: int = 0):
    """Install the Memory adapter as a named bank beside the generation adapters and return its identity record.

    The generation (Stage2) adapters must already be part of the base -- merged, as ``infer`` does -- or frozen: the
    Memory bank is evaluated INSTEAD of the primary adapter while memory rows are installed, so only a merged base gives
    the composition "Stage2 + Memory".  A fresh bank must contribute exactly zero (its up-projections are zero); a given
    ``memory_state`` (``{parameter name ending in __memory: tensor}``) is loaded strictly.  Afterwards nothing in the model
    trains.  (reference: attach_memory_adapter, solar/backends/minimax_h3/memory_adapter.py:11-61)"""
    import torch

    from ..models.h3 import LoRALinear

    mods = [m for m in model.modules() if isinstance(m, LoRALinear)]
    if any(m.rank > 0 and any(p.requires_grad for p in (m.lora_A, m.lora_B)) for m in mods):
        raise ValueError("the generation adapters must be merged into the base or frozen before the Memory bank is attached")
    if any(hasattr(m, "lora_A__memory") for m in mods):
        raise ValueError("a Memory bank is already attached")
    model.add_adapter("memory", rank=int(rank), seed=int(seed))
    own = {k: v for k, v in model.named_parameters() if k.endswith("__memory")}
    if memory_state is None:
        if any(int(torch.count_nonzero(p)) for k, p in own.items() if "lora_B__" in k):
            raise ValueError("a new Memory bank must initially contribute zero")
        digest = "fresh-zero"
    else:
        if set(memory_state) != set(own):
            odd = sorted(set(memory_state) ^ set(own))[:4]
            raise ValueError(f"the Memory adapter's tensors do not match the bank (e.g. {odd})")
        with torch.no_grad():
            for k, p in own.items():
                if tuple(memory_state[k].shape) != tuple(p.shape):
                    raise ValueError(f"{k}: shape {tuple(memory_state[k].shape)} does not fit {tuple(p.shape)}")
                p.copy_(memory_state[k].to(p))
        digest = adapter_digest(memory_state)
    model.requires_grad_(False)
    return {"frozen_adapter": str(frozen_identity), "memory_adapter": digest, "rank": int(rank),
            "parameter_count": int(sum(p.numel() for p in own.values())), "tensors": len(own), "active_with_memory_rows": ["merged-base", "memory"]}
