"""Scene admission for the realtime engine: reject a bad scene on every rank at once, before any device collective.

A scene (prompt embedding, anchor latent, geometry) is checked by every rank on its own copy; the verdicts are
exchanged on the control group (gloo, host only) and either every rank proceeds or every rank raises the same
``SceneRejected`` carrying ``pre_call_collective_agreement=True``.  Because the agreement happens before the first
device-side exchange of the scene, a rejection leaves the resident model, its caches and its captured graphs
untouched: the worker parks the scene (``recover``) and keeps serving.  Any other error -- or a rejection that was
not agreed collectively -- is not recoverable and tears the session down
(reference behaviour: deploy/solar_wm/backends/standard/runtime/engine.py:245-272).
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional

import torch

from ..errors import BackendContractError
from ..runtime.distributed import propagate_collective_error


class SceneRejected(BackendContractError):
    def __init__(self, message: str, *, stage: str, pre_call_collective_agreement: bool):
        super().__init__(message)
        self.stage = stage
        self.pre_call_collective_agreement = bool(pre_call_collective_agreement)


def check_scene(scene: Mapping[str, torch.Tensor], *, text_dim: int, latent_channels: int, grid_hw,
                max_prompt_tokens: int = 4096) -> Optional[str]:
    """A rank-local verdict: ``None`` when the scene can be served, else the reason."""
    text, anchor = scene.get("text"), scene.get("anchor_latent")
    if not isinstance(text, torch.Tensor) or text.dim() != 2 or text.shape[1] != text_dim:
        return f"prompt embedding must be [tokens, {text_dim}]"
    if not 1 <= text.shape[0] <= max_prompt_tokens:
        return f"prompt has {text.shape[0]} tokens, allowed 1..{max_prompt_tokens}"
    h, w = grid_hw
    want = (latent_channels, 1, 2 * h, 2 * w)
    if not isinstance(anchor, torch.Tensor) or tuple(anchor.shape) != want:
        return f"anchor latent must be {want}"
    if not bool(torch.isfinite(text.float()).all()) or not bool(torch.isfinite(anchor.float()).all()):
        return "scene tensors hold non-finite values"
    return None


def admit_scene(verdict: Optional[str], *, dist=None, rank=None, world_size=None, stage: str = "scene_start") -> None:
    """Exchange the rank-local verdicts; raise the same ``SceneRejected`` everywhere if any rank objects."""
    try:
        propagate_collective_error(verdict, dist=dist, label=stage, rank=rank, world_size=world_size)
    except BackendContractError as exc:
        raise SceneRejected(str(exc), stage=stage, pre_call_collective_agreement=True) from None


def recover(error: BaseException, park: Callable[[], None]) -> str:
    """Park the rejected scene and report its stage; anything but a coordinated pre-call rejection is re-raised."""
    if not isinstance(error, SceneRejected) or not error.pre_call_collective_agreement:
        raise RuntimeError("only a coordinated pre-call rejection is recoverable") from error
    if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
        raise RuntimeError("cannot recover in the middle of a graph capture") from error
    park()
    return error.stage
