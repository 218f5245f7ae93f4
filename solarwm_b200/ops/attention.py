"""Attention front end.

``attention(q, k, v)`` takes ``[B, S, H, D]`` tensors.  On CUDA it launches the hand-written
sm_100a flash-attention kernels (``csrc/attention.cu``: S = QK^T and O += PV on tcgen05 with
accumulators in TMEM, K/V tiles streamed by TMA, online softmax in registers); on CPU it runs
the fp32 PyTorch statement.  ``backend="library"`` selects torch SDPA and exists only as the
baseline arm for comparisons -- it is never the default on a GPU.

Replaces flash_attn varlen / SDPA of the reference
(solar/backends/wan22/runtime/modeling/attention.py:34-188).
"""
from __future__ import annotations

import math
import os

import torch

from . import _lib, reference
from ._lib import count

_BACKEND = os.environ.get("SOLAR_B200_ATTENTION", "native")


def set_backend(name: str) -> None:
    global _BACKEND
    if name not in ("native", "library"):
        raise ValueError(name)
    _BACKEND = name


def get_backend() -> str:
    return _BACKEND


def _library_attention(q, k, v, scale):
    o = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=scale)
    return o.transpose(1, 2).contiguous()


def native_supported(q, k) -> bool:
    return _lib.available() and hasattr(_lib.load(), "solar_attn_fwd") and q.shape[-1] in (64, 128)


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, memo):
        from .attention_native import attn_fwd

        # ``memo`` = (dict, key): under activation checkpointing the first forward stores the
        # attention output and log-sum-exp there and the recompute pass takes them back instead
        # of running the kernel a second time (attention is the one op too costly to recompute).
        cached = None if memo is None else memo[0].pop(memo[1], None)
        if cached is not None:
            o, lse = cached
        else:
            o, lse = attn_fwd(q, k, v, scale)
            if memo is not None and memo[0].get("__store__", False):
                memo[0][memo[1]] = (o, lse)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        from .attention_native import attn_bwd

        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = attn_bwd(q, k, v, o, lse, do.contiguous(), ctx.scale)
        return dq, dk, dv, None, None


def attention(q, k, v, *, scale=None, backend=None, memo=None):
    """Bidirectional softmax attention; q ``[B, Sq, H, D]``, k/v ``[B, Sk, H, D]`` -> ``[B, Sq, H, D]``.
    ``memo`` is an optional ``(dict, key)`` slot used to carry the output across a checkpoint recompute."""
    d = q.shape[-1]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    if not q.is_cuda:
        return reference.attention(q, k, v, scale=scale)
    backend = backend or _BACKEND
    if backend == "native":
        if not native_supported(q, k):
            raise _lib.NativeError(f"native attention does not support head_dim={d}")
        return _AttnFn.apply(q, k, v, scale, memo)
    count("library_sdpa")
    return _library_attention(q, k, v, scale)
