"""ctypes front end of ``csrc/attention_bwd.cu`` (dK/dV and dQ kernels on tcgen05/TMEM)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from .attention_native import _bshd
from .functional import status_word


_overlap_set = False


def set_tail_overlap(enable: bool) -> bool:
    """dQ kernel on a side stream so that it fills the partly empty last wave of the dK/dV kernel (matters when a
    rank owns few heads).  Returns the previous setting."""
    global _overlap_set
    _overlap_set = True
    return bool(_lib.load().solar_attn_bwd_overlap(c_int(1 if enable else 0)))


def ensure_tail_overlap_default() -> None:
    """First use: apply ``SOLAR_ATTN_BWD_OVERLAP`` (default on) unless ``set_tail_overlap`` was called already."""
    if not _overlap_set:
        import os

        set_tail_overlap(os.environ.get("SOLAR_ATTN_BWD_OVERLAP", "1") != "0")


def attn_bwd_native(q, k, v, o, lse, do, scale: float):
    ensure_tail_overlap_default()
    q, k, v, o, do = _bshd(q), _bshd(k), _bshd(v), _bshd(o), _bshd(do)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    dk = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
    dv = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
    sq_pad = (Sq + 127) // 128 * 128
    scratch = torch.empty(2 * B * H * sq_pad, dtype=torch.float32, device=q.device)
    lib = _lib.load()
    rc = lib.solar_attn_bwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(dq), ptr(dk), ptr(dv),
                            ptr(scratch), c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(D),
                            c_ll(q.stride(1)), c_ll(q.stride(0)), c_ll(k.stride(1)), c_ll(k.stride(0)),
                            c_ll(v.stride(1)), c_ll(v.stride(0)), c_ll(o.stride(1)), c_ll(o.stride(0)),
                            c_ll(do.stride(1)), c_ll(do.stride(0)), c_float(scale), ptr(status_word(q.device)),
                            stream_handle())
    check(rc, "solar_attn_bwd")
    count("attn_bwd", 3)
    return dq, dk, dv
