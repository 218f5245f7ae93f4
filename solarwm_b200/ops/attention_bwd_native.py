"""ctypes front end of ``csrc/attention_bwd.cu`` (dK/dV and dQ kernels on tcgen05/TMEM)."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from .attention_native import _bshd
from .functional import status_word


def attn_bwd_native(q, k, v, o, lse, do, scale: float):
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
