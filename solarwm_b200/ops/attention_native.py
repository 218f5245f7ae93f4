"""ctypes front end of ``csrc/attention.cu`` (flash attention forward on tcgen05/TMEM) and of the
attention backward kernels."""
from __future__ import annotations

import torch

from . import _lib
from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from .functional import status_word


def _bshd(t: torch.Tensor) -> torch.Tensor:
    """Accept any [B, S, H, D] view with unit stride on D, stride D on H and 16-byte aligned rows."""
    B, S, H, D = t.shape
    ok = (t.stride(3) == 1 and t.stride(2) == D and (t.stride(1) * 2) % 16 == 0 and (t.stride(0) * 2) % 16 == 0
          and t.data_ptr() % 16 == 0)
    return t if ok else t.contiguous()


def attn_fwd(q, k, v, scale: float, need_lse: bool = True):
    assert q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16
    q, k, v = _bshd(q), _bshd(k), _bshd(v)
    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    o = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if need_lse else None
    lib = _lib.load()
    rc = lib.solar_attn_fwd(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(B), c_int(Sq), c_int(Sk), c_int(H),
                            c_int(D), c_ll(q.stride(1)), c_ll(q.stride(0)), c_ll(k.stride(1)), c_ll(k.stride(0)),
                            c_ll(v.stride(1)), c_ll(v.stride(0)), c_ll(o.stride(1)), c_ll(o.stride(0)),
                            c_float(scale), ptr(status_word(q.device)), stream_handle())
    check(rc, "solar_attn_fwd")
    count("attn_fwd")
    return o, lse


def attn_bwd(q, k, v, o, lse, do, scale: float):
    """dq, dk, dv.  Uses the native backward kernels when the library exports them; until then the
    gradient is obtained from the library SDPA (counted as ``library_sdpa_bwd``)."""
    lib = _lib.load()
    if hasattr(lib, "solar_attn_bwd"):
        from .attention_bwd_native import attn_bwd_native

        return attn_bwd_native(q, k, v, o, lse, do, scale)
    count("library_sdpa_bwd")
    with torch.enable_grad():
        qq, kk, vv = (t.detach().transpose(1, 2).requires_grad_(True) for t in (q, k, v))
        out = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, scale=scale)
        dq, dk, dv = torch.autograd.grad(out, (qq, kk, vv), do.transpose(1, 2))
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)
