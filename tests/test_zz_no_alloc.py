"""The allocation-free attention-backward entry point, called through its exported C symbol.

Some embedders may not allocate device memory when they call into the library (fixed memory
arenas, plug-ins inside another allocator, hosts that forbid cudaMalloc after start-up).  For them
``solar_attn_bwd_noalloc`` keeps its work vectors in a device array inside the library.  The test
checks, on two calls in a row (the array keeps the first call's contents), that it returns what the
regular entry point returns, and that an oversized problem is refused with a readable message.
This file sorts last on purpose: a run that stops at the first failure has already run the rest.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, q, k, v, o, lse, do, scale):
    from solarwm_b200.ops._lib import c_float, c_int, c_ll, ptr, stream_handle
    from solarwm_b200.ops.functional import status_word

    B, Sq, H, D = q.shape
    Sk = k.shape[1]
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    fn = lib.solar_attn_bwd_noalloc
    fn.restype = ctypes.c_int
    rc = fn(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(dq), ptr(dk), ptr(dv), c_int(B), c_int(Sq),
            c_int(Sk), c_int(H), c_int(D), c_ll(q.stride(1)), c_ll(q.stride(0)), c_ll(k.stride(1)), c_ll(k.stride(0)),
            c_ll(v.stride(1)), c_ll(v.stride(0)), c_ll(o.stride(1)), c_ll(o.stride(0)), c_ll(do.stride(1)),
            c_ll(do.stride(0)), c_float(scale), ptr(status_word(q.device)), stream_handle())
    return rc, dq, dk, dv


def _problem(B, Sq, Sk, H, D, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    mk = lambda n: torch.randn(B, n, H, D, generator=g, device="cuda").to(torch.bfloat16)
    return mk(Sq), mk(Sk), mk(Sk), mk(Sq)


def test_noalloc_entry_matches_regular_entry_twice_and_rejects_oversize():
    from solarwm_b200 import ops
    from solarwm_b200.ops import _lib
    from solarwm_b200.ops.attention_bwd_native import attn_bwd_native
    from solarwm_b200.ops.attention_native import attn_fwd

    lib = _lib.load()
    assert hasattr(lib, "solar_attn_bwd_noalloc")
    # two different shapes back to back: the second call sees the first call's leftovers
    for B, Sq, Sk, H, D, seed in ((1, 700, 520, 2, 128, 1), (2, 300, 384, 3, 64, 2)):
        q, k, v, do = _problem(B, Sq, Sk, H, D, seed)
        scale = 1.0 / math.sqrt(D)
        o, lse = attn_fwd(q, k, v, scale)
        want = attn_bwd_native(q, k, v, o, lse, do, scale)
        rc, dq, dk, dv = _call_noalloc(lib, q, k, v, o, lse, do, scale)
        assert rc == 0, lib.solar_last_error()
        torch.cuda.synchronize()
        ops.check_status()
        for name, got, ref in (("dq", dq, want[0]), ("dk", dk, want[1]), ("dv", dv, want[2])):
            rel = ((got.float() - ref.float()).norm() / ref.float().norm()).item()
            assert rel < 2e-2, (name, rel)
            assert torch.equal(got, ref), f"{name}: the two entry points run the same kernels on the same inputs"
    # 2 * B * H * round_up(Sq, 128) floats must fit the built-in array (1 Mi floats)
    q, k, v, do = _problem(1, 128, 128, 1, 128, 3)
    o, lse = attn_fwd(q, k, v, 0.1)
    # (no pointer is dereferenced here: the size check comes before any launch)
    from solarwm_b200.ops._lib import c_float, c_int, c_ll, ptr, stream_handle

    rc = lib.solar_attn_bwd_noalloc(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(q), ptr(k), ptr(v),
                                    c_int(1), c_int(600_000), c_int(128), c_int(1), c_int(128), c_ll(128), c_ll(128),
                                    c_ll(128), c_ll(128), c_ll(128), c_ll(128), c_ll(128), c_ll(128), c_ll(128),
                                    c_ll(128), c_float(0.1), ptr(None), stream_handle())
    assert rc != 0
    msg = lib.solar_last_error().decode()
    assert "scratch floats" in msg and "1048576" in msg
