"""Autograd-aware front ends of the native sm_100a kernels.

Every op takes 2-D ``[rows, features]`` bf16 activations.  On CUDA tensors the native kernel
is launched (and a launch counter is bumped); on CPU tensors the PyTorch statement from
``ops.reference`` runs, which is what the gloo/CPU tests exercise.  There is no silent
fallback on CUDA: if the native library cannot be loaded the call raises.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib, reference
from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle

NT, NN, TN = 0, 1, 2

_status: dict[int, torch.Tensor] = {}
_scratch: dict[int, torch.Tensor] = {}


def status_word(device) -> torch.Tensor:
    """Per-device int32 word that kernels with bounded waits set when a wait gave up."""
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def read_status(device="cuda", clear: bool = True) -> int:
    """Synchronising read of the bounded-wait status word: 0 = every wait completed, otherwise the code of the wait
    that gave up (5 = a peer's flag never arrived).  ``clear`` resets a non-zero word."""
    w = status_word(device)
    code = int(w.item())
    if code != 0 and clear:
        w.zero_()
    return code


def check_status(device="cuda") -> None:
    """``read_status`` that raises on a non-zero word."""
    code = read_status(device)
    if code != 0:
        raise _lib.NativeError(f"a device-side bounded wait gave up (code {code})")


def _scratch_f32(device, n=2048) -> torch.Tensor:
    dev = torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    if idx not in _scratch or _scratch[idx].numel() < n:
        _scratch[idx] = torch.empty(n, dtype=torch.float32, device=torch.device("cuda", idx))
    return _scratch[idx]


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    if t.dim() != 2:
        raise ValueError(f"expected a 2-D tensor, got {tuple(t.shape)}")
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
    return t


# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------
_GEMM_BACKEND = "native"


def set_gemm_backend(name: str) -> str:
    """``native``: this library's tcgen05 kernels (default).  ``library``: ``torch.matmul`` (cuBLAS) with the bias /
    activation / accumulate steps as separate torch ops -- only for A/B baselines (``bench.py --impl baseline``); the
    fused-exchange entry points always run the native kernels.  Returns the previous setting."""
    global _GEMM_BACKEND
    if name not in ("native", "library"):
        raise ValueError("gemm backend must be 'native' or 'library'")
    previous, _GEMM_BACKEND = _GEMM_BACKEND, name
    return previous


def gemm(a, b, layout=NT, *, bias=None, act=None, out=None, out_dtype=None, accumulate=False,
         max_ctas=0):
    """C = op(A) op(B) with bf16 operands and fp32 accumulation.

    layout NT: a [M,K], b [N,K];  NN: a [M,K], b [K,N];  TN: a [K,M], b [K,N].
    """
    if a.is_cuda and _GEMM_BACKEND == "library":
        c = a @ b.t() if layout == NT else (a @ b if layout == NN else a.t() @ b)
        count("library_gemm")
        if bias is not None:
            c = c + bias
        if act == "gelu":
            c = torch.nn.functional.gelu(c, approximate="tanh")
        elif act == "swiglu":
            g, u = c.view(c.shape[0], -1, 2, 64).unbind(2)
            c = (torch.nn.functional.silu(g.float()) * u.float()).reshape(c.shape[0], -1).to(c.dtype)
        if out is not None:
            if accumulate:
                out.add_(c.to(out.dtype))
            else:
                out.copy_(c)
            return out
        return c.to(out_dtype) if out_dtype is not None else c
    if not a.is_cuda:
        af, bf = a.float(), b.float()
        c = af @ bf.t() if layout == NT else (af @ bf if layout == NN else af.t() @ bf)
        if bias is not None:
            c = c + bias.float()
        if act == "gelu":
            c = torch.nn.functional.gelu(c, approximate="tanh")
        elif act == "swiglu":
            g, u = c.view(c.shape[0], -1, 2, 64).unbind(2)
            c = (torch.nn.functional.silu(g) * u).reshape(c.shape[0], -1)
        dt = out_dtype or (out.dtype if out is not None else a.dtype)
        if out is not None:
            if accumulate:
                out.add_(c.to(out.dtype))
            else:
                out.copy_(c.to(out.dtype))
            return out
        return c.to(dt)
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "gemm operands must be bf16"
    a = _rowmajor(a)
    b = _rowmajor(b)
    if layout == NT:
        M, K = a.shape
        N, K2 = b.shape
    elif layout == NN:
        M, K = a.shape
        K2, N = b.shape
    else:
        K, M = a.shape
        K2, N = b.shape
    if K != K2:
        raise ValueError(f"gemm inner dimensions differ: {K} vs {K2}")
    n_out = N // 2 if act == "swiglu" else N
    if out is None:
        out = torch.empty((M, n_out), dtype=out_dtype or torch.bfloat16, device=a.device)
        accumulate = False
    else:
        if out.shape != (M, n_out) or out.stride(1) != 1:
            raise ValueError("gemm: bad output tensor")
    if bias is not None:
        assert bias.dtype == torch.bfloat16 and bias.is_contiguous()
    lib = _lib.load()
    rc = lib.solar_gemm_bf16(
        ptr(a), ptr(b), ptr(out), ptr(bias), c_int(M), c_int(N), c_int(K),
        c_ll(a.stride(0)), c_ll(b.stride(0)), c_ll(out.stride(0)), c_int(layout),
        c_int({"gelu": 1, "swiglu": 2}.get(act, 0)), c_int(1 if out.dtype == torch.float32 else 0),
        c_int(1 if accumulate else 0), ptr(status_word(a.device)), c_int(max_ctas), stream_handle())
    check(rc, "solar_gemm_bf16")
    count("gemm")
    return out


def colsum(a, splits=None):
    """Column sums of a 2-D bf16 tensor -> fp32 [D] (deterministic two-stage reduction)."""
    if not a.is_cuda:
        return a.float().sum(0)
    a = _rowmajor(a)
    R, D = a.shape
    splits = splits or max(1, min(64, 600 // max(1, (D + 63) // 64)))
    part = torch.empty((splits, 1, D), dtype=torch.float32, device=a.device)
    lib = _lib.load()
    rc = lib.solar_colreduce(ptr(a), c_ll(a.stride(0)), ptr(None), c_ll(0), ptr(None), ptr(None), ptr(None),
                             ptr(None), c_ll(0), c_int(0), ptr(part), ptr(None), c_ll(R), c_int(R),
                             c_int(1), c_int(splits), c_int(D), c_int(3), c_int(0), c_int(1), stream_handle())
    check(rc, "solar_colreduce")
    count("colreduce")
    return part.sum(0).view(D)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        return gemm(x, w, NT, bias=b)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = _rowmajor(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, NN)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy, x, TN, out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = colsum(dy)
        return dx, dw, db


def linear(x, w, b=None, act=None):
    """y = x w^T (+ b) (-> GELU-tanh when act == 'gelu', inference only)."""
    if not x.is_cuda:
        return reference.linear(x, w, b, act)
    if act is not None:
        if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad):
            raise RuntimeError("fused activation epilogue is forward-only; use gelu() when training")
        return gemm(x, w, NT, bias=b, act=act)
    if hasattr(w, "main_grad"):
        return _LinearMainGradFn.apply(x, w, b)
    return _LinearFn.apply(x, w, b)


class _LoRALinearFn(torch.autograd.Function):
    """y = x W^T + b + s (x A^T) B^T with W and b frozen: the adapter product lands in the base GEMM's output through
    the reduce-add epilogue, and backward is four GEMMs (dt = s dy B; dx = dy W + dt A; dA = dt^T x; dB = s dy^T t)."""

    @staticmethod
    def forward(ctx, x, w, b, a, bb, scale):
        y = gemm(x, w, NT, bias=b)
        t = gemm(x, a, NT)
        bs = bb if scale == 1.0 else (bb * scale).to(bb.dtype)
        gemm(t, bs, NT, out=y, accumulate=True)
        ctx.save_for_backward(x, w, a, bs, t)
        ctx.scale = scale
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, a, bs, t = ctx.saved_tensors
        dy = _rowmajor(dy)
        dt = gemm(dy, bs, NN)                           # [M, r], the scale is folded into bs
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy, w, NN)
            gemm(dt, a, NN, out=dx, accumulate=True)
        da = gemm(dt, x, TN, out_dtype=a.dtype)
        db = gemm(dy, t, TN, out_dtype=bs.dtype)
        if ctx.scale != 1.0:
            db = (db * ctx.scale).to(db.dtype)
        return dx, None, None, da, db, None


def pad_adapter_rank(lora_a, lora_b):
    """The GEMM kernels take inner and outer extents in multiples of 8.  The released rank (384) is one; a rank that is not
    (small test models) is zero-padded for the call: zero rows of A times zero columns of B add nothing, the padding is a
    differentiable view-and-copy, and its gradient slices fall away."""
    r = lora_a.shape[0]
    if r % 8 == 0:
        return lora_a, lora_b
    extra = 8 - r % 8
    return torch.nn.functional.pad(lora_a, (0, 0, 0, extra)), torch.nn.functional.pad(lora_b, (0, extra))


def lora_linear(x, w, b, lora_a, lora_b, scale: float = 1.0):
    """A frozen linear with a trainable low-rank update: ``lora_a`` [r, in], ``lora_b`` [out, r]."""
    if not x.is_cuda:
        y = x.float() @ w.float().t() + scale * ((x.float() @ lora_a.float().t()) @ lora_b.float().t())
        if b is not None:
            y = y + b.float()
        return y.to(x.dtype)
    lora_a, lora_b = pad_adapter_rank(lora_a, lora_b)
    return _LoRALinearFn.apply(x, w, b, lora_a, lora_b, float(scale))


# Weights (by address) whose forward product is not needed right now: the last GEMM of a segment that is being
# re-run in backward only to rebuild what that GEMM's own backward keeps (its input), not its output.
_SKIP_FORWARD: set = set()


def _forward_needed(w) -> bool:
    return not _SKIP_FORWARD or w.data_ptr() not in _SKIP_FORWARD


class _SegmentFn(torch.autograd.Function):
    """``fn(*args)`` that keeps only ``args`` for backward.  Backward re-runs ``fn`` with gradients on -- with the
    forward product of the segment's LAST linear skipped (``tail_weight``), since nothing reads it -- and
    back-propagates through the rebuilt graph.  Parameters used inside ``fn`` receive their gradients there."""

    @staticmethod
    def forward(ctx, fn, tail_weight, *args):
        ctx.fn, ctx.tail = fn, tail_weight
        ctx.save_for_backward(*args)
        with torch.no_grad():
            return fn(*args)

    @staticmethod
    def backward(ctx, dy):
        args = [a.detach().requires_grad_(need) for a, need in zip(ctx.saved_tensors, ctx.needs_input_grad[2:])]
        key = None if ctx.tail is None else ctx.tail.data_ptr()
        with torch.enable_grad():
            if key is not None:
                _SKIP_FORWARD.add(key)
            try:
                out = ctx.fn(*args)
            finally:
                _SKIP_FORWARD.discard(key)
        torch.autograd.backward(out, dy)
        return (None, None) + tuple(a.grad for a in args)


def recompute_segment(fn, tail_weight, *args):
    """Run ``fn(*args)`` keeping only its inputs (see ``_SegmentFn``); plain call when gradients are off."""
    if not torch.is_grad_enabled():
        return fn(*args)
    return _SegmentFn.apply(fn, tail_weight, *args)


class _SplitColumnsFn(torch.autograd.Function):
    """Column views of a fused projection output (q | k | v).  Plain slicing would have autograd build a zero-filled
    full-width gradient per slice and add them up; here backward is one concatenation."""

    @staticmethod
    def forward(ctx, x, *sizes):
        outs, c0 = [], 0
        for n in sizes:
            outs.append(x[:, c0:c0 + n])
            c0 += n
        return tuple(outs)

    @staticmethod
    def backward(ctx, *grads):
        return (torch.cat(grads, dim=1),) + (None,) * len(grads)


def split_columns(x, sizes):
    """``x [rows, sum(sizes)]`` -> column views, with a single-pass backward."""
    if not (torch.is_grad_enabled() and x.requires_grad):
        outs, c0 = [], 0
        for n in sizes:
            outs.append(x[:, c0:c0 + n])
            c0 += n
        return tuple(outs)
    return _SplitColumnsFn.apply(x, *sizes)


class _LinearMainGradFn(torch.autograd.Function):
    """Linear whose parameter gradients are written straight into flat ``main_grad`` buffers."""

    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x)
        ctx.w, ctx.b = w, b
        if not _forward_needed(w):
            return x.new_empty((x.shape[0], w.shape[0]))
        return gemm(x, w, NT, bias=b)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        w, b = ctx.w, ctx.b
        dy = _rowmajor(dy)
        dgrad = (lambda: gemm(dy, w, NN)) if ctx.needs_input_grad[0] else (lambda: None)
        dx = wgrad_beside(dy, x, w, dgrad) if w.requires_grad else dgrad()
        if b is not None and b.requires_grad:
            accumulate_main_grad(b, colsum(dy))
        return dx, None, None


# The weight-gradient GEMM of a linear has no consumer until its block's gradients are reduced, and it is independent
# of the input-gradient GEMM.  Both are persistent kernels that fill the GPU, so run back to back each pays its own
# partial last wave -- at 8-way sequence parallelism a [3410 x 3072] product is 168 CTA-pair tiles over 74 pairs: 2.27
# waves that take 3.  Launched on two streams, the CTAs of the second kernel start on SMs as the first one's CTAs run
# out of tiles, so the pair pays one tail instead of two.  The main stream joins the side stream before anything else
# is enqueued, so every later kernel (and the allocator's reuse of ``dy``) is ordered after both.
_WGRAD_SIDE: dict = {}
_WGRAD_OVERLAP = os.environ.get("SOLAR_WGRAD_OVERLAP", "auto")      # "1" / "0" / "auto": on when more than one rank runs


def _wgrad_overlap_on() -> bool:
    if _WGRAD_OVERLAP in ("0", "1"):
        return _WGRAD_OVERLAP == "1"
    import torch.distributed as dist

    # with sequence parallelism the GEMMs shrink to a few waves and the partial last wave matters (measured at 8 ranks:
    # 323.7 -> 320.1 ms per step, gradients bit-identical); on one GPU the step does not change (1.877 vs 1.885 s)
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def wgrad_beside(dy, x, w, dgrad):
    """``w.main_grad (+)= dy^T x`` on a side stream while ``dgrad()`` (the input-gradient work) is enqueued on the
    current one; returns what ``dgrad`` returns."""
    def wgrad():
        gemm(dy, x, TN, out=w.main_grad, accumulate=_grad_is_live(w))
        _mark_grad_live(w)

    if not (dy.is_cuda and _wgrad_overlap_on()):
        wgrad()
        return dgrad()
    main = torch.cuda.current_stream()
    side = _WGRAD_SIDE.get(dy.device.index)
    if side is None:
        side = _WGRAD_SIDE[dy.device.index] = torch.cuda.Stream(device=dy.device)
    side.wait_stream(main)
    with torch.cuda.stream(side):
        wgrad()
    out = dgrad()
    main.wait_stream(side)
    return out


def _grad_is_live(p) -> bool:
    """Has ``main_grad`` of this parameter been written since the last ``zero_grads``?  A fused
    view over several parameters carries them in ``_anchors`` and shares their state."""
    anchors = getattr(p, "_anchors", None) or (p,)
    return bool(getattr(anchors[0], "grad_live", False))


def _mark_grad_live(p) -> None:
    for a in getattr(p, "_anchors", None) or (p,):
        a.grad_live = True


def accumulate_main_grad(p, g) -> None:
    """Add (or first-write) a gradient into a parameter's flat ``main_grad`` view."""
    if _grad_is_live(p):
        p.main_grad.add_(g.to(p.main_grad.dtype).view_as(p.main_grad))
    else:
        p.main_grad.copy_(g.view_as(p.main_grad))
    _mark_grad_live(p)


# --------------------------------------------------------------------------------------
# norm + adaLN modulation
# --------------------------------------------------------------------------------------
def _mod_args(shift, scale):
    if scale is None:
        return ptr(None), ptr(None), c_ll(0)
    assert shift.dtype == torch.float32 and scale.dtype == torch.float32
    assert shift.stride(-1) == 1 and scale.stride(-1) == 1 and shift.stride(0) == scale.stride(0)
    return ptr(shift), ptr(scale), c_ll(scale.stride(0))


def _splits_for(D, groups):
    blocks = ((D + 63) // 64) * max(groups, 1)
    return max(1, min(32, 600 // blocks))


class _NormModFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale, w, b, mode, eps, rpg, goff, table):
        x = _rowmajor(x)
        R, D = x.shape
        y = torch.empty((R, D), dtype=x.dtype, device=x.device)
        stats = torch.empty((R, 2), dtype=torch.float32, device=x.device)
        sh, sc, ms = _mod_args(shift, scale)
        lib = _lib.load()
        rc = lib.solar_norm_modulate_fwd(ptr(x), c_ll(x.stride(0)), ptr(y), c_ll(D), ptr(stats), ptr(w),
                                         ptr(b), sh, sc, ms, ptr(table), c_int(rpg), c_int(goff),
                                         c_ll(R), c_int(D), c_float(eps), c_int(mode), stream_handle())
        check(rc, "solar_norm_modulate_fwd")
        count("norm_modulate_fwd")
        ctx.save_for_backward(x, stats, scale, w, b, table)
        ctx.cfg = (mode, rpg, goff, None if scale is None else scale.shape[0])
        return y

    @staticmethod
    def backward(ctx, dy):
        x, stats, scale, w, b, table = ctx.saved_tensors
        mode, rpg, goff, G = ctx.cfg
        dy = _rowmajor(dy)
        R, D = x.shape
        lib = _lib.load()
        dx = dshift = dscale = dw = db = None
        _, sc, ms = _mod_args(scale, scale)
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x)
            rc = lib.solar_norm_modulate_bwd(ptr(dy), c_ll(dy.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(dx),
                                             c_ll(dx.stride(0)), ptr(stats), ptr(w), sc, ms, ptr(table),
                                             c_int(rpg), c_int(goff), c_ll(R), c_int(D), c_int(mode),
                                             c_int(0), stream_handle())
            check(rc, "solar_norm_modulate_bwd")
            count("norm_modulate_bwd")
        if scale is not None and (ctx.needs_input_grad[1] or ctx.needs_input_grad[2]):
            if table is not None:
                raise RuntimeError("modulation gradients with an explicit group table are not supported")
            gl = (R + rpg - 1) // rpg
            splits = _splits_for(D, gl)
            o0 = torch.empty((splits, gl, D), dtype=torch.float32, device=x.device)
            o1 = torch.empty_like(o0)
            rc = lib.solar_colreduce(ptr(dy), c_ll(dy.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(stats), ptr(w),
                                     ptr(b), ptr(None), c_ll(0), c_int(0), ptr(o0), ptr(o1), c_ll(R),
                                     c_int(rpg), c_int(gl), c_int(splits), c_int(D), c_int(0), c_int(mode),
                                     c_int(1), stream_handle())
            check(rc, "solar_colreduce")
            count("colreduce")
            dscale = torch.zeros((G, D), dtype=torch.float32, device=x.device)
            dshift = torch.zeros_like(dscale)
            dscale[goff:goff + gl] = o0.sum(0)
            dshift[goff:goff + gl] = o1.sum(0)
        if mode >= 1 and w is not None and ctx.needs_input_grad[3]:
            splits = _splits_for(D, 1)
            o0 = torch.empty((splits, 1, D), dtype=torch.float32, device=x.device)
            o1 = torch.empty_like(o0)
            rc = lib.solar_colreduce(ptr(dy), c_ll(dy.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(stats),
                                     ptr(None), ptr(None), sc, ms, c_int(goff), ptr(o0), ptr(o1), c_ll(R),
                                     c_int(R), c_int(1), c_int(splits), c_int(D),
                                     c_int(1), c_int(mode), c_int(rpg), stream_handle())
            check(rc, "solar_colreduce")
            count("colreduce")
            dw = o0.sum(0).view(D)
            if mode == 2:
                db = o1.sum(0).view(D)
        return dx, dshift, dscale, dw, db, None, None, None, None, None


def norm_modulate(x, shift=None, scale=None, *, mode=0, w=None, b=None, eps=1e-6, rows_per_group=1,
                  group_offset=0, table=None):
    """y = norm(x) [*w + b] * (1 + scale[g]) + shift[g];  shift/scale are fp32 ``[G, D]`` views."""
    if not x.is_cuda:
        return reference.norm_modulate(x, shift, scale, mode=mode, w=w, b=b, eps=eps,
                                       rows_per_group=rows_per_group, group_offset=group_offset, table=table)
    if mode >= 1 and scale is not None and w is not None and w.requires_grad and torch.is_grad_enabled():
        # dw with modulation needs the per-row scale; colreduce kind 1 handles contiguous groups only.
        if table is not None:
            raise RuntimeError("trainable norm weight with a group table is not supported")
    return _NormModFn.apply(x, shift, scale, w, b, int(mode), float(eps), int(rows_per_group),
                            int(group_offset), table)


class _GatedResidualFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, res, y, gate, rpg, goff, table):
        res = _rowmajor(res)
        y = _rowmajor(y)
        R, D = res.shape
        out = torch.empty((R, D), dtype=res.dtype, device=res.device)
        lib = _lib.load()
        gs = c_ll(0 if gate is None else gate.stride(0))
        rc = lib.solar_gated_residual(ptr(res), c_ll(res.stride(0)), ptr(y), c_ll(y.stride(0)), ptr(out),
                                      c_ll(D), ptr(gate), gs, ptr(table), c_int(rpg), c_int(goff), c_ll(R),
                                      c_int(D), c_int(0), stream_handle())
        check(rc, "solar_gated_residual")
        count("gated_residual")
        need_y = gate is not None and gate.requires_grad
        ctx.save_for_backward(y if need_y else None, gate, table)
        ctx.cfg = (rpg, goff)
        return out

    @staticmethod
    def backward(ctx, dout):
        y, gate, table = ctx.saved_tensors
        rpg, goff = ctx.cfg
        dout = _rowmajor(dout)
        R, D = dout.shape
        lib = _lib.load()
        dy = dgate = None
        if ctx.needs_input_grad[1]:
            if gate is None:
                dy = dout
            else:
                dy = torch.empty_like(dout)
                rc = lib.solar_gated_residual(ptr(None), c_ll(0), ptr(dout), c_ll(dout.stride(0)), ptr(dy),
                                              c_ll(D), ptr(gate), c_ll(gate.stride(0)), ptr(table), c_int(rpg),
                                              c_int(goff), c_ll(R), c_int(D), c_int(1), stream_handle())
                check(rc, "solar_gated_residual")
                count("gated_residual_bwd")
        if gate is not None and ctx.needs_input_grad[2]:
            if table is not None:
                raise RuntimeError("gate gradients with an explicit group table are not supported")
            gl = (R + rpg - 1) // rpg
            splits = _splits_for(D, gl)
            o0 = torch.empty((splits, gl, D), dtype=torch.float32, device=dout.device)
            rc = lib.solar_colreduce(ptr(dout), c_ll(dout.stride(0)), ptr(y), c_ll(y.stride(0)), ptr(None),
                                     ptr(None), ptr(None), ptr(None), c_ll(0), c_int(0), ptr(o0), ptr(None),
                                     c_ll(R), c_int(rpg), c_int(gl), c_int(splits), c_int(D), c_int(2),
                                     c_int(0), c_int(1), stream_handle())
            check(rc, "solar_colreduce")
            count("colreduce")
            dgate = torch.zeros((gate.shape[0], D), dtype=torch.float32, device=dout.device)
            dgate[goff:goff + gl] = o0.sum(0)
        return dout if ctx.needs_input_grad[0] else None, dy, dgate, None, None, None


def gated_residual(res, y, gate=None, *, rows_per_group=1, group_offset=0, table=None):
    """out = res + gate[g] * y  (gate fp32 ``[G, D]`` view, or None for a plain residual add)."""
    if not res.is_cuda:
        return reference.gated_residual(res, y, gate, rows_per_group=rows_per_group,
                                        group_offset=group_offset, table=table)
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.stride(-1) == 1
    return _GatedResidualFn.apply(res, y, gate, int(rows_per_group), int(group_offset), table)


# --------------------------------------------------------------------------------------
# full-width RMSNorm + RoPE
# --------------------------------------------------------------------------------------
class _RmsRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, rope, eps, no_norm):
        x = _rowmajor(x)
        R, D = x.shape
        y = torch.empty((R, D), dtype=x.dtype, device=x.device)
        rstd = torch.empty((R,), dtype=torch.float32, device=x.device)
        half = 0 if rope is None else rope.shape[1]
        lib = _lib.load()
        rc = lib.solar_rmsnorm_rope_fwd(ptr(x), c_ll(x.stride(0)), ptr(y), c_ll(D), ptr(w), ptr(rope),
                                        c_int(half), ptr(rstd), c_ll(R), c_int(D), c_float(eps),
                                        c_int(1 if no_norm else 0), stream_handle())
        check(rc, "solar_rmsnorm_rope_fwd")
        count("rmsnorm_rope_fwd")
        ctx.save_for_backward(x, w, rope, rstd)
        ctx.no_norm = no_norm
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rope, rstd = ctx.saved_tensors
        dy = _rowmajor(dy)
        R, D = x.shape
        half = 0 if rope is None else rope.shape[1]
        need_dw = (not ctx.no_norm) and w is not None and ctx.needs_input_grad[1]
        splits = _splits_for(D, 1)
        part = torch.empty((splits, D), dtype=torch.float32, device=x.device) if need_dw else None
        dx = torch.empty_like(x)
        lib = _lib.load()
        rc = lib.solar_rmsnorm_rope_bwd(ptr(dy), c_ll(dy.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(dx),
                                        c_ll(dx.stride(0)), ptr(w), ptr(rope), c_int(half), ptr(rstd),
                                        ptr(part), c_int(splits), c_ll(R), c_int(D),
                                        c_int(1 if ctx.no_norm else 0), stream_handle())
        check(rc, "solar_rmsnorm_rope_bwd")
        count("rmsnorm_rope_bwd")
        dw = part.sum(0) if need_dw else None
        return dx, dw, None, None, None


def rmsnorm_rope(x, w, rope, *, eps=1e-6, no_norm=False):
    """Full-width RMSNorm * w then per-head interleaved RoPE; rope fp32 ``[R, hd/2, 2]`` or None."""
    if not x.is_cuda:
        return reference.rmsnorm_rope(x, w, rope, eps=eps, no_norm=no_norm)
    if rope is not None:
        assert rope.dtype == torch.float32 and rope.is_contiguous() and rope.shape[0] == x.shape[0]
    if w is not None:
        assert w.dtype == torch.float32
    return _RmsRopeFn.apply(x, w, rope, float(eps), bool(no_norm))


# --------------------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------------------
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        x = x.contiguous()
        y = torch.empty_like(x)
        lib = _lib.load()
        check(lib.solar_gelu(ptr(x), ptr(None), ptr(y), ptr(None), c_ll(x.numel()), c_int(0), stream_handle()),
              "solar_gelu")
        count("gelu_fwd")
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        lib = _lib.load()
        check(lib.solar_gelu(ptr(x), ptr(dy), ptr(dx), ptr(None), c_ll(x.numel()), c_int(1), stream_handle()),
              "solar_gelu")
        count("gelu_bwd")
        return dx


def gelu(x):
    if not x.is_cuda:
        return reference.gelu_tanh(x)
    return _GeluFn.apply(x)


def _gelu_launch(x, dy, out, backward: int):
    lib = _lib.load()
    check(lib.solar_gelu(ptr(x), ptr(dy), ptr(out), ptr(None), c_ll(x.numel()), c_int(backward), stream_handle()), "solar_gelu")
    count("gelu_bwd" if backward else "gelu_fwd")


class _GeluLinearMainGradFn(torch.autograd.Function):
    """``linear(gelu(h), w, b)`` that keeps only ``h`` for backward: the activation ``gelu(h)`` (the widest
    tensor of a transformer block) is rebuilt by one elementwise pass when the weight gradient needs it,
    instead of living in memory from forward to backward."""

    @staticmethod
    def forward(ctx, h, w, b):
        h = h.contiguous()
        ctx.save_for_backward(h)
        ctx.w, ctx.b = w, b
        if not _forward_needed(w):
            return h.new_empty((h.shape[0], w.shape[0]))
        a = torch.empty_like(h)
        _gelu_launch(h, None, a, 0)
        return gemm(a, w, NT, bias=b)

    @staticmethod
    def backward(ctx, dy):
        (h,) = ctx.saved_tensors
        w, b = ctx.w, ctx.b
        dy = _rowmajor(dy)
        def dgrad():
            if not ctx.needs_input_grad[0]:
                return None
            da = gemm(dy, w, NN)
            dh = torch.empty_like(h)
            _gelu_launch(h, da, dh, 1)
            return dh

        if w.requires_grad:
            a = torch.empty_like(h)
            _gelu_launch(h, None, a, 0)
            dh = wgrad_beside(dy, a, w, dgrad)
            del a
        else:
            dh = dgrad()
        if b is not None and b.requires_grad:
            accumulate_main_grad(b, colsum(dy))
        return dh, None, None


def gelu_linear(h, w, b=None):
    """``linear(gelu_tanh(h), w, b)``; on the device with flat-gradient parameters the activation is not kept."""
    if h.is_cuda and hasattr(w, "main_grad") and torch.is_grad_enabled():
        return _GeluLinearMainGradFn.apply(h, w, b)
    return linear(gelu(h), w, b)


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        gu = gu.contiguous()
        M, N2 = gu.shape
        y = torch.empty((M, N2 // 2), dtype=gu.dtype, device=gu.device)
        lib = _lib.load()
        check(lib.solar_swiglu(ptr(gu), ptr(None), ptr(y), c_ll(M), c_int(N2 // 2), c_int(0), stream_handle()),
              "solar_swiglu")
        count("swiglu_fwd")
        ctx.save_for_backward(gu)
        return y

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        dy = dy.contiguous()
        M, N2 = gu.shape
        dgu = torch.empty_like(gu)
        lib = _lib.load()
        check(lib.solar_swiglu(ptr(gu), ptr(dy), ptr(dgu), c_ll(M), c_int(N2 // 2), c_int(1), stream_handle()),
              "solar_swiglu")
        count("swiglu_bwd")
        return dgu


def swiglu(gu):
    """[M, 2N] (gate | up) -> up * silu(gate)."""
    if not gu.is_cuda:
        return reference.swiglu(gu)
    return _SwigluFn.apply(gu)


# --------------------------------------------------------------------------------------
# optimizer / reductions / scheduler math / loss
# --------------------------------------------------------------------------------------
def adamw_(master, m, v, grad, *, live=None, ema=None, lr, beta1, beta2, eps, wd, step,
           grad_scale: Optional[torch.Tensor] = None, skip: Optional[torch.Tensor] = None,
           ema_decay: float = 0.0):
    """In-place fused AdamW over flat fp32 shards; refreshes the bf16 live copy and EMA shadow."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    if not master.is_cuda:
        gs = 1.0 if grad_scale is None else float(grad_scale)
        if skip is not None and int(skip) != 0:
            return
        reference.adamw_step(master, m, v, grad, lr=lr, beta1=beta1, beta2=beta2, eps=eps, wd=wd,
                             step=step, grad_scale=gs)
        if live is not None:
            live.copy_(master.to(live.dtype))
        if ema is not None:
            ema.mul_(ema_decay).add_(master, alpha=1.0 - ema_decay)
        return
    n = master.numel()
    assert n % 4 == 0 and grad.numel() == n
    lib = _lib.load()
    rc = lib.solar_adamw(ptr(master), ptr(m), ptr(v), ptr(live), ptr(ema), ptr(grad),
                         c_int(1 if grad.dtype == torch.float32 else 0), ptr(grad_scale), ptr(skip), c_ll(n),
                         c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(wd),
                         c_float(bc1), c_float(bc2), c_float(ema_decay), stream_handle())
    check(rc, "solar_adamw")
    count("adamw")


def sumsq(x, out=None, accumulate=False):
    """Sum of squares of a flat bf16/fp32 tensor into a 1-element fp32 tensor."""
    if not x.is_cuda:
        s = x.float().pow(2).sum().view(1)
        if out is None:
            return s
        out.copy_(out + s if accumulate else s)
        return out
    x = x.contiguous().view(-1)
    assert x.numel() % 8 == 0
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    lib = _lib.load()
    rc = lib.solar_sumsq(ptr(x), c_int(1 if x.dtype == torch.float32 else 0), c_ll(x.numel()),
                         ptr(_scratch_f32(x.device)), ptr(out), c_int(1 if accumulate else 0), stream_handle())
    check(rc, "solar_sumsq")
    count("sumsq", 2)
    return out


def flow_op(a, b, sigma, sigma2, op, group_size, want_second=False):
    out0 = torch.empty_like(a)
    out1 = torch.empty_like(a) if want_second else None
    lib = _lib.load()
    rc = lib.solar_flow(ptr(a), ptr(b), ptr(sigma), ptr(sigma2), ptr(out0), ptr(out1), c_ll(a.numel()),
                        c_ll(group_size), c_int(op), stream_handle())
    check(rc, "solar_flow")
    count("flow")
    return out0, out1


def add_noise(x0, noise, sigma):
    """x_t = (1-s) x0 + s n and velocity target n - x0; sigma fp32 [G], x0 [G, ...]."""
    G = sigma.numel()
    if not x0.is_cuda:
        shape = (G,) + (1,) * (x0.dim() - 1)
        s = sigma.float().view(shape)
        return ((1 - s) * x0.float() + s * noise.float()).to(x0.dtype), (noise.float() - x0.float()).to(x0.dtype)
    x0 = x0.contiguous()
    noise = noise.contiguous()
    return flow_op(x0, noise, sigma.contiguous(), None, 0, x0.numel() // G, want_second=True)


def flow_to_x0(x_t, v, sigma):
    G = sigma.numel()
    if not x_t.is_cuda:
        s = sigma.float().view((G,) + (1,) * (x_t.dim() - 1))
        return (x_t.float() - s * v.float()).to(x_t.dtype)
    return flow_op(x_t.contiguous(), v.contiguous(), sigma.contiguous(), None, 1, x_t.numel() // G)[0]


def euler_step(x_t, v, sigma, sigma_next):
    G = sigma.numel()
    if not x_t.is_cuda:
        d = (sigma_next.float() - sigma.float()).view((G,) + (1,) * (x_t.dim() - 1))
        return (x_t.float() + d * v.float()).to(x_t.dtype)
    return flow_op(x_t.contiguous(), v.contiguous(), sigma.contiguous(), sigma_next.contiguous(), 2,
                   x_t.numel() // G)[0]


class _MseFn(torch.autograd.Function):
    """The kernel sums ``w m^2 (pred - target)^2`` with a unit denominator; the division by ``denom`` (a host number or
    a one-element device tensor) happens on the device afterwards, so a mask-dependent denominator costs no host read."""

    @staticmethod
    def forward(ctx, pred, target, weight, mask, denom):
        pred = pred.contiguous()
        target = target.contiguous()
        G = pred.shape[0]
        loss = torch.empty(1, dtype=torch.float32, device=pred.device)
        inv = (1.0 / denom) if torch.is_tensor(denom) else torch.full((1,), 1.0 / float(denom), dtype=torch.float32,
                                                                      device=pred.device)
        lib = _lib.load()
        rc = lib.solar_mse(ptr(pred), ptr(target), ptr(weight), ptr(mask), c_ll(pred.numel()),
                           c_ll(pred.numel() // G), c_float(1.0), ptr(_scratch_f32(pred.device)),
                           ptr(loss), ptr(None), ptr(None), stream_handle())
        check(rc, "solar_mse")
        count("mse_fwd", 2)
        ctx.save_for_backward(pred, target, weight, mask, inv)
        return (loss * inv).view(())

    @staticmethod
    def backward(ctx, gloss):
        pred, target, weight, mask, inv = ctx.saved_tensors
        G = pred.shape[0]
        dpred = torch.empty_like(pred)
        gl = (gloss.reshape(1).float() * inv).contiguous()
        lib = _lib.load()
        rc = lib.solar_mse(ptr(pred), ptr(target), ptr(weight), ptr(mask), c_ll(pred.numel()),
                           c_ll(pred.numel() // G), c_float(1.0), ptr(_scratch_f32(pred.device)),
                           ptr(None), ptr(dpred), ptr(gl), stream_handle())
        check(rc, "solar_mse")
        count("mse_bwd")
        return dpred, None, None, None, None


def weighted_masked_mse(pred, target, weight=None, mask=None, denom=None):
    """sum_g w[g] m[g] |pred_g - target_g|^2 / denom with pred/target ``[G, ...]`` bf16.
    ``denom`` defaults to (number of unmasked groups) x (elements per group), computed on the device."""
    if not pred.is_cuda:
        return reference.weighted_masked_mse(pred, target, weight, mask)
    G = pred.shape[0]
    weight = None if weight is None else weight.float().contiguous()
    mask = None if mask is None else mask.float().contiguous()
    if denom is None:
        per_group = pred.numel() // G
        denom = float(G * per_group) if mask is None else (mask.sum().clamp_min(1.0) * per_group).view(1)
    return _MseFn.apply(pred, target, weight, mask, denom)


def rgb8(frame_chw, mean=(0.485, 0.456, 0.406), std=(0.229, 0.224, 0.225)):
    """bf16 ``[3, H, W]`` -> uint8 ``[H, W, 3]`` on the tensor's device; raises on a NaN pixel."""
    import ctypes

    assert frame_chw.dtype == torch.bfloat16 and frame_chw.dim() == 3 and frame_chw.shape[0] == 3
    H, W = frame_chw.shape[1:]
    m3 = (ctypes.c_float * 3)(*mean)
    s3 = (ctypes.c_float * 3)(*std)
    lib = _lib.load()
    if frame_chw.is_cuda:
        out = torch.empty((H, W, 3), dtype=torch.uint8, device=frame_chw.device)
        flag = torch.zeros(1, dtype=torch.int32, device=frame_chw.device)
        rc = lib.solar_rgb8(ptr(frame_chw), ptr(out), c_int(H), c_int(W), c_ll(frame_chw.stride(0)),
                            c_ll(frame_chw.stride(1)), c_ll(frame_chw.stride(2)), m3, s3, ptr(flag),
                            stream_handle())
        check(rc, "solar_rgb8")
        count("rgb8")
        return out, flag
    out = torch.empty((H, W, 3), dtype=torch.uint8)
    lib.solar_host_rgb8_bf16.restype = ctypes.c_int
    ok = lib.solar_host_rgb8_bf16(ptr(frame_chw), ctypes.c_size_t(H), ctypes.c_size_t(W),
                                  ctypes.c_size_t(frame_chw.stride(0)), ctypes.c_size_t(frame_chw.stride(1)),
                                  ctypes.c_size_t(frame_chw.stride(2)), m3, s3, ptr(out))
    if not ok:
        raise FloatingPointError("nonfinite RGB pixel")
    return out, None


def interleave_gate_up(w: torch.Tensor) -> torch.Tensor:
    """``[gate (F rows) | up (F rows)]`` -> rows in blocks of 64: 64 gate rows, their 64 up rows, ...  (F a multiple of
    64), the layout the GEMM's SwiGLU epilogue reads; works for a bias vector too."""
    f2 = w.shape[0]
    if f2 % 128:
        raise ValueError("the fused gate|up width must be a multiple of 128")
    half = f2 // 2
    g, u = w[:half], w[half:]
    rest = w.shape[1:]
    return torch.stack([g.reshape(half // 64, 64, *rest), u.reshape(half // 64, 64, *rest)], 1).reshape(f2, *rest).contiguous()


def linear_swiglu(x, w_interleaved, b_interleaved=None):
    """``silu(x Wg^T + bg) * (x Wu^T + bu)`` with the activation in the GEMM epilogue: the ``[rows, 2F]`` product is never
    written.  Weights / bias in the ``interleave_gate_up`` layout.  Inference only (no autograd)."""
    return gemm(x, w_interleaved, NT, bias=b_interleaved, act="swiglu")


# --------------------------------------------------------------------------------------
# streaming ViT decoder step: q/k head RMSNorm + rotary + k/v cache write; tile blend + compensation
# --------------------------------------------------------------------------------------
def vit_qkv_to_cache(qkv, q_w, k_w, cos, sin, k_cache, v_cache, lo: int, *, heads: int, eps: float = 1e-6):
    """qkv bf16 ``[B, N, 3*heads*dh]`` -> q ``[B, N, heads*dh]``; k and v are written into rows
    ``[lo, lo + N)`` of ``k_cache`` / ``v_cache`` ``[B, rows, heads*dh]`` (no autograd; inference only).

    Same arithmetic as per-head RMSNorm (rounded to bf16) followed by rotate-half rotary with per-row
    ``cos`` / ``sin`` ``[N, dh]`` (``None`` = no rotation)."""
    B, N, three_a = qkv.shape
    a = three_a // 3
    dh = a // heads
    if not qkv.is_cuda:
        def norm(x, w):
            v = x.reshape(B, N, heads, dh).float()
            return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(qkv.dtype)

        def rot(x):
            if cos is None:
                return x
            v = x.float()
            r = torch.cat([-v[..., dh // 2:], v[..., :dh // 2]], dim=-1)
            return (v * cos.view(1, N, 1, dh) + r * sin.view(1, N, 1, dh)).to(qkv.dtype)

        q = rot(norm(qkv[..., :a], q_w)).reshape(B, N, a)
        k_cache[:, lo:lo + N] = rot(norm(qkv[..., a:2 * a], k_w)).reshape(B, N, a)
        v_cache[:, lo:lo + N] = qkv[..., 2 * a:]
        return q
    assert qkv.dtype == torch.bfloat16 and qkv.stride(2) == 1 and qkv.stride(0) == N * qkv.stride(1)
    assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.shape[2] == a
    assert q_w.dtype == torch.float32 and k_w.dtype == torch.float32
    if cos is not None:
        assert cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous() and cos.shape == (N, dh)
    q = torch.empty((B, N, a), dtype=qkv.dtype, device=qkv.device)
    rc = _lib.load().solar_vit_qkv(ptr(qkv), c_ll(qkv.stride(1)), ptr(q_w), ptr(k_w), ptr(cos), ptr(sin), ptr(q),
                                   ptr(k_cache), ptr(v_cache), c_ll(k_cache.stride(0)), c_ll(lo), c_ll(B), c_ll(N),
                                   c_int(heads), c_int(dh), c_float(eps), stream_handle())
    check(rc, "solar_vit_qkv")
    count("vit_qkv")
    return q


def tile_blend(tiles, offsets, H: int, W: int, overlap_px: int, coef=None):
    """tiles bf16 ``[T, 3, F, tH, tW]`` on CUDA (inner two dims contiguous), ``offsets`` the pixel ``(y, x)`` of
    each tile -> fp32 ``[3, F, H, W]``: ramp-weighted mean over the tiles that cover a pixel, then
    ``x - (a + b x + c x^2)`` with ``coef`` a host fp32 tensor ``[3 (a, b, c), 3, F]`` (``None`` = identity)."""
    import ctypes

    T, C, F_n, tH, tW = tiles.shape
    assert tiles.is_cuda and tiles.dtype == torch.bfloat16 and C == 3
    assert tiles.stride(4) == 1 and tiles.stride(3) == tW and len(offsets) == T
    out = torch.empty((3, F_n, H, W), dtype=torch.float32, device=tiles.device)
    py = (ctypes.c_int * T)(*[int(o[0]) for o in offsets])
    px = (ctypes.c_int * T)(*[int(o[1]) for o in offsets])
    cf = None
    if coef is not None:
        flat = coef.detach().to("cpu", torch.float32).contiguous().view(-1).tolist()
        assert len(flat) == 9 * F_n
        cf = (ctypes.c_float * len(flat))(*flat)
    rc = _lib.load().solar_tile_blend(ptr(tiles), c_ll(tiles.stride(0)), c_ll(tiles.stride(1)), c_ll(tiles.stride(2)),
                                      ptr(out), c_int(T), c_int(F_n), c_int(tH), c_int(tW), c_int(H), c_int(W),
                                      c_int(overlap_px), py, px, cf, stream_handle())
    check(rc, "solar_tile_blend")
    count("tile_blend")
    return out


# --------------------------------------------------------------------------------------
# implicit-GEMM convolution on channels-last activations (VAE)
# --------------------------------------------------------------------------------------
def pack_conv_weight(weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """``[Cout, Cin, kt, kh, kw]`` -> bf16 ``[Cout8, taps * ceil(Cin/64) * 64]`` (tap-major, each tap's input
    channels zero-padded to a multiple of 64; Cout rounded up to a multiple of 8) and the matching bf16 bias."""
    cout, cin, kt, kh, kw = weight.shape
    kpt = (cin + 63) // 64
    c8 = (cout + 7) // 8 * 8
    packed = torch.zeros(c8, kt * kh * kw, kpt * 64, dtype=torch.bfloat16, device=weight.device)
    packed[:cout, :, :cin] = weight.detach().permute(0, 2, 3, 4, 1).reshape(cout, kt * kh * kw, cin).to(torch.bfloat16)
    b = torch.zeros(c8, dtype=torch.bfloat16, device=weight.device)
    if bias is not None:
        b[:cout] = bias.detach().to(torch.bfloat16)
    return packed.view(c8, -1), b


def conv3d_channels_last(x, packed_w, packed_b, kernel, *, history=None, out_channels: Optional[int] = None):
    """Stride-1 convolution of bf16 ``x [T, H, W, Cin]`` ("same" padding in H / W, causal in T) with weights from
    ``pack_conv_weight``.  ``history`` ``[kt-1, H, W, Cin]`` supplies the frames before ``x`` (zeros if None).
    Returns ``[T, H, W, Cout8]`` (slice with ``out_channels`` to drop the channel padding).  CUDA only."""
    kt, kh, kw = kernel
    T, H, W, cin = x.shape
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and cin % 8 == 0
    if history is not None and kt > 1:
        xin = torch.cat([history, x], 0)
        shift = 0
    else:
        xin, shift = x, -(kt - 1)
    c8 = packed_w.shape[0]
    assert packed_w.shape[1] == kt * kh * kw * ((cin + 63) // 64) * 64
    y = torch.empty((T, H, W, c8), dtype=torch.bfloat16, device=x.device)
    rc = _lib.load().solar_conv3d_bf16(ptr(xin), ptr(packed_w), ptr(y), ptr(packed_b), c_int(xin.shape[0]), c_int(H),
                                       c_int(W), c_int(cin), c_int(T), c_int(c8), c_int(kt), c_int(kh), c_int(kw),
                                       c_int(shift), ptr(status_word(x.device)), c_int(0), stream_handle())
    check(rc, "solar_conv3d_bf16")
    count("conv3d")
    return y if out_channels is None or out_channels == c8 else y[..., :out_channels]


def rms_silu_channels_last(x, gamma, silu: bool = True):
    """bf16 ``x [..., C]`` (contiguous, channels last) -> ``x / max(||x||, 1e-12) * sqrt(C) * gamma`` (then SiLU), one pass."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
    C = x.shape[-1]
    g = gamma.detach().float().contiguous()
    y = torch.empty_like(x)
    rc = _lib.load().solar_rms_silu_cl(ptr(x), ptr(y), ptr(g), c_ll(x.numel() // C), c_int(C), c_int(1 if silu else 0),
                                       stream_handle())
    check(rc, "solar_rms_silu_cl")
    count("rms_silu_cl")
    return y


# --------------------------------------------------------------------------------------
# per-head RMSNorm + MM-RoPE + PRoPE (H3 attention path)
# --------------------------------------------------------------------------------------
class _HeadOpFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cos, sin, mats, heads, rot_dims, sections, eps):
        x = _rowmajor(x)
        S = x.shape[0]
        y = torch.empty((S, x.shape[1]), dtype=x.dtype, device=x.device)
        rstd = torch.empty((S, heads), dtype=torch.float32, device=x.device) if w is not None else None
        lib = _lib.load()
        rc = lib.solar_headop(ptr(x), c_ll(x.stride(0)), ptr(y), c_ll(y.stride(0)), ptr(w), ptr(cos), ptr(sin), ptr(mats),
                              ptr(rstd), c_ll(S), c_int(heads), c_int(128), c_int(rot_dims), c_int(sections), c_float(eps),
                              c_int(0), stream_handle())
        check(rc, "solar_headop")
        count("headop_fwd")
        ctx.save_for_backward(x, w, cos, sin, mats, rstd)
        ctx.cfg = (heads, rot_dims, sections, eps)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, cos, sin, mats, rstd = ctx.saved_tensors
        heads, rot_dims, sections, eps = ctx.cfg
        dy = _rowmajor(dy)
        S = x.shape[0]
        g = torch.empty_like(x)
        lib = _lib.load()
        rc = lib.solar_headop(ptr(dy), c_ll(dy.stride(0)), ptr(g), c_ll(g.stride(0)), ptr(None), ptr(cos), ptr(sin), ptr(mats),
                              ptr(None), c_ll(S), c_int(heads), c_int(128), c_int(rot_dims), c_int(sections), c_float(eps),
                              c_int(1), stream_handle())
        check(rc, "solar_headop")
        count("headop_bwd")
        if w is not None:
            dx = torch.empty_like(x)
            rc = lib.solar_headnorm_bwd(ptr(g), c_ll(g.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(dx), c_ll(dx.stride(0)),
                                        ptr(w), ptr(rstd), c_ll(S), c_int(heads), stream_handle())
            check(rc, "solar_headnorm_bwd")
            count("headnorm_bwd")
            g = dx
        return g, None, None, None, None, None, None, None, None


def head_norm_rope_prope(x, w=None, cos=None, sin=None, mats=None, *, heads, rot_dims=96, sections=2, eps=1e-6):
    """y = PRoPE(MM-RoPE(RMSNorm_head(x) * w)) for head_dim 128 (weights are frozen: only dx is produced)."""
    if not x.is_cuda:
        return reference.head_norm_rope_prope(x, w, cos, sin, mats, heads=heads, rot_dims=rot_dims, sections=sections, eps=eps)
    for t in (w, cos, sin, mats):
        assert t is None or (t.dtype == torch.float32 and t.is_contiguous())
    return _HeadOpFn.apply(x, w, cos, sin, mats, int(heads), int(rot_dims), int(sections), float(eps))
