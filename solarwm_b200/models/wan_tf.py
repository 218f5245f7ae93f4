"""Teacher-forcing and cache-free sliding-window forwards of the causal Wan DiT.

``forward_teacher_forcing``: one pass over the concatenated ``[clean | noisy]`` token sequence;
clean frames carry timestep 0, noisy frames their sampled timestep (and AnyFlow target time
``r``), both halves share RoPE positions, and self-attention follows the block-causal window
rule of ``teacher_forcing_mask`` (reference: CausalWanModel.forward_train_tf,
solar/backends/wan22/runtime/modeling/causal_model.py:2093-2345, which builds a FlexAttention
block mask; here each chunk and role runs one dense attention over its visible key span).

``forward_window``: cache-free inference over ``[history window | current chunk]`` with per-frame
timesteps and absolute frame positions (reference: forward_inference_window, :2350-2619).

With sequence parallelism the ``2F`` (or window) frames are sharded whole-frame over the ranks and
the Ulysses exchange hands every rank the full sequence for ``H / P`` heads, so the structured
attention runs unchanged on the exchanged tensors.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..ops import functional as F_
from .wan import WanDiT, rope_table
from .wan_causal import teacher_forcing_attention


_MASKS: dict = {}


def _cached_mask(kind: str, *key):
    """Structured masks are pure functions of their geometry: build each once (tables are cached per device inside)."""
    from ..ops import attention_mask as am

    if (kind, key) not in _MASKS:
        _MASKS[(kind, key)] = am.block_causal_mask(*key) if kind == "causal" else am.teacher_forcing_segment_mask(*key)
    return _MASKS[(kind, key)]


def _masked_kernel_ok(q) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and ops.get_backend() == "native"


def block_causal_attention(q, k, v, *, frame_tokens: int, chunk_frames: int, window_chunks: int,
                           sink_frames: int = 0):
    """Chunk i attends sink + chunks max(0, i-W) .. i of the same sequence; tensors [1, L, H, D].  On the device this
    is ONE masked flash-attention call (per-row key ranges, tiles outside the window skipped); the chunk loop below is
    the CPU form of the same rule."""
    ct = chunk_frames * frame_tokens
    if _masked_kernel_ok(q):
        from ..ops.attention_mask import masked_attention

        return masked_attention(q, k, v, _cached_mask("causal", q.shape[1], ct, window_chunks, sink_frames * frame_tokens))
    n = (q.shape[1] + ct - 1) // ct
    sink = sink_frames * frame_tokens
    outs = []
    for i in range(n):
        lo = max(0, i - window_chunks) * ct
        hi = min((i + 1) * ct, q.shape[1])
        if sink and lo > 0:
            kk = torch.cat([k[:, :sink], k[:, lo:hi]], 1)
            vv = torch.cat([v[:, :sink], v[:, lo:hi]], 1)
        else:
            kk, vv = k[:, lo:hi], v[:, lo:hi]
        outs.append(ops.attention(q[:, i * ct:hi], kk, vv))
    return torch.cat(outs, 1)


def _run(model: WanDiT, tok, t_frames, r_frames, context, frame_positions, grid_hw, attn_fn, out_frames, y_camera=None):
    """Shared body: tok [F_all*ft, dim] (B = 1), per-frame times, explicit frame positions; ``y_camera`` =
    ``{"viewmats": [1, F_all, 4, 4], "Ks": [1, F_all, 3, 3] or None, "transform": str}`` (one camera per packed
    frame) conditions the self-attention as in the bidirectional forward."""
    cfg = model.cfg
    P = model.stem.params
    h, w = grid_hw
    ft = h * w
    f_all = tok.shape[0] // ft
    e, e0 = model.time_condition(t_frames, r_frames)
    ctx = model.embed_text(context)
    sp = model.sp
    f0, fl = 0, f_all
    if sp.size > 1:
        base, rem = divmod(f_all, sp.size)
        fl = base + int(sp.rank < rem)
        f0 = sp.rank * base + min(sp.rank, rem)
        tok = tok[f0 * ft:(f0 + fl) * ft]
        sp.set_layout(1, f_all, ft)
    rope = rope_table((fl, h, w), cfg.head_dim, tok.device, frame_positions=frame_positions[f0:f0 + fl])
    kw = dict(B=1, L=f_all * ft, frame_tokens=ft, group_offset=f0 if sp.size > 1 else 0, sp=sp, attn_fn=attn_fn)
    if y_camera is not None:
        from . import camera_prope

        Ks = y_camera.get("Ks")
        mats = camera_prope.prope_matrices(y_camera["viewmats"][0, f0:f0 + fl].to(tok.device),
                                           None if Ks is None else Ks[0, f0:f0 + fl].to(tok.device),
                                           transform=y_camera.get("transform", "linear"))
        kw["camera"] = tuple(camera_prope.per_row(m_, ft) for m_ in mats)
    xs = tok
    for bi, block in enumerate(model.blocks):
        if model.checkpointing != "none" and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            xs = checkpoint(lambda a, b, c, blk=block: blk(a, b, rope, c, **kw), xs, e0, ctx, use_reentrant=False)
        else:
            xs = block(xs, e0, rope, ctx, **kw)
    if sp.size > 1:
        xs = sp.gather_sequence(xs, 1)
    lo, hi = out_frames
    xs = xs[lo * ft:hi * ft]
    hm = (P["head.modulation"].float().view(1, 2, cfg.dim) + e.float().view(-1, 1, cfg.dim)[lo:hi]).contiguous()
    xh = F_.norm_modulate(xs, hm[:, 0], hm[:, 1], eps=cfg.eps, rows_per_group=ft, **model.blocks[0]._norm_kw(xs))
    out = F_.linear(xh, P["head.head.weight"], P["head.head.bias"])
    return model.unpatchify(out, 1, (hi - lo, h, w))


def _embed(model: WanDiT, x):
    rows, grid = model.patchify(x.to(model.dtype))
    pw = model.stem.params["patch_embedding.weight"]
    return F_.linear(rows, pw.view(pw.shape[0], -1), model.stem.params["patch_embedding.bias"]), grid


def forward_teacher_forcing(model: WanDiT, clean, noisy, t, context, *, r: Optional[torch.Tensor] = None,
                            chunk_frames: int = 3, window_chunks: int = 6, sink_frames: int = 0,
                            capture: Optional[list] = None, y_camera=None):
    """clean / noisy [1, C, F, H, W]; t (and r) [1, F] on the 1000-step grid; returns the prediction
    for the noisy half [1, C_out, F, H, W].  With ``capture`` (an empty list) every block appends the detached
    keys / values of the clean half (this rank's heads): clean rows never see a noisy row, so they are the same in
    every evaluation of a step and ``forward_noisy_suffix`` can reuse them."""
    if clean.shape[0] != 1:
        raise ValueError("teacher forcing packs one video per call")
    if y_camera is not None:
        if capture is not None and model.cfg.camera_attention_mode == "parallel":
            raise ValueError("key / value capture follows one attention per block; the parallel camera branch adds a second")
        twice = lambda v: None if v is None else torch.cat([v, v], dim=1)      # noqa: E731  clean | noisy share cameras
        y_camera = dict(y_camera, viewmats=twice(y_camera["viewmats"]), Ks=twice(y_camera.get("Ks")))
    tok_c, grid = _embed(model, clean)
    tok_n, _ = _embed(model, noisy)
    f, h, w = grid
    ft = h * w
    zeros = torch.zeros_like(t)
    t_all = torch.cat([zeros, t], dim=1)
    r_all = None if r is None else torch.cat([zeros, r], dim=1)
    pos = torch.arange(f).repeat(2)

    def attn(q, k, v):
        L = f * ft
        if capture is not None and len(capture) < len(model.blocks):      # a checkpoint recompute must not append again
            capture.append((k[:, :L].detach(), v[:, :L].detach()))
        if _masked_kernel_ok(q):
            # one masked kernel over the whole [clean | noisy] sequence: no per-chunk launches, no key concatenation
            from ..ops.attention_mask import masked_attention

            return masked_attention(q, k, v, _cached_mask("tf", L, chunk_frames * ft, window_chunks, sink_frames * ft, 0))
        oc, on = teacher_forcing_attention(q[:, :L], k[:, :L], v[:, :L], q[:, L:], k[:, L:], v[:, L:],
                                           frame_tokens=ft, chunk_frames=chunk_frames,
                                           window_chunks=window_chunks, sink_frames=sink_frames)
        return torch.cat([oc, on], 1)

    return _run(model, torch.cat([tok_c, tok_n], 0), t_all, r_all, context, pos, (h, w), attn, (f, 2 * f), y_camera)


@torch.no_grad()
def forward_noisy_suffix(model: WanDiT, noisy, t, context, captured, *, r: Optional[torch.Tensor] = None,
                         chunk_frames: int = 3, window_chunks: int = 6, sink_frames: int = 0):
    """The noisy half alone against the clean keys / values captured by ``forward_teacher_forcing(capture=...)``:
    the same prediction as the full teacher-forcing evaluation gives for these noisy frames, without recomputing
    the clean half (about half the cost).  For the no-grad central-difference probes of the AnyFlow objective
    (reference: prefix-KV capture / suffix reuse, solar/backends/minimax_h3/w6_attention.py:218-324, applied here to
    the Wan teacher-forcing mask)."""
    if len(captured) != len(model.blocks):
        raise ValueError("one captured (k, v) pair per block is required")
    tok_n, grid = _embed(model, noisy)
    f, h, w = grid
    ft = h * w
    ct = chunk_frames * ft
    L = f * ft
    sink = sink_frames * ft
    layer = [0]

    def attn(q, k, v):
        ck, cv = captured[layer[0]]
        layer[0] += 1
        outs = []
        for i in range(-(-L // ct)):
            lo = max(0, i - window_chunks) * ct
            hi = min((i + 1) * ct, L)
            seg = [slice(0, sink)] if (sink and lo > 0) else []
            kk = [ck[:, s] for s in seg] + [ck[:, lo:i * ct], k[:, i * ct:hi]]
            vv = [cv[:, s] for s in seg] + [cv[:, lo:i * ct], v[:, i * ct:hi]]
            outs.append(ops.attention(q[:, i * ct:hi], torch.cat(kk, 1), torch.cat(vv, 1)))
        return torch.cat(outs, 1)

    return _run(model, tok_n, t, r, context, torch.arange(f), (h, w), attn, (0, f))


def forward_window(model: WanDiT, frames, t, context, *, first_frame: int, current_frames: int,
                   chunk_frames: int = 3, window_chunks: int = 6, r: Optional[torch.Tensor] = None, y_camera=None):
    """frames [1, C, Fw, H, W] = clean history followed by the current noisy chunk; t [1, Fw] (0 on the
    history); ``first_frame`` = absolute index of the window's first frame.  Returns the prediction for
    the last ``current_frames`` frames."""
    tok, grid = _embed(model, frames)
    f, h, w = grid
    pos = torch.arange(f) + int(first_frame)

    def attn(q, k, v):
        return block_causal_attention(q, k, v, frame_tokens=h * w, chunk_frames=chunk_frames,
                                      window_chunks=window_chunks)

    return _run(model, tok, t, r, context, pos, (h, w), attn, (f - current_frames, f), y_camera)
