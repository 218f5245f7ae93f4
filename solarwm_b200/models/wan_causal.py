"""Block-causal (chunk-wise autoregressive) execution of the Wan DiT with a rolling KV cache.

Per transformer block the cache holds, for every cached token, the normalised AND ROTATED key and
the value: ``[sink frames | local window | current chunk]``.  Keys are written once with the RoPE of
the position they have at that moment; a denoising evaluation therefore reads the window as it is
(no pass over the cached keys per layer and step).  Positions follow the reference's re-basing rule
(solar/backends/wan22/runtime/modeling/causal_model.py:88-220, 657-876, 1028-1235, 1948-2088): sink
frames keep positions ``0 ..``; the newest frame sits at ``min(absolute index, position_cap - 1)`` and
the window counts down from there, so a rollout longer than the training length keeps seeing positions
it was trained on.  ``position_cap`` is the cache capacity by default (window-relative positions), the
training length for block-relative RoPE, or a finite ``pmax`` for EchoRoPE.  When the rule moves the
history (the window slides, or the cap is reached) the cached window keys are re-based by ONE delta
rotation per chunk -- RoPE rotations compose and only the temporal pairs move -- fused with the
window shift.  ``rope_at_read=True`` keeps the original form (un-rotated keys, RoPE at every read) as
the oracle the tests compare against.

Differences from the reference, on purpose:
  * a forward with ``commit=False`` (the denoising steps of a chunk) writes the chunk's K/V into the
    staging slots behind the committed tokens and never touches committed state; ``commit=True``
    (the clean forward after the last step) advances the committed length and, when the window is
    full, shifts the window once.  The reference clones the whole cache of every block on every
    step (causal_model.py:1054-1067).
  * text keys/values of the cross-attention are projected once per prompt and reused.
  * under head-parallel inference (SP > 1, reference P4) every rank keeps all tokens but only its
    heads in the cache and the attention outputs are all-gathered on the head axis.

Teacher forcing (Stage 1) uses ``teacher_forcing_attention``: the ``[clean | noisy]`` block mask is
executed as one dense attention per chunk over its visible key segments (sink + bounded clean
window + own chunk) instead of a FlexAttention block mask (causal_model.py:329-471).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from ..ops import functional as F_
from .wan import WanDiT, rope_table


@dataclass
class LayerCache:
    k: torch.Tensor          # [capacity_tokens, dim_local]  normalised, un-rotated keys
    v: torch.Tensor          # [capacity_tokens, dim_local]
    text_k: Optional[torch.Tensor] = None   # [T, dim] projected + normalised text keys
    text_v: Optional[torch.Tensor] = None
    cam_k: Optional[torch.Tensor] = None    # the parallel camera branch's own cache: keys / values stored AFTER the
    cam_v: Optional[torch.Tensor] = None    # P^-1 of their own frame (no rotary positions, so a slide is a plain move)


@dataclass
class KVCache:
    layers: List[LayerCache]
    frame_tokens: int
    sink_frames: int
    window_frames: int        # committed frames kept besides the sink
    chunk_frames: int
    committed_frames: int = 0          # frames currently held (sink + window part)
    total_frames: int = 0              # frames generated so far (absolute)
    grid_hw: tuple = (0, 0)
    cam_inv: Optional[torch.Tensor] = None   # [capacity_frames, 4, 4] P^-1 of every cached frame (camera runs)
    position_cap: int = 0              # the newest frame's RoPE position never exceeds position_cap - 1
    newest_pos: int = -1               # position the newest committed non-sink frame was rotated to

    def reset(self) -> None:
        """Start a new stream in the same buffers (nothing is cleared: rows beyond ``committed_frames`` are never read);
        the projected text of the previous stream is dropped."""
        self.committed_frames = self.total_frames = 0
        self.newest_pos = -1
        if self.cam_inv is not None:
            self.cam_inv.copy_(torch.eye(4, device=self.cam_inv.device).expand_as(self.cam_inv))
        for lc in self.layers:
            lc.text_k = lc.text_v = None

    @property
    def positions_saturated(self) -> bool:
        """The newest position has reached the cap: from here on every chunk moves the history by its own length."""
        return self.total_frames >= self.position_cap - self.chunk_frames

    @property
    def capacity_frames(self) -> int:
        return self.sink_frames + self.window_frames + self.chunk_frames


def allocate_kv_cache(model: WanDiT, *, grid_hw, chunk_frames: int, window_frames: Optional[int] = None,
                      sink_frames: Optional[int] = None, heads_local: Optional[int] = None, device=None,
                      position_cap: Optional[int] = None) -> KVCache:
    """``position_cap``: RoPE positions of the newest frame are clamped to ``position_cap - 1`` (default: the cache
    capacity in frames = window-relative positions; pass the training length for block-relative RoPE)."""
    cfg = model.cfg
    h, w = grid_hw
    ft = h * w
    sink = cfg.sink_size if sink_frames is None else sink_frames
    window = (cfg.local_attn_size if cfg.local_attn_size > 0 else 21) if window_frames is None else window_frames
    window = max(window - sink, chunk_frames)
    hl = cfg.num_heads if heads_local is None else heads_local
    dim_local = hl * cfg.head_dim
    dev = device or next(model.parameters()).device
    cap = (sink + window + chunk_frames) * ft
    buf = lambda: torch.zeros(cap, dim_local, dtype=model.dtype, device=dev)   # noqa: E731
    layers = [LayerCache(buf(), buf()) for _ in model.blocks]
    if cfg.camera_attention_mode == "parallel":
        for lc in layers:
            lc.cam_k, lc.cam_v = buf(), buf()
    cap_frames = sink + window + chunk_frames
    if position_cap is not None and position_cap < cap_frames:
        raise ValueError(f"position_cap {position_cap} is below the cache capacity of {cap_frames} frames")
    return KVCache(layers, ft, sink, window, chunk_frames, grid_hw=(h, w),
                   position_cap=cap_frames if position_cap is None else int(position_cap))


class CausalWanRunner:
    """Chunk-by-chunk forward of a ``WanDiT`` against a ``KVCache`` (inference; no autograd)."""

    def __init__(self, model: WanDiT, sp=None, rope_at_read: bool = False):
        self.model = model
        self.sp = sp
        self.rope_at_read = bool(rope_at_read)
        self._rope_cache = {}

    # -- positions ------------------------------------------------------------------------------------------------
    @staticmethod
    def chunk_first_position(cache: KVCache, f: int) -> int:
        """RoPE position of the first frame of the chunk that comes next (absolute until the cap, then clamped)."""
        a0 = cache.total_frames
        if a0 + f <= cache.sink_frames:
            return a0
        return min(a0 + f - 1, cache.position_cap - 1) - f + 1

    def _delta_table(self, n_tokens: int, delta_frames: int, device):
        """(cos, sin) per token that rotates the temporal RoPE pairs by ``delta_frames`` positions and leaves the
        spatial pairs alone."""
        key = ("delta", n_tokens, delta_frames, str(device))
        if key not in self._rope_cache:
            from .wan import rope_axis_dims

            hd = self.model.cfg.head_dim
            cf, ch, cw = rope_axis_dims(hd)
            inv = 1.0 / torch.pow(10000.0, torch.arange(0, 2 * cf, 2, dtype=torch.float64) / (2 * cf))
            ang = torch.cat([float(delta_frames) * inv, torch.zeros(ch + cw, dtype=torch.float64)])
            tab = torch.stack([torch.cos(ang), torch.sin(ang)], -1).to(torch.float32)
            self._rope_cache[key] = tab.unsqueeze(0).expand(n_tokens, -1, -1).contiguous().to(device)
        return self._rope_cache[key]

    def _rebase_window(self, cache: KVCache, delta_frames: int) -> None:
        """Move the cached (non-sink) window keys by ``delta_frames`` positions: one rotation pass per layer."""
        ft = cache.frame_tokens
        a = cache.sink_frames * ft
        b = cache.committed_frames * ft
        if b > a and delta_frames != 0:
            tab = self._delta_table(b - a, delta_frames, cache.layers[0].k.device)
            for lc in cache.layers:
                lc.k[a:b] = F_.rmsnorm_rope(lc.k[a:b], None, tab, no_norm=True)
        cache.newest_pos += delta_frames

    def _rope(self, frames, hw, device, first=0):
        key = (frames, hw, first, str(device))
        if key not in self._rope_cache:
            self._rope_cache[key] = rope_table((frames, hw[0], hw[1]), self.model.cfg.head_dim, device, frame_offset=first)
        return self._rope_cache[key]

    @torch.no_grad()
    def encode_text(self, cache: KVCache, context: torch.Tensor) -> None:
        """Project the prompt once: per block, normalised text keys and values for the cross-attention."""
        m = self.model
        ctx = m.embed_text(context)
        D = m.cfg.dim
        for blk, lc in zip(m.blocks, cache.layers):
            kv = blk._fused_linear(ctx, "cross_attn.k", "cross_attn.v", 2 * D)
            lc.text_k = F_.rmsnorm_rope(kv[:, :D], blk._p("cross_attn.norm_k.weight").float(), None, eps=m.cfg.eps)
            lc.text_v = kv[:, D:].contiguous()

    @torch.no_grad()
    def forward_chunk(self, cache: KVCache, x: torch.Tensor, t: torch.Tensor, *, commit: bool, y=None,
                      y_camera=None) -> torch.Tensor:
        """x [1, C, f, H, W] (f = chunk frames), t [1, f] -> prediction [1, C_out, f, H, W].

        ``y_camera`` = ``{"viewmats": [1, f, 4, 4], "Ks": [1, f, 3, 3] or None, "transform": str}`` switches on
        PRoPE with separate query / key cameras: queries take P^T of the chunk's cameras, every cached key
        (after RoPE) and value takes the P^-1 of ITS OWN frame, the output takes P of the chunk
        (reference: prope_qkv_separate, camera_prope.py:93-180)."""
        m, cfg = self.model, self.model.cfg
        P_ = m.stem.params
        if y is not None:
            x = torch.cat([x, y], dim=1)
        rows, (f, h, w) = m.patchify(x.to(m.dtype))
        ft = h * w
        assert ft == cache.frame_tokens and f <= cache.chunk_frames
        pw = P_["patch_embedding.weight"]
        xs = F_.linear(rows, pw.view(pw.shape[0], -1), P_["patch_embedding.bias"])
        e, e0 = m.time_condition(t)
        D, H, hd = cfg.dim, cfg.num_heads, cfg.head_dim
        ctx_frames = cache.committed_frames
        n_ctx, n_new = ctx_frames * ft, f * ft
        if self.rope_at_read:
            rope_all = self._rope(ctx_frames + f, (h, w), xs.device)
            rope_q = rope_all[n_ctx:]
        else:
            # keys are cached rotated: bring the history to where this chunk expects it (a no-op in the steady state,
            # where the commit of the previous chunk already did it), then rotate only the new rows
            first = self.chunk_first_position(cache, f)
            if ctx_frames > cache.sink_frames and cache.newest_pos != first - 1:
                self._rebase_window(cache, first - 1 - cache.newest_pos)
            rope_all = None
            rope_q = self._rope(f, (h, w), xs.device, first=first)
        sp = self.sp
        P = 1 if sp is None else sp.size
        hl = H // P
        h0 = 0 if sp is None else sp.rank * hl
        gk = dict(rows_per_group=ft)
        cam = None
        parallel = cfg.camera_attention_mode == "parallel"
        if y_camera is not None:
            from . import camera_prope

            Ks = y_camera.get("Ks")
            PT, Pinv, Pm = camera_prope.prope_matrices(y_camera["viewmats"][0].to(xs.device),
                                                       None if Ks is None else Ks[0].to(xs.device),
                                                       transform=y_camera.get("transform", "linear"))
            if cache.cam_inv is None:
                cache.cam_inv = torch.eye(4, device=xs.device).repeat(cache.capacity_frames, 1, 1)
            cache.cam_inv[ctx_frames:ctx_frames + f] = Pinv
            cam = (camera_prope.per_row(PT, ft), camera_prope.per_row(Pinv, ft), camera_prope.per_row(Pm, ft),
                   camera_prope.per_row(cache.cam_inv[:ctx_frames + f], ft))
        for blk, lc in zip(m.blocks, cache.layers):
            mod = (blk._p("modulation").float().view(1, 6, D) + e0).contiguous()
            xm = F_.norm_modulate(xs, mod[:, 0], mod[:, 1], mode=0, eps=cfg.eps, **gk)
            qkv = blk._fused_linear(xm, "self_attn.q", "self_attn.v", 3 * D)
            q = F_.rmsnorm_rope(qkv[:, :D], blk._p("self_attn.norm_q.weight").float(), rope_q, eps=cfg.eps)
            k_raw = F_.rmsnorm_rope(qkv[:, D:2 * D], blk._p("self_attn.norm_k.weight").float(),
                                    None if self.rope_at_read else rope_q, eps=cfg.eps)
            cs = slice(h0 * hd, (h0 + hl) * hd)
            v_new = qkv[:, 2 * D:][:, cs]
            q_loc = q[:, cs]
            own = cam is not None and not parallel          # cameras on the block's own attention
            if own:
                q_loc = camera_prope.apply(q_loc.contiguous(), cam[0], hl)
                v_new = camera_prope.apply(v_new.contiguous(), cam[1], hl)       # values are cached transformed
            lc.k[n_ctx:n_ctx + n_new] = k_raw[:, cs]
            lc.v[n_ctx:n_ctx + n_new] = v_new
            k_all = F_.rmsnorm_rope(lc.k[:n_ctx + n_new], None, rope_all, no_norm=True) if self.rope_at_read \
                else lc.k[:n_ctx + n_new]
            if own:
                k_all = camera_prope.apply(k_all, cam[3], hl)                    # after RoPE, each key with its own camera
            o = ops.attention(q_loc.reshape(1, n_new, hl, hd), k_all.view(1, n_ctx + n_new, hl, hd),
                              lc.v[:n_ctx + n_new].view(1, n_ctx + n_new, hl, hd))
            o = o.reshape(n_new, hl * hd)
            if own:
                o = camera_prope.apply(o, cam[2], hl)
            if P > 1:
                o = sp.all_gather_heads(o)
            if cfg.gated_attention:
                gate = 2.0 * torch.sigmoid(F_.linear(xm, blk._p("self_attn.to_gate_logits.weight"),
                                                     blk._p("self_attn.to_gate_logits.bias")).float())
                o = (o.view(n_new, H, hd) * gate.to(o.dtype).unsqueeze(-1)).reshape(n_new, D)
            yb = blk._linear(o, "self_attn.o.weight", "self_attn.o.bias")
            if cam is not None and parallel:
                # the camera branch: no rotary positions, keys and values enter ITS cache already in their own
                # frame's camera coordinates, so the history is read as it is
                cqkv = blk._fused_linear(xm, "cam_self_attn.q_proj", "cam_self_attn.v_proj", 3 * D)
                cq = F_.rmsnorm_rope(cqkv[:, :D], blk._p("cam_self_attn.norm_q.weight").float(), None, eps=cfg.eps)
                ck = F_.rmsnorm_rope(cqkv[:, D:2 * D], blk._p("cam_self_attn.norm_k.weight").float(), None, eps=cfg.eps)
                cq = camera_prope.apply(cq[:, cs].contiguous(), cam[0], hl)
                lc.cam_k[n_ctx:n_ctx + n_new] = camera_prope.apply(ck[:, cs].contiguous(), cam[1], hl)
                lc.cam_v[n_ctx:n_ctx + n_new] = camera_prope.apply(cqkv[:, 2 * D:][:, cs].contiguous(), cam[1], hl)
                oc_ = ops.attention(cq.reshape(1, n_new, hl, hd), lc.cam_k[:n_ctx + n_new].view(1, n_ctx + n_new, hl, hd),
                                    lc.cam_v[:n_ctx + n_new].view(1, n_ctx + n_new, hl, hd)).reshape(n_new, hl * hd)
                oc_ = camera_prope.apply(oc_, cam[2], hl)
                if P > 1:
                    oc_ = sp.all_gather_heads(oc_)
                yb = yb + blk._linear(oc_, "cam_self_attn.out_proj.weight", "cam_self_attn.out_proj.bias")
            xs = F_.gated_residual(xs, yb, mod[:, 2], **gk)
            xn = F_.norm_modulate(xs, mode=2, w=blk._p("norm3.weight").float(), b=blk._p("norm3.bias").float(),
                                  eps=cfg.eps) if cfg.cross_attn_norm else xs
            qc = blk._linear(xn, "cross_attn.q.weight", "cross_attn.q.bias")
            qc = F_.rmsnorm_rope(qc, blk._p("cross_attn.norm_q.weight").float(), None, eps=cfg.eps)
            T = lc.text_k.shape[0]
            oc = ops.attention(qc.view(1, n_new, H, hd), lc.text_k.view(1, T, H, hd), lc.text_v.view(1, T, H, hd))
            xs = F_.gated_residual(xs, blk._linear(oc.reshape(n_new, D), "cross_attn.o.weight", "cross_attn.o.bias"), None)
            xm = F_.norm_modulate(xs, mod[:, 3], mod[:, 4], mode=0, eps=cfg.eps, **gk)
            hmid = F_.linear(xm, blk._p("ffn.0.weight"), blk._p("ffn.0.bias"), act="gelu") if xs.is_cuda else \
                F_.gelu(F_.linear(xm, blk._p("ffn.0.weight"), blk._p("ffn.0.bias")))
            xs = F_.gated_residual(xs, blk._linear(hmid, "ffn.2.weight", "ffn.2.bias"), mod[:, 5], **gk)
        hm = (P_["head.modulation"].float().view(1, 2, D) + e.float().view(-1, 1, D)).contiguous()
        xh = F_.norm_modulate(xs, hm[:, 0], hm[:, 1], mode=0, eps=cfg.eps, rows_per_group=ft)
        out = m.unpatchify(F_.linear(xh, P_["head.head.weight"], P_["head.head.bias"]), 1, (f, h, w))
        if commit:
            if not self.rope_at_read and cache.total_frames + f > cache.sink_frames:
                cache.newest_pos = self.chunk_first_position(cache, f) + f - 1
            self._commit(cache, f)
        return out

    def _commit(self, cache: KVCache, f: int) -> None:
        """Keep the chunk just written; when sink + window is exceeded drop the oldest window frames."""
        ft = cache.frame_tokens
        cache.committed_frames += f
        cache.total_frames += f
        limit = cache.sink_frames + cache.window_frames
        extra = cache.committed_frames - limit
        if extra > 0:
            s0 = cache.sink_frames * ft
            keep = (cache.committed_frames - cache.sink_frames - extra) * ft
            for lc in cache.layers:
                for buf in (lc.k, lc.v, lc.cam_k, lc.cam_v):
                    if buf is not None:
                        buf[s0:s0 + keep] = buf[s0 + extra * ft:s0 + extra * ft + keep].clone()
            if cache.cam_inv is not None:
                fs, fk = cache.sink_frames, keep // ft
                cache.cam_inv[fs:fs + fk] = cache.cam_inv[fs + extra:fs + extra + fk].clone()
            cache.committed_frames = limit
        if not self.rope_at_read and cache.committed_frames > cache.sink_frames:
            # re-base now for the chunk that comes next (assumed to have this chunk's length), so that a captured
            # commit contains the rotation and the next evaluations read the window as it is
            nxt = self.chunk_first_position(cache, f)
            if cache.newest_pos != nxt - 1:
                self._rebase_window(cache, nxt - 1 - cache.newest_pos)


def teacher_forcing_attention(q_clean, k_clean, v_clean, q_noisy, k_noisy, v_noisy, *, frame_tokens: int,
                              chunk_frames: int, window_chunks: int, sink_frames: int = 0):
    """Block-causal ``[clean | noisy]`` attention for teacher forcing; all tensors ``[1, F*ft, H, D]``.

    clean chunk i sees  sink + clean chunks max(0, i-W) .. i
    noisy chunk i sees  sink + clean chunks max(0, i-W) .. i-1 + its own noisy chunk
    Returns (o_clean, o_noisy).  Executed as one dense attention per chunk and role.
    """
    ft = frame_tokens
    ct = chunk_frames * ft
    L = q_clean.shape[1]
    n_chunks = -(-L // ct)                       # the last chunk may hold fewer frames
    sink = sink_frames * ft
    outs_c, outs_n = [], []
    for i in range(n_chunks):
        lo = max(0, i - window_chunks) * ct
        seg = [slice(0, sink)] if (sink and lo > 0) else []
        c_hi = min((i + 1) * ct, L)
        ks = [k_clean[:, s] for s in seg] + [k_clean[:, lo:c_hi]]
        vs = [v_clean[:, s] for s in seg] + [v_clean[:, lo:c_hi]]
        kc, vc = (ks[0], vs[0]) if len(ks) == 1 else (torch.cat(ks, 1), torch.cat(vs, 1))   # one span: no copy
        outs_c.append(ops.attention(q_clean[:, i * ct:c_hi], kc, vc))
        kn = [k_clean[:, s] for s in seg] + [k_clean[:, lo:i * ct], k_noisy[:, i * ct:c_hi]]
        vn = [v_clean[:, s] for s in seg] + [v_clean[:, lo:i * ct], v_noisy[:, i * ct:c_hi]]
        outs_n.append(ops.attention(q_noisy[:, i * ct:c_hi], torch.cat(kn, 1), torch.cat(vn, 1)))
    return torch.cat(outs_c, 1), torch.cat(outs_n, 1)


def teacher_forcing_mask(num_frames: int, frame_tokens: int, chunk_frames: int, window_chunks: int,
                         sink_frames: int = 0) -> torch.Tensor:
    """Dense boolean mask ``[2L, 2L]`` (True = visible) over ``[clean | noisy]`` tokens; the oracle
    for ``teacher_forcing_attention`` and for direct block-mask construction."""
    L = num_frames * frame_tokens
    ct = chunk_frames * frame_tokens
    chunk = torch.arange(L) // ct
    is_sink = torch.arange(L) < sink_frames * frame_tokens
    qc, kc = chunk.view(-1, 1), chunk.view(1, -1)
    clean_clean = ((kc <= qc) & (kc >= qc - window_chunks)) | is_sink.view(1, -1) & (kc <= qc)
    noisy_clean = ((kc < qc) & (kc >= qc - window_chunks)) | is_sink.view(1, -1) & (kc < qc)
    noisy_noisy = kc == qc
    top = torch.cat([clean_clean, torch.zeros(L, L, dtype=torch.bool)], 1)
    bottom = torch.cat([noisy_clean, noisy_noisy], 1)
    return torch.cat([top, bottom], 0)
