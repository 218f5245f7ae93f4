"""Windowed ViT video decoder with latent-by-latent streaming, tile blending and pixel compensation.

The decoder is a transformer over the tokens of a *window* of ``window`` latent frames that starts
on a multiple of ``stride`` (7 and 5 for the H3-style codec); every latent token carries
``frames x patch x patch x 3`` output pixels.  ``StreamingViTDecoder`` decodes every latent the
moment it arrives:

* **step**: the new latent runs alone at its slot of the current window, with the RoPE position of
  that slot, and attends to the register tokens and to the cached keys / values of the slots before
  it.  Its frames are emitted at once and never revised: one frame for a latent that opens a group
  of ``stride`` latents, ``frames_per_latent`` for the others.
* **shift**: when the window moves by ``stride``, the ``window - stride`` latents shared with the
  previous window run again at slots 0.. of the new window, in the pass of the window's next latent;
  this only refills the cache.
* **compensate**: ``a + b x`` (``+ c x^2`` on the first frame of the stream) is taken off every emitted
  pixel, ``x`` being the pixel's own value, with per-slot, per-channel, per-frame constants.
* **tiles**: the latent grid is cut into overlapping spatial tiles (the batch axis of the
  transformer); decoded tiles are blended with linear ramps over the overlap.  ``distributed=True`` splits
  the tiles over a process group and gathers the decoded tiles on rank 0.

Keys are cached after RoPE, one ``[tiles, registers + window * hw, heads * dim_head]`` buffer per
layer; a step reads the first ``registers + (slot + 1) * hw`` rows in place.  The attention and the
GEMMs run on this package's kernels (head_dim 64); the norms, RoPE and residuals use the row kernels.

Reference: deploy/solar_wm/shared/vae/streaming.py:1-473 (StreamingDecoder), tile_parallel.py:11-80.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import functional as F_


@dataclass
class ViTDecoderConfig:
    latent_channels: int = 24
    dim: int = 1024
    depth: int = 36
    heads: int = 16
    dim_head: int = 64
    ffn_dim: int = 2816
    registers: int = 5              # register + cls tokens in front of every window
    window: int = 7
    stride: int = 5
    frames_per_latent: int = 4
    patch: int = 16                 # output pixels per latent pixel, per side
    eps: float = 1e-6

    @classmethod
    def tiny(cls):
        return cls(latent_channels=4, dim=64, depth=2, heads=2, dim_head=32, ffn_dim=128, registers=2, patch=2)


def _axis_rope(n_pairs: int, coords: torch.Tensor, theta: float = 100.0) -> torch.Tensor:
    inv = 1.0 / torch.pow(theta, torch.arange(n_pairs, dtype=torch.float64) / max(n_pairs, 1))
    return torch.outer(coords.to(torch.float64), inv * math.pi)


def rope_tables(slot: int, window: int, h: int, w: int, dim_head: int):
    """cos / sin [h*w, dim_head] (rotate-half layout) of one slot of a window; coordinates are the
    length-normalised centres in [-1, 1] of a ``window x h x w`` grid."""
    pairs = dim_head // 2
    pt = pairs // 3
    ph = pairs // 3
    pw = pairs - pt - ph
    norm = lambda i, n: 2.0 * ((i + 0.5) / n) - 1.0   # noqa: E731
    t = torch.full((h * w,), norm(slot, window), dtype=torch.float64)
    ys = norm(torch.arange(h, dtype=torch.float64), h).repeat_interleave(w)
    xs = norm(torch.arange(w, dtype=torch.float64), w).repeat(h)
    ang = torch.cat([_axis_rope(pt, t), _axis_rope(ph, ys), _axis_rope(pw, xs)], dim=1)      # [hw, pairs]
    full = torch.cat([ang, ang], dim=1)
    return torch.cos(full).float(), torch.sin(full).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int) -> torch.Tensor:
    """x [B, N, heads*dh]; cos/sin [N, dh]; rotate-half within each head."""
    B, N, _ = x.shape
    v = x.view(B, N, heads, -1).float()
    half = v.shape[-1] // 2
    rot = torch.cat([-v[..., half:], v[..., :half]], dim=-1)
    out = v * cos.view(1, N, 1, -1) + rot * sin.view(1, N, 1, -1)
    return out.to(x.dtype).view(B, N, -1)


class ViTBlock(nn.Module):
    def __init__(self, c: ViTDecoderConfig, device, dtype, gen):
        super().__init__()
        a = c.heads * c.dim_head
        mk = lambda o, i: nn.Parameter((torch.randn(o, i, generator=gen, device=gen.device) / math.sqrt(i)).to(device, dtype),  # noqa: E731
                                       requires_grad=False)
        self.qkv, self.out = mk(3 * a, c.dim), mk(c.dim, a)
        self.gate_up, self.down = mk(2 * c.ffn_dim, c.dim), mk(c.dim, c.ffn_dim)
        self.norm1 = nn.Parameter(torch.ones(c.dim, device=device), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(c.dim, device=device), requires_grad=False)
        self.q_norm = nn.Parameter(torch.ones(c.dim_head, device=device), requires_grad=False)
        self.k_norm = nn.Parameter(torch.ones(c.dim_head, device=device), requires_grad=False)


def _head_rms(x, w, heads, eps):
    B, N, _ = x.shape
    v = x.view(B, N, heads, -1).float()
    v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return v.to(x.dtype).view(B, N, -1)


class ViTVideoDecoder(nn.Module):
    def __init__(self, cfg: ViTDecoderConfig = ViTDecoderConfig(), device="cpu", dtype=torch.bfloat16, seed: int = 0):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        g = torch.Generator(device=device).manual_seed(seed)
        mk = lambda o, i, s=None: nn.Parameter((torch.randn(o, i, generator=g, device=g.device) * (s or 1 / math.sqrt(i))).to(device, dtype),  # noqa: E731
                                               requires_grad=False)
        self.embed = mk(cfg.dim, cfg.latent_channels)
        self.registers = nn.Parameter((torch.randn(cfg.registers, cfg.dim, generator=g, device=g.device) * 0.02).to(device, dtype),
                                      requires_grad=False)
        self.blocks = nn.ModuleList([ViTBlock(cfg, device, dtype, g) for _ in range(cfg.depth)])
        self.norm_out = nn.Parameter(torch.ones(cfg.dim, device=device), requires_grad=False)
        self.unembed = mk(cfg.frames_per_latent * cfg.patch * cfg.patch * 3, cfg.dim, 0.02)

    # one block on ``x`` [B, N, dim] whose keys/values are appended to (k_all, v_all) by the caller
    def block_qkv(self, blk: ViTBlock, x, cos, sin):
        c = self.cfg
        B, N, _ = x.shape
        a = c.heads * c.dim_head
        xm = F_.norm_modulate(x.reshape(B * N, -1), mode=1, w=blk.norm1, eps=c.eps)
        qkv = F_.linear(xm, blk.qkv).view(B, N, 3 * a)
        q = _head_rms(qkv[..., :a], blk.q_norm, c.heads, c.eps)
        k = _head_rms(qkv[..., a:2 * a], blk.k_norm, c.heads, c.eps)
        if cos is not None:
            q, k = apply_rope(q, cos, sin, c.heads), apply_rope(k, cos, sin, c.heads)
        return q, k, qkv[..., 2 * a:]

    def block_q_cached(self, blk: ViTBlock, x, cos, sin, k_cache, v_cache, lo: int):
        """The streaming form of ``block_qkv``: q is returned, k / v land in cache rows [lo, lo + N) through
        one fused kernel (head norms, rotary and the cache write share one pass over the qkv rows)."""
        c = self.cfg
        B, N, _ = x.shape
        xm = F_.norm_modulate(x.reshape(B * N, -1), mode=1, w=blk.norm1, eps=c.eps)
        qkv = F_.linear(xm, blk.qkv).view(B, N, -1)
        return F_.vit_qkv_to_cache(qkv, blk.q_norm, blk.k_norm, cos, sin, k_cache, v_cache, lo, heads=c.heads, eps=c.eps)

    def block_finish(self, blk: ViTBlock, x, o):
        c = self.cfg
        B, N, _ = x.shape
        x2 = F_.gated_residual(x.reshape(B * N, -1), F_.linear(o.reshape(B * N, -1), blk.out), None)
        xm = F_.norm_modulate(x2, mode=1, w=blk.norm2, eps=c.eps)
        if xm.is_cuda and blk.gate_up.shape[0] % 128 == 0:
            # gate|up product and SwiGLU in one kernel: the [rows, 2 * ffn] tensor is never written
            il = getattr(blk, "_gate_up_interleaved", None)
            if il is None or il.device != xm.device or il._version_src != blk.gate_up._version:
                il = F_.interleave_gate_up(blk.gate_up.detach())
                il._version_src = blk.gate_up._version
                blk._gate_up_interleaved = il
            y = F_.linear(F_.linear_swiglu(xm, il), blk.down)
        else:
            y = F_.linear(F_.swiglu(F_.linear(xm, blk.gate_up)), blk.down)
        return F_.gated_residual(x2, y, None).view(B, N, -1)

    def attend(self, q, k, v):
        c = self.cfg
        B, Nq, _ = q.shape
        Nk = k.shape[1]
        return ops.attention(q.view(B, Nq, c.heads, c.dim_head), k.reshape(B, Nk, c.heads, c.dim_head),
                             v.reshape(B, Nk, c.heads, c.dim_head)).reshape(B, Nq, -1)

    def to_pixels(self, x, h, w):
        """x [B, h*w, dim] -> frames [B, 3, frames_per_latent, h*patch, w*patch]."""
        c = self.cfg
        B = x.shape[0]
        y = F_.linear(F_.norm_modulate(x.reshape(B * h * w, -1), mode=1, w=self.norm_out, eps=c.eps), self.unembed)
        y = y.view(B, h, w, 3, c.frames_per_latent, c.patch, c.patch)
        return y.permute(0, 3, 4, 1, 5, 2, 6).reshape(B, 3, c.frames_per_latent, h * c.patch, w * c.patch)

    @torch.no_grad()
    def decode_window(self, latents: torch.Tensor) -> torch.Tensor:
        """Oracle: latents [B, C, n <= window, h, w] decoded in one pass with the same visibility the
        streaming decoder has (slot i sees the registers and slots <= i; registers see registers).
        Returns [B, 3, n * frames_per_latent, H, W]."""
        c = self.cfg
        B, C, n, h, w = latents.shape
        hw = h * w
        tok = F_.linear(latents.permute(0, 2, 3, 4, 1).reshape(B * n * hw, C).to(self.dtype), self.embed).view(B, n * hw, -1)
        x = torch.cat([self.registers.unsqueeze(0).expand(B, -1, -1), tok], dim=1)
        cs = [rope_tables(s, c.window, h, w, c.dim_head) for s in range(n)]
        R = c.registers
        cos = torch.cat([torch.ones(R, c.dim_head)] + [t[0] for t in cs]).to(x.device)
        sin = torch.cat([torch.zeros(R, c.dim_head)] + [t[1] for t in cs]).to(x.device)
        for blk in self.blocks:
            q, k, v = self.block_qkv(blk, x, cos, sin)
            outs = [self.attend(q[:, :R], k[:, :R], v[:, :R])]
            for s in range(n):
                hi = R + (s + 1) * hw
                outs.append(self.attend(q[:, R + s * hw:hi], k[:, :hi], v[:, :hi]))
            x = self.block_finish(blk, x, torch.cat(outs, dim=1))
        frames = [self.to_pixels(x[:, R + s * hw:R + (s + 1) * hw], h, w) for s in range(n)]
        return torch.cat(frames, dim=2)


def tile_plan(h: int, w: int, tile: int, overlap: int):
    """Start offsets of square-ish tiles covering an ``h x w`` latent grid with the given overlap."""
    def starts(n):
        if n <= tile:
            return [0]
        step = tile - overlap
        s = list(range(0, n - tile, step)) + [n - tile]
        return sorted(set(s))
    return [(y, x) for y in starts(h) for x in starts(w)]


def blend_tiles(tiles: List[torch.Tensor], plan, h: int, w: int, tile: int, overlap: int, patch: int) -> torch.Tensor:
    """tiles: list of [3, F, th*patch, tw*patch] in plan order -> [3, F, h*patch, w*patch] with linear ramps
    over the overlaps (weights sum to one everywhere)."""
    F_n = tiles[0].shape[1]
    out = torch.zeros(3, F_n, h * patch, w * patch, dtype=torch.float32, device=tiles[0].device)
    acc = torch.zeros(1, 1, h * patch, w * patch, dtype=torch.float32, device=tiles[0].device)
    ov = overlap * patch

    def ramp(n, lo, hi):
        wgt = torch.ones(n)
        if lo and ov:
            wgt[:ov] = torch.linspace(0, 1, ov + 2)[1:-1]
        if hi and ov:
            wgt[-ov:] = torch.linspace(1, 0, ov + 2)[1:-1]
        return wgt

    for t, (y, x) in zip(tiles, plan):
        th, tw = t.shape[2], t.shape[3]
        wy = ramp(th, y > 0, y + th // patch < h).to(t.device)
        wx = ramp(tw, x > 0, x + tw // patch < w).to(t.device)
        wgt = (wy.view(-1, 1) * wx.view(1, -1)).view(1, 1, th, tw)
        out[:, :, y * patch:y * patch + th, x * patch:x * patch + tw] += t.float() * wgt
        acc[:, :, y * patch:y * patch + th, x * patch:x * patch + tw] += wgt
    return out / acc.clamp_min(1e-8)


@dataclass
class CompensationTable:
    """Per (slot, channel, frame) constants of ``x - (a + b x [+ c x^2])``; ``c`` applies to the first frame
    of the stream only."""
    a: torch.Tensor          # [window, 3, frames_per_latent]
    b: torch.Tensor
    c: Optional[torch.Tensor] = None

    @classmethod
    def zeros(cls, window: int, frames: int):
        z = torch.zeros(window, 3, frames)
        return cls(z.clone(), z.clone(), z.clone())

    def folded_affine(self, slot: int, frame: int, mean: torch.Tensor, std: torch.Tensor):
        """Per-channel constants (std', mean') such that ``x * std' + mean'`` equals de-normalising the
        compensated pixel ``(x - (a + b x)) * std + mean``: the linear part of the compensation rides on the
        RGB8 conversion kernel's own affine step, so emitting a frame stays one pass over the pixels."""
        a, b = self.a[slot, :, frame].to(std), self.b[slot, :, frame].to(std)
        return std * (1.0 - b), mean - a * std

    def coefficients(self, slot: int, n_frames: int, first_of_stream: bool) -> torch.Tensor:
        """Host tensor [3 (a, b, c), 3 channels, n_frames] for the last ``n_frames`` positions of ``slot``;
        the quadratic term is kept for the first emitted frame of a stream only."""
        out = torch.zeros(3, 3, n_frames)
        out[0], out[1] = self.a[slot, :, -n_frames:], self.b[slot, :, -n_frames:]
        if first_of_stream and self.c is not None:
            out[2, :, 0] = self.c[slot, :, -n_frames:][:, 0]
        return out

    def apply(self, frames: torch.Tensor, slot: int, first_of_stream: bool) -> torch.Tensor:
        """frames [3, F, H, W] (F <= frames_per_latent, the last F positions of the slot)."""
        F_n = frames.shape[1]
        a = self.a[slot, :, -F_n:].to(frames.device).view(3, F_n, 1, 1)
        b = self.b[slot, :, -F_n:].to(frames.device).view(3, F_n, 1, 1)
        x = frames.float()
        y = x - (a + b * x)
        if first_of_stream and self.c is not None:
            y[:, :1] = y[:, :1] - self.c[slot, :, -F_n:][:, :1].to(frames.device).view(3, 1, 1, 1) * x[:, :1] ** 2
        return y


class StreamingViTDecoder:
    def __init__(self, model: ViTVideoDecoder, grid_hw, *, tile: Optional[int] = None, overlap: int = 0,
                 table: Optional[CompensationTable] = None, group=None, distributed: bool = False):
        self.m, self.cfg = model, model.cfg
        self.h, self.w = grid_hw
        self.tile = tile or max(self.h, self.w)
        self.overlap = overlap
        self.plan = tile_plan(self.h, self.w, self.tile, overlap) if tile else [(0, 0)]
        self.th, self.tw = (min(self.tile, self.h), min(self.tile, self.w)) if tile else (self.h, self.w)
        self.table = table
        self.group = group
        self.rank, self.world = 0, 1
        if distributed:                      # tiles are dealt round-robin to the ranks of ``group``
            import torch.distributed as dist

            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.my_tiles = [i for i in range(len(self.plan)) if i % self.world == self.rank]
        self.reset()

    def reset(self) -> None:
        c = self.cfg
        dev = self.m.embed.device
        rows = c.registers + c.window * self.th * self.tw
        a = c.heads * c.dim_head
        n = max(len(self.my_tiles), 1)
        self.k = [torch.zeros(n, rows, a, dtype=self.m.dtype, device=dev) for _ in self.m.blocks]
        self.v = [torch.zeros(n, rows, a, dtype=self.m.dtype, device=dev) for _ in self.m.blocks]
        self.count = 0                      # latents received
        self.recent: List[torch.Tensor] = []   # the last window - stride latents (for the shift refill)
        self._rope = {s: tuple(t.to(dev, torch.float32).contiguous() for t in rope_tables(s, c.window, self.th, self.tw, c.dim_head))
                      for s in range(c.window)}
        self._registers_ready = False

    # -------------------------------------------------------------------------------------
    def _tiles_of(self, latent: torch.Tensor) -> torch.Tensor:
        """latent [C, h, w] -> [my tiles, th*tw, C]"""
        parts = []
        for i in self.my_tiles:
            y, x = self.plan[i]
            parts.append(latent[:, y:y + self.th, x:x + self.tw].permute(1, 2, 0).reshape(self.th * self.tw, -1))
        return torch.stack(parts)

    def _fill_registers(self) -> None:
        c, m = self.cfg, self.m
        n = len(self.my_tiles)
        x = m.registers.unsqueeze(0).expand(n, -1, -1)
        self._reg_x = []
        for li, blk in enumerate(m.blocks):
            self._reg_x.append(x)
            q = m.block_q_cached(blk, x, None, None, self.k[li], self.v[li], 0)
            x = m.block_finish(blk, x, m.attend(q, self.k[li][:, :c.registers], self.v[li][:, :c.registers]))
        self._registers_ready = True

    def _run_slot(self, latent: torch.Tensor, slot: int, emit: bool):
        """One latent through all blocks at ``slot``; writes its keys / values; returns token states."""
        c, m = self.cfg, self.m
        hw = self.th * self.tw
        tok = self._tiles_of(latent.to(m.dtype))
        n = tok.shape[0]
        x = F_.linear(tok.reshape(n * hw, -1), m.embed).view(n, hw, -1)
        cos, sin = self._rope[slot]
        lo = c.registers + slot * hw
        for li, blk in enumerate(m.blocks):
            q = m.block_q_cached(blk, x, cos, sin, self.k[li], self.v[li], lo)
            o = m.attend(q, self.k[li][:, :lo + hw], self.v[li][:, :lo + hw])
            x = m.block_finish(blk, x, o)
        return x if emit else None

    @torch.no_grad()
    def push(self, latent: torch.Tensor) -> Optional[torch.Tensor]:
        """latent [C, h, w] (the next latent of the stream).  Returns its frames [3, F, H, W] on rank 0
        (F = 1 for a latent that opens a group of ``stride``, else ``frames_per_latent``); other ranks get None."""
        c = self.cfg
        if not self.my_tiles:
            i = self.count
            self.count += 1
            if self.m.embed.is_cuda and self.m.dtype == torch.bfloat16 and len(self.plan) <= 32:
                n_f = 1 if i % c.stride == 0 else c.frames_per_latent      # join the device gather with no tiles
                self._gather_device(torch.zeros(0, 3, n_f, self.th * c.patch, self.tw * c.patch, dtype=self.m.dtype,
                                                device=self.m.embed.device))
                return None
            return self._gather(None)
        if not self._registers_ready:
            self._fill_registers()
        i = self.count
        # windows start at multiples of ``stride`` and span ``window`` slots; the first window takes latents
        # 0 .. window-1, afterwards a new window begins with its (window - stride + 1)-th latent
        shared = c.window - c.stride
        start = ((i - shared) // c.stride) * c.stride if i >= c.window else 0
        slot = i - start
        if start > 0 and slot == shared:
            # the window moved: refill slots 0 .. shared-1 with the latents shared with the previous window
            for s, old in enumerate(self.recent[-shared:]):
                self._run_slot(old, s, emit=False)
        x = self._run_slot(latent, slot, emit=True)
        self.recent = (self.recent + [latent.clone()])[-(c.window - c.stride):]
        frames = self.m.to_pixels(x, self.th, self.tw)                      # [tiles, 3, F, th*p, tw*p]
        first_of_group = i % c.stride == 0
        if first_of_group:
            frames = frames[:, :, -1:]
        self.count += 1
        if frames is not None and frames.is_cuda and frames.dtype == torch.bfloat16 and len(self.plan) <= 32:
            # one pass over the pixels: ramp-weighted tile mean and the compensation polynomial together
            tiles = frames if self.world == 1 else self._gather_device(frames)
            if tiles is None:
                return None
            coef = None if self.table is None else self.table.coefficients(slot, frames.shape[2], first_of_stream=(i == 0))
            order = [t for r in range(self.world) for t in range(len(self.plan)) if t % self.world == r]
            offs = [(self.plan[t][0] * c.patch, self.plan[t][1] * c.patch) for t in order]
            return F_.tile_blend(tiles, offs, self.h * c.patch, self.w * c.patch, self.overlap * c.patch, coef)
        out = self._gather(frames)
        if out is None:
            return None
        if self.table is not None:
            out = self.table.apply(out, slot, first_of_stream=(i == 0))
        return out

    def _gather_device(self, frames: torch.Tensor) -> Optional[torch.Tensor]:
        """Tiles of every rank -> rank 0, on the device (one gather collective): [all tiles in rank-major order,
        3, F, th*p, tw*p] on rank 0, None elsewhere.  Ranks own ceil or floor of tiles / world; all send the
        padded count."""
        import torch.distributed as dist

        per = -(-len(self.plan) // self.world)
        send = frames.contiguous()
        if send.shape[0] < per:
            send = torch.cat([send, send.new_zeros(per - send.shape[0], *send.shape[1:])])
        bufs = [torch.empty_like(send) for _ in range(self.world)] if self.rank == 0 else None
        dist.gather(send, bufs, dst=dist.get_global_rank(self.group, 0) if self.group is not None else 0, group=self.group)
        if self.rank != 0:
            return None
        counts = [len([t for t in range(len(self.plan)) if t % self.world == r]) for r in range(self.world)]
        return torch.cat([b[:n] for b, n in zip(bufs, counts)])

    def _gather(self, frames: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        c = self.cfg
        if self.world == 1:
            tiles = [frames[j] for j in range(frames.shape[0])]
            return blend_tiles(tiles, self.plan, self.h, self.w, self.tile, self.overlap, c.patch) if len(self.plan) > 1 \
                else frames[0].float()
        import torch.distributed as dist

        gathered = [None] * self.world if self.rank == 0 else None
        dist.gather_object(None if frames is None else frames.cpu(), gathered, dst=0, group=self.group)
        if self.rank != 0:
            return None
        tiles: List[Optional[torch.Tensor]] = [None] * len(self.plan)
        for r, fr in enumerate(gathered):
            owned = [i for i in range(len(self.plan)) if i % self.world == r]
            for j, i in enumerate(owned):
                tiles[i] = fr[j]
        return blend_tiles(tiles, self.plan, self.h, self.w, self.tile, self.overlap, c.patch)


class TensorParallelViT:
    """Head / FFN-column tensor parallelism of ``ViTVideoDecoder`` blocks over a process group.

    Rank r keeps heads ``[r H/P, (r+1) H/P)`` of the fused q|k|v projection with the matching input columns
    of the output projection, and FFN columns ``[r F/P, (r+1) F/P)`` of gate / up with the matching input
    columns of the down projection.  The two row-parallel products give partial sums that are formed in
    fp32, summed with one all-reduce each, and only then rounded to the activation dtype -- the same
    rounding point as the unsharded product (reference: deploy/solar_wm/shared/vae/streamrender_tp.py:63-113).
    Every rank holds all tokens; keys / values are cached per rank for its own heads only.
    """

    def __init__(self, model: ViTVideoDecoder, group=None):
        import torch.distributed as dist

        self.m, self.cfg, self.group = model, model.cfg, group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        c = self.cfg
        if c.heads % self.world or c.ffn_dim % self.world:
            raise ValueError("heads and ffn_dim must be divisible by the tensor-parallel size")
        self.hl, self.fl = c.heads // self.world, c.ffn_dim // self.world
        a, al = c.heads * c.dim_head, self.hl * c.dim_head
        r = self.rank
        self.shards = []
        for blk in model.blocks:
            qkv = torch.cat([blk.qkv[i * a + r * al:i * a + (r + 1) * al] for i in range(3)]).contiguous()
            gate_up = torch.cat([blk.gate_up[r * self.fl:(r + 1) * self.fl],
                                 blk.gate_up[c.ffn_dim + r * self.fl:c.ffn_dim + (r + 1) * self.fl]]).contiguous()
            self.shards.append({"qkv": qkv, "out": blk.out[:, r * al:(r + 1) * al].contiguous(), "gate_up": gate_up,
                                "down": blk.down[:, r * self.fl:(r + 1) * self.fl].contiguous()})

    def _row_parallel(self, x, w):
        import torch.distributed as dist

        part = x.float() @ w.float().t()                          # fp32 partial sum of this rank's input columns
        dist.all_reduce(part, group=self.group)
        return part.to(x.dtype)

    def block(self, li: int, x, cos, sin, k_cache=None, v_cache=None, lo: int = 0):
        """x [B, N, dim] -> [B, N, dim].  With caches ([B, rows, hl*dh]) the new keys / values are written at
        ``[lo, lo+N)`` and attention reads ``[0, lo+N)``."""
        c, blk, sh = self.cfg, self.m.blocks[li], self.shards[li]
        B, N, _ = x.shape
        al = self.hl * c.dim_head
        xm = F_.norm_modulate(x.reshape(B * N, -1), mode=1, w=blk.norm1, eps=c.eps)
        qkv = F_.linear(xm, sh["qkv"]).view(B, N, 3 * al)
        q = _head_rms(qkv[..., :al], blk.q_norm, self.hl, c.eps)
        k = _head_rms(qkv[..., al:2 * al], blk.k_norm, self.hl, c.eps)
        v = qkv[..., 2 * al:]
        if cos is not None:
            q, k = apply_rope(q, cos, sin, self.hl), apply_rope(k, cos, sin, self.hl)
        if k_cache is not None:
            k_cache[:, lo:lo + N], v_cache[:, lo:lo + N] = k, v
            k, v = k_cache[:, :lo + N], v_cache[:, :lo + N]
        Nk = k.shape[1]
        o = ops.attention(q.reshape(B, N, self.hl, c.dim_head), k.reshape(B, Nk, self.hl, c.dim_head),
                          v.reshape(B, Nk, self.hl, c.dim_head)).reshape(B * N, al)
        x2 = F_.gated_residual(x.reshape(B * N, -1), self._row_parallel(o, sh["out"]), None)
        xm = F_.norm_modulate(x2, mode=1, w=blk.norm2, eps=c.eps)
        y = self._row_parallel(F_.swiglu(F_.linear(xm, sh["gate_up"])), sh["down"])
        return F_.gated_residual(x2, y, None).view(B, N, -1)
