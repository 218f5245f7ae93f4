"""MiniMax-H3-shaped DiT: one packed heterogeneous token document, per-row adaLN tables, per-head
q/k RMSNorm + MM-RoPE + camera PRoPE, SwiGLU FFN, LoRA adapters on a frozen bf16 base.

The H3 architecture itself is external to the reference (it subclasses a diffusers model); the
dimensions used here are the ones recoverable from it (hidden 5376, head_dim 128, 56 heads ->
attention width 7168, FFN 14336, 50 blocks + 2 text-refiner blocks, text width 5120, 24-channel
latents patched 1x2x2 -> 96-wide rows, 32-wide audio rows; solar/backends/minimax_h3/model.py:
346-879, lora.py:55-71, stage0p5.py:72-76) and are all configurable.

Packed document  [text | anchor | observations | audio | video]  as ONE ``[S, hidden]`` matrix:
  * every row carries a modality tag (0 video, 1 text, 2 audio) and a timestep index; the adaLN
    vectors of a row are looked up as ``table[t_idx * 3 + tag]`` (K1/K2 of the reference's Triton set,
    here ``ops.norm_modulate(table=...)`` / ``ops.gated_residual(table=...)``)
  * position ids ``[S, 3]`` (t, h, w) feed the MM-RoPE tables; rows with a camera carry a 4x4
    projection on head channels [96, 128): ``P^T`` for queries, ``P^-1`` for keys and values, ``P`` for
    the attention output (``ops.head_norm_rope_prope``)
  * attention is plain bidirectional attention over the document (segment plans of block-causal
    variants come from ``models.wan_causal.teacher_forcing_attention``-style chunk loops)

LoRA: ``y = x W^T + (x A^T) B^T``; the low-rank product is accumulated into the base GEMM's output
by the GEMM epilogue's reduce-add store (``accumulate=True``), so no extra pass over ``y``
(reference: torch.addmm epilogue, solar/backends/minimax_h3/lora.py:402-471).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from ..ops import functional as F_

TAG_VIDEO, TAG_TEXT, TAG_AUDIO = 0, 1, 2


@dataclass
class H3Config:
    hidden_size: int = 5376
    num_attention_heads: int = 56
    attention_head_dim: int = 128
    num_layers: int = 50
    num_refiner_layers: int = 2
    ffn_dim: int = 14336
    text_dim: int = 5120
    latent_row_dim: int = 96          # 24 channels x (1,2,2) patch
    audio_row_dim: int = 32
    time_embed_hidden_dim: int = 256
    time_embed_dim: int = 1024
    rot_dims: int = 96
    rope_sections: int = 2
    lora_rank: int = 0                # 0 = no adapters
    eps: float = 1e-5

    @property
    def attn_dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim


def h3_preset(name: str) -> H3Config:
    if name in ("h3_33b", "minimax_h3"):
        return H3Config()
    if name == "tiny":
        return H3Config(hidden_size=256, num_attention_heads=2, num_layers=2, num_refiner_layers=1, ffn_dim=512,
                        text_dim=64, time_embed_hidden_dim=32, time_embed_dim=64)
    raise KeyError(name)


class _LoRAFn(torch.autograd.Function):
    """y = x W^T + (x A^T) B^T with frozen W; gradients for x, A and B."""

    @staticmethod
    def forward(ctx, x, w, a, b):
        y = F_.gemm(x, w, F_.NT)
        t = F_.gemm(x, a, F_.NT)
        F_.gemm(t, b, F_.NT, out=y, accumulate=True)
        ctx.save_for_backward(x, w, a, b, t)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, a, b, t = ctx.saved_tensors
        dy = F_._rowmajor(dy)
        dt = F_.gemm(dy, b, F_.NN)                      # [M, r]
        dx = F_.gemm(dy, w, F_.NN)
        F_.gemm(dt, a, F_.NN, out=dx, accumulate=True)
        da = F_.gemm(dt, x, F_.TN, out_dtype=a.dtype)
        db = F_.gemm(dy, t, F_.TN, out_dtype=b.dtype)
        return dx, None, da, db


class LoRALinear(nn.Module):
    def __init__(self, d_in, d_out, rank, device, dtype, gen):
        super().__init__()
        bound = math.sqrt(6.0 / (d_in + d_out))
        self.weight = nn.Parameter(((torch.rand(d_out, d_in, generator=gen, device=gen.device) * 2 - 1) * bound).to(device, dtype),
                                   requires_grad=rank == 0)
        self.rank = rank
        if rank > 0:
            self.lora_A = nn.Parameter((torch.randn(rank, d_in, generator=gen, device=gen.device) / math.sqrt(d_in)).to(device, dtype))
            self.lora_B = nn.Parameter(torch.zeros(d_out, rank, device=device, dtype=dtype))

        self._bank = None          # name of the active extra adapter bank (None: the primary lora_A / lora_B)

    def add_bank(self, name: str, rank: int, gen) -> None:
        """A second, independently trained adapter over the same frozen weight (e.g. the Memory adapter)."""
        d_out, d_in = self.weight.shape
        dev, dt = self.weight.device, self.weight.dtype
        setattr(self, f"lora_A__{name}", nn.Parameter((torch.randn(rank, d_in, generator=gen, device=gen.device) / math.sqrt(d_in)).to(dev, dt)))
        setattr(self, f"lora_B__{name}", nn.Parameter(torch.zeros(d_out, rank, device=dev, dtype=dt)))

    def use_bank(self, name) -> None:
        if name is not None and not hasattr(self, f"lora_A__{name}"):
            raise KeyError(f"no adapter bank {name!r}")
        self._bank = name

    def _adapter(self):
        if self._bank is not None:
            return getattr(self, f"lora_A__{self._bank}"), getattr(self, f"lora_B__{self._bank}")
        return (self.lora_A, self.lora_B) if self.rank > 0 else (None, None)

    def forward(self, x):
        a, b = self._adapter()
        if a is None:
            return F_.linear(x, self.weight)
        if not x.is_cuda:
            return (x.float() @ self.weight.float().t() + (x.float() @ a.float().t()) @ b.float().t()).to(x.dtype)
        a, b = F_.pad_adapter_rank(a, b)
        return _LoRAFn.apply(x, self.weight, a, b)

    @torch.no_grad()
    def merge_(self):
        """Fold the adapter into the base weight (released-weight merge)."""
        if self.rank > 0:
            self.weight.add_((self.lora_B.float() @ self.lora_A.float()).to(self.weight.dtype))
            self.lora_B.zero_()


class H3Block(nn.Module):
    def __init__(self, cfg: H3Config, device, dtype, gen, modulated=True):
        super().__init__()
        self.cfg, self.modulated = cfg, modulated
        h, a, f, r = cfg.hidden_size, cfg.attn_dim, cfg.ffn_dim, cfg.lora_rank
        mk = lambda i, o: LoRALinear(i, o, r, device, dtype, gen)
        self.to_q, self.to_k, self.to_v, self.to_out = mk(h, a), mk(h, a), mk(h, a), mk(a, h)
        self.ffn_gate_up, self.ffn_down = mk(h, 2 * f), mk(f, h)
        self.norm1 = nn.Parameter(torch.ones(h, device=device), requires_grad=False)
        self.norm2 = nn.Parameter(torch.ones(h, device=device), requires_grad=False)
        self.norm_q = nn.Parameter(torch.ones(cfg.attention_head_dim, device=device), requires_grad=False)
        self.norm_k = nn.Parameter(torch.ones(cfg.attention_head_dim, device=device), requires_grad=False)
        if modulated:
            self.adaln_proj = nn.Parameter((torch.randn(3 * 6 * h, cfg.time_embed_dim, generator=gen, device=gen.device) * 0.02).to(device, dtype),
                                           requires_grad=False)

    def tables(self, temb):
        """temb [T, time_embed_dim] -> adaLN table fp32 [T*3, 6, hidden] (row = t_idx*3 + tag)."""
        t = F_.linear(torch.nn.functional.silu(temb.float()).to(temb.dtype), self.adaln_proj)
        return t.float().view(-1, 6, self.cfg.hidden_size).contiguous()

    def forward(self, x, table, idx, rope_cos, rope_sin, cam_q, cam_kv, cam_o, sp=None, attn_fn=None, memo=None):
        cfg = self.cfg
        H, hd = cfg.num_attention_heads, cfg.attention_head_dim
        kw = dict(rot_dims=cfg.rot_dims, sections=cfg.rope_sections, eps=cfg.eps)
        if self.modulated:
            xm = F_.norm_modulate(x, table[:, 0], table[:, 1], mode=1, w=self.norm1, eps=cfg.eps, table=idx)
        else:
            xm = F_.norm_modulate(x, mode=1, w=self.norm1, eps=cfg.eps)
        q = ops.head_norm_rope_prope(self.to_q(xm), self.norm_q, rope_cos, rope_sin, cam_q, heads=H, **kw)
        k = ops.head_norm_rope_prope(self.to_k(xm), self.norm_k, rope_cos, rope_sin, cam_kv, heads=H, **kw)
        v = self.to_v(xm)
        if cam_kv is not None:
            v = ops.head_norm_rope_prope(v, None, None, None, cam_kv, heads=H, **kw)
        S = x.shape[0]
        q, k, v = (t.view(1, S, H, hd) for t in (q, k, v))
        if sp is not None and sp.size > 1:
            q, k, v = sp.scatter_heads(q, k, v)
        o = attn_fn(q, k, v) if attn_fn is not None else ops.attention(q, k, v, memo=None if memo is None else (memo, "self"))
        if sp is not None and sp.size > 1:
            o = sp.gather_heads(o)
        o = o.reshape(S, H * hd)
        if cam_o is not None:
            o = ops.head_norm_rope_prope(o, None, None, None, cam_o, heads=H, **kw)
        y = self.to_out(o)
        x = F_.gated_residual(x, y, table[:, 2], table=idx) if self.modulated else F_.gated_residual(x, y, None)
        if self.modulated:
            xm = F_.norm_modulate(x, table[:, 3], table[:, 4], mode=1, w=self.norm2, eps=cfg.eps, table=idx)
        else:
            xm = F_.norm_modulate(x, mode=1, w=self.norm2, eps=cfg.eps)
        y = self.ffn_down(F_.swiglu(self.ffn_gate_up(xm)))
        return F_.gated_residual(x, y, table[:, 5], table=idx) if self.modulated else F_.gated_residual(x, y, None)


def mm_rope_tables(position_ids: torch.Tensor, rot_dims: int = 96, sections: int = 2, theta: float = 10000.0):
    """position_ids [S, 3] (t, h, w; float64) -> (cos, sin) fp32 [S, rot_dims] in rotate-half layout:
    each section holds its frequencies twice (first half | second half).  The rot_dims/2 frequency
    slots are dealt to the three axes in equal thirds."""
    S = position_ids.shape[0]
    pairs = rot_dims // 2
    per_axis = pairs // 3
    pos = position_ids.to(torch.float64)
    ang = []
    for axis in range(3):
        n = per_axis if axis < 2 else pairs - 2 * per_axis
        inv = 1.0 / torch.pow(theta, torch.arange(n, dtype=torch.float64, device=pos.device) / n)
        ang.append(pos[:, axis:axis + 1] * inv)
    ang = torch.cat(ang, dim=1)                                     # [S, pairs]
    per_sec = pairs // sections
    blocks = [torch.cat([ang[:, s * per_sec:(s + 1) * per_sec]] * 2, dim=1) for s in range(sections)]
    full = torch.cat(blocks, dim=1)
    return torch.cos(full).float().contiguous(), torch.sin(full).float().contiguous()


def prope_row_matrices(viewmats: torch.Tensor, fx: float, fy: float):
    """viewmats [S, 4, 4] (identity for rows without a camera) -> (P^T for q, P^-1 for k/v, P for the output),
    each fp32 [S, 4, 4], with P = diag(fx, fy, 1, 1) @ view."""
    v = viewmats.to(torch.float64)
    lift = torch.diag(torch.tensor([fx, fy, 1.0, 1.0], dtype=torch.float64, device=v.device))
    P = lift @ v
    Pinv = torch.linalg.inv(P)
    f = lambda m: m.float().contiguous()
    return f(P.transpose(-1, -2)), f(Pinv), f(P)


class H3DiT(nn.Module):
    def __init__(self, cfg: H3Config, device="cpu", dtype=torch.bfloat16, seed: int = 0):
        super().__init__()
        self.cfg, self.dtype = cfg, dtype
        g = torch.Generator(device=device).manual_seed(seed)   # weights are drawn on the target device
        h = cfg.hidden_size
        lin = lambda i, o, s=None: nn.Parameter((torch.randn(o, i, generator=g, device=g.device) * (s or 1.0 / math.sqrt(i))).to(device, dtype),
                                                requires_grad=False)
        self.proj_in, self.audio_proj_in = lin(cfg.latent_row_dim, h), lin(cfg.audio_row_dim, h)
        self.context_embedder = lin(cfg.text_dim, h)
        self.time_in, self.time_out = lin(cfg.time_embed_hidden_dim, cfg.time_embed_dim), lin(cfg.time_embed_dim, cfg.time_embed_dim)
        self.refiner = nn.ModuleList([H3Block(cfg, device, dtype, g, modulated=False) for _ in range(cfg.num_refiner_layers)])
        self.blocks = nn.ModuleList([H3Block(cfg, device, dtype, g) for _ in range(cfg.num_layers)])
        self.norm_out = nn.Parameter(torch.ones(h, device=device), requires_grad=False)
        self.proj_out, self.audio_proj_out = lin(h, cfg.latent_row_dim, 0.02), lin(h, cfg.audio_row_dim, 0.02)
        self.sp = None
        # training under sequence parallelism: ``forward`` keeps this rank's balanced share of the packed rows through
        # the blocks (attention exchanges heads for rows) and returns the predictions of ITS rows only;
        # ``local_video_rows`` / ``local_audio_rows`` then give their ranges in video / audio row coordinates.  The
        # streaming generator shards its rows itself and leaves this off.
        self.shard_rows = False
        self.local_video_rows = self.local_audio_rows = None
        # inference-only caches installed by renderer.service (None = off)
        # activation checkpointing of the main blocks: "none" | "full" (recompute the block in backward) |
        # "selective" (recompute everything but the attention call, whose output is carried across the recompute;
        # reference policy: solar/backends/minimax_h3/fsdp.py:146-165)
        self.checkpointing = "none"
        self.fixed_tables = None        # {tuple of unique timesteps: [per-block adaLN tables]}
        self.text_cache = None          # {"input": rows, "output": refined rows, "hits": n}

    def trainable_parameters(self):
        return [p for p in self.parameters() if p.requires_grad]

    @torch.no_grad()
    def fuse_qkv_(self) -> int:
        """Inference: make the q, k and v projection weights of every adapter-free block views of ONE ``[3 A, hidden]``
        buffer (``block.qkv_weight``), so that a caller can run the three projections as one GEMM.  At a few hundred
        rows per rank one projection is 84 CTA-pair tiles on 74 pairs -- two waves for 1.13 -- and the fused one is
        252 tiles in four waves instead of six.  No memory is added (the parameters move into the buffer); the
        per-projection modules keep working.  Returns the number of blocks fused."""
        done = 0
        for blk in list(self.refiner) + list(self.blocks):
            mods = (blk.to_q, blk.to_k, blk.to_v)
            if getattr(blk, "qkv_weight", None) is not None or any(m.rank > 0 or m._bank is not None for m in mods):
                continue
            a = mods[0].weight.shape[0]
            fused = torch.cat([m.weight.data for m in mods], dim=0)
            for i, m in enumerate(mods):
                m.weight.data = fused[i * a:(i + 1) * a]
            blk.qkv_weight = fused
            done += 1
        return done

    # named adapter banks: independent LoRA sets over the same frozen base, one active at a time ----------
    def add_adapter(self, name: str, rank: int, seed: int = 0) -> None:
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for mod in self.modules():
            if isinstance(mod, LoRALinear):
                mod.add_bank(name, rank, gen)

    def set_adapter(self, name) -> None:
        """``None`` selects the primary adapter (or the bare base when ``lora_rank`` is 0)."""
        for mod in self.modules():
            if isinstance(mod, LoRALinear):
                mod.use_bank(name)
        self.active_adapter = name

    def adapter_state(self, name: str) -> dict:
        tag = f"__{name}"
        return {k: v.detach().clone() for k, v in self.state_dict().items() if k.endswith(tag)}

    def time_embed(self, timesteps):
        """unique timesteps [T] in [0, 1] -> [T, time_embed_dim]"""
        from .wan import sinusoidal_embedding

        e = sinusoidal_embedding(self.cfg.time_embed_hidden_dim, timesteps * 1000.0).to(self.dtype)
        e = F_.linear(e, self.time_in)
        return F_.linear(torch.nn.functional.silu(e.float()).to(self.dtype), self.time_out)

    def forward(self, *, video_rows, text_rows, audio_rows=None, anchor_rows=None, timesteps, t_index, tags,
                position_ids, viewmats=None, fx=0.505, fy=0.898, attn_fn=None):
        """Rows are packed in the order [text | anchor | audio | video]; ``t_index`` / ``tags`` /
        ``position_ids`` / ``viewmats`` are per packed row.  Returns (video prediction [Nv, 96],
        audio prediction [Na, 32] or None)."""
        cfg = self.cfg
        dt = self.dtype
        parts, n_text = [], text_rows.shape[0]
        cos, sin = mm_rope_tables(position_ids.to(self.proj_in.device), cfg.rot_dims, cfg.rope_sections)
        tc = self.text_cache if not torch.is_grad_enabled() else None
        if tc is not None and tc.get("input") is not None and tc["input"].shape == text_rows.shape \
                and torch.equal(tc["input"], text_rows):
            txt = tc["output"]
            tc["hits"] = tc.get("hits", 0) + 1
        else:
            txt = F_.linear(text_rows.to(dt), self.context_embedder)
            for blk in self.refiner:       # text-only refiner blocks (no modulation, no camera)
                txt = blk(txt, None, None, cos[:n_text].contiguous(), sin[:n_text].contiguous(), None, None, None)
            if tc is not None:
                tc["input"], tc["output"] = text_rows.detach().clone(), txt
        parts.append(txt)
        if anchor_rows is not None:
            parts.append(F_.linear(anchor_rows.to(dt), self.proj_in))
        n_audio = 0
        if audio_rows is not None:
            n_audio = audio_rows.shape[0]
            parts.append(F_.linear(audio_rows.to(dt), self.audio_proj_in))
        n_video = video_rows.shape[0]
        parts.append(F_.linear(video_rows.to(dt), self.proj_in))
        x = torch.cat(parts, dim=0)
        S = x.shape[0]
        assert t_index.shape[0] == S and tags.shape[0] == S and position_ids.shape[0] == S
        idx = (t_index.to(torch.int32) * 3 + tags.to(torch.int32)).contiguous()
        tables = None
        if self.fixed_tables is not None and not torch.is_grad_enabled():
            key = tuple(round(float(t), 6) for t in timesteps.float().cpu().tolist())
            if key not in self.fixed_tables:
                raise ValueError(f"timestep set {key} was not prepared; refusing to use stale modulation tables")
            tables = self.fixed_tables[key]
        else:
            temb = self.time_embed(timesteps.to(x.device).float())
        cam_q = cam_kv = cam_o = None
        if viewmats is not None:
            cam_q, cam_kv, cam_o = prope_row_matrices(viewmats.to(x.device), fx, fy)
        lo, hi = 0, S
        if self.shard_rows and self.sp is not None and self.sp.size > 1:
            from ..parallel.ulysses import balanced_bounds, balanced_lengths

            if tables is not None:
                raise ValueError("fixed modulation tables are an inference cache; row-sharded training builds its own")
            self.sp.set_layout_rows(1, balanced_lengths(S, self.sp.size))
            lo, hi = balanced_bounds(S, self.sp.size, self.sp.rank)
            x, idx, cos, sin = x[lo:hi], idx[lo:hi].contiguous(), cos[lo:hi].contiguous(), sin[lo:hi].contiguous()
            if cam_q is not None:
                cam_q, cam_kv, cam_o = (m[lo:hi].contiguous() for m in (cam_q, cam_kv, cam_o))
        ckpt = self.checkpointing if torch.is_grad_enabled() else "none"
        for bi, blk in enumerate(self.blocks):
            if ckpt in ("full", "selective"):
                from torch.utils.checkpoint import checkpoint

                memo = {"__store__": True} if (ckpt == "selective" and x.is_cuda and attn_fn is None) else None
                x = checkpoint(lambda a, te, b=blk, mm=memo: b(a, b.tables(te), idx, cos, sin, cam_q, cam_kv, cam_o, sp=self.sp,
                                                              attn_fn=attn_fn, memo=mm), x, temb, use_reentrant=False)
                continue
            x = blk(x, tables[bi] if tables is not None else blk.tables(temb), idx, cos, sin, cam_q, cam_kv, cam_o,
                    sp=self.sp, attn_fn=attn_fn)
        xn = F_.norm_modulate(x, mode=1, w=self.norm_out, eps=cfg.eps)

        def part(first, last):                       # packed rows [first, last) that this rank holds
            a, b = min(max(first, lo), hi), min(max(last, lo), hi)
            return a - lo, b - lo, (a - first, b - first)

        va, vb, self.local_video_rows = part(S - n_video, S)
        vid = F_.linear(xn[va:vb], self.proj_out)
        aud = None
        if n_audio:
            aa, ab, self.local_audio_rows = part(S - n_video - n_audio, S - n_video)
            aud = F_.linear(xn[aa:ab], self.audio_proj_out)
        return vid, aud
