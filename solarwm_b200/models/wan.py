"""Wan2.2-style video DiT (TI2V-5B, I2V-A14B and tiny test shapes) on the fused sm_100a operators.

Architecture (same parameter names and shapes as the reference so checkpoints interchange;
reference: solar/backends/wan22/runtime/modeling/model.py:286-561 and
causal_model.py:1610-1710, 1734-1870, 2621-2854):

  patch embedding Conv3d(k = s = (1,2,2)) as a GEMM -> L tokens of width ``dim``
  time path: sinusoid(freq_dim) -> Linear/SiLU/Linear -> SiLU -> Linear(dim, 6*dim), per latent frame
  text path: Linear(text_dim, dim) -> GELU-tanh -> Linear(dim, dim), 512 tokens
  block:  x += gate_msa * SelfAttn(LN(x) * (1 + scale_msa) + shift_msa)      q/k: full-width RMSNorm, 3-axis RoPE
          x += CrossAttn(LN_affine(x), text)
          x += gate_mlp * FFN(LN(x) * (1 + scale_mlp) + shift_mlp)           FFN: Linear/GELU-tanh/Linear
  head:   Linear(LN(x) * (1 + scale) + shift) -> unpatchify

Execution model: activations are kept as one 2-D ``[B*L, dim]`` bf16 matrix; every projection is a
tcgen05 GEMM (QKV fused into one ``[3*dim, dim]`` GEMM through adjacent flat-buffer slots), every
norm/modulate/gate/rope step is a single row kernel, attention is the flash kernel.  Under
Ulysses sequence parallelism each rank holds whole latent frames; ``self.sp`` exchanges
heads<->sequence around the attention.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass
from typing import Optional, Sequence

import torch
import torch.nn as nn

from .. import ops
from ..ops import functional as F_
from ..parallel.flat import FlatUnit
from ..utils.trace import span


@dataclass
class WanConfig:
    model_type: str = "t2v"
    patch_size: tuple = (1, 2, 2)
    text_len: int = 512
    in_dim: int = 16
    dim: int = 2048
    ffn_dim: int = 8192
    freq_dim: int = 256
    text_dim: int = 4096
    out_dim: int = 16
    num_heads: int = 16
    num_layers: int = 32
    qk_norm: bool = True
    cross_attn_norm: bool = True
    eps: float = 1e-6
    local_attn_size: int = -1
    sink_size: int = 0
    num_frame_per_block: int = 3
    flow_objective: str = "flow_matching"   # or "anyflow_forward_map"
    anyflow_gate: float = 0.25
    # "none" / "fused_prope": cameras (when given) transform the heads of the block's own self-attention;
    # "parallel": every block owns a second, zero-initialised self-attention that sees positions only through the
    # cameras (reference: CausalPropeSelfAttention, runtime/modeling/causal_model.py:1238-1525)
    camera_attention_mode: str = "none"
    norm_type: str = "layer"                # "layer": LayerNorm without affine (Wan); "rms": RMSNorm (LTX)
    # per-head output gate of the self-attention: o_h <- o_h * 2 sigmoid(x_mod W_g^T + b_g)_h with W_g, b_g zero at
    # initialisation (gate 1), applied after the camera output transform and before the output projection
    # (reference: to_gate_logits / gated_attention_function, solar/backends/ltx25/torch_model.py:259-261, order
    # "native_head_gate_and_output_projection" in solar/backends/ltx25/adapter.py:14-20)
    gated_attention: bool = False

    @property
    def head_dim(self) -> int:
        return self.dim // self.num_heads

    def to_dict(self):
        return asdict(self)


def wan_preset(name: str) -> WanConfig:
    """Named architectures (reference: runtime/architectures/{ti2v_5b,i2v_a14b}.json)."""
    if name in ("ti2v_5b", "wan22_ti2v_5b"):
        return WanConfig(model_type="ti2v", in_dim=48, out_dim=48, dim=3072, ffn_dim=14336, num_heads=24,
                         num_layers=30, local_attn_size=12, sink_size=3)
    if name in ("i2v_a14b", "wan22_i2v_a14b"):
        return WanConfig(model_type="i2v", in_dim=36, out_dim=16, dim=5120, ffn_dim=13824, num_heads=40,
                         num_layers=40, local_attn_size=21, sink_size=0)
    if name in ("ltx_video_2b", "ltx25_video"):
        # LTX-Video-2B-shaped: 28 blocks, dim 2048, 32 heads x 64, 128-channel latents, patch 1, RMSNorm
        return WanConfig(model_type="t2v", patch_size=(1, 1, 1), in_dim=128, out_dim=128, dim=2048, ffn_dim=8192,
                         num_heads=32, num_layers=28, text_dim=4096, text_len=128, norm_type="rms", cross_attn_norm=False)
    if name in ("ltx25_video_13b", "ltx25_13b"):
        # the released LTX-2.5 video core: 48 blocks, 32 heads x 128, 128-channel latents, 1024 caption tokens of
        # width 4096, per-head attention gates (reference layout check: solar/backends/ltx25/checkpoint.py:308-322)
        return WanConfig(model_type="t2v", patch_size=(1, 1, 1), in_dim=128, out_dim=128, dim=4096, ffn_dim=16384,
                         num_heads=32, num_layers=48, text_dim=4096, text_len=1024, norm_type="rms", cross_attn_norm=False,
                         gated_attention=True)
    if name == "tiny":
        return WanConfig(model_type="t2v", in_dim=16, out_dim=16, dim=128, ffn_dim=512, num_heads=4,
                         num_layers=2, text_dim=256, text_len=32, freq_dim=64)
    raise KeyError(name)


# --------------------------------------------------------------------------------------------
# position / time tables
# --------------------------------------------------------------------------------------------
def rope_axis_dims(head_dim: int):
    c = head_dim // 2
    return c - 2 * (c // 3), c // 3, c // 3


def rope_table(grid: Sequence[int], head_dim: int, device, frame_offset: int = 0, theta: float = 10000.0,
               frame_positions: Optional[torch.Tensor] = None):
    """(cos, sin) per token for the 3-axis RoPE: ``[F*H*W, head_dim/2, 2]`` fp32, angles in fp64.

    The complex pairs of a head are split ``[c - 2(c//3), c//3, c//3]`` over (frame, row, column);
    each axis uses ``theta^(-2i/d_axis)`` with ``d_axis`` twice the number of pairs of that axis.
    ``frame_positions`` overrides the frame coordinate (rolling-window / block-relative positions).
    """
    f, h, w = (int(v) for v in grid)
    cf, ch, cw = rope_axis_dims(head_dim)

    def axis(n_pairs, pos):
        d = 2 * n_pairs
        inv = 1.0 / torch.pow(theta, torch.arange(0, d, 2, dtype=torch.float64) / d)
        return torch.outer(pos.to(torch.float64), inv)

    fpos = torch.arange(f, dtype=torch.float64) + frame_offset if frame_positions is None \
        else frame_positions.to(torch.float64).cpu()
    af = axis(cf, fpos).view(f, 1, 1, cf).expand(f, h, w, cf)
    ah = axis(ch, torch.arange(h)).view(1, h, 1, ch).expand(f, h, w, ch)
    aw = axis(cw, torch.arange(w)).view(1, 1, w, cw).expand(f, h, w, cw)
    ang = torch.cat([af, ah, aw], dim=-1).reshape(f * h * w, cf + ch + cw)
    return torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).to(device).contiguous()


def sinusoidal_embedding(dim: int, position: torch.Tensor) -> torch.Tensor:
    """[N] -> [N, dim] (cos | sin), evaluated in fp64 like the reference (model.py:16-25)."""
    half = dim // 2
    pos = position.to(torch.float64)
    freqs = torch.pow(10000.0, -torch.arange(half, dtype=torch.float64, device=pos.device) / half)
    s = torch.outer(pos, freqs)
    return torch.cat([torch.cos(s), torch.sin(s)], dim=1)


def _identity_attention(q, k, v):
    """Skipped attention: the output of a token is its own value."""
    return v


class _UnitReady(torch.autograd.Function):
    """Identity placed at a block's input.  Its backward runs when the gradient of the block input is complete,
    i.e. after every node of the block (it is the block's oldest node and the engine runs newer ready nodes first),
    and tells ``hook`` that the block's parameter gradients are final -- the sharded optimizer starts the block's
    reduce-scatter there, under the backward of the blocks below."""

    @staticmethod
    def forward(ctx, x, hook, unit):
        ctx.hook, ctx.unit = hook, unit
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.hook(ctx.unit)
        return g, None, None


class _BlockGate(torch.autograd.Function):
    """Identity on a block's OUTPUT: its backward runs before any node of the block and asks the parameter provider
    to make the block's (sharded) weights resident again and to clear its gradient slot for writing."""

    @staticmethod
    def forward(ctx, x, provider, index):
        ctx.provider, ctx.index = provider, index
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.provider.acquire(ctx.index, backward=True)
        return g, None, None


class _NoSP:
    size = 1
    rank = 0

    def scatter_heads(self, q, k, v):
        return q, k, v

    def gather_heads(self, o):
        return o


# --------------------------------------------------------------------------------------------
# modules
# --------------------------------------------------------------------------------------------
class _Named(nn.Module):
    """Container that only holds parameters under reference-compatible names."""


def _register(module: nn.Module, dotted: str, p: nn.Parameter) -> None:
    parts = dotted.split(".")
    for name in parts[:-1]:
        if not hasattr(module, name):
            module.add_module(name, _Named())
        module = getattr(module, name)
    module.register_parameter(parts[-1], p)


def _block_specs(cfg: WanConfig):
    d, f = cfg.dim, cfg.ffn_dim
    specs = []
    for attn in ("self_attn", "cross_attn"):
        for n in ("q", "k", "v"):
            specs.append((f"{attn}.{n}.weight", (d, d), False))
        for n in ("q", "k", "v"):
            specs.append((f"{attn}.{n}.bias", (d,), False))
        specs.append((f"{attn}.o.weight", (d, d), False))
        specs.append((f"{attn}.o.bias", (d,), False))
        specs.append((f"{attn}.norm_q.weight", (d,), True))
        specs.append((f"{attn}.norm_k.weight", (d,), True))
    specs += [("ffn.0.weight", (f, d), False), ("ffn.0.bias", (f,), False),
              ("ffn.2.weight", (d, f), False), ("ffn.2.bias", (d,), False),
              ("modulation", (1, 6, d), True)]
    if cfg.cross_attn_norm:
        specs += [("norm3.weight", (d,), True), ("norm3.bias", (d,), True)]
    if cfg.gated_attention:
        specs += [("self_attn.to_gate_logits.weight", (cfg.num_heads, d), False),
                  ("self_attn.to_gate_logits.bias", (cfg.num_heads,), False)]
    if cfg.camera_attention_mode == "parallel":
        pre = "cam_self_attn"
        specs += [(f"{pre}.{n}_proj.weight", (d, d), False) for n in ("q", "k", "v")]
        specs += [(f"{pre}.{n}_proj.bias", (d,), False) for n in ("q", "k", "v")]
        specs += [(f"{pre}.out_proj.weight", (d, d), False), (f"{pre}.out_proj.bias", (d,), False),
                  (f"{pre}.norm_q.weight", (d,), True), (f"{pre}.norm_k.weight", (d,), True)]
    return specs


# adjacent projection slots that one GEMM serves, by the name of the first
_SPAN_NAMES = {"q": ("q", "k", "v"), "k": ("k", "v"), "q_proj": ("q_proj", "k_proj", "v_proj")}


class WanBlock(nn.Module):
    def __init__(self, cfg: WanConfig, device, dtype, shard_pad: int = 1):
        super().__init__()
        self.cfg = cfg
        self.unit = FlatUnit(_block_specs(cfg), device, dtype, pad_to=shard_pad)
        for name in self.unit.slots:
            _register(self, name, self.unit.parameter(name))
        self.lora = None            # ModuleDict of low-rank adapters once ``models.lora.inject_lora`` ran

    def _adapter(self, wname: str):
        if not self.lora:
            return None
        key = wname[:-len(".weight")].replace(".", "__")
        return self.lora[key] if key in self.lora else None

    # parameters through the unit (fused views where slots are adjacent) ------------------
    def _p(self, name):
        return self.unit.params[name]

    def _use_main_grad(self) -> bool:
        return self.unit.grad is not None and torch.is_grad_enabled()

    def _norm_kw(self, x):
        """Pre-modulation norm: LayerNorm without affine (Wan) or weight-free RMSNorm (LTX)."""
        if self.cfg.norm_type == "layer":
            return {"mode": 0}
        ones = getattr(self, "_ones", None)
        if ones is None or ones.device != x.device:
            ones = self._ones = torch.ones(self.cfg.dim, dtype=torch.float32, device=x.device)
        return {"mode": 1, "w": ones}

    def _linear(self, x, wname, bname):
        ad = self._adapter(wname)
        if ad is not None:
            return F_.lora_linear(x, self._p(wname), self._p(bname), ad.lora_A, ad.lora_B, ad.scale)
        return F_.linear(x, self._p(wname), self._p(bname))

    def _fused_params(self, first, last, n_out):
        """Views over the adjacent weight / bias slots ``first..last`` (e.g. q|k|v), wired to the flat
        gradient buffers when gradients are on."""
        d_in = self.unit.slots[first + ".weight"].shape[1]
        w = self.unit.span(first + ".weight", last + ".weight", (n_out, d_in))
        b = self.unit.span(first + ".bias", last + ".bias", (n_out,))
        if torch.is_grad_enabled() and self.unit.grad is not None:
            w.main_grad = self.unit.grad_span(first + ".weight", last + ".weight", (n_out, d_in))
            b.main_grad = self.unit.grad_span(first + ".bias", last + ".bias", (n_out,))
            names = _SPAN_NAMES[first.rsplit(".", 1)[1]]
            pre = first.rsplit(".", 1)[0]
            w._anchors = tuple(self._p(f"{pre}.{n}.weight") for n in names)
            b._anchors = tuple(self._p(f"{pre}.{n}.bias") for n in names)
            w.requires_grad_(True)
            b.requires_grad_(True)
        return w, b

    def _fused_linear(self, x, first, last, n_out):
        """One GEMM over adjacent weight slots ``first..last`` (e.g. q|k|v)."""
        if self.lora:               # adapters are per projection: issue the parts one by one
            pre = first.rsplit(".", 1)[0]
            return torch.cat([self._linear(x, f"{pre}.{n}.weight", f"{pre}.{n}.bias")
                              for n in _SPAN_NAMES[first.rsplit(".", 1)[1]]], dim=1)
        if not x.is_cuda or (torch.is_grad_enabled() and self.unit.grad is None):
            names = _SPAN_NAMES[first.rsplit(".", 1)[1]]
            pre = first.rsplit(".", 1)[0]
            w = torch.cat([self._p(f"{pre}.{n}.weight") for n in names], 0)
            b = torch.cat([self._p(f"{pre}.{n}.bias") for n in names], 0)
            return F_.linear(x, w, b)
        w, b = self._fused_params(first, last, n_out)
        if torch.is_grad_enabled():
            return F_._LinearMainGradFn.apply(x, w, b)
        return F_.gemm(x, w, F_.NT, bias=b)

    def forward(self, x, e0, rope, context, *, B, L, frame_tokens, group_offset=0, sp=None, memo=None, attn_fn=None,
                camera=None):
        """x [B*L_local, dim]; e0 fp32 [G, 6, dim] (G = B * frames); context [B*T, dim]."""
        cfg = self.cfg
        D, H, hd = cfg.dim, cfg.num_heads, cfg.head_dim
        sp = sp or _NoSP()
        mod = (self._p("modulation").float().view(1, 6, D) + e0).contiguous()
        gk = dict(rows_per_group=frame_tokens, group_offset=group_offset)

        # ---- self attention
        nk = self._norm_kw(x)
        # lean: the three norm outputs and the FFN hidden activation are not kept; backward rebuilds them from the
        # block's residual stream (two row passes and one GEMM) -- 8 of the block's 22 row-widths of activations
        lean = bool(getattr(self, "lean", False)) and torch.is_grad_enabled()
        Ll = x.shape[0] // B
        branch = camera is not None and cfg.camera_attention_mode == "parallel"
        cam_branch, camera = (camera, None) if branch else (None, camera)
        fused_sp = attn_fn is None and camera is None and not self.lora and not cfg.gated_attention and \
            bool(getattr(sp, "fused", False)) and x.is_cuda and B == 1 and sp.size > 1 and \
            (not torch.is_grad_enabled() or self.unit.grad is not None)
        xm = None if (lean and not fused_sp) else F_.norm_modulate(x, mod[:, 0], mod[:, 1], eps=cfg.eps, **nk, **gk)
        if fused_sp:
            # Ulysses exchanges ride on the producing kernels in both directions (parallel/fused_ulysses.py); the
            # out-projection belongs to the same function because its dgrad GEMM carries the backward exchange
            from ..parallel.fused_ulysses import FusedSelfAttention

            parity = sp.next_parity()
            w, b = self._fused_params("self_attn.q", "self_attn.v", 3 * D)
            y = FusedSelfAttention.apply(xm, w, b, self._p("self_attn.norm_q.weight"), self._p("self_attn.norm_k.weight"),
                                         rope, self._p("self_attn.o.weight"), self._p("self_attn.o.bias"), cfg.eps,
                                         1.0 / math.sqrt(hd), sp, parity, None if memo is None else (memo, "self"))
        else:
            if lean:
                qkv = F_.recompute_segment(
                    lambda a, s0, s1: self._fused_linear(F_.norm_modulate(a, s0, s1, eps=cfg.eps, **nk, **gk),
                                                         "self_attn.q", "self_attn.v", 3 * D),
                    self._p("self_attn.q.weight"), x, mod[:, 0], mod[:, 1])
            else:
                qkv = self._fused_linear(xm, "self_attn.q", "self_attn.v", 3 * D)
            q_raw, k_raw, v = F_.split_columns(qkv, (D, D, D))
            q = F_.rmsnorm_rope(q_raw, self._p("self_attn.norm_q.weight").float(), rope, eps=cfg.eps)
            k = F_.rmsnorm_rope(k_raw, self._p("self_attn.norm_k.weight").float(), rope, eps=cfg.eps)
            if camera is not None:          # PRoPE on the whole head: q <- P^T, k / v <- P^-1 (per local row)
                from . import camera_prope

                q = camera_prope.apply(q, camera[0], H)
                k = camera_prope.apply(k, camera[1], H)
                v = camera_prope.apply(v, camera[1], H)
            q, k, v = (t.reshape(B, Ll, H, hd) for t in (q, k, v))
            q, k, v = sp.scatter_heads(q, k, v)
            if attn_fn is not None:     # structured (block-causal / teacher-forcing) self attention
                o = attn_fn(q, k, v)
            else:
                o = ops.attention(q, k, v, memo=None if memo is None else (memo, "self"))
            o = sp.gather_heads(o).reshape(B * Ll, D)
            if camera is not None:
                o = camera_prope.apply(o, camera[2], H)
            if cfg.gated_attention:
                if xm is None:
                    xm = F_.norm_modulate(x, mod[:, 0], mod[:, 1], eps=cfg.eps, **nk, **gk)
                gate = 2.0 * torch.sigmoid(F_.linear(xm, self._p("self_attn.to_gate_logits.weight"),
                                                     self._p("self_attn.to_gate_logits.bias")).float())
                o = (o.view(B * Ll, H, hd) * gate.to(o.dtype).unsqueeze(-1)).reshape(B * Ll, D)
            y = self._linear(o, "self_attn.o.weight", "self_attn.o.bias")
        if cam_branch is not None:
            if xm is None:
                xm = F_.norm_modulate(x, mod[:, 0], mod[:, 1], eps=cfg.eps, **nk, **gk)
            y = y + self.camera_attention(xm, cam_branch, B=B, sp=sp, attn_fn=attn_fn)
        x = F_.gated_residual(x, y, mod[:, 2], **gk)

        # ---- cross attention (text keys/values are replicated on every SP rank)
        if cfg.cross_attn_norm and lean:
            qc = F_.recompute_segment(
                lambda a: self._linear(F_.norm_modulate(a, mode=2, w=self._p("norm3.weight").float(),
                                                        b=self._p("norm3.bias").float(), eps=cfg.eps),
                                       "cross_attn.q.weight", "cross_attn.q.bias"),
                self._p("cross_attn.q.weight"), x)
        else:
            if cfg.cross_attn_norm:
                xn = F_.norm_modulate(x, mode=2, w=self._p("norm3.weight").float(), b=self._p("norm3.bias").float(),
                                      eps=cfg.eps)
            else:
                xn = x
            qc = self._linear(xn, "cross_attn.q.weight", "cross_attn.q.bias")
        qc = F_.rmsnorm_rope(qc, self._p("cross_attn.norm_q.weight").float(), None, eps=cfg.eps)
        kvc = self._fused_linear(context, "cross_attn.k", "cross_attn.v", 2 * D)
        kc = F_.rmsnorm_rope(kvc[:, :D], self._p("cross_attn.norm_k.weight").float(), None, eps=cfg.eps)
        vc = kvc[:, D:]
        T = context.shape[0] // B
        with span("cross_attention"):
            oc = ops.attention(qc.reshape(B, Ll, H, hd), kc.reshape(B, T, H, hd), vc.reshape(B, T, H, hd),
                               memo=None if memo is None else (memo, "cross"))
        yc = self._linear(oc.reshape(B * Ll, D), "cross_attn.o.weight", "cross_attn.o.bias")
        x = F_.gated_residual(x, yc, None)

        # ---- feed forward
        def ffn(a, s3, s4):
            hm = F_.norm_modulate(a, s3, s4, eps=cfg.eps, **nk, **gk)
            if self._adapter("ffn.2.weight") is not None:      # the adapter reads the activation, so it is kept
                return self._linear(F_.gelu(self._linear(hm, "ffn.0.weight", "ffn.0.bias")), "ffn.2.weight", "ffn.2.bias")
            return F_.gelu_linear(self._linear(hm, "ffn.0.weight", "ffn.0.bias"), self._p("ffn.2.weight"), self._p("ffn.2.bias"))

        with span("ffn.fwd"):
            y = F_.recompute_segment(ffn, self._p("ffn.2.weight"), x, mod[:, 3], mod[:, 4]) if lean else ffn(x, mod[:, 3], mod[:, 4])
        x = F_.gated_residual(x, y, mod[:, 5], **gk)
        return x


def _camera_attention(self, xm, camera, *, B, sp, attn_fn=None):
    """The parallel camera branch on the block's modulated input: its own q | k | v projection (one GEMM), RMS-normed
    q and k WITHOUT rotary positions, the camera transforms on whole heads (q <- P^T, k / v <- P^-1, output <- P), the
    same attention pattern as the main branch, and a zero-initialised output projection."""
    from . import camera_prope

    cfg = self.cfg
    D, H, hd = cfg.dim, cfg.num_heads, cfg.head_dim
    Ll = xm.shape[0] // B
    qkv = self._fused_linear(xm, "cam_self_attn.q_proj", "cam_self_attn.v_proj", 3 * D)
    q, k, v = F_.split_columns(qkv, (D, D, D))
    q = F_.rmsnorm_rope(q, self._p("cam_self_attn.norm_q.weight").float(), None, eps=cfg.eps)
    k = F_.rmsnorm_rope(k, self._p("cam_self_attn.norm_k.weight").float(), None, eps=cfg.eps)
    q = camera_prope.apply(q, camera[0], H)
    k = camera_prope.apply(k, camera[1], H)
    v = camera_prope.apply(v.contiguous(), camera[1], H)
    q, k, v = sp.scatter_heads(*(t.reshape(B, Ll, H, hd) for t in (q, k, v)))
    o = attn_fn(q, k, v) if attn_fn is not None else ops.attention(q, k, v)
    o = camera_prope.apply(sp.gather_heads(o).reshape(B * Ll, D), camera[2], H)
    return self._linear(o, "cam_self_attn.out_proj.weight", "cam_self_attn.out_proj.bias")


WanBlock.camera_attention = _camera_attention


def _stem_specs(cfg: WanConfig):
    d = cfg.dim
    pp = cfg.patch_size[0] * cfg.patch_size[1] * cfg.patch_size[2]
    specs = [("patch_embedding.weight", (d, cfg.in_dim, *cfg.patch_size), False),
             ("patch_embedding.bias", (d,), False),
             ("text_embedding.0.weight", (d, cfg.text_dim), False), ("text_embedding.0.bias", (d,), False),
             ("text_embedding.2.weight", (d, d), False), ("text_embedding.2.bias", (d,), False),
             ("time_embedding.0.weight", (d, cfg.freq_dim), False), ("time_embedding.0.bias", (d,), False),
             ("time_embedding.2.weight", (d, d), False), ("time_embedding.2.bias", (d,), False),
             ("time_projection.1.weight", (6 * d, d), False), ("time_projection.1.bias", (6 * d,), False),
             ("head.head.weight", (cfg.out_dim * pp, d), False), ("head.head.bias", (cfg.out_dim * pp,), False),
             ("head.modulation", (1, 2, d), True)]
    if cfg.flow_objective == "anyflow_forward_map":
        specs += [("delta_embedding.0.weight", (d, cfg.freq_dim), False), ("delta_embedding.0.bias", (d,), False),
                  ("delta_embedding.2.weight", (d, d), False), ("delta_embedding.2.bias", (d,), False)]
    return specs


class WanDiT(nn.Module):
    """Bidirectional / block-causal Wan DiT.  ``forward`` mirrors the reference call
    ``model(x, t, context, seq_len, y=...)`` with batched tensors instead of Python lists."""

    def __init__(self, cfg: WanConfig, device="cpu", dtype=torch.bfloat16, seed: Optional[int] = 0,
                 shard_pad: int = 1):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype
        self.stem = FlatUnit(_stem_specs(cfg), device, dtype, pad_to=shard_pad)
        for name in self.stem.slots:
            _register(self, name, self.stem.parameter(name))
        self.blocks = nn.ModuleList([WanBlock(cfg, device, dtype, shard_pad) for _ in range(cfg.num_layers)])
        self.sp = _NoSP()
        self.checkpointing = "none"  # "none" | "full" | "selective"
        self.keep_blocks = 0         # the last ``keep_blocks`` blocks keep their activations (no recompute)
        self.lean_kept = False       # kept blocks drop their norm outputs and FFN hidden (rebuilt in backward)
        self._rope_cache: dict = {}
        self.grad_ready_hook = None  # callable(unit): a block's parameter gradients are final (set by the trainer)
        self.param_provider = None   # parallel.shard_params.ShardedParameters when block weights are sharded
        if seed is not None:
            self.init_weights(seed)

    # ----------------------------------------------------------------------------------
    def units(self):
        return [self.stem] + [b.unit for b in self.blocks]

    def ensure_grads(self):
        for u in self.units():
            u.ensure_grads()

    def zero_grads(self):
        for u in self.units():
            u.zero_grads()

    def finalize_grads(self):
        for u in self.units():
            u.finalize_grads()

    @torch.no_grad()
    def init_weights(self, seed: int = 0):
        """Xavier-uniform linears, N(0, 0.02) text/time MLPs, zero head, N(0,1)/sqrt(dim) modulation
        (reference model.py:534-561), generated on the parameter's own device."""
        g = torch.Generator(device="cpu").manual_seed(int(seed))
        dev_gen = None
        if self.stem.device.type == "cuda":
            dev_gen = torch.Generator(device=self.stem.device).manual_seed(int(seed))

        def fill(p, kind, std=0.02):
            gen = dev_gen if p.is_cuda else g
            if kind == "xavier":
                fan_out = p.shape[0]
                fan_in = p[0].numel()
                bound = math.sqrt(6.0 / (fan_in + fan_out))
                p.copy_((torch.rand(p.shape, generator=gen, device=p.device) * 2 - 1) * bound)
            elif kind == "normal":
                p.copy_(torch.randn(p.shape, generator=gen, device=p.device) * std)
            elif kind == "ones":
                p.fill_(1.0)
            else:
                p.zero_()

        d = self.cfg.dim
        for name, p in self.named_parameters():
            leaf = name.split(".")[-1]
            if "modulation" in name:
                fill(p, "normal", 1.0 / math.sqrt(d))
            elif "norm" in name:
                fill(p, "ones" if leaf == "weight" else "zeros")
            elif leaf == "bias":
                fill(p, "zeros")
            elif name.startswith(("text_embedding", "time_embedding", "delta_embedding")):
                fill(p, "normal", 0.02)
            elif name.startswith("head.head") or ".cam_self_attn.out_proj." in name or ".to_gate_logits." in name:
                fill(p, "zeros")
            else:
                fill(p, "xavier")

    # ----------------------------------------------------------------------------------
    def patchify(self, x):
        """[B, C, F, H, W] -> [B*L, C*pt*ph*pw] rows ordered (f, h, w) and the token grid."""
        B, C, F, H, W = x.shape
        pt, ph, pw = self.cfg.patch_size
        f, h, w = F // pt, H // ph, W // pw
        x = x.view(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B * f * h * w, C * pt * ph * pw), (f, h, w)

    def unpatchify(self, y, B, grid):
        f, h, w = grid
        pt, ph, pw = self.cfg.patch_size
        c = self.cfg.out_dim
        y = y.view(B, f, h, w, pt, ph, pw, c).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return y.reshape(B, c, f * pt, h * ph, w * pw)

    def _rope(self, grid, device, frame_offset=0, B=1):
        key = (tuple(grid), str(device), frame_offset, B)
        if key not in self._rope_cache:
            t = rope_table(grid, self.cfg.head_dim, device, frame_offset)
            self._rope_cache[key] = t.repeat(B, 1, 1) if B > 1 else t
        return self._rope_cache[key]

    def time_condition(self, t_frames, r_frames=None):
        """Per-frame timestep embedding e [G, dim] and modulation e0 fp32 [G, 6, dim]."""
        cfg = self.cfg
        P = self.stem.params
        dt = self.dtype
        emb = sinusoidal_embedding(cfg.freq_dim, t_frames.reshape(-1)).to(dt)
        e = F_.linear(emb, P["time_embedding.0.weight"], P["time_embedding.0.bias"])
        e = torch.nn.functional.silu(e.float()).to(dt)
        e = F_.linear(e, P["time_embedding.2.weight"], P["time_embedding.2.bias"])
        if cfg.flow_objective == "anyflow_forward_map" and r_frames is not None:
            # second time MLP on the interval start r, mixed with a fixed gate (reference
            # causal_model.py:1872-1908)
            demb = sinusoidal_embedding(cfg.freq_dim, r_frames.reshape(-1)).to(dt)
            de = F_.linear(demb, P["delta_embedding.0.weight"], P["delta_embedding.0.bias"])
            de = torch.nn.functional.silu(de.float()).to(dt)
            de = F_.linear(de, P["delta_embedding.2.weight"], P["delta_embedding.2.bias"])
            g = cfg.anyflow_gate
            e = ((1.0 - g) * e.float() + g * de.float()).to(dt)
        e_act = torch.nn.functional.silu(e.float()).to(dt)
        e0 = F_.linear(e_act, P["time_projection.1.weight"], P["time_projection.1.bias"])
        return e, e0.float().view(-1, 6, cfg.dim)

    def embed_text(self, context):
        """[B, T, text_dim] -> [B*T, dim]"""
        P = self.stem.params
        B, T, _ = context.shape
        c = context.reshape(B * T, -1).to(self.dtype)
        c = F_.linear(c, P["text_embedding.0.weight"], P["text_embedding.0.bias"])
        c = F_.gelu(c)
        return F_.linear(c, P["text_embedding.2.weight"], P["text_embedding.2.bias"])

    def _run_block(self, block, x, e0, rope, ctx, kw, index=0):
        """``checkpointing``: "none" keeps every activation; "full" recomputes the whole block in
        backward; "selective" recomputes the block except its two attention calls, whose outputs are
        carried across the recompute (the reference's saved-attention policy,
        solar/backends/minimax_h3/fsdp.py:146-165).  The last ``keep_blocks`` blocks are exempt: with
        memory to spare their activations stay resident and their recompute is saved."""
        with span(f"block.{index:02d}"):
            return self._run_block_inner(block, x, e0, rope, ctx, kw, index)

    def _run_block_inner(self, block, x, e0, rope, ctx, kw, index):
        prov = self.param_provider
        k = None if prov is None else prov.index_of(block.unit)
        training = torch.is_grad_enabled() and x.requires_grad
        if self.grad_ready_hook is not None and training:
            x = _UnitReady.apply(x, self._block_done if k is not None else self.grad_ready_hook, block.unit)
        if k is not None:
            prov.acquire(k)                       # the block's weights are gathered (prefetched one block ahead)
        out = self._run_block_compute(block, x, e0, rope, ctx, kw, index)
        if k is not None:
            prov.release(k)
            if training:
                out = _BlockGate.apply(out, prov, k)
        return out

    def _block_done(self, unit) -> None:
        """Backward of a block with sharded weights is complete: reduce its gradients, then free its slots."""
        self.grad_ready_hook(unit)
        self.param_provider.release(self.param_provider.index_of(unit))

    def _run_block_compute(self, block, x, e0, rope, ctx, kw, index):
        exempt = index >= len(self.blocks) - int(self.keep_blocks)
        if self.checkpointing in ("full", "selective") and torch.is_grad_enabled() and not exempt:
            from torch.utils.checkpoint import checkpoint

            memo = {"__store__": True} if (self.checkpointing == "selective" and x.is_cuda) else None
            block.lean = False
            return checkpoint(lambda a, b, c: block(a, b, rope, c, memo=memo, **kw), x, e0, ctx, use_reentrant=False)
        block.lean = bool(self.lean_kept)
        return block(x, e0, rope, ctx, **kw)

    def forward(self, x, t, context, y=None, r=None, y_camera=None, perturb_blocks=()):
        """x [B, C, F, H, W] noisy latents; t [B, F] (or [B]) timesteps in [0, 1000];
        context [B, T, text_dim]; y optional channel-concatenated conditioning (I2V);
        y_camera optional ``{"viewmats": [B, F, 4, 4], "Ks": [B, F, 3, 3] or None, "transform": str}``:
        PRoPE camera conditioning of the self-attention (reference: causal_model.py:925-1000);
        ``perturb_blocks``: indices of blocks whose self-attention is skipped (every token keeps its own
        value) -- the perturbed evaluation of spatio-temporal guidance."""
        cfg = self.cfg
        P = self.stem.params
        if y is not None:
            x = torch.cat([x, y], dim=1)
        B = x.shape[0]
        rows, grid = self.patchify(x.to(self.dtype))
        f, h, w = grid
        frame_tokens = h * w
        L = f * frame_tokens
        if t.dim() == 1:
            t = t.view(B, 1).expand(B, f)
        elif t.shape[1] == L:
            t = t[:, ::frame_tokens]
        if r is not None and r.dim() == 1:
            r = r.view(B, 1).expand(B, f)
        pw = P["patch_embedding.weight"]
        tok = F_.linear(rows, pw.view(pw.shape[0], -1), P["patch_embedding.bias"])
        e, e0 = self.time_condition(t, r)
        ctx = self.embed_text(context)

        # sequence parallel: whole latent frames per rank (uneven allowed)
        sp = self.sp
        f0, fl = 0, f
        if sp.size > 1:
            base, rem = divmod(f, sp.size)
            fl = base + int(sp.rank < rem)
            f0 = sp.rank * base + min(sp.rank, rem)
            tok = tok.view(B, L, -1)[:, f0 * frame_tokens:(f0 + fl) * frame_tokens].reshape(B * fl * frame_tokens, -1)
            sp.set_layout(B, f, frame_tokens)
        rope = self._rope((fl, h, w), tok.device, frame_offset=f0, B=B)
        # group (= batch, frame) of a local row: b * f + f0 + local_frame; with B == 1 this is a
        # plain offset, for B > 1 under SP the e0 rows are re-packed per rank instead.
        if sp.size > 1 and B > 1:
            e0_l = e0.view(B, f, 6, cfg.dim)[:, f0:f0 + fl].reshape(B * fl, 6, cfg.dim)
            goff = 0
        else:
            e0_l, goff = e0, f0 if sp.size > 1 else 0
        kw = dict(B=B, L=L, frame_tokens=frame_tokens, group_offset=goff, sp=sp)
        if y_camera is not None:
            from . import camera_prope

            vm = y_camera["viewmats"][:, f0:f0 + fl].reshape(B * fl, 4, 4).to(tok.device)
            Ks = y_camera.get("Ks")
            Ks = None if Ks is None else Ks[:, f0:f0 + fl].reshape(B * fl, 3, 3).to(tok.device)
            mats = camera_prope.prope_matrices(vm, Ks, transform=y_camera.get("transform", "linear"))
            kw["camera"] = tuple(camera_prope.per_row(m, frame_tokens) for m in mats)
        xs = tok
        skip = {int(i) for i in perturb_blocks}
        for bi, block in enumerate(self.blocks):
            kw_b = dict(kw, attn_fn=_identity_attention) if bi in skip else kw
            xs = self._run_block(block, xs, e0_l, rope, ctx, kw_b, index=bi)
        if sp.size > 1:
            xs = sp.gather_sequence(xs, B)
        # head
        hm = (P["head.modulation"].float().view(1, 2, cfg.dim) + e.float().view(-1, 1, cfg.dim)).contiguous()
        xh = F_.norm_modulate(xs, hm[:, 0], hm[:, 1], eps=cfg.eps, rows_per_group=frame_tokens,
                              **self.blocks[0]._norm_kw(xs))
        out = F_.linear(xh, P["head.head.weight"], P["head.head.bias"])
        return self.unpatchify(out, B, grid)
