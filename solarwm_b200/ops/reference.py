"""Plain PyTorch statements of every fused op (fp32 math, autograd-differentiable).

These are the oracles the GPU numerics tests compare the sm_100a kernels against, and the
code path used on CPU (gloo tests, contract tests).  They follow the eager chains of the
reference model: LayerNorm -> (1+scale)*x+shift, gate*y+x, full-width RMSNorm + interleaved
complex RoPE (solar/backends/wan22/runtime/modeling/model.py:38-110,
causal_model.py:1636-1707).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def group_index(rows: int, rows_per_group: int, group_offset: int, table, device):
    if table is not None:
        return table.long()
    return torch.arange(rows, device=device) // max(int(rows_per_group), 1) + int(group_offset)


def norm_modulate(x, shift, scale, *, mode=0, w=None, b=None, eps=1e-6, rows_per_group=1,
                  group_offset=0, table=None):
    """mode 0: LayerNorm without affine; 1: RMSNorm * w; 2: LayerNorm * w + b.
    shift/scale: [G, D] (or None)."""
    xf = x.float()
    if mode == 1:
        n = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        n = (xf - mu) * torch.rsqrt(var + eps)
    if mode >= 1:
        n = n * w.float()
    if mode == 2:
        n = n + b.float()
    if scale is not None:
        g = group_index(x.shape[0], rows_per_group, group_offset, table, x.device)
        n = n * (1.0 + scale.float()[g]) + shift.float()[g]
    return n.to(x.dtype)


def gated_residual(res, y, gate, *, rows_per_group=1, group_offset=0, table=None):
    if gate is None:
        return (res.float() + y.float()).to(res.dtype)
    g = group_index(res.shape[0], rows_per_group, group_offset, table, res.device)
    return (res.float() + gate.float()[g] * y.float()).to(res.dtype)


def rmsnorm_rope(x, w, rope, *, eps=1e-6, head_dim=None, no_norm=False):
    """x [R, D]; rope [R, hd/2, 2] (cos, sin) or None; interleaved (2i, 2i+1) pairs per head."""
    xf = x.float()
    if not no_norm:
        xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    if rope is not None:
        R, D = xf.shape
        hd = rope.shape[1] * 2
        v = xf.view(R, D // hd, hd // 2, 2)
        cos = rope[:, None, :, 0].float()
        sin = rope[:, None, :, 1].float()
        a, b = v[..., 0], v[..., 1]
        xf = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).reshape(R, D)
    return xf.to(x.dtype)


def gelu_tanh(x):
    return F.gelu(x.float(), approximate="tanh").to(x.dtype)


def swiglu(gu):
    n = gu.shape[-1] // 2
    g, u = gu[..., :n].float(), gu[..., n:].float()
    return (u * F.silu(g)).to(gu.dtype)


def linear(x, w, b=None, act=None):
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    if act == "gelu":
        y = F.gelu(y, approximate="tanh")
    return y.to(x.dtype)


def attention(q, k, v, *, scale=None, mask=None):
    """q [B, Sq, H, D], k/v [B, Sk, H, D]; mask broadcastable to [B, H, Sq, Sk] (True = keep)."""
    d = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    s = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, vf).transpose(1, 2).to(q.dtype)


def adamw_step(master, m, v, grad, *, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    g = grad.float() * grad_scale
    master.mul_(1.0 - lr * wd)
    m.mul_(beta1).add_(g, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v / bc2).sqrt_().add_(eps)
    master.addcdiv_(m, denom, value=-lr / bc1)
    return master


def weighted_masked_mse(pred, target, weight=None, mask=None):
    """pred/target [G, ...]; weight/mask [G] broadcast over the remaining axes.  The mask is
    applied to both operands before the subtraction; the mean runs over selected elements."""
    p, t = pred.float(), target.float()
    G = p.shape[0]
    shape = (G,) + (1,) * (p.dim() - 1)
    mk = torch.ones(G, device=p.device) if mask is None else mask.float()
    wt = torch.ones(G, device=p.device) if weight is None else weight.float()
    diff = p * mk.view(shape) - t * mk.view(shape)
    per = diff.pow(2) * wt.view(shape)
    denom = mk.sum().clamp_min(1.0) * (p.numel() // G)
    return per.sum() / denom


def head_norm_rope_prope(x, w, cos, sin, mats, *, heads: int, rot_dims: int = 96, sections: int = 2, eps: float = 1e-6):
    """Per-head RMSNorm * w, rotate-half RoPE inside each of ``sections`` blocks of the first
    ``rot_dims`` channels, then a 4x4 matrix on every 4-vector of the remaining channels.
    x [S, heads*128]; cos/sin [S, rot_dims]; mats [S, 4, 4]; any of w / cos / mats may be None."""
    S = x.shape[0]
    v = x.float().view(S, heads, -1)
    hd = v.shape[-1]
    if w is not None:
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    if cos is not None:
        sec = rot_dims // sections
        rot = v[..., :rot_dims].reshape(S, heads, sections, sec)
        a, b = rot[..., :sec // 2], rot[..., sec // 2:]
        half = torch.cat([-b, a], dim=-1)
        c = cos.float().view(S, 1, sections, sec)
        s_ = sin.float().view(S, 1, sections, sec)
        v = torch.cat([(rot * c + half * s_).reshape(S, heads, rot_dims), v[..., rot_dims:]], dim=-1)
    if mats is not None:
        cam = v[..., rot_dims:].reshape(S, heads, (hd - rot_dims) // 4, 4)
        cam = torch.einsum("sij,shnj->shni", mats.float().view(S, 4, 4), cam)
        v = torch.cat([v[..., :rot_dims], cam.reshape(S, heads, hd - rot_dims)], dim=-1)
    return v.reshape(S, heads * hd).to(x.dtype)
