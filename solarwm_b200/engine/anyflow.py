"""AnyFlow v1.5 forward-map objective math (backbone independent).

* shift ``s t / (1 + (s-1) t)``
* ``(t, r)`` pairs: two fp32 uniforms per sample (all ``u1`` then all ``u2``), ``t = u1``,
  ``r = u2 t``; sample types are assigned over the GLOBAL data-parallel batch by flat index:
  the first ``round(diffusion_ratio * N)`` samples are diffusion (``r = t``), the next
  ``round(consistency_ratio * N)`` are consistency (``r = 0``), the rest are flow-map samples with
  strict ``0 < r < t`` (enforced with ``nextafter``, no extra random draws)
* bounded central difference window ``t+ = min(t + eps, N)``, ``t- = max(t - eps, r)``, eps = 5
* Gaussian timestep weights on the shifted 1000-step grid, min-subtracted, mean one
* adaptive rescale of non-diffusion losses toward the global mean diffusion loss

Reference: solar/training/anyflow.py:27-316.
"""
from __future__ import annotations

from typing import Callable, NamedTuple, Optional

import torch

DIFFUSION, CONSISTENCY, FLOW_MAP = 0, 1, 2


class TimePairs(NamedTuple):
    t: torch.Tensor
    r: torch.Tensor
    is_diffusion: torch.Tensor
    is_consistency: torch.Tensor
    sample_type: torch.Tensor


def apply_timestep_shift(x, shift: float):
    x = torch.as_tensor(x)
    if not x.is_floating_point():
        x = x.float()
    shift = float(shift)
    if not (shift > 0) or shift != shift or shift == float("inf"):
        raise ValueError(f"shift must be positive and finite, got {shift}")
    return x if shift == 1.0 else shift * x / (1.0 + (shift - 1.0) * x)


def sample_time_pairs(batch: int, *, dp_rank: int = 0, dp_world: int = 1, diffusion_ratio: float = 0.5,
                      consistency_ratio: float = 0.25, generator=None, device="cpu") -> TimePairs:
    if batch < 1 or dp_world < 1 or not 0 <= dp_rank < dp_world:
        raise ValueError("invalid batch / data-parallel coordinates")
    if not 0 <= diffusion_ratio <= 1 or not 0 <= consistency_ratio <= 1 or diffusion_ratio + consistency_ratio > 1:
        raise ValueError("diffusion_ratio and consistency_ratio must lie in [0,1] and sum to at most 1")
    u1 = torch.rand(batch, dtype=torch.float32, device=device, generator=generator)
    u2 = torch.rand(batch, dtype=torch.float32, device=device, generator=generator)
    t, r = u1, u2 * u1
    n_global = batch * dp_world
    idx = torch.arange(batch, device=device) + dp_rank * batch
    n_diff = round(diffusion_ratio * n_global)
    n_cons = round(consistency_ratio * n_global)
    is_diff = idx < n_diff
    is_cons = (idx >= n_diff) & (idx < n_diff + n_cons)
    is_map = ~(is_diff | is_cons)
    r = torch.where(is_diff, t, r)
    r = torch.where(is_cons, torch.zeros_like(r), r)
    zero, one = torch.zeros((), device=device), torch.ones((), device=device)
    tiny = torch.nextafter(zero, one)
    r_pos = torch.where(r > 0, r, tiny)
    t_gt = torch.where(t > r_pos, t, torch.nextafter(r_pos, one))
    r = torch.where(is_map, r_pos, r)
    t = torch.where(is_map, t_gt, t)
    kind = torch.full((batch,), FLOW_MAP, dtype=torch.int8, device=device)
    kind = torch.where(is_diff, torch.full_like(kind, DIFFUSION), kind)
    kind = torch.where(is_cons, torch.full_like(kind, CONSISTENCY), kind)
    return TimePairs(t, r, is_diff, is_cons, kind)


def difference_window(t, r, *, epsilon: float = 5.0, num_train_timesteps: int = 1000):
    if epsilon <= 0 or num_train_timesteps <= 0:
        raise ValueError("epsilon and num_train_timesteps must be positive")
    t = torch.as_tensor(t)
    r = torch.as_tensor(r, device=t.device, dtype=t.dtype)
    t, r = torch.broadcast_tensors(t, r)
    return (t + epsilon).clamp_max(num_train_timesteps), torch.maximum(t - epsilon, r)


def _trail(v, ndim):
    return v.reshape(*v.shape, *((1,) * (ndim - v.ndim)))


@torch.no_grad()
def central_difference(u_plus, u_minus, t_plus, t_minus):
    if u_plus.shape != u_minus.shape:
        raise ValueError("u_plus and u_minus must have identical shapes")
    tp = torch.as_tensor(t_plus, device=u_plus.device, dtype=torch.float32)
    tm = torch.as_tensor(t_minus, device=u_plus.device, dtype=torch.float32)
    tp, tm = torch.broadcast_tensors(tp, tm)
    width = _trail((tp - tm).clamp_min(1e-6), u_plus.ndim)
    return ((u_plus.detach().float() - u_minus.detach().float()) / width).detach()


@torch.no_grad()
def gaussian_timestep_weights(shifted_raw_t, *, shift: float, num_train_timesteps: int = 1000):
    x = torch.as_tensor(shifted_raw_t)
    dt = torch.float64 if x.dtype == torch.float64 else torch.float32
    n = int(num_train_timesteps)
    grid = apply_timestep_shift(torch.linspace(1.0, 0.0, n + 1, dtype=dt, device=x.device)[:-1], shift) * n
    w = torch.exp(-2.0 * ((grid - n / 2.0) / n).square())
    w = w - w.min()
    if not bool(torch.isfinite(w.sum())) or not bool(w.sum() > 0):
        raise ValueError("gaussian training-grid weights have invalid normalization")
    w = w * (n / w.sum())
    flat = x.to(dt).reshape(-1)
    nearest = torch.argmin((grid[:, None] - flat[None, :]).abs(), dim=0)
    return w[nearest].reshape(x.shape)


def anyflow_residual(u_pred, du_dt, t, r, velocity_target, *, num_train_timesteps: int = 1000):
    """``u + (t - r) du/dt - (noise - x0)`` with times on the raw grid scaled to [0, 1]."""
    span = _trail(((torch.as_tensor(t) - torch.as_tensor(r)) / num_train_timesteps).float().to(u_pred.device), u_pred.ndim)
    return u_pred.float() + span * du_dt.float() - velocity_target.float()


def adaptive_rescale(per_sample_loss, is_diffusion, *, gather_fn: Optional[Callable] = None, process_group=None,
                     eps: float = 1e-5):
    if gather_fn is not None and process_group is not None:
        raise ValueError("provide at most one of gather_fn and process_group")
    if per_sample_loss.ndim != 1 or per_sample_loss.shape != is_diffusion.shape:
        raise ValueError("per_sample_loss and is_diffusion must be 1-D with the same shape")
    if eps <= 0:
        raise ValueError("eps must be positive")
    is_diffusion = is_diffusion.to(per_sample_loss.device, torch.bool)

    def gather(x):
        x = x.detach()
        if gather_fn is not None:
            got = gather_fn(x)
            parts = [got] if torch.is_tensor(got) else list(got)
            return torch.cat([p.to(per_sample_loss.device).reshape(-1) for p in parts])
        if process_group is not None:
            import torch.distributed as dist

            parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group=process_group))]
            dist.all_gather(parts, x, group=process_group)
            return torch.cat([p.reshape(-1) for p in parts])
        return x.reshape(-1)

    g_loss, g_diff = gather(per_sample_loss), gather(is_diffusion).bool()
    if g_loss.numel() != g_diff.numel():
        raise ValueError("gathered loss and sample-type mask lengths differ")
    with torch.no_grad():
        ref = g_loss[g_diff]
        ref = ref[torch.isfinite(ref)]
        if ref.numel() == 0 or bool(is_diffusion.all()):
            return per_sample_loss
        scale = ref.mean().to(per_sample_loss) / (per_sample_loss.detach() + eps)
        scale = torch.where(torch.isfinite(scale), scale, torch.ones_like(scale))
    return torch.where(is_diffusion, per_sample_loss, per_sample_loss * scale)
