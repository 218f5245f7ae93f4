"""Omni flow-matching core of the renderer.

A sample is a packed H3 document ``[text | anchor | structure rows | target video rows]``:

* the **structure** stream (depth / edge / layout latents of the same geometry as the target) enters
  as clean video-tagged rows that share the target's positions and cameras -- the model reads the
  scene structure off them through ordinary attention;
* every **target** row carries its own known degree from an observation plan: the row holds
  ``t x0 + (1 - t) n`` at its own ``t`` and its adaLN table entry is looked up by that ``t``;
* the loss is the flow-matching error ``|| v - (x0 - n) ||^2`` over the plan's loss rows only.

``render`` integrates the same field with the data-ward Euler rule over a fixed time grid while the
rows a plan marks as known are pinned to their degree at every step
(reference: solar/renderer/core.py:49-, render.py:21-293).
"""
from __future__ import annotations

from typing import Mapping, Optional

import numpy as np
import torch

from ..backends.minimax_h3 import flow
from ..backends.minimax_h3.layout import TAG_TEXT, TAG_VIDEO, patchify_latents, spatial_axis, temporal_positions, unpatchify_rows
from ..engine.master_adamw import FP32MasterAdamW
from ..models.h3 import H3DiT
from .known_degree import ObservationPlan, ObservationProfile, sample_plan


def _positions(n_text: int, frames: int, h: int, w: int, copies: int):
    """text rows, anchor frame, then ``copies`` video streams that share the native frame positions."""
    rows = h * w
    pos_text = torch.zeros(n_text, 3, dtype=torch.float64)
    pos_text[:, 0] = torch.arange(n_text)
    grid = torch.from_numpy(np.stack(np.meshgrid(spatial_axis(h, w), spatial_axis(w, h), indexing="ij"), -1).reshape(rows, 2))
    tpos = torch.from_numpy(temporal_positions(frames + 1, origin=float(n_text)))

    def frames_at(ts):
        p = torch.zeros(len(ts) * rows, 3, dtype=torch.float64)
        p[:, 0] = torch.as_tensor(ts, dtype=torch.float64).repeat_interleave(rows)
        p[:, 1:] = grid.repeat(len(ts), 1)
        return p

    vid = frames_at(tpos[1:].tolist())
    return torch.cat([pos_text, frames_at([float(tpos[0])])] + [vid] * copies)


def packed_forward(model: H3DiT, *, prompt, anchor_rows, structure_rows, target_rows, row_times: torch.Tensor,
                   grid_hw, cameras: Optional[torch.Tensor] = None, attn_fn=None):
    """Returns the network output on the target rows [L, 96].  ``row_times`` [L] in [0, 1]; ``structure_rows`` may
    be None (plain generation / dropped control)."""
    h, w = grid_hw
    rows = h * w
    L = target_rows.shape[0]
    F = L // rows
    n_text = prompt.shape[0]
    dev = target_rows.device
    n_struct = 0 if structure_rows is None else structure_rows.shape[0]
    values = torch.cat([torch.tensor([1.0, 0.999]), row_times.detach().float().cpu()])
    uniq, inverse = torch.unique(values, return_inverse=True)
    t_index = torch.cat([torch.full((n_text,), int(inverse[0])), torch.full((anchor_rows.shape[0],), int(inverse[1])),
                         torch.full((n_struct,), int(inverse[0])), inverse[2:]]).to(torch.int32)
    tags = torch.cat([torch.full((n_text,), TAG_TEXT), torch.full((anchor_rows.shape[0] + n_struct + L,), TAG_VIDEO)]).to(torch.int32)
    pos = _positions(n_text, F, h, w, copies=2 if n_struct else 1)
    view = None
    if cameras is not None:
        per = cameras[1:].float().repeat_interleave(rows, dim=0)
        view = torch.cat([torch.eye(4).repeat(n_text, 1, 1), cameras[:1].float().repeat(anchor_rows.shape[0], 1, 1)]
                         + [per] * (2 if n_struct else 1))
    video = target_rows if structure_rows is None else torch.cat([structure_rows, target_rows])
    out, _ = model(video_rows=video, text_rows=prompt, anchor_rows=anchor_rows, timesteps=uniq,
                   t_index=t_index.to(dev), tags=tags.to(dev), position_ids=pos, viewmats=view, attn_fn=attn_fn)
    return out[n_struct:]


class OmniFlowTrainer:
    def __init__(self, cfg, device, profile: ObservationProfile = ObservationProfile(), lr: float = 1e-4, seed: int = 0,
                 model: Optional[H3DiT] = None, optimizer: Optional[FP32MasterAdamW] = None):
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.device = torch.device(device)
        self.model = model or H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        self.opt = optimizer or FP32MasterAdamW(self.model.trainable_parameters(), lr=lr)
        self.profile = profile
        self.rng = np.random.default_rng(seed)
        self.gen = torch.Generator(device=self.device).manual_seed(seed * 100003 + 29)
        self.last_plan: Optional[ObservationPlan] = None

    def compute_loss(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        """The plan-weighted flow-matching loss of one sample, with its graph (the caller runs backward)."""
        dev, dt = self.device, self.model.dtype
        lat = sample["target_latents"].to(dev)
        C, F, H, W = lat.shape
        h, w = H // 2, W // 2
        base_t = float(1.0 - flow.shifted_sigma(torch.tensor(self.rng.random()), flow.VIDEO_SHIFT))
        plan = sample_plan(self.profile, frames=F, grid_height=h, grid_width=w, base_time=base_t,
                           shift=flow.VIDEO_SHIFT, rng=self.rng, given=sample.get("known_degree"))
        self.last_plan = plan
        t_rows = torch.from_numpy(plan.row_times).to(dev)
        noise = torch.randn(lat.shape, generator=self.gen, device=dev, dtype=torch.float32)
        x0_rows, n_rows = patchify_latents(lat).float(), patchify_latents(noise)
        x_rows = (t_rows.view(-1, 1) * x0_rows + (1.0 - t_rows.view(-1, 1)) * n_rows).to(dt)
        structure = sample.get("structure_latents") if plan.use_control else None
        anchor = sample["anchor_latents"].to(dev) if plan.use_anchor else torch.zeros_like(sample["anchor_latents"]).to(dev)
        pred = packed_forward(self.model, prompt=sample["prompt_embeds"].to(dev, dt),
                              anchor_rows=patchify_latents(anchor).to(dt),
                              structure_rows=None if structure is None else patchify_latents(structure.to(dev)).to(dt),
                              target_rows=x_rows, row_times=t_rows, grid_hw=(h, w),
                              cameras=sample.get("camera_w2c") if plan.use_camera else None)
        keep = torch.from_numpy(plan.loss_rows).to(dev)
        err = (pred.float() - (x0_rows - n_rows)).pow(2).mean(dim=1)
        return (err * keep).sum() / keep.sum().clamp_min(1)

    def train_step(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        loss = self.compute_loss(sample)
        loss.backward()
        self.opt.gather_grads()
        self.opt.clip_(1.0)
        self.opt.step()
        self.opt.zero_grad()
        return loss.detach()


@torch.no_grad()
def render(model: H3DiT, sample: Mapping[str, torch.Tensor], *, steps: int = 8, known: Optional[torch.Tensor] = None,
           known_degree: Optional[torch.Tensor] = None, seed: int = 0, shift: float = flow.VIDEO_SHIFT) -> torch.Tensor:
    """Sample target latents [C, F, H, W].  ``known`` [C, F, H, W] with ``known_degree`` [F*h*w] in [0, 1] pins
    observed rows: at time t a row of degree d holds ``max(t, d)``-level content of the known clip."""
    dev, dt = model.proj_in.device, model.dtype
    C, F, H, W = sample["shape"]
    h, w = H // 2, W // 2
    g = torch.Generator(device=dev).manual_seed(seed)
    noise_rows = torch.randn(F * h * w, C * 4, generator=g, device=dev)
    x = noise_rows.clone()
    times = flow.rollout_times(steps, shift)                      # increasing towards 1
    deg = None if known_degree is None else known_degree.to(dev).float().view(-1, 1)
    known_rows = None if known is None else patchify_latents(known.to(dev)).float()
    structure = sample.get("structure_latents")
    structure_rows = None if structure is None else patchify_latents(structure.to(dev)).to(dt)
    anchor_rows = patchify_latents(sample["anchor_latents"].to(dev)).to(dt)
    for i, t in enumerate(times[:steps]):
        t_rows = torch.full((F * h * w,), float(t), device=dev)
        if deg is not None:
            t_rows = torch.maximum(t_rows, deg.view(-1))
            pinned = t_rows.view(-1, 1) * known_rows + (1.0 - t_rows.view(-1, 1)) * noise_rows
            x = torch.where(deg > float(t), pinned, x)
        v = packed_forward(model, prompt=sample["prompt_embeds"].to(dev, dt), anchor_rows=anchor_rows,
                           structure_rows=structure_rows, target_rows=x.to(dt), row_times=t_rows, grid_hw=(h, w),
                           cameras=sample.get("camera_w2c")).float()
        t_next = float(times[i + 1]) if i + 1 < len(times) else 1.0
        x = x + (torch.clamp(torch.full_like(t_rows, t_next) - t_rows, min=0.0)).view(-1, 1) * v   # data-ward Euler
    return unpatchify_rows(x.to(dt), C, F, H, W)
