"""Wan Stage1: block-causal teacher-forcing training (flow matching or AnyFlow v1.5).

Every chunk of ``chunk_frames`` latent frames draws its own timestep; the model sees the clean video
and the per-chunk-noised video in one ``[clean | noisy]`` pass (``models/wan_tf.py``) and is trained
on the noisy half.

* ``tf_fm``: velocity target ``noise - clean`` with the scheduler's Gaussian timestep weights
  (reference: solar/backends/wan22/runtime/stage1.py:45-194).
* ``anyflow``: per-chunk ``(t, r)`` pairs (diffusion / consistency / flow-map sample types assigned
  over the global data-parallel batch), the trainable evaluation ``u(x_t, t, r)`` plus two no-grad
  evaluations at ``t+`` / ``t-`` for the bounded central difference, the residual
  ``u + (t - r) du/dt - v`` and the adaptive rescale of non-diffusion samples
  (reference: solar/backends/wan22/runtime/stage1_anyflow.py:162-450, solar/training/anyflow.py).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional

import torch

from ... import ops
from ...engine import anyflow as af
from ...engine.flow import logit_normal_sigmas
from ...models.wan_tf import forward_noisy_suffix, forward_teacher_forcing
from .stage0p5 import Stage0p5Options, WanStage0p5Trainer


@dataclass
class Stage1Options(Stage0p5Options):
    objective: str = "tf_fm"            # "tf_fm" | "anyflow"
    chunk_frames: int = 3
    window_chunks: int = 6
    sink_frames: int = 0
    diffusion_ratio: float = 0.5
    consistency_ratio: float = 0.25
    difference_epsilon: float = 5.0
    dp_rank: int = 0
    dp_world: int = 1
    reuse_prefix: bool = True           # AnyFlow probes reuse the clean half's keys / values of the trainable pass


class WanStage1Trainer(WanStage0p5Trainer):
    def __init__(self, cfg, device, opts: Stage1Options = Stage1Options(), sp=None, model=None, dp_group=None, **kw):
        super().__init__(cfg, device, opts, sp=sp, model=model, dp_group=dp_group, **kw)

    # ------------------------------------------------------------------------------------
    def _per_chunk(self, values: torch.Tensor, F: int) -> torch.Tensor:
        """[n_chunks] -> [1, F]: every frame of a chunk carries the chunk's value."""
        return values.repeat_interleave(self.opts.chunk_frames)[:F].view(1, F)

    def _noised(self, latents, noise, t_frames):
        F = latents.shape[1]
        sigma = (t_frames.reshape(F) / self.scheduler.num_train_timesteps).float()
        x_t, target = ops.add_noise(latents[0], noise[0], sigma)
        return x_t.unsqueeze(0), target.unsqueeze(0)

    def _predict(self, clean, x_t, t, text, r=None, capture=None, captured=None):
        o = self.opts
        kw = dict(r=r, chunk_frames=o.chunk_frames, window_chunks=o.window_chunks, sink_frames=o.sink_frames)
        if captured is not None:                                # probe: the noisy half against the captured clean half
            pred = forward_noisy_suffix(self.model, x_t.permute(0, 2, 1, 3, 4), t, text, captured, **kw)
        else:
            pred = forward_teacher_forcing(self.model, clean.permute(0, 2, 1, 3, 4), x_t.permute(0, 2, 1, 3, 4), t, text,
                                           capture=capture, y_camera=getattr(self, "y_camera", None), **kw)
        return pred.permute(0, 2, 1, 3, 4)                      # [1, F, C, H, W]

    def microbatch(self, latents: torch.Tensor, text: torch.Tensor, y: Optional[torch.Tensor] = None):
        """latents [1, F, C, H, W]; one packed video per call."""
        o = self.opts
        if latents.shape[0] != 1:
            raise ValueError("stage1 packs one video per microbatch")
        F = latents.shape[1]
        n_chunks = (F + o.chunk_frames - 1) // o.chunk_frames
        noise = torch.randn(latents.shape, generator=self.gen, device=self.device, dtype=torch.float32).to(latents.dtype)
        if o.objective == "tf_fm":
            sig = logit_normal_sigmas(n_chunks, o.timestep_shift, generator=self.gen, device=self.device)
            if self.sp is not None and self.sp.size > 1:
                self.sp.broadcast_(sig, noise)
            t_chunk = sig * self.scheduler.num_train_timesteps
            t = self._per_chunk(t_chunk, F)
            x_t, target = self._noised(latents, noise, t)
            pred = self._predict(latents, x_t, t, text)
            weight = self._per_chunk(self.scheduler.training_weight(t_chunk), F).reshape(F)
            loss = ops.weighted_masked_mse(pred[0].contiguous(), target[0][:, :pred.shape[2]].contiguous(),
                                           weight.float(), torch.ones(F, device=self.device))
        elif o.objective == "anyflow":
            loss = self._anyflow_loss(latents, noise, text, n_chunks)
        else:
            raise ValueError(f"unknown stage1 objective {o.objective!r}")
        (loss / (o.grad_accum * self.sp_size * self.dp_size)).backward()
        return loss.detach()

    def _anyflow_loss(self, latents, noise, text, n_chunks):
        o = self.opts
        N = self.scheduler.num_train_timesteps
        F = latents.shape[1]
        pairs = af.sample_time_pairs(n_chunks, dp_rank=o.dp_rank, dp_world=o.dp_world,
                                     diffusion_ratio=o.diffusion_ratio, consistency_ratio=o.consistency_ratio,
                                     generator=self.gen, device=self.device)
        t_c = af.apply_timestep_shift(pairs.t, o.timestep_shift) * N
        r_c = af.apply_timestep_shift(pairs.r, o.timestep_shift) * N
        if self.sp is not None and self.sp.size > 1:
            self.sp.broadcast_(t_c, r_c, noise)
        t, r = self._per_chunk(t_c, F), self._per_chunk(r_c, F)
        x_t, target = self._noised(latents, noise, t)
        need = ~pairs.is_diffusion                                  # diffusion samples (r = t) have no du/dt term
        probes = bool(need.any())
        if self.sp is not None and self.sp.size > 1:                # SP peers take the same branch
            flag = torch.tensor([float(probes)], device=self.device)
            self.sp.broadcast_(flag)
            probes = bool(flag.item())
        # the clean half is the same in the trainable evaluation and in both probes: its keys / values are kept
        # (the suffix evaluation carries no cameras, so camera-conditioned steps evaluate the probes in full)
        prefix = [] if (probes and o.reuse_prefix and getattr(self, "y_camera", None) is None) else None
        u = self._predict(latents, x_t, t, text, r=r, capture=prefix)
        # central difference along the interpolation path x(t') = (1 - s') x0 + s' n, s' = t' / N
        tp_c, tm_c = af.difference_window(t_c, r_c, epsilon=o.difference_epsilon, num_train_timesteps=N)
        if probes:
            with torch.no_grad():
                tp, tm = self._per_chunk(tp_c, F), self._per_chunk(tm_c, F)
                x_p, _ = self._noised(latents, noise, tp)
                x_m, _ = self._noised(latents, noise, tm)
                u_p = self._predict(latents, x_p, tp, text, r=r, captured=prefix)
                u_m = self._predict(latents, x_m, tm, text, r=r, captured=prefix)
                du = af.central_difference(u_p[0], u_m[0], tp.reshape(F) / N, tm.reshape(F) / N)
        else:
            du = torch.zeros_like(u[0], dtype=torch.float32)
        resid = af.anyflow_residual(u[0], du, t.reshape(F), r.reshape(F), target[0][:, :u.shape[2]],
                                    num_train_timesteps=N)
        per_frame = resid.square().mean(dim=(1, 2, 3))
        w = self._per_chunk(af.gaussian_timestep_weights(t_c, shift=o.timestep_shift, num_train_timesteps=N), F).reshape(F)
        per_chunk = (per_frame * w.to(per_frame)).view(-1)
        ids = torch.arange(F, device=self.device) // o.chunk_frames
        chunk_loss = torch.zeros(n_chunks, device=self.device).index_add_(0, ids, per_chunk) / \
            torch.zeros(n_chunks, device=self.device).index_add_(0, ids, torch.ones_like(per_chunk))
        chunk_loss = af.adaptive_rescale(chunk_loss, pairs.is_diffusion, process_group=self.dp_group)
        return chunk_loss.mean()


def run_stage1_training(config: Mapping[str, Any]):
    """Config-driven entry used by the backend boundary: builds the trainer from the resolved config and
    runs the generic training engine with the stage-1 step."""
    from .runtime import build_training_run

    train = config["train"]
    causal = config["model"].get("causal", {}) or {}
    extra = dict(objective="anyflow" if str(train.get("objective", "")).startswith("anyflow") else "tf_fm",
                 chunk_frames=int(causal.get("chunk_frames", 3)), window_chunks=int(causal.get("window_chunks", 6)),
                 sink_frames=int(causal.get("sink_frames", 0)),
                 diffusion_ratio=float(train.get("diffusion_ratio", 0.5)),
                 consistency_ratio=float(train.get("consistency_ratio", 0.25)))
    return build_training_run(config, trainer_cls=WanStage1Trainer, options_cls=Stage1Options,
                              extra_options=extra).run()
