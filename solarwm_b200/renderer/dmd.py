"""Few-step distillation of the renderer (distribution matching, structure-guided teacher).

The student renders in ``student_steps`` Euler steps.  For one sample: the student's render (with
gradients on its last step) is re-noised to a random level; the frozen teacher scores it twice --
with and without the structure stream -- and the two are combined as
``free + guidance * (real - free)``; the critic (trained by flow matching on the student's renders)
gives the fake score; the student follows the KL-gradient surrogate of ``engine/sgf.py``
(reference: solar/renderer/dmd.py:20-, dmd_runtime.py:34-344).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ..backends.minimax_h3 import flow
from ..backends.minimax_h3.layout import patchify_latents
from ..backends.minimax_h3.stage2 import share_base
from ..engine.master_adamw import FP32MasterAdamW
from ..engine.sgf import sgf_kl_gradient, sgf_student_loss, should_update_student
from ..models.h3 import H3DiT, LoRALinear
from .core import packed_forward, render


def structure_guided(real: torch.Tensor, free: torch.Tensor, guidance: float) -> torch.Tensor:
    return free + guidance * (real - free)


class RendererDMDTrainer:
    def __init__(self, cfg, device, *, student_steps: int = 4, guidance: float = 2.0, critic_updates_per_student: int = 5,
                 lr_student: float = 2e-6, lr_critic: float = 4e-7, seed: int = 0):
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.device = torch.device(device)
        self.student = H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        self.critic = H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        share_base(self.critic, self.student)
        self.opt_s = FP32MasterAdamW(self.student.trainable_parameters(), lr=lr_student, betas=(0.0, 0.999))
        self.opt_c = FP32MasterAdamW(self.critic.trainable_parameters(), lr=lr_critic, betas=(0.0, 0.999))
        self.steps, self.guidance, self.ratio = student_steps, guidance, critic_updates_per_student
        self.gen = torch.Generator(device=self.device).manual_seed(seed * 100003 + 31)
        self.global_step = self.student_step = 0
        self.teacher = None                 # ``set_teacher``: the control-trained renderer as a frozen third role
        self.sync = None                    # ``sync(params, flat_fp32_grad)``: the runtime's reduction over the replicas

    def set_teacher(self, adapter_state: Mapping[str, torch.Tensor]) -> None:
        """The teacher of a renderer distillation is the control-trained renderer: the shared base with ITS adapters,
        frozen.  Without one the base alone (the student with its adapters off) stands in."""
        t = H3DiT(self.student.cfg, device=self.device, dtype=self.student.dtype, seed=0)
        share_base(t, self.student)
        own = {n: p for n, p in t.named_parameters() if p.requires_grad}
        if set(own) != set(adapter_state):
            raise ValueError("the teacher's adapter file does not hold exactly this architecture's adapter tensors")
        with torch.no_grad():
            for n, p in own.items():
                p.copy_(adapter_state[n].to(p))
        self.teacher = t.eval().requires_grad_(False)

    def _finish(self, opt, label: str) -> float:
        flat = opt.gather_grads()
        if self.sync is not None:
            self.sync(opt.params, flat)
        norm = float(opt.clip_(10.0))
        if not (norm == norm and norm != float("inf")):
            opt.zero_grad()
            raise FloatingPointError(f"non-finite renderer distillation {label} gradient norm")
        opt.step()
        opt.zero_grad()
        return norm

    def _teacher(self):
        student = self.student

        class _Off:
            def __enter__(s):
                s.saved = [(m, m.rank) for m in student.modules() if isinstance(m, LoRALinear)]
                for m, _ in s.saved:
                    m.rank = 0

            def __exit__(s, *a):
                for m, r in s.saved:
                    m.rank = r
        return _Off()

    def _x0(self, model, sample, x_rows, t: float, with_structure: bool):
        dev, dt = self.device, model.dtype
        C, F, H, W = sample["shape"]
        structure = sample.get("structure_latents") if with_structure else None
        v = packed_forward(model, prompt=sample["prompt_embeds"].to(dev, dt),
                           anchor_rows=patchify_latents(sample["anchor_latents"].to(dev)).to(dt),
                           structure_rows=None if structure is None else patchify_latents(structure.to(dev)).to(dt),
                           target_rows=x_rows.to(dt), row_times=torch.full((x_rows.shape[0],), float(t), device=dev),
                           grid_hw=(H // 2, W // 2), cameras=sample.get("camera_w2c"))
        return x_rows.float() + (1.0 - float(t)) * v.float(), v

    def train_outer_step(self, sample: Mapping[str, torch.Tensor]) -> Mapping[str, float]:
        dev = self.device
        update_student = should_update_student(self.global_step, self.ratio)
        # student render: all but the last step without gradients
        times = flow.rollout_times(self.steps, flow.VIDEO_SHIFT)
        with torch.no_grad():
            lat = render(self.student, sample, steps=self.steps - 1, seed=int(torch.randint(0, 2 ** 31 - 1, (1,), generator=self.gen, device=dev)))
        x_rows = patchify_latents(lat).float()
        t_last = float(times[self.steps - 1])
        noise = torch.randn(x_rows.shape, generator=self.gen, device=dev)
        x_in = t_last * x_rows + (1 - t_last) * noise
        with torch.set_grad_enabled(update_student):
            out, _ = self._x0(self.student, sample, x_in, t_last, True)
        result = {}
        if update_student:
            t_s = float(0.02 + 0.96 * torch.rand(1, generator=self.gen, device=dev))
            n2 = torch.randn(x_rows.shape, generator=self.gen, device=dev)
            x_t = t_s * out.detach() + (1 - t_s) * n2
            with torch.no_grad():
                fake, _ = self._x0(self.critic, sample, x_t, t_s, True)
                if self.teacher is not None:
                    real, _ = self._x0(self.teacher, sample, x_t, t_s, True)
                    free, _ = self._x0(self.teacher, sample, x_t, t_s, False)
                else:
                    with self._teacher():
                        real, _ = self._x0(self.student, sample, x_t, t_s, True)
                        free, _ = self._x0(self.student, sample, x_t, t_s, False)
                real = structure_guided(real, free, self.guidance)
                if not bool(torch.isfinite(fake).all() and torch.isfinite(real).all()):
                    raise FloatingPointError("non-finite renderer distillation score")
            g = sgf_kl_gradient(fake_x0=fake.unsqueeze(0), real_x0=real.unsqueeze(0), student_output=out.detach().unsqueeze(0))
            loss_s = sgf_student_loss(out.unsqueeze(0), g)
            loss_s.backward()
            result["student_grad_norm"] = self._finish(self.opt_s, "student")
            result["student"] = float(loss_s.detach())
            self.student_step += 1
        t_c = float(0.02 + 0.96 * torch.rand(1, generator=self.gen, device=dev))
        n3 = torch.randn(x_rows.shape, generator=self.gen, device=dev)
        x0 = out.detach()
        _, vel = self._x0(self.critic, sample, t_c * x0 + (1 - t_c) * n3, t_c, True)
        loss_c = (vel.float() - (x0 - n3)).pow(2).mean()
        if not bool(torch.isfinite(loss_c)):
            raise FloatingPointError("non-finite renderer distillation critic loss")
        loss_c.backward()
        result["critic_grad_norm"] = self._finish(self.opt_c, "critic")
        result["critic"] = float(loss_c.detach())
        self.global_step += 1
        return result
