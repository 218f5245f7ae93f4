"""H3 Stage2: self-gradient forcing of the block-causal student.

Roles share one frozen bf16 base; they differ only in their adapters:
  * student  (LoRA trained)  -- block-causal, rolled out with the streaming generator;
  * critic   (LoRA trained)  -- bidirectional "fake" score, flow matching on the student's samples;
  * teacher  (no adapter)    -- bidirectional "real" score, classifier-free guided.

Outer step: no-grad streaming rollout (4 denoise + 1 commit evaluations per chunk, random exit step) ->
one teacher-forcing replay with gradients under the W6 visibility rule -> critic update every step,
student update every ``critic_updates_per_student``-th step with the KL-gradient surrogate
(reference: solar/backends/minimax_h3/stage2.py:16-150, stage2_runtime.py, sgf_rollout.py:147-330,
solar/training/sgf.py).
"""
from __future__ import annotations

from typing import Mapping

import torch

from ...engine.master_adamw import FP32MasterAdamW
from ...engine.sgf import sgf_kl_gradient, sgf_student_loss, should_update_student
from ...models.h3 import H3DiT, LoRALinear
from ...serve.h3_stream import H3StreamConfig, H3StreamingGenerator
from . import flow
from .layout import build_layout, expand_cameras, patchify_latents
from .stage1 import teacher_forcing_forward


def share_base(dst: H3DiT, src: H3DiT) -> None:
    """Alias every frozen tensor of ``dst`` to ``src``'s (adapters stay private): three roles, one base."""
    src_mods = dict(src.named_modules())
    for name, mod in dst.named_modules():
        if isinstance(mod, LoRALinear):
            mod.weight = src_mods[name].weight
    src_params = dict(src.named_parameters())
    for name, p in list(dst.named_parameters()):
        if not p.requires_grad and "lora_" not in name and name in src_params:
            parent, _, leaf = name.rpartition(".")
            setattr(dst.get_submodule(parent) if parent else dst, leaf, src_params[name])


class H3Stage2Trainer:
    def __init__(self, cfg, device, *, chunk_latents: int = 5, window_chunks: int = 5, denoise_steps: int = 4,
                 grid_hw=(4, 4), lr_student: float = 2e-6, lr_critic: float = 4e-7, critic_updates_per_student: int = 5,
                 guidance_scale: float = 3.0, seed: int = 0):
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.device = torch.device(device)
        self.student = H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        self.critic = H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        share_base(self.critic, self.student)
        self.opt_s = FP32MasterAdamW(self.student.trainable_parameters(), lr=lr_student, betas=(0.0, 0.999))
        self.opt_c = FP32MasterAdamW(self.critic.trainable_parameters(), lr=lr_critic, betas=(0.0, 0.999))
        self.stream_cfg = H3StreamConfig(grid_hw=grid_hw, latent_channels=cfg.latent_row_dim // 4,
                                         chunk_latents=chunk_latents, window_chunks=window_chunks,
                                         denoise_steps=denoise_steps, use_cuda_graph=False, seed=seed)
        self.ratio, self.scale = critic_updates_per_student, guidance_scale
        self.gen = torch.Generator(device=self.device).manual_seed(seed * 100003 + 11)
        self.global_step = self.student_step = 0
        self.teacher = None                    # ``set_teacher``: a third role with its own frozen adapters
        self.sync = None                       # ``sync(params, flat_fp32_grad)``: the runtime's reduction over ranks
        self.silence = None                    # packed rows of encoded silence [Na, 32]: the replay's and the scores' audio

    def set_teacher(self, adapter_state: Mapping[str, torch.Tensor], seed: int = 0) -> None:
        """Build the teacher role: the shared frozen base with the given adapter weights, never trained."""
        t = H3DiT(self.student.cfg, device=self.device, dtype=self.student.dtype, seed=seed)
        share_base(t, self.student)
        own = dict(t.named_parameters())
        wanted = {n for n, p in own.items() if p.requires_grad}
        if set(adapter_state) != wanted:
            raise ValueError("the teacher's adapter file does not hold exactly this architecture's adapter tensors")
        with torch.no_grad():
            for n in wanted:
                own[n].copy_(adapter_state[n].to(own[n]))
        self.teacher = t.eval().requires_grad_(False)

    # ------------------------------------------------------------------------------------
    def _adapters_off(self, model):
        class _Off:
            def __enter__(s):
                s.saved = [(m, m.rank) for m in model.modules() if isinstance(m, LoRALinear)]
                for m, _ in s.saved:
                    m.rank = 0
            def __exit__(s, *a):
                for m, r in s.saved:
                    m.rank = r
        return _Off()

    def _audio(self):
        """The silent soundtrack at a freshly drawn audio time, ``(rows, t_audio)``, or None when no silence is set."""
        if self.silence is None:
            return None
        from .silence import noised_silence

        return noised_silence(self.silence, self.gen, self.device)

    def _bidirectional_x0(self, model, x_t, t: float, sample, cameras, audio=None):
        """x0 prediction of a bidirectional evaluation on the packed document; x_t [C, F, H, W]; ``audio`` as ``_audio``
        returns it (evaluations that are compared with one another get the same one)."""
        dev, dt = self.device, model.dtype
        C, F, H, W = x_t.shape
        prompt = sample["prompt_embeds"].to(dev, dt)
        layout = build_layout(n_text=prompt.shape[0], latent_frames=F, grid_hw=(H // 2, W // 2), t_video=float(t),
                              n_audio=0 if audio is None else audio[0].shape[0], t_audio=0.5 if audio is None else audio[1])
        view = None if cameras is None else expand_cameras(layout, cameras)
        vid, _ = model(video_rows=patchify_latents(x_t).to(dt), text_rows=prompt,
                       audio_rows=None if audio is None else audio[0].to(dt),
                       anchor_rows=patchify_latents(sample["anchor_latents"].to(dev)).to(dt), timesteps=layout.timesteps,
                       t_index=layout.t_index.to(dev), tags=layout.tags.to(dev), position_ids=layout.position_ids,
                       viewmats=view)
        return patchify_latents(x_t).float() + (1.0 - float(t)) * vid.float(), vid

    @torch.no_grad()
    def rollout(self, sample, n_chunks: int, cameras):
        gen = H3StreamingGenerator(self.student, self.stream_cfg)
        gen.gen = self.gen
        gen.start(sample["prompt_embeds"].to(self.device), sample["anchor_latents"].to(self.device),
                  None if cameras is None else cameras[0])
        k = self.stream_cfg.chunk_latents
        chunks = [gen.next_chunk(None if cameras is None else cameras[1 + i * k:1 + (i + 1) * k]) for i in range(n_chunks)]
        exit_index = int(torch.randint(0, len(gen.times), (1,), generator=self.gen, device=self.device).item())
        return torch.cat(chunks, dim=1), float(gen.times[exit_index])

    def _replay(self, sample, n_chunks: int, *, grad: bool):
        """Roll the student out (no gradient), then evaluate it once under teacher forcing at the exit time; returns
        the student's clean-sample rows (with a graph when ``grad``) and the latent geometry."""
        dev = self.device
        cams = sample.get("camera_w2c")
        generated, t_exit = self.rollout(sample, n_chunks, cams)                     # [C, F, H, W]
        C, F, H, W = generated.shape
        dt = self.student.dtype
        noise = torch.randn(generated.shape, generator=self.gen, device=dev, dtype=torch.float32)
        clean_rows = patchify_latents(generated).to(dt)
        noisy_rows = (t_exit * clean_rows.float() + (1 - t_exit) * patchify_latents(noise)).to(dt)
        anchor_rows = patchify_latents(sample["anchor_latents"].to(dev)).to(dt)
        audio = self._audio()
        extra = {} if audio is None else {"audio_rows": audio[0].to(dt), "t_audio": audio[1]}
        with torch.set_grad_enabled(grad):
            v = teacher_forcing_forward(self.student, prompt=sample["prompt_embeds"].to(dev, dt), anchor_rows=anchor_rows, **extra,
                                        clean_rows=clean_rows, noisy_rows=noisy_rows,
                                        t_chunks=torch.full((n_chunks,), t_exit, device=dev), grid_hw=(H // 2, W // 2),
                                        chunk_latents=self.stream_cfg.chunk_latents,
                                        window_chunks=self.stream_cfg.window_chunks, cameras=cams)
            out_rows = noisy_rows.float() + (1 - t_exit) * v.float()                 # student x0 (rows)
        return out_rows, (C, F, H, W)

    def _finish(self, opt, label: str) -> float:
        """Pack the gradients, let the runtime reduce them over the ranks, refuse non-finite norms, clip, step."""
        flat = opt.gather_grads()
        if self.sync is not None:
            self.sync(opt.params, flat)
        norm = float(opt.clip_(10.0))
        if not (norm == norm and norm != float("inf")):
            opt.zero_grad()
            raise FloatingPointError(f"non-finite H3 SGF {label} gradient norm")
        opt.step()
        opt.zero_grad()
        return norm

    def _real_x0(self, x_t, t_s, sample, cams, audio=None):
        """The guided "real" score: the teacher role when one was built, else the student with its adapters off."""
        import contextlib

        model = self.teacher if self.teacher is not None else self.student
        scope = contextlib.nullcontext() if self.teacher is not None else self._adapters_off(self.student)
        with scope:
            real, _ = self._bidirectional_x0(model, x_t, t_s, sample, cams, audio)
            if self.scale != 1.0:
                null = dict(sample, prompt_embeds=torch.zeros_like(sample["prompt_embeds"]))
                real_u, _ = self._bidirectional_x0(model, x_t, t_s, null, cams, audio)
                real = real_u + self.scale * (real - real_u)
        return real

    def student_phase(self, sample: Mapping[str, torch.Tensor], n_chunks: int = 2) -> Mapping[str, float]:
        from .layout import unpatchify_rows

        dev, dt, cams = self.device, self.student.dtype, sample.get("camera_w2c")
        out_rows, (C, F, H, W) = self._replay(sample, n_chunks, grad=True)
        out_lat = unpatchify_rows(out_rows.detach().to(dt), C, F, H, W)
        t_s = float(0.02 + 0.96 * torch.rand(1, generator=self.gen, device=dev))
        n2 = torch.randn((C, F, H, W), generator=self.gen, device=dev, dtype=torch.float32).to(dt)
        x_t = flow.interpolate(out_lat, n2, t_s)
        audio = self._audio()                       # one silent soundtrack for the scores that are subtracted
        with torch.no_grad():
            fake, _ = self._bidirectional_x0(self.critic, x_t, t_s, sample, cams, audio)
            real = self._real_x0(x_t, t_s, sample, cams, audio)
            if not bool(torch.isfinite(fake).all() and torch.isfinite(real).all()):
                raise FloatingPointError("non-finite H3 SGF score output")
        g = sgf_kl_gradient(fake_x0=fake.unsqueeze(0), real_x0=real.unsqueeze(0), student_output=out_rows.detach().unsqueeze(0))
        loss_s = sgf_student_loss(out_rows.unsqueeze(0), g)
        loss_s.backward()
        norm = self._finish(self.opt_s, "student")
        self.student_step += 1
        return {"student": float(loss_s.detach()), "student_grad_norm": norm}

    def critic_phase(self, sample: Mapping[str, torch.Tensor], n_chunks: int = 2, replayed=None) -> Mapping[str, float]:
        """Flow matching of the critic on the student's sample (``replayed``: rows and geometry of a replay that was
        just made on the same sample, so the single-sample form of the outer step does not roll out twice)."""
        from .layout import unpatchify_rows

        dev, dt, cams = self.device, self.student.dtype, sample.get("camera_w2c")
        out_rows, (C, F, H, W) = replayed if replayed is not None else self._replay(sample, n_chunks, grad=False)
        out_lat = unpatchify_rows(out_rows.detach().to(dt), C, F, H, W)
        t_c = float(0.02 + 0.96 * torch.rand(1, generator=self.gen, device=dev))
        n3 = torch.randn((C, F, H, W), generator=self.gen, device=dev, dtype=torch.float32).to(dt)
        x_tc = flow.interpolate(out_lat, n3, t_c)
        _, vel = self._bidirectional_x0(self.critic, x_tc, t_c, sample, cams, self._audio())
        target = patchify_latents(out_lat.float() - n3.float())
        loss_c = (vel.float() - target).pow(2).mean()
        if not bool(torch.isfinite(loss_c)):
            raise FloatingPointError("non-finite H3 SGF critic loss")
        loss_c.backward()
        norm = self._finish(self.opt_c, "critic")
        return {"critic": float(loss_c.detach()), "critic_grad_norm": norm}

    def train_outer_step(self, sample: Mapping[str, torch.Tensor], n_chunks: int = 2, critic_sample=None) -> Mapping[str, float]:
        """One outer step: the student phase on every ``critic_updates_per_student``-th step, the critic phase always.
        With ``critic_sample`` the two phases see different samples (two rollouts, as the training runtime does);
        without it the critic learns from the replay the student phase just made."""
        result = {}
        update_student = should_update_student(self.global_step, self.ratio)
        if critic_sample is None:
            out_rows, geometry = self._replay(sample, n_chunks, grad=update_student)
            if update_student:
                held = self._replay
                self._replay = lambda *a, **k: (out_rows, geometry)          # the phase consumes the replay made above
                try:
                    result.update(self.student_phase(sample, n_chunks))
                finally:
                    self._replay = held
            result.update(self.critic_phase(sample, n_chunks, replayed=(out_rows.detach(), geometry)))
        else:
            if update_student:
                result.update(self.student_phase(sample, n_chunks))
            result.update(self.critic_phase(critic_sample, n_chunks))
        self.global_step += 1
        return result
