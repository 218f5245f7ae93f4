"""Wan Stage2: self-gradient forcing (distribution-matching distillation of a few-step causal student).

Three networks share one architecture:
  * **student** (trainable, block-causal): rolls a video out chunk by chunk with its own KV cache;
  * **teacher** (frozen, bidirectional): the "real" score, evaluated with classifier-free guidance;
  * **critic** (trainable, bidirectional): the "fake" score, trained by flow matching on the
    student's samples.

One outer step (``train_outer_step``):
  1. ``rollout``: no-grad chunked rollout through the denoising grid with the rolling KV cache; a
     random exit index (shared by all chunks and SP ranks) picks the step whose input the gradient
     pass will see; every chunk is committed clean to the cache.
  2. one gradient pass: teacher-forcing replay of the whole clip, ``[generated clean | re-noised at
     the exit step]`` -> student x0 ``out``.
  3. critic update (every step): flow matching on ``add_noise(out.detach(), t')``.
  4. student update (every ``critic_updates_per_student``-th step): ``g = (fake_x0 - real_x0) /
     mean|out - real_x0|`` and the surrogate ``0.5 ||out - (out - g).detach()||^2``.

Reference: stage2_camera_rollout, _stage2_self_forcing_latents and Wan5BStage2Runtime.train_outer_step
(solar/backends/wan22/runtime/stage2.py:408-771, 2055), solar/training/sgf.py:9-78.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Sequence

import torch

from ... import ops
from ...engine.flow import FlowMatchScheduler
from ...engine.optim import FlatAdamW
from ...errors import BackendContractError
from ...engine.sgf import sgf_kl_gradient, sgf_student_loss, should_update_student
from ...models.wan import WanConfig, WanDiT
from ...models.wan_causal import CausalWanRunner, allocate_kv_cache
from ...models.wan_tf import forward_teacher_forcing


@dataclass
class Stage2Options:
    lr_student: float = 2e-6
    lr_critic: float = 4e-7
    betas: tuple = (0.0, 0.999)
    weight_decay: float = 0.01
    max_grad_norm: Optional[float] = 10.0
    timestep_shift: float = 5.0
    denoising_steps: Sequence[float] = (1000.0, 750.0, 500.0, 250.0)
    chunk_frames: int = 3
    window_chunks: int = 6
    sink_frames: int = 0
    critic_updates_per_student: int = 5
    guidance_scale: float = 3.0
    min_score_t: float = 20.0
    max_score_t: float = 980.0
    checkpointing: str = "none"
    ema_decay: Optional[float] = None      # per-role EMA: a fp32 shadow of the student, updated after each of its steps
    ema_start_step: int = 39               # until this outer step the shadow simply follows the student (decay 0)
    seed: int = 0


def _to_bcfhw(x):
    return x.permute(0, 2, 1, 3, 4)


class WanStage2Trainer:
    def __init__(self, cfg: WanConfig, device, opts: Stage2Options = Stage2Options(), sp=None,
                 dtype=torch.bfloat16, student: Optional[WanDiT] = None, teacher: Optional[WanDiT] = None,
                 critic: Optional[WanDiT] = None):
        self.cfg, self.opts, self.device = cfg, opts, torch.device(device)
        self.sp = sp
        self.sp_size = 1 if sp is None else sp.size
        self.dp_group, self.dp_size = None, 1      # ``run_stage2_training`` sets them for data-parallel replicas
        mk = lambda seed: WanDiT(cfg, device=device, dtype=dtype, seed=seed)   # noqa: E731
        self.student = student or mk(opts.seed)
        self.teacher = teacher or mk(opts.seed)
        self.critic = critic or mk(opts.seed)
        for m in (self.student, self.teacher, self.critic):
            if sp is not None:
                m.sp = sp
            m.checkpointing = opts.checkpointing
        for p in self.teacher.parameters():
            p.requires_grad_(False)
        self.student.ensure_grads()
        self.critic.ensure_grads()
        kw = dict(betas=opts.betas, eps=1e-8, weight_decay=opts.weight_decay)
        self.opt_student = FlatAdamW(self.student.units(), lr=opts.lr_student, **kw)
        self.opt_critic = FlatAdamW(self.critic.units(), lr=opts.lr_critic, **kw)
        self.scheduler = FlowMatchScheduler(shift=opts.timestep_shift)
        self.gen = torch.Generator(device=self.device).manual_seed(opts.seed * 100003 + 7)
        self.global_step = 0
        self.ema_student = None
        if opts.ema_decay is not None:
            from ...engine.ema import ShardedEMA

            self.ema_student = ShardedEMA(self.student, decay=float(opts.ema_decay), device=self.device, dtype=torch.float32)

    # ------------------------------------------------------------------------------------
    def _sigma(self, t):
        return (torch.as_tensor(t, device=self.device, dtype=torch.float32) / self.scheduler.num_train_timesteps)

    def _add_noise(self, x0, noise, t_frames):
        """x0 / noise [1, F, C, H, W], t_frames [F] -> x_t [1, F, C, H, W]."""
        x_t, _ = ops.add_noise(x0[0].contiguous(), noise[0].contiguous(), self._sigma(t_frames))
        return x_t.unsqueeze(0)

    def _x0(self, x_t, v, t_frames):
        return ops.flow_to_x0(x_t[0].contiguous(), v[0].contiguous(), self._sigma(t_frames)).unsqueeze(0)

    def _randn(self, shape, dtype):
        return torch.randn(shape, generator=self.gen, device=self.device, dtype=torch.float32).to(dtype)

    # ------------------------------------------------------------------------------------
    def rollout_cache(self, grid_hw):
        """The student's rolling KV cache (sink + window + one chunk, per block) for a token grid, allocated ONCE per
        geometry and reset between rollouts, so no step of the training loop allocates cache memory (reference:
        allocate_kv_cache / allocate_crossattn_cache, solar/backends/wan22/runtime/stage2.py:1758-1854; the projected
        text keys / values, its cross-attention cache, are rebuilt per sample by ``encode_text``)."""
        caches = self.__dict__.setdefault("_rollout_caches", {})
        key = tuple(int(v) for v in grid_hw)
        cache = caches.get(key)
        if cache is None:
            o = self.opts
            cache = caches[key] = allocate_kv_cache(self.student, grid_hw=key, chunk_frames=o.chunk_frames,
                                                    window_frames=o.window_chunks * o.chunk_frames + o.sink_frames,
                                                    sink_frames=o.sink_frames, device=self.device)
        cache.reset()
        return cache

    @torch.no_grad()
    def rollout(self, text, shape, dtype, exit_index: Optional[int] = None):
        """Chunked no-grad rollout.  Returns (generated x0 [1,F,C,H,W], exit timestep, exit_index)."""
        o = self.opts
        _, F, C, H, W = shape
        steps = list(o.denoising_steps)
        if exit_index is None:
            idx = torch.randint(0, len(steps), (1,), generator=self.gen, device=self.device)
            if self.sp is not None and self.sp.size > 1:
                self.sp.broadcast_(idx)
            exit_index = int(idx.item())
        runner = CausalWanRunner(self.student, sp=None)
        ph, pw = self.cfg.patch_size[1], self.cfg.patch_size[2]
        cache = self.rollout_cache((H // ph, W // pw))
        runner.encode_text(cache, text)
        outs = []
        cam_all = getattr(self, "y_camera", None)      # set per batch by ``train_outer_step``: every chunk carries its cameras

        def cams(a, b):
            if cam_all is None:
                return {}
            return {"y_camera": {"viewmats": cam_all["viewmats"][:, a:b], "Ks": None if cam_all["Ks"] is None else cam_all["Ks"][:, a:b],
                                 "transform": cam_all["transform"]}}

        for f0 in range(0, F, o.chunk_frames):
            f = min(o.chunk_frames, F - f0)
            x = self._randn((1, f, C, H, W), dtype)
            x0 = x
            for si, t in enumerate(steps):
                tt = torch.full((1, f), float(t), device=self.device)
                v = runner.forward_chunk(cache, _to_bcfhw(x), tt, commit=False, **cams(f0, f0 + f))
                x0 = self._x0(x, _to_bcfhw(v), tt[0])
                if si + 1 < len(steps):
                    x = self._add_noise(x0, self._randn(x0.shape, dtype), torch.full((f,), float(steps[si + 1])))
            runner.forward_chunk(cache, _to_bcfhw(x0), torch.zeros((1, f), device=self.device), commit=True, **cams(f0, f0 + f))
            outs.append(x0)
        return torch.cat(outs, dim=1), float(steps[exit_index]), exit_index

    def student_replay(self, generated, text, exit_t: float):
        """One gradient pass over the clip: the student denoises ``generated`` re-noised at ``exit_t`` while
        attending to the clean ``generated`` history.  Returns x0 [1,F,C,H,W] with grad."""
        o = self.opts
        F = generated.shape[1]
        t = torch.full((F,), float(exit_t), device=self.device)
        noisy = self._add_noise(generated, self._randn(generated.shape, generated.dtype), t)
        v = forward_teacher_forcing(self.student, _to_bcfhw(generated), _to_bcfhw(noisy), t.view(1, F), text,
                                    chunk_frames=o.chunk_frames, window_chunks=o.window_chunks,
                                    sink_frames=o.sink_frames, y_camera=getattr(self, "y_camera", None))
        v = _to_bcfhw(v)
        sig = self._sigma(t).view(1, F, 1, 1, 1)
        return (noisy.float() - sig * v.float())

    def _score_x0(self, model, x_t, t_frames, text, null_text=None, scale: float = 1.0):
        F = x_t.shape[1]
        tt = t_frames.view(1, F)
        cam = getattr(self, "y_camera", None)          # the scores see the same trajectory the student rolled out along
        v = model(_to_bcfhw(x_t), tt, text, y_camera=cam)
        if null_text is not None and scale != 1.0:
            vu = model(_to_bcfhw(x_t), tt, null_text, y_camera=cam)
            v = vu + scale * (v - vu)
        sig = self._sigma(t_frames).view(1, F, 1, 1, 1)
        return x_t.float() - sig * _to_bcfhw(v).float()

    def _apply(self, model, opt):
        model.finalize_grads()
        if self.sp is not None and self.sp.size > 1:
            self.sp.sum_gradients_([g for u in model.units() for g in (u.grad, u.grad_v)])
        if self.dp_size > 1:                       # replicas rolled out different prompts: average their gradients
            import torch.distributed as dist

            for u in model.units():
                for g in (u.grad, u.grad_v):
                    dist.all_reduce(g, group=self.dp_group)
                    g.mul_(1.0 / self.dp_size)
        norm = opt.local_grad_sumsq().sqrt()
        opt.set_clip(norm, self.opts.max_grad_norm)
        opt.step()
        model.zero_grads()
        return norm

    def train_outer_step(self, batch: Mapping[str, Any]):
        """batch: ``latents`` (shape/dtype template only; SGF trains data-free), ``text`` and optional
        ``null_text`` [1, T, text_dim].  Returns a dict of scalar losses."""
        o = self.opts
        dev = self.device
        lat = batch["latents"].to(dev, non_blocking=True)
        text = batch["text"].to(dev, non_blocking=True)
        from .runtime import camera_condition

        self.y_camera = camera_condition(batch, self.cfg, getattr(self, "camera_transform", "linear"), dev)
        null = batch.get("null_text")
        null = torch.zeros_like(text) if null is None else null.to(dev, non_blocking=True)
        F = lat.shape[1]
        generated, exit_t, _ = self.rollout(text, lat.shape, lat.dtype)
        update_student = should_update_student(self.global_step, o.critic_updates_per_student)
        result = {}
        with torch.set_grad_enabled(update_student):
            out = self.student_replay(generated, text, exit_t)                      # fp32 [1,F,C,H,W]
        # one score timestep per clip, shared by both score networks and by the SP group
        u = torch.rand(1, generator=self.gen, device=dev)
        if self.sp is not None and self.sp.size > 1:
            self.sp.broadcast_(u)
        t_score = (o.min_score_t + (o.max_score_t - o.min_score_t) * u).expand(F).contiguous()
        noise = self._randn(out.shape, lat.dtype)
        if update_student:
            x_t = self._add_noise(out.detach().to(lat.dtype), noise, t_score)
            with torch.no_grad():
                real = self._score_x0(self.teacher, x_t, t_score, text, null, o.guidance_scale)
                fake = self._score_x0(self.critic, x_t, t_score, text)
            g = sgf_kl_gradient(fake_x0=fake, real_x0=real, student_output=out.detach())
            loss_s = sgf_student_loss(out, g)
            (loss_s / self.sp_size).backward()
            result["student"] = float(loss_s.detach())
            result["student_grad_norm"] = float(self._apply(self.student, self.opt_student))
            if self.ema_student is not None:             # the role's own average: only student steps advance it
                from ...engine.ema import ema_decay_for_step

                self.ema_student.update(self.student, decay=ema_decay_for_step(
                    target_decay=self.opts.ema_decay, global_step=self.global_step, warmup_steps=self.opts.ema_start_step))
        # critic: flow matching on the student's sample
        x0 = out.detach().to(lat.dtype)
        u2 = torch.rand(1, generator=self.gen, device=dev)
        if self.sp is not None and self.sp.size > 1:
            self.sp.broadcast_(u2)
        t_c = (o.min_score_t + (o.max_score_t - o.min_score_t) * u2).expand(F).contiguous()
        noise_c = self._randn(out.shape, lat.dtype)
        x_tc, target = ops.add_noise(x0[0].contiguous(), noise_c[0].contiguous(), self._sigma(t_c))
        pred = self.critic(_to_bcfhw(x_tc.unsqueeze(0)), t_c.view(1, F), text)
        pred = _to_bcfhw(pred)[0].contiguous()
        loss_c = ops.weighted_masked_mse(pred, target[:, :pred.shape[1]].contiguous(),
                                         torch.ones(F, device=dev), torch.ones(F, device=dev))
        (loss_c / self.sp_size).backward()
        result["critic"] = float(loss_c.detach())
        result["critic_grad_norm"] = float(self._apply(self.critic, self.opt_critic))
        self.global_step += 1
        return result

    # -- role checkpoints ------------------------------------------------------------------
    def role_state(self) -> Mapping[str, Any]:
        return {"student": self.student.state_dict(), "critic": self.critic.state_dict(),
                "opt_student": self.opt_student.state_dict(), "opt_critic": self.opt_critic.state_dict(),
                "global_step": self.global_step, "objective_gen": self.gen.get_state().cpu(),
                **({} if self.ema_student is None else {"ema_student": self.ema_student.state_dict(),
                                                        "ema_student_updates": self.ema_student.num_updates})}

    def load_role_state(self, state: Mapping[str, Any]) -> None:
        self.student.load_state_dict(state["student"])
        self.critic.load_state_dict(state["critic"])
        self.opt_student.load_state_dict(state["opt_student"])
        self.opt_critic.load_state_dict(state["opt_critic"])
        self.global_step = int(state["global_step"])
        self.gen.set_state(state["objective_gen"])
        if self.ema_student is not None:
            if "ema_student" not in state:
                raise BackendContractError("the checkpoint carries no student EMA but ema_decay is set")
            self.ema_student.load_state_dict(state["ema_student"], num_updates=int(state["ema_student_updates"]))


def load_role_weights(model: WanDiT, source, *, role: str, weight_source: str = "live") -> Mapping[str, Any]:
    """Fill one role from an earlier run: a Stage2 checkpoint (``role.pt``: its ``student`` or ``critic``, or the student's
    average with ``weight_source: ema``) or a Stage0.5 / Stage1 checkpoint (``model.pt``: live or averaged weights).  The
    checkpoint is verified first; the receipt names what was taken."""
    from ...checkpoint.store import verify_checkpoint

    if weight_source not in ("live", "ema"):
        raise BackendContractError("weight_source is live or ema")
    verified = verify_checkpoint(source)
    root = verified.path
    if (root / "role.pt").is_file():
        doc = torch.load(root / "role.pt", map_location="cpu", weights_only=True)
        key = "ema_student" if weight_source == "ema" else ("critic" if role == "critic" else "student")
        if key not in doc:
            raise BackendContractError(f"{root} holds no {key} weights")
        state, taken = doc[key], f"role.pt:{key}"
    elif (root / "model.pt").is_file():
        doc = torch.load(root / "model.pt", map_location="cpu", weights_only=True)
        key = "ema" if weight_source == "ema" else "model"
        if doc.get(key) is None:
            raise BackendContractError(f"{root} holds no {key} weights")
        state, taken = doc[key], f"model.pt:{key}"
    else:
        raise BackendContractError(f"{root} holds neither role.pt nor model.pt")
    own = model.state_dict()
    if set(state) != set(own):
        missing, extra = sorted(set(own) - set(state))[:4], sorted(set(state) - set(own))[:4]
        raise BackendContractError(f"{taken} of {root} does not match the architecture: missing {missing}, unexpected {extra}")
    model.load_state_dict({k: v.to(own[k].dtype) for k, v in state.items()})
    return {"role": role, "source": str(root), "taken": taken, "checkpoint": verified.manifest_digest, "step": int(verified.step),
            "stage": verified.contract.stage}


def expected_student_updates(outer_steps: int, ratio: int) -> int:
    """How many of the first ``outer_steps`` outer steps updated the student (the rule of ``should_update_student``)."""
    return sum(1 for k in range(outer_steps) if should_update_student(k, ratio))


def run_stage2_training(config: Mapping[str, Any]) -> Mapping[str, Any]:
    """Config-driven entry.  Roles start from ``checkpoint.initialization.{student, teacher, critic}`` (``{path,
    weight_source}``; a role without one keeps its seeded random weights, a critic without one starts from the teacher's
    as the recipe does); ``checkpoint.resume_from`` restores both trainable roles, their optimizers, the student's
    average, every rank's random streams and the batch position, and checks that the saved counters agree with the
    update schedule; every outer step is an event line; role checkpoints go through the transactional store every
    ``runtime.save_every`` steps, at ``checkpoint.save_steps`` and at the end."""
    import torch.distributed as dist

    from ...checkpoint.store import CheckpointTransaction, verify_checkpoint
    from ...config.routes import validate_route
    from ...engine.train_engine import JsonlEventSink
    from ...parallel import dist_init
    from ...runtime import distributed as rdist
    from ...runtime.output_layout import checkpoint_model_dir, events_path, output_root
    from ...runtime.safe_state import capture_rank_state, restore_rank_state
    from .checkpoint import build_contract
    from .contracts import architecture
    from .runtime import encoded_batches, synthetic_batches

    dist_cfg = config.get("distributed", {}) or {}
    ctx = dist_init.initialize(int(dist_cfg.get("sequence_parallel_size", 1)),
                               device=str(config.get("runtime", {}).get("device", "auto")))
    try:
        topo = ctx.topology
        arch = architecture(config)
        train, rt, ck = config["train"], config.get("runtime", {}) or {}, config.get("checkpoint", {}) or {}
        causal = config["model"].get("causal", {}) or {}
        opts = Stage2Options(
            lr_student=float((train.get("optimizer", {}) or {}).get("lr", 2e-6)),
            lr_critic=float((train.get("critic_optimizer", {}) or {}).get("lr", 4e-7)),
            timestep_shift=float(config["model"].get("timestep_shift", 5.0)),
            denoising_steps=tuple(train.get("denoising_steps", (1000.0, 750.0, 500.0, 250.0))),
            chunk_frames=int(causal.get("chunk_frames", 3)), window_chunks=int(causal.get("window_chunks", 6)),
            sink_frames=int(causal.get("sink_frames", 0)),
            critic_updates_per_student=int(train.get("critic_updates_per_student", 5)),
            guidance_scale=float(train.get("guidance_scale", 3.0)), seed=int(config["data"].get("seed", 0)),
            ema_decay=(float(train["ema"]["decay"]) if (train.get("ema", {}) or {}).get("enabled") else None),
            ema_start_step=int((train.get("ema", {}) or {}).get("start_step", 39)))
        dtype = torch.bfloat16 if ctx.device.type == "cuda" else torch.float32
        trainer = WanStage2Trainer(arch, ctx.device, opts, sp=ctx.sp, dtype=dtype)
        trainer.dp_group, trainer.dp_size = ctx.dp_group, topo.dp_size
        trainer.camera_transform = str(config["model"].get("camera_translation_transform", "linear"))
        # replicas draw different noise; SP peers of one replica must draw the same
        trainer.gen.manual_seed(opts.seed * 100003 + 7 + 7919 * topo.dp_rank)
        receipts = {}
        init = ck.get("initialization", {}) or {}
        for role, model in (("student", trainer.student), ("teacher", trainer.teacher), ("critic", trainer.critic)):
            spec = init.get(role)
            if spec:
                spec = {"path": spec} if isinstance(spec, str) else dict(spec)
                receipts[role] = dict(load_role_weights(model, spec["path"], role=role, weight_source=str(spec.get("weight_source", "live"))))
        if "teacher" in receipts and "critic" not in receipts:
            trainer.critic.load_state_dict(trainer.teacher.state_dict())
            receipts["critic"] = dict(receipts["teacher"], role="critic", taken=receipts["teacher"]["taken"] + " (teacher's)")
        for role, opt, model in (("student", trainer.opt_student, trainer.student), ("critic", trainer.opt_critic, trainer.critic)):
            if role in receipts:
                opt.adopt_live_weights()
        if trainer.ema_student is not None and "student" in receipts:
            trainer.ema_student.update(trainer.student, decay=0.0)          # the average restarts at the loaded weights
            trainer.ema_student.num_updates = 0
        if str(config["data"].get("source", "synthetic")) == "index":       # prompts (and the shape template) from a corpus
            batches = encoded_batches(config, arch, ctx.device, topo.dp_rank, topo.dp_size)
        else:
            batches = synthetic_batches(dict(config, data=dict(config["data"], seed=int(config["data"].get("seed", 0)) + topo.dp_rank)),
                                        arch, ctx.device)
        consumed = 0
        if ck.get("resume_from"):
            verified = verify_checkpoint(str(ck["resume_from"]))
            run = torch.load(verified.path / "runtime.pt", weights_only=True)
            ranks = torch.load(verified.path / "rank-state.pt", weights_only=True)
            if int(ranks["world_size"]) != topo.raw_world_size or int(ranks["sp_size"]) != topo.sp_size:
                raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks (SP {ranks['sp_size']}); "
                                           f"{topo.raw_world_size} (SP {topo.sp_size}) are running")
            if run.get("initialization") != receipts:
                raise BackendContractError("the checkpoint's roles started from other weights than this configuration names")
            trainer.load_role_state(torch.load(verified.path / "role.pt", map_location=ctx.device, weights_only=True))
            want = expected_student_updates(trainer.global_step, opts.critic_updates_per_student)
            if int(run["student_updates"]) != want or int(run["global_step"]) != trainer.global_step:
                raise BackendContractError(f"checkpoint counters disagree with the update schedule: {run['student_updates']} student "
                                           f"updates at outer step {run['global_step']}, the schedule gives {want}")
            mine = ranks["ranks"][topo.raw_rank]
            restore_rank_state(mine, ctx.device)
            trainer.gen.set_state(mine["objective_gen"])
            for _ in range(int(mine["batches_consumed"])):
                next(batches)
            consumed = int(mine["batches_consumed"])
        max_steps = int(rt.get("max_steps_override") or train["max_steps"])
        save_every = int(rt.get("save_every", 0))
        save_steps = {int(v) for v in ck.get("save_steps", ())} | ({max_steps} if save_every > 0 or ck.get("save_steps") else set())
        sink = JsonlEventSink(events_path(output_root(config), topo.raw_rank))
        route = validate_route(config)

        def save(step: int) -> str:
            state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in capture_rank_state(ctx.device).items()}
            state.update(objective_gen=trainer.gen.get_state().cpu(), batches_consumed=consumed)
            states = [state]
            if topo.raw_world_size > 1:
                states = [None] * topo.raw_world_size
                dist.all_gather_object(states, state)
            target = checkpoint_model_dir(output_root(config), step)

            def write():
                with CheckpointTransaction(target) as tx:
                    torch.save(dict(trainer.role_state()), tx.path / "role.pt")
                    torch.save({"ranks": states, "world_size": topo.raw_world_size, "sp_size": topo.sp_size}, tx.path / "rank-state.pt")
                    torch.save({"global_step": int(step), "initialization": receipts,
                                "student_updates": expected_student_updates(step, opts.critic_updates_per_student)}, tx.path / "runtime.pt")
                    done = tx.commit(step=int(step), contract=build_contract(config, route, topo.sp_size),
                                     required_components=("role.pt", "rank-state.pt", "runtime.pt"),
                                     metadata={"roles": ["student", "critic"], "initialization": receipts})
                return done.manifest_digest

            return rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None, label="checkpoint commit")

        last, ident, saved_at = {}, None, None
        while trainer.global_step < max_steps:
            last = trainer.train_outer_step(next(batches))
            consumed += 1
            step = trainer.global_step
            sink({"event": "train_step", "step": step, **{k: float(v) for k, v in last.items()}})
            if step in save_steps or (save_every > 0 and step % save_every == 0):
                ident, saved_at = save(step), step
        return {"final_step": trainer.global_step, "losses": last, "checkpoint": ident, "initialization": receipts,
                "checkpoint_dir": None if saved_at is None else str(checkpoint_model_dir(output_root(config), saved_at))}
    finally:
        dist_init.shutdown(ctx)
