"""Training runtime of H3 Stage2 (self-gradient forcing): three roles over one frozen base, with the checkpoint,
resume, averaging and event lifecycle of the other H3 stages.

  roles        student (adapters trained, block-causal), critic (adapters trained, bidirectional), teacher (frozen:
               the base alone, or the base with the adapters of ``checkpoint.initialization.teacher``).  The base is
               ONE set of bf16 tensors that the three modules alias (``stage2.share_base``), so a 180 GB GPU holds
               the 33B base once; the reference builds three FSDP-wrapped copies.
  outer step   every ``train.critic_updates_per_student``-th step starts with a student update (rollout -> replay with
               gradients -> critic and teacher scores -> KL-gradient surrogate), then every step updates the critic on
               a SECOND sample (rollout -> replay without gradients -> flow matching).  Non-finite scores, losses or
               gradient norms raise ``FloatingPointError`` before any weight changes.
  ranks        data parallel: each replica rolls out its own samples; the flat fp32 adapter gradients of the role
               being updated are averaged over the replicas (``runtime.sync_adapter_gradients``).
  averaging    an fp32 EMA of the student's master weights that is CREATED at ``checkpoint.ema.start_step`` student
               updates; a checkpoint taken before that boundary holds none, and a resume checks that the two agree.
  checkpoint   ``adapter.pt`` (student), ``critic.pt``, both optimizers, ``ema.pt``, every rank's random streams and
               the two step counters; ``checkpoint.resume_from`` continues bit-exactly.

Reference: H3SGFTrainingRuntime and run_sgf_training (solar/backends/minimax_h3/stage2_runtime.py:55-306).
"""
from __future__ import annotations

import time
from typing import Any, Mapping

import torch

from ... import ops
from ...checkpoint.store import CheckpointContract, CheckpointTransaction, verify_checkpoint
from ...config.routes import validate_route
from ...engine.train_engine import JsonlEventSink, StepPolicy
from ...errors import BackendContractError
from ...parallel import dist_init
from ...runtime import distributed as rdist
from ...runtime.output_layout import checkpoint_model_dir, events_path, output_root
from ...runtime.randomness import model_init_seed, objective_seed
from ...runtime.safe_state import capture_rank_state, restore_rank_state
from .runtime import ADAPTER_SCHEMA, EMA_SCHEMA, AdapterEMA, sync_adapter_gradients
from .stage2 import H3Stage2Trainer

COMPONENTS = ("adapter.pt", "critic.pt", "optimizer.pt", "critic-optimizer.pt", "ema.pt", "rank-state.pt", "runtime.pt")


def _adapter_state(model) -> dict:
    return {n: p.detach().cpu().clone() for n, p in model.named_parameters() if p.requires_grad}


def _read_adapter(path) -> dict:
    doc = torch.load(str(path), map_location="cpu", weights_only=True)
    if not isinstance(doc, dict) or doc.get("schema") != ADAPTER_SCHEMA or not isinstance(doc.get("state"), dict):
        raise BackendContractError(f"{path} is not an H3 adapter file")
    return doc["state"]


def _adopt(model, optimizer, state: Mapping[str, torch.Tensor], what: str) -> None:
    """Adapter tensors into the live views AND the optimizer's fp32 master."""
    own = {n: p for n, p in model.named_parameters() if p.requires_grad}
    if set(own) != set(state):
        raise BackendContractError(f"{what}: the adapter file does not hold exactly this architecture's adapter tensors")
    with torch.no_grad():
        for n, p in own.items():
            if tuple(state[n].shape) != tuple(p.shape):
                raise BackendContractError(f"{what}: {n} has shape {tuple(state[n].shape)}, the model {tuple(p.shape)}")
            p.copy_(state[n].to(p))
        optimizer.master.copy_(optimizer.live.float())


class H3SGFRuntime:
    def __init__(self, config: Mapping[str, Any], *, model_config, load_released=None):
        self.config, self.route = config, validate_route(config)
        if self.route.stage != "stage2":
            raise BackendContractError("the SGF runtime serves the stage2 routes")
        train, data = config["train"], config["data"]
        dist_cfg = config.get("distributed", {}) or {}
        if int(dist_cfg.get("sequence_parallel_size", 1)) != 1:
            raise BackendContractError("H3 Stage2 training is data parallel here: sequence_parallel_size must be 1")
        self.ctx = dist_init.initialize(1, device=str(config.get("runtime", {}).get("device", "auto")))
        topo = self.topology = self.ctx.topology
        dev = self.device = self.ctx.device
        self.seed = int(data.get("seed", 0))
        causal = config["model"].get("causal", {}) or {}
        self.k = int(causal.get("chunk_latents", 5))
        self.frames = int(data.get("latent_frames", 2 * self.k))
        if self.frames % self.k:
            raise BackendContractError("data.latent_frames must be a whole number of chunks")
        self.size = (int(data.get("latent_height", 8)), int(data.get("latent_width", 8)))
        o, oc = train.get("optimizer", {}) or {}, train.get("critic_optimizer", {}) or {}
        lr = float(o.get("lr", o.get("learning_rate", 2e-6)))
        self.trainer = H3Stage2Trainer(
            model_config, dev, chunk_latents=self.k, window_chunks=int(causal.get("window_chunks", 5)),
            grid_hw=(self.size[0] // 2, self.size[1] // 2), denoise_steps=int(train.get("denoise_steps", 4)), lr_student=lr,
            lr_critic=float(oc.get("lr", oc.get("learning_rate", lr * 0.2))),
            critic_updates_per_student=int(train.get("critic_updates_per_student", 5)),
            guidance_scale=float(train.get("guidance_scale", 3.0)), seed=model_init_seed("minimax_h3", self.seed) % (2 ** 31))
        tr = self.trainer
        if load_released is not None:
            load_released(tr.student, config)              # the critic and the teacher alias the same base tensors
        tr.gen = torch.Generator(device=dev).manual_seed(objective_seed(self.seed, topo.dp_rank))
        if data.get("silence_latents_path"):
            from .silence import load_silence_latents, silence_rows

            tr.silence = silence_rows(load_silence_latents(data["silence_latents_path"], pixel_frames=int(data.get("pixel_frames", 158))))
        if topo.dp_size > 1:
            tr.sync = lambda params, flat: sync_adapter_gradients(params, flat, sp_group=None, sp_size=1,
                                                                  dp_group=self.ctx.dp_group,
                                                                  dp_size=topo.dp_size)
        ck = self.ck = config.get("checkpoint", {}) or {}
        self.initialization = {"student": "init:random", "critic": "init:random", "teacher": "base"}
        init = ck.get("initialization", {}) or {}
        for role, (model, opt) in (("student", (tr.student, tr.opt_s)), ("critic", (tr.critic, tr.opt_c))):
            if init.get(role):
                _adopt(model, opt, _read_adapter(init[role]), role)
                self.initialization[role] = str(init[role])
        if init.get("teacher"):
            tr.set_teacher(_read_adapter(init["teacher"]))
            self.initialization["teacher"] = str(init["teacher"])
        e = ck.get("ema", {}) or {}
        self.ema_start, self.ema_decay, self.ema = int(e.get("start_step", 0)), float(e.get("decay", 0.999)), None
        self.ema_enabled = bool(e.get("enabled", True))
        self.max_steps = int(config.get("runtime", {}).get("max_steps_override") or train["max_steps"])
        self.batches_consumed = 0
        self.checkpoint_id = "init:random"
        if ck.get("resume_from"):
            self.load_checkpoint(str(ck["resume_from"]))
        self._check_ema_boundary()

    # -- state ------------------------------------------------------------------------------------------------------------
    @property
    def global_step(self) -> int:
        return self.trainer.global_step

    @property
    def student_step(self) -> int:
        return self.trainer.student_step

    def _check_ema_boundary(self) -> None:
        expected = self.ema_enabled and self.student_step >= self.ema_start and self.student_step > 0
        if expected != (self.ema is not None):
            raise BackendContractError("the student EMA's presence differs from the saved student-update boundary "
                                       f"(student_step={self.student_step}, start_step={self.ema_start})")

    def _ema_update(self) -> None:
        if not self.ema_enabled or self.student_step < self.ema_start:
            return
        if self.ema is None:
            self.ema = AdapterEMA(self.trainer.opt_s, self.ema_decay)       # starts AT the current weights
        else:
            self.ema.update()

    def _next_sample(self):
        from ...data.synthetic import h3_sample

        ordinal = self.batches_consumed * self.topology.dp_size + self.topology.dp_rank
        self.batches_consumed += 1
        data, cfg = self.config["data"], self.trainer.student.cfg
        s = h3_sample(latent_frames=self.frames, height=self.size[0], width=self.size[1], prompt_len=int(data.get("prompt_len", 8)),
                      text_dim=cfg.text_dim, seed=self.seed * 100003 + ordinal)
        s["camera_w2c"] = torch.eye(4).repeat(self.frames + 1, 1, 1)
        return s

    # -- one outer step -----------------------------------------------------------------------------------------------------
    def train_outer_step(self) -> Mapping[str, float]:
        from ...engine.sgf import should_update_student

        tr, t0 = self.trainer, time.monotonic()
        n_chunks = self.frames // self.k
        update_student = should_update_student(tr.global_step, tr.ratio)
        stats = {"student_updated": float(update_student), "loss_student": 0.0, "student_grad_norm": 0.0}
        if update_student:
            got = tr.student_phase(self._next_sample(), n_chunks)
            stats.update(loss_student=got["student"], student_grad_norm=got["student_grad_norm"])
            self._ema_update()
        got = tr.critic_phase(self._next_sample(), n_chunks)
        tr.global_step += 1
        stats.update(loss_critic=got["critic"], critic_grad_norm=got["critic_grad_norm"], student_step=float(tr.student_step),
                     loss=stats["loss_student"] if update_student else got["critic"], lr=tr.opt_s.lr, critic_lr=tr.opt_c.lr,
                     compute_time_s=time.monotonic() - t0)
        if self.topology.is_main:
            print(f"[h3-sgf] outer_step={tr.global_step} student_step={tr.student_step} student_loss={stats['loss_student']:.6f} "
                  f"critic_loss={stats['loss_critic']:.6f} compute_time_s={stats['compute_time_s']:.2f} "
                  f"ema={'present' if self.ema is not None else 'not_started'}", flush=True)
        return stats

    # -- checkpoints --------------------------------------------------------------------------------------------------------
    def _contract(self) -> CheckpointContract:
        r = self.route
        return CheckpointContract(family="minimax_h3", stage=r.stage, causal_mode=r.causal_mode, objective=r.objective,
                                  objective_variant=r.variant, camera_translation_transform="logd4", parameterization="lora",
                                  sp_size=1, data_generation=str(self.config["data"].get("source", "synthetic")))

    def _rank_state(self) -> dict:
        state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in capture_rank_state(self.device).items()}
        state["objective_gen"] = self.trainer.gen.get_state().cpu()
        state["batches_consumed"] = int(self.batches_consumed)
        return state

    def save_checkpoint(self, step: int) -> str:
        import torch.distributed as dist

        topo, tr = self.topology, self.trainer
        states = [self._rank_state()]
        if topo.raw_world_size > 1:
            states = [None] * topo.raw_world_size
            dist.all_gather_object(states, self._rank_state())
        target = checkpoint_model_dir(output_root(self.config), step)

        def write():
            with CheckpointTransaction(target) as tx:
                rank = tr.student.cfg.lora_rank
                torch.save({"schema": ADAPTER_SCHEMA, "state": _adapter_state(tr.student), "rank": rank}, tx.path / "adapter.pt")
                torch.save({"schema": ADAPTER_SCHEMA, "state": _adapter_state(tr.critic), "rank": rank}, tx.path / "critic.pt")
                torch.save(tr.opt_s.state_dict(), tx.path / "optimizer.pt")
                torch.save(tr.opt_c.state_dict(), tx.path / "critic-optimizer.pt")
                torch.save(self.ema.state_dict(tr.student) if self.ema is not None else {"schema": EMA_SCHEMA, "state": None},
                           tx.path / "ema.pt")
                torch.save({"ranks": states, "world_size": topo.raw_world_size}, tx.path / "rank-state.pt")
                torch.save({"global_step": int(tr.global_step), "student_step": int(tr.student_step),
                            "initialization": dict(self.initialization)}, tx.path / "runtime.pt")
                done = tx.commit(step=int(step), contract=self._contract(), required_components=list(COMPONENTS),
                                 metadata={"initialization": dict(self.initialization)})
            return done.manifest_digest

        self.checkpoint_id = rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None,
                                                             label="checkpoint commit")
        return self.checkpoint_id

    def load_checkpoint(self, path: str) -> None:
        verified = verify_checkpoint(path)
        root, tr, topo = verified.path, self.trainer, self.topology
        ranks = torch.load(root / "rank-state.pt", weights_only=True)
        if int(ranks["world_size"]) != topo.raw_world_size:
            raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks; {topo.raw_world_size} are running")
        for name, opt in (("optimizer.pt", tr.opt_s), ("critic-optimizer.pt", tr.opt_c)):
            state = torch.load(root / name, weights_only=True)
            opt.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in state.items()})
            opt.lr = float(state["lr"])
        run = torch.load(root / "runtime.pt", weights_only=True)
        tr.global_step, tr.student_step = int(run["global_step"]), int(run["student_step"])
        ema = torch.load(root / "ema.pt", weights_only=True)
        if ema.get("state") is not None:
            self.ema = AdapterEMA(tr.opt_s, self.ema_decay)
            self.ema.load_state_dict(ema, tr.student)
        mine = ranks["ranks"][topo.raw_rank]
        restore_rank_state(mine, self.device)
        tr.gen.set_state(mine["objective_gen"])
        self.batches_consumed = int(mine["batches_consumed"])
        self.checkpoint_id = verified.manifest_digest

    def validate(self, step: int) -> Mapping[str, Any]:
        tr = self.trainer
        report = {"step": int(step), "student_step": int(tr.student_step), "student_adapter_norm": float(tr.opt_s.master.norm()),
                  "critic_adapter_norm": float(tr.opt_c.master.norm())}
        if self.ema is not None:
            report["ema_norm"] = float(self.ema.shadow.norm())
        return report

    def close(self) -> None:
        dist_init.shutdown(self.ctx)


def run_sgf_training(config: Mapping[str, Any], *, model_config, load_released=None) -> Mapping[str, Any]:
    runtime = H3SGFRuntime(config, model_config=model_config, load_released=load_released)
    try:
        rt, ck = config.get("runtime", {}) or {}, config.get("checkpoint", {}) or {}
        policy = StepPolicy(max_steps=runtime.max_steps, grad_accum=1,
                            save_every=int(ck.get("save_every_steps", rt.get("save_every", 0))),
                            validate_every=int((config.get("validation", {}) or {}).get("validate_every_steps", rt.get("validate_every", 0))),
                            save_steps=tuple(int(s) for s in ck.get("save_steps", ())) + ((runtime.max_steps,) if rt.get("save_final", True) else ()))
        sink = JsonlEventSink(events_path(output_root(config), runtime.topology.raw_rank))
        last: Mapping[str, float] = {}
        saved = None
        while runtime.global_step < policy.max_steps:
            last = runtime.train_outer_step()
            step = runtime.global_step
            sink({"event": "train_step", "step": step, **last})
            if policy.should_save(step):
                runtime.save_checkpoint(step)
                saved = step
            if policy.should_validate(step):
                sink({"event": "validation", "step": step, "report": dict(runtime.validate(step))})
        return {"final_step": runtime.global_step, "student_step": runtime.student_step, "last": dict(last),
                "last_loss": last.get("loss"), "checkpoint_id": runtime.checkpoint_id,
                "checkpoint": None if saved is None else str(checkpoint_model_dir(output_root(config), saved)),
                "native_launches": ops.total_launches()}
    finally:
        runtime.close()
