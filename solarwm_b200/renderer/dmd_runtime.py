"""Config-driven few-step distillation of the renderer, with the checkpoint / resume / event lifecycle of the other runtimes.

  roles        student (adapters trained; starts from ``train.dmd.student_init`` or from the control adapters), critic
               (adapters trained; starts from ``train.dmd.critic_init`` or from the control adapters), teacher (the
               control-trained renderer ``train.dmd.control``, frozen).  One bf16 base aliased by all three.
  data         the omni corpus (``renderer.data.OmniStream``): prompts, first frames, structure streams, cameras; the
               target latents of the clips are not used (distribution matching is data-free beyond the conditions).
  step         ``dmd.RendererDMDTrainer.train_outer_step``: student render, structure-guided teacher score, critic score,
               KL-gradient surrogate on every ``critic_updates_per_student``-th step, critic flow matching every step;
               flat fp32 gradients averaged over the replicas; non-finite scores / losses / norms refuse the update.
  checkpoint   ``adapter.pt`` (student), ``critic.pt``, both optimizers, every rank's random streams and reader position,
               both step counters, and the identities of the parents; no EMA (a checkpoint that holds one is refused).

Reference: H3OmniDMDRuntime and run_omni_dmd_training (solar/renderer/dmd_runtime.py:22-368).
"""
from __future__ import annotations

import time
from typing import Any, Mapping

import torch

from .. import ops
from ..backends.minimax_h3.runtime import ADAPTER_SCHEMA, EMA_SCHEMA, sync_adapter_gradients
from ..checkpoint.store import CheckpointContract, CheckpointTransaction, verify_checkpoint
from ..engine.train_engine import JsonlEventSink
from ..errors import BackendContractError, ConfigurationError
from ..models.h3 import h3_preset
from ..parallel import dist_init
from ..runtime import distributed as rdist
from ..runtime.output_layout import checkpoint_model_dir, events_path, output_root
from ..runtime.randomness import model_init_seed, objective_seed
from ..runtime.safe_state import capture_rank_state, restore_rank_state
from .data import MemberContract, OmniStream
from .dmd import RendererDMDTrainer
from .runtime import read_adapter, validate_config, weight_identity

COMPONENTS = ("adapter.pt", "critic.pt", "optimizer.pt", "critic-optimizer.pt", "ema.pt", "rank-state.pt", "runtime.pt")


def _adopt(model, optimizer, state: Mapping[str, torch.Tensor], what: str) -> None:
    own = {n: p for n, p in model.named_parameters() if p.requires_grad}
    if set(own) != set(state):
        raise BackendContractError(f"{what}: the adapter file does not hold exactly this architecture's adapter tensors")
    with torch.no_grad():
        for n, p in own.items():
            p.copy_(state[n].to(p))
        optimizer.master.copy_(optimizer.live.float())


class RendererDMDRuntime:
    def __init__(self, config: Mapping[str, Any]):
        validate_config(config)
        train, data, model_cfg = config["train"], config["data"], config["model"]
        if train.get("objective") != "dmd" or not isinstance(train.get("dmd"), Mapping):
            raise ConfigurationError("the distillation runtime needs train.objective: dmd and a train.dmd section")
        dmd = train["dmd"]
        if not dmd.get("control"):
            raise ConfigurationError("train.dmd.control names the control-trained adapters the teacher uses")
        self.config = config
        self.ctx = dist_init.initialize(1, device=str(config["runtime"].get("device", "auto")))
        topo = self.topology = self.ctx.topology
        dev = self.device = self.ctx.device
        self.seed = int(data.get("seed", 42))
        cfg = h3_preset(str(model_cfg.get("architecture", "h3_33b")))
        cfg.lora_rank = int((model_cfg.get("adapter", {}) or {}).get("rank", cfg.lora_rank or 8))
        o, oc = train.get("optimizer", {}) or {}, train.get("critic_optimizer", {}) or {}
        lr = float(o.get("lr", 2e-6))
        tr = self.trainer = RendererDMDTrainer(cfg, dev, student_steps=int(dmd.get("student_steps", 4)), guidance=float(dmd.get("guidance", 2.0)),
                                               critic_updates_per_student=int(dmd.get("critic_updates_per_student", 5)), lr_student=lr,
                                               lr_critic=float(oc.get("lr", lr * 0.2)), seed=model_init_seed("minimax_h3", self.seed) % (2 ** 31))
        tr.gen = torch.Generator(device=dev).manual_seed(objective_seed(self.seed, topo.dp_rank))
        if topo.dp_size > 1:
            tr.sync = lambda params, flat: sync_adapter_gradients(params, flat, sp_group=None, sp_size=1, dp_group=self.ctx.dp_group,
                                                                  dp_size=topo.dp_size)
        control = read_adapter(dmd["control"])
        tr.set_teacher(control)
        self.parents = {"control": self._identity(dmd["control"])}
        for role, key, model, opt in (("student", "student_init", tr.student, tr.opt_s), ("critic", "critic_init", tr.critic, tr.opt_c)):
            source = dmd.get(key) or dmd["control"]
            _adopt(model, opt, control if source == dmd["control"] else read_adapter(source), role)
            self.parents[key] = self._identity(source)
        c = data.get("member_contract", {}) or {}
        contract = MemberContract(latent_channels=int(c.get("latent_channels", 24)), text_dim=int(c.get("text_dim", cfg.text_dim)),
                                  grids=tuple(tuple(int(v) for v in g) for g in c.get("grids", ((48, 84), (84, 48)))),
                                  frames_period=int(c.get("frames_period", 5)), frames_offset=int(c.get("frames_offset", 2)))
        self.reader = OmniStream(root=data["omni_root"], index=data["omni_index"], dp_rank=topo.dp_rank, dp_size=topo.dp_size, seed=self.seed,
                                 shuffle=bool(data.get("shuffle", True)), length_buckets=bool(data.get("omni_length_buckets", True)), contract=contract)
        self.max_steps = int(config["runtime"].get("max_steps_override") or train["max_steps"])
        self.checkpoint_id = "init:" + self.parents["control"]
        ck = config.get("checkpoint", {}) or {}
        if ck.get("resume_from"):
            self.load_checkpoint(str(ck["resume_from"]))

    @staticmethod
    def _identity(path) -> str:
        from pathlib import Path

        p = Path(path)
        return weight_identity(p / "adapter.pt" if p.is_dir() else p)

    @property
    def global_step(self) -> int:
        return self.trainer.global_step

    def train_outer_step(self) -> Mapping[str, float]:
        import torch.distributed as dist

        t0 = time.monotonic()
        sample = rdist.collective_call(self.reader.next, dist=dist if self.topology.raw_world_size > 1 else None, label="renderer data read")
        got = dict(self.trainer.train_outer_step(sample.as_training_sample()))
        stats = {"student_updated": float("student" in got), "loss_student": got.get("student", 0.0), "loss_critic": got["critic"],
                 "student_grad_norm": got.get("student_grad_norm", 0.0), "critic_grad_norm": got["critic_grad_norm"],
                 "student_step": float(self.trainer.student_step), "loss": got.get("student", got["critic"]),
                 "compute_time_s": time.monotonic() - t0}
        return stats

    # -- checkpoints --------------------------------------------------------------------------------------------------------
    def _metadata(self) -> dict:
        return {"parents": dict(self.parents), "data_plan": self.reader.plan_fingerprint, "dmd": {k: v for k, v in self.config["train"]["dmd"].items()
                                                                                                   if k not in ("control", "student_init", "critic_init")}}

    def _rank_state(self) -> dict:
        state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in capture_rank_state(self.device).items()}
        state["objective_gen"] = self.trainer.gen.get_state().cpu()
        state["reader"] = self.reader.state_dict()
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
                for name, model in (("adapter.pt", tr.student), ("critic.pt", tr.critic)):
                    torch.save({"schema": ADAPTER_SCHEMA, "rank": rank,
                                "state": {n: p.detach().cpu() for n, p in model.named_parameters() if p.requires_grad}}, tx.path / name)
                torch.save(tr.opt_s.state_dict(), tx.path / "optimizer.pt")
                torch.save(tr.opt_c.state_dict(), tx.path / "critic-optimizer.pt")
                torch.save({"schema": EMA_SCHEMA, "state": None}, tx.path / "ema.pt")          # distillation keeps no average
                torch.save({"ranks": states, "world_size": topo.raw_world_size}, tx.path / "rank-state.pt")
                torch.save({"global_step": int(tr.global_step), "student_step": int(tr.student_step), **self._metadata()}, tx.path / "runtime.pt")
                done = tx.commit(step=int(step), contract=CheckpointContract(
                    family="minimax_h3_renderer", stage="fewstep", causal_mode="bidirectional", objective="dmd",
                    objective_variant="structure_guided", camera_translation_transform="logd4", parameterization=f"lora-r{rank}", sp_size=1,
                    data_generation="solarrenderer.omni.v1"), required_components=list(COMPONENTS), metadata=self._metadata())
            return done.manifest_digest

        self.checkpoint_id = rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None, label="checkpoint commit")
        return self.checkpoint_id

    def load_checkpoint(self, path: str) -> None:
        verified = verify_checkpoint(path)
        root, tr, topo = verified.path, self.trainer, self.topology
        run = torch.load(root / "runtime.pt", weights_only=True)
        mine = self._metadata()
        for key in ("parents", "data_plan", "dmd"):
            if run.get(key) != mine[key]:
                raise BackendContractError(f"the checkpoint was distilled under another {key.replace('_', ' ')}")
        if torch.load(root / "ema.pt", weights_only=True).get("state") is not None:
            raise BackendContractError("a renderer distillation checkpoint unexpectedly holds an average")
        ranks = torch.load(root / "rank-state.pt", weights_only=True)
        if int(ranks["world_size"]) != topo.raw_world_size:
            raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks; {topo.raw_world_size} are running")
        for name, opt in (("optimizer.pt", tr.opt_s), ("critic-optimizer.pt", tr.opt_c)):
            state = torch.load(root / name, weights_only=True)
            opt.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in state.items()})
            opt.lr = float(state["lr"])
        tr.global_step, tr.student_step = int(run["global_step"]), int(run["student_step"])
        state = ranks["ranks"][topo.raw_rank]
        restore_rank_state(state, self.device)
        tr.gen.set_state(state["objective_gen"])
        self.reader.load_state_dict(state["reader"])
        self.checkpoint_id = verified.manifest_digest

    def close(self) -> None:
        self.reader.close()
        dist_init.shutdown(self.ctx)


def run_dmd_training(config: Mapping[str, Any]) -> Mapping[str, Any]:
    runtime = RendererDMDRuntime(config)
    try:
        ck = config.get("checkpoint", {}) or {}
        every = int(ck.get("save_every_steps", 0))
        at = {int(s) for s in ck.get("save_steps", ())} | {runtime.max_steps}
        sink = JsonlEventSink(events_path(output_root(config), runtime.topology.raw_rank))
        last, saved = {}, None
        while runtime.global_step < runtime.max_steps:
            last = runtime.train_outer_step()
            step = runtime.global_step
            sink({"event": "train_step", "step": step, **last})
            if step in at or (every and step % every == 0):
                runtime.save_checkpoint(step)
                saved = step
        return {"final_step": runtime.global_step, "student_step": runtime.trainer.student_step, "last": dict(last),
                "checkpoint_id": runtime.checkpoint_id, "checkpoint": None if saved is None else str(checkpoint_model_dir(output_root(config), saved)),
                "native_launches": ops.total_launches()}
    finally:
        runtime.close()
