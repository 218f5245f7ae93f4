"""Multi-rank LTX adapter training behind the shared optimizer-step engine.

The recipe trains rank-384 adapters on a frozen 13B video core.  On 180 GB GPUs the frozen bf16 base is REPLICATED (26 GB)
rather than wrapped in a sharding layer whose every block gathers weights, and the adapters -- which a sharding wrapper
would have to be told to ignore and which the reference then synchronises by hand -- are plain replicated parameters
whose gradients live in the optimizer's one flat fp32 buffer:

  sequence        Ulysses SP through the blocks (the NCCL transport; the fused transport is off while adapters are on);
                  SP peers see the same sample, the same noise and the same sigma (broadcast from the group's first rank);
  gradients       summed over SP (complementary tokens), averaged over DP (different samples): one fp32 all-reduce of the
                  flat buffer after the ranks agreed on which adapters received a gradient;
  optimizer       fp32-master AdamW over the flat buffer, warm-up + cosine schedule, fp32 average of the trainable weights;
  checkpoint      ``adapter.pt`` under the released key inventory with its metadata record, ``optimizer.pt``,
                  ``scheduler.pt``, ``ema.pt``, ``rank-state.pt``, ``runtime.pt`` holding the run's fingerprint
                  (``checkpoint.runtime_fingerprint``); a full resume must present the identical fingerprint and the exact
                  adapter target inventory (``checkpoint.validate_full_resume``).

Reference: solar/backends/ltx25/torch_training.py:82-593, runtime.py:119-488, checkpoint.py:669-763.
"""
from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from ... import ops
from ...checkpoint.store import CheckpointContract, CheckpointTransaction, verify_checkpoint
from ...config.routes import validate_route
from ...engine.train_engine import (BatchIdentity, GradientStatus, JsonlEventSink, MicrobatchResult, StepPolicy,
                                    TrainingEngine)
from ...errors import BackendContractError
from ...parallel import dist_init
from ...runtime import distributed as rdist
from ...runtime.output_layout import checkpoint_model_dir, events_path, output_root
from ...runtime.randomness import objective_seed
from ...runtime.safe_state import capture_rank_state, restore_rank_state
from ..minimax_h3.runtime import WarmupCosine, sync_adapter_gradients
from .checkpoint import EMARecipe, LoRARecipe, TrainingCheckpointManifest, runtime_fingerprint, validate_full_resume
from .flow import masked_flow_loss, noisy_input_and_target, sample_sigmas

COMPONENTS = ("adapter.pt", "optimizer.pt", "scheduler.pt", "ema.pt", "rank-state.pt", "runtime.pt")
EMA_SCHEMA = "solarwm.ltx25.adapter-ema.v1"


class LTXTrainingRuntime:
    def __init__(self, config: Mapping[str, Any]):
        from .backend import LTXTrainer, _arch

        self.config, self.route = config, validate_route(config)
        train, data = config["train"], config["data"]
        adapter = config["model"].get("adapter") or {}
        if int(adapter.get("rank", 0)) < 1:
            raise BackendContractError("the LTX training runtime trains adapters: model.adapter.rank must be positive")
        dist_cfg = config.get("distributed", {}) or {}
        self.ctx = dist_init.initialize(int(dist_cfg.get("sequence_parallel_size", 1)), device=str(config.get("runtime", {}).get("device", "auto")))
        topo = self.topology = self.ctx.topology
        self.device = self.ctx.device
        self.seed = int(data.get("seed", 0))
        o = train.get("optimizer", {}) or {}
        self.arch = _arch(config)
        fsdp = train.get("fsdp", {}) or {}
        ac = fsdp.get("activation_checkpointing", False)
        self.core = LTXTrainer(self.arch, self.device, lr=float(o.get("lr", 1e-4)), seed=self.seed, sp=self.ctx.sp,
                               checkpointing=("full" if ac is True else (ac or "none")), lora_rank=int(adapter["rank"]), lora_alpha=adapter.get("alpha"),
                               base_weights=config["model"].get("base_weights"))
        self.core.gen.manual_seed(objective_seed(self.seed, topo.dp_rank))
        self.optimizer, self.lora = self.core.opt, self.core.lora
        self.clip = float(o.get("grad_clip", 1.0))
        self.max_steps = int(config.get("runtime", {}).get("max_steps_override") or train["max_steps"])
        self.scheduler = WarmupCosine(self.optimizer, warmup=int(o.get("warmup_steps", train.get("warmup_steps", 0))), total=self.max_steps,
                                      min_ratio=float(o.get("min_lr_ratio", 0.1)))
        e = train.get("ema", {}) or {}
        self.ema_recipe = EMARecipe(enabled=bool(e.get("enabled", True)), start_step=int(e.get("start_step", 0)),
                                    update_every_steps=int(e.get("update_every_steps", 1)), decay=float(e.get("decay", 0.999)))
        self.ema = self.optimizer.master.clone() if self.ema_recipe.enabled else None
        self.ema_updates = 0
        self.targets = tuple(self.lora.metadata()["targets"])
        self.fingerprint = runtime_fingerprint(
            camera_translation_transform=str(config["model"].get("camera_translation_transform", "linear")),
            data_generation=str(data.get("generation", data.get("source", "synthetic"))),
            lora=LoRARecipe(rank=self.lora.rank, alpha=int(self.lora.alpha), target_count=len(self.targets),
                            trainable_parameters=sum(p.numel() for p in self.lora.parameters)), ema=self.ema_recipe)
        self._corpus = None
        if str(data.get("source", "synthetic")) == "index":
            from ..wan22.runtime import iter_encoded_samples

            self._corpus = iter_encoded_samples(data, topo.dp_rank, topo.dp_size)
        self._shape = (1, self.arch.in_dim, int(data.get("latent_frames", 4)), int(data.get("latent_height", 8)), int(data.get("latent_width", 8)))
        self._global_step, self.batches_consumed = 0, 0
        self.checkpoint_id = "init:random"
        self.plan_fingerprint = f"ltx25-seed{self.seed}-dp{topo.dp_size}"
        ck = config.get("checkpoint", {}) or {}
        if ck.get("mode") == "full_resume" and ck.get("resume_from"):
            self.load_checkpoint(str(ck["resume_from"]))

    # -- engine hooks -------------------------------------------------------------------------------------------------------
    @property
    def global_step(self) -> int:
        return self._global_step

    def set_global_step(self, step: int) -> None:
        self._global_step = int(step)

    def zero_grad(self) -> None:
        self.optimizer.zero_grad()

    def _next_sample(self):
        ordinal = self.batches_consumed * self.topology.dp_size + self.topology.dp_rank
        self.batches_consumed += 1
        if self._corpus is not None:
            row, enc = next(self._corpus)
            if enc["latents"].shape[1] != self.arch.in_dim or tuple(enc["text"].shape) != (self.arch.text_len, self.arch.text_dim):
                raise BackendContractError(f"{row.sample_id}: latents / text do not match the architecture")
            self._cameras = enc["camera_c2w"].float().unsqueeze(0) if "camera_c2w" in enc else None
            return str(row.sample_id), ordinal, enc["latents"].permute(1, 0, 2, 3).unsqueeze(0).float(), enc["text"].unsqueeze(0).float()
        g = torch.Generator().manual_seed(self.seed * 100003 + ordinal)
        lat, txt = torch.randn(self._shape, generator=g), torch.randn(1, self.arch.text_len, self.arch.text_dim, generator=g)
        self._cameras = None
        if self.config["data"].get("cameras"):      # a seeded dolly for the camera-conditioned recipe
            frames = self._shape[2]
            c2w = torch.eye(4).repeat(1, frames, 1, 1)
            c2w[0, :, 2, 3] = torch.arange(frames) * 0.05 * (1.0 + float(torch.rand(1, generator=g)))
            self._cameras = c2w
        return f"synthetic-{ordinal:08d}", ordinal, lat, txt

    def _camera_condition(self):
        """Parameter-free PRoPE with the family's fixed intrinsics over world-to-camera matrices relative to the clip's
        first camera; ``None`` when the sample carries no cameras."""
        if getattr(self, "_cameras", None) is None:
            return None
        from ...models.ltx import ltx_camera_condition

        c2w = self._cameras.to(self.device, torch.float64)
        rel = torch.linalg.inv(c2w[:, :1]) @ c2w
        rel[:, 0] = torch.eye(4, dtype=torch.float64, device=self.device)
        return ltx_camera_condition(torch.linalg.inv(rel).float(), str(self.config["model"].get("camera_translation_transform", "linear")))

    def train_microbatch(self, micro_index: int, grad_accum: int) -> MicrobatchResult:
        ident, ordinal, latents, text = self._next_sample()
        core, sp = self.core, self.ctx.sp
        lat = latents.to(self.device).to(core.model.dtype)
        B, C, F, H, W = lat.shape
        sigma = sample_sigmas(B, F * H * W, generator=core.gen, device=self.device)
        noise = torch.randn(lat.shape, generator=core.gen, device=self.device, dtype=torch.float32).to(lat.dtype)
        if sp is not None and sp.size > 1:
            sp.broadcast_(sigma, noise)
        x_t, target, per_frame = noisy_input_and_target(lat, noise, sigma)
        loss = masked_flow_loss(core.model(x_t, per_frame * 1000.0, text.to(self.device), y_camera=self._camera_condition()), target)
        (loss / (grad_accum * (1 if sp is None else sp.size))).backward()
        value = float(loss.detach())
        if not math.isfinite(value):
            raise BackendContractError(f"non-finite loss on {ident}")
        identity = BatchIdentity((ident,), (0,), (objective_seed(self.seed, self.topology.dp_rank) + ordinal,), self.checkpoint_id, self.plan_fingerprint)
        return MicrobatchResult(identity, {"loss": value})

    def assert_sp_peer_identity(self, identity: BatchIdentity) -> None:
        if self.topology.sp_size == 1:
            return
        import torch.distributed as dist

        seen = [None] * self.topology.sp_size
        dist.all_gather_object(seen, identity, group=self.ctx.sp_group)
        if any(other != seen[0] for other in seen):
            raise BackendContractError(f"sequence-parallel peers trained on different microbatches: {seen}")

    def prepare_optimizer_step(self) -> GradientStatus:
        topo = self.topology
        flat = self.optimizer.gather_grads()
        sync_adapter_gradients(self.optimizer.params, flat, sp_group=self.ctx.sp_group, sp_size=topo.sp_size, dp_group=self.ctx.dp_group,
                               dp_size=topo.dp_size)
        norm = float(self.optimizer.clip_(self.clip))
        return GradientStatus(finite=math.isfinite(norm), norm=norm)

    def optimizer_step(self) -> None:
        self.optimizer.step()

    def scheduler_step(self) -> None:
        self.scheduler.step()

    def ema_update(self, step: int) -> None:
        r = self.ema_recipe
        if self.ema is not None and step >= r.start_step and step % r.update_every_steps == 0:
            self.ema.lerp_(self.optimizer.master, 1.0 - r.decay)
            self.ema_updates += 1

    # -- checkpoints --------------------------------------------------------------------------------------------------------
    def _rank_state(self) -> dict:
        state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in capture_rank_state(self.device).items()}
        state["objective_gen"] = self.core.gen.get_state().cpu()
        state["batches_consumed"] = int(self.batches_consumed)
        return state

    def save_checkpoint(self, step: int) -> str:
        import torch.distributed as dist

        topo = self.topology
        states = [self._rank_state()]
        if topo.raw_world_size > 1:
            states = [None] * topo.raw_world_size
            dist.all_gather_object(states, self._rank_state())
        target = checkpoint_model_dir(output_root(self.config), step)

        def write():
            with CheckpointTransaction(target) as tx:
                torch.save({"metadata": self.lora.metadata(), "state": {k: v.cpu() for k, v in self.lora.state_dict().items()}}, tx.path / "adapter.pt")
                torch.save(self.optimizer.state_dict(), tx.path / "optimizer.pt")
                torch.save(self.scheduler.state_dict(), tx.path / "scheduler.pt")
                torch.save({"schema": EMA_SCHEMA, "targets": list(self.targets), "num_updates": self.ema_updates,
                            "flat": None if self.ema is None else self.ema.cpu()}, tx.path / "ema.pt")
                torch.save({"ranks": states, "world_size": topo.raw_world_size, "sp_size": topo.sp_size}, tx.path / "rank-state.pt")
                torch.save({"global_step": int(step), "fingerprint": self.fingerprint, "adapter_targets": list(self.targets)}, tx.path / "runtime.pt")
                r = self.route
                done = tx.commit(step=int(step), contract=CheckpointContract(
                    family="ltx25_video", stage=r.stage, causal_mode=r.causal_mode, objective=r.objective, objective_variant=r.variant,
                    camera_translation_transform=str(self.config["model"].get("camera_translation_transform", "linear")), parameterization="lora",
                    sp_size=topo.sp_size, data_generation=self.fingerprint["data_generation"]), required_components=list(COMPONENTS), metadata={})
            return done.manifest_digest

        self.checkpoint_id = rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None, label="checkpoint commit")
        return self.checkpoint_id

    def load_checkpoint(self, path: str) -> None:
        verified = verify_checkpoint(path)
        root, topo = verified.path, self.topology
        run = torch.load(root / "runtime.pt", weights_only=True)
        ema = torch.load(root / "ema.pt", weights_only=True)
        manifest = TrainingCheckpointManifest(int(run["global_step"]), run["fingerprint"], tuple(run["adapter_targets"]), tuple(ema.get("targets", ())),
                                              (root / "optimizer.pt").is_file(), (root / "scheduler.pt").is_file())
        validate_full_resume(manifest, self.fingerprint, self.targets)
        ranks = torch.load(root / "rank-state.pt", weights_only=True)
        if int(ranks["world_size"]) != topo.raw_world_size or int(ranks["sp_size"]) != topo.sp_size:
            raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks (SP {ranks['sp_size']}); "
                                       f"{topo.raw_world_size} (SP {topo.sp_size}) are running")
        adapter = torch.load(root / "adapter.pt", weights_only=True)
        self.lora.load_state_dict({k: v.to(self.device) for k, v in adapter["state"].items()}, broadcast=False)
        opt = torch.load(root / "optimizer.pt", weights_only=True)
        self.optimizer.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in opt.items()})
        self.optimizer.lr = float(opt["lr"])
        self.scheduler.load_state_dict(torch.load(root / "scheduler.pt", weights_only=True))
        if self.ema is not None:
            if ema.get("flat") is None or ema["flat"].shape != self.ema.shape:
                raise BackendContractError("the checkpoint's average does not fit the trainable adapters")
            self.ema.copy_(ema["flat"])
            self.ema_updates = int(ema["num_updates"])
        mine = ranks["ranks"][topo.raw_rank]
        restore_rank_state(mine, self.device)
        self.core.gen.set_state(mine["objective_gen"])
        self.batches_consumed = int(mine["batches_consumed"])
        if self._corpus is not None:
            for _ in range(self.batches_consumed):
                next(self._corpus)
        self._global_step = int(run["global_step"])
        self.checkpoint_id = verified.manifest_digest

    def validate(self, step: int) -> Mapping[str, Any]:
        """Adapter norms and, with ``validation.index``, the flow loss at fixed noise levels (seeded per clip and level) on
        the run's frozen, source-balanced validation clips (the selection machinery of ``minimax_h3.validation``)."""
        report = {"step": int(step), "adapter_norm": float(self.optimizer.master.norm())}
        if self.ema is not None:
            report["ema_norm"] = float(self.ema.norm())
        val = self.config.get("validation", {}) or {}
        if val.get("index"):
            report["validation"] = self._validation_loss(val)
        return report

    def _validation_loss(self, val: Mapping[str, Any]) -> Mapping[str, Any]:
        import torch.distributed as dist
        from pathlib import Path

        from ...data.index import read_index
        from ...preencode.shards import read_encoded_sample
        from ..minimax_h3.validation import IndexedValidation, score

        topo, core = self.topology, self.core
        if getattr(self, "_validation", None) is None:
            index = Path(str(val["index"]))
            root = Path(str(val.get("root") or index.parent))

            def read(row):
                enc = read_encoded_sample(root, row.values)
                if enc["latents"].shape[1] != self.arch.in_dim or tuple(enc["text"].shape) != (self.arch.text_len, self.arch.text_dim):
                    raise BackendContractError(f"{row.sample_id}: latents / text do not match the architecture")
                return {"latents": enc["latents"].permute(1, 0, 2, 3).unsqueeze(0).float(), "text": enc["text"].unsqueeze(0).float()}

            self._validation = IndexedValidation(read_index(index), read, sample_count=int(val.get("sample_count", 8)), seed=int(val.get("seed", 42)),
                                                 dp_rank=topo.dp_rank, dp_size=topo.dp_size, balance=bool(val.get("balance_sources", True)),
                                                 freeze_path=output_root(self.config) / "validation-selection.json")
            self._validation.prepare(dist if topo.raw_world_size > 1 else None)

        def loss_at(sample, sigma, gen):
            lat = sample["latents"].to(self.device).to(core.model.dtype)
            noise = torch.randn(lat.shape, generator=gen, device=self.device, dtype=torch.float32).to(lat.dtype)
            x_t, target, per_frame = noisy_input_and_target(lat, noise, torch.full((1,), float(sigma), device=self.device))
            return masked_flow_loss(core.model(x_t, per_frame * 1000.0, sample["text"].to(self.device)), target)

        return dict(score(self._validation, loss_at, device=self.device, dist=dist if topo.dp_size > 1 else None, group=self.ctx.dp_group))

    def close(self) -> None:
        dist_init.shutdown(self.ctx)


def adapter_weights(checkpoint, weight_source: str = "live"):
    """``(metadata, {released key: tensor})`` of a verified adapter checkpoint: the live adapters, or the averaged ones
    unpacked from the flat fp32 buffer (the optimizer's layout: parameters in key order, each padded to 64 elements)."""
    if weight_source not in ("live", "ema"):
        raise BackendContractError("weight_source is live or ema")
    verified = verify_checkpoint(checkpoint)
    doc = torch.load(verified.path / "adapter.pt", map_location="cpu", weights_only=True)
    meta, state = doc["metadata"], doc["state"]
    if weight_source == "ema":
        ema = torch.load(verified.path / "ema.pt", map_location="cpu", weights_only=True)
        flat = ema.get("flat")
        if flat is None:
            raise BackendContractError("the checkpoint holds no averaged adapters")
        out, at = {}, 0
        for key in meta["state_keys"]:
            n = state[key].numel()
            out[key] = flat[at:at + n].view(state[key].shape).to(state[key].dtype)
            at += (n + 63) // 64 * 64
        if at != flat.numel():
            raise BackendContractError("the averaged buffer does not match the adapter inventory")
        state = out
    return meta, state, verified


def run_training(config: Mapping[str, Any]) -> Mapping[str, Any]:
    runtime = LTXTrainingRuntime(config)
    try:
        train, rt = config["train"], config.get("runtime", {}) or {}
        policy = StepPolicy(max_steps=runtime.max_steps, grad_accum=int(train.get("grad_accum", train.get("gradient_accumulation_steps", 1))),
                            save_every=int(rt.get("save_every", 0)), validate_every=int(rt.get("validate_every", 0)),
                            save_steps=(runtime.max_steps,) if rt.get("save_final", True) else ())
        write = JsonlEventSink(events_path(output_root(config), runtime.topology.raw_rank))
        last = {}

        def sink(event):
            write(event)
            if event.get("event") == "optimizer_step":
                last.update(event["losses"])

        final = TrainingEngine(runtime, policy, event_sink=sink).run()
        return {"final_step": final, "checkpoint_id": runtime.checkpoint_id, "last_loss": last.get("loss"),
                "checkpoint": str(checkpoint_model_dir(output_root(config), final)), "native_launches": ops.total_launches()}
    finally:
        runtime.close()
