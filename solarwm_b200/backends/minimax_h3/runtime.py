"""Multi-rank H3 adapter training behind the shared optimizer-step engine.

The 33B base is frozen bf16 and only low-rank adapters train, so the state that has to be kept consistent across ranks
is small.  The design for one 8 x 180 GB node therefore differs from the reference's (a frozen-base FSDP/HSDP wrap
whose every block gathers its weights, plus adapters that FSDP ignores and that are synchronised separately):

  base weights      REPLICATED on every GPU (66 GB of 180): no parameter gather sits on the step's critical path;
  activations       activation checkpointing per main block (``train.activation_checkpointing``: none | selective |
                    full; selective carries the attention output across the recompute);
  sequence          SP ranks hold balanced shares of the packed rows through the blocks (head exchange around
                    attention); each computes the loss of its own video rows, so adapter gradients are
                    COMPLEMENTARY over SP and REPLICATED work over DP;
  adapter gradients live in the optimizer's ONE flat fp32 buffer: summed over SP and averaged over DP with a single
                    fp32 all-reduce (two when the groups do not tile the world), after the ranks agreed on which
                    parameters received a gradient;
  optimizer / EMA   fp32 master AdamW over the flat buffer (one launch), an fp32 EMA of the master saved as ``ema.pt``.

``H3TrainingRuntime`` implements the hooks ``engine.train_engine.TrainingEngine`` drives; checkpoints hold
``adapter.pt``, ``optimizer.pt``, ``scheduler.pt``, ``ema.pt``, ``rank-state.pt`` (every rank's random streams) and
``runtime.pt``, and ``checkpoint.mode: full_resume`` continues a run exactly.

Reference: H3TrainingRuntime (solar/backends/minimax_h3/runtime.py:491-930), sync_lora_gradients
(solar/backends/minimax_h3/distributed.py:483-546), the FSDP wrap it replaces (solar/backends/minimax_h3/fsdp.py:45-233).
"""
from __future__ import annotations

import math
from typing import Any, Mapping, Optional, Sequence

import torch

from ... import ops
from ...checkpoint.store import CheckpointContract, CheckpointTransaction, verify_checkpoint
from ...config.routes import validate_route
from ...engine.master_adamw import FP32MasterAdamW
from ...engine.train_engine import (BatchIdentity, GradientStatus, JsonlEventSink, MicrobatchResult, StepPolicy,
                                    TrainingEngine)
from ...errors import BackendContractError
from ...models.h3 import H3DiT
from ...parallel import dist_init
from ...runtime import distributed as rdist
from ...runtime.output_layout import checkpoint_model_dir, events_path, output_root
from ...runtime.randomness import model_init_seed, objective_seed
from ...runtime.safe_state import capture_rank_state, restore_rank_state
from . import flow
from .layout import build_layout, expand_cameras, patchify_latents

ADAPTER_SCHEMA = "solarwm.minimax-h3-lora.v1"
EMA_SCHEMA = "solarwm.minimax-h3-ema.v1"
COMPONENTS = ("adapter.pt", "optimizer.pt", "scheduler.pt", "ema.pt", "rank-state.pt", "runtime.pt")


# ---------------------------------------------------------------------------------------------------------------------
# adapter gradient synchronisation
# ---------------------------------------------------------------------------------------------------------------------
def sync_adapter_gradients(params: Sequence[torch.nn.Parameter], flat: torch.Tensor, *, sp_group, sp_size: int,
                           dp_group, dp_size: int) -> None:
    """``flat`` is the optimizer's packed fp32 gradient (already gathered from ``params``).  The ranks first agree
    on WHICH parameters received a gradient (a rank whose graph dropped an adapter would otherwise silently add
    zeros), then the buffer is summed over SP (complementary rows of one sample) and averaged over DP (different
    samples).  The reduction is fp32 whatever the adapters' dtype."""
    import torch.distributed as dist

    world = sp_size * dp_size
    if world == 1:
        return
    flags = torch.tensor([int(p.grad is not None) for p in params], device=flat.device, dtype=torch.int32)
    dist.all_reduce(flags)
    ranks = dist.get_world_size()
    if bool(((flags != 0) & (flags != ranks)).any().item()):
        odd = [i for i, f in enumerate(flags.tolist()) if f not in (0, ranks)]
        raise BackendContractError(f"ranks disagree on which adapter parameters received a gradient (indices {odd[:8]})")
    if ranks == world:                      # the two groups tile the world: one collective, then the DP mean
        dist.all_reduce(flat)
        if dp_size > 1:
            flat.mul_(1.0 / dp_size)
        return
    if sp_size > 1:
        dist.all_reduce(flat, group=sp_group)
    if dp_size > 1:
        dist.all_reduce(flat, group=dp_group)
        flat.mul_(1.0 / dp_size)


class WarmupCosine:
    """lr(step) = base * (step / warmup while warming up, then a cosine from 1 down to ``min_ratio`` at ``total``)."""

    def __init__(self, optimizer: FP32MasterAdamW, *, warmup: int, total: int, min_ratio: float = 0.1):
        self.optimizer, self.base = optimizer, float(optimizer.lr)
        self.warmup, self.total, self.min_ratio = int(warmup), int(total), float(min_ratio)
        self.last_step = 0
        optimizer.lr = self.base * self.scale(0)

    def scale(self, step: int) -> float:
        if step < self.warmup:
            return step / max(1, self.warmup)
        progress = min(1.0, (step - self.warmup) / max(1, self.total - self.warmup))
        return self.min_ratio + (1.0 - self.min_ratio) * 0.5 * (1.0 + math.cos(math.pi * progress))

    def step(self) -> None:
        self.last_step += 1
        self.optimizer.lr = self.base * self.scale(self.last_step)

    def state_dict(self):
        return {"last_step": self.last_step, "base_lr": self.base}

    def load_state_dict(self, state) -> None:
        self.last_step = int(state["last_step"])
        self.optimizer.lr = self.base * self.scale(self.last_step)


class AdapterEMA:
    """fp32 exponential average of the optimizer's packed master weights (one ``lerp_`` per update)."""

    def __init__(self, optimizer: FP32MasterAdamW, decay: float):
        self.optimizer, self.decay = optimizer, float(decay)
        self.shadow = optimizer.master.clone()
        self.num_updates = 0

    def update(self) -> None:
        self.shadow.lerp_(self.optimizer.master, 1.0 - self.decay)
        self.num_updates += 1

    def named(self, model) -> dict:
        """The averaged adapters under the model's parameter names."""
        by_id = {id(p): n for n, p in model.named_parameters()}
        out = {}
        for p, off in zip(self.optimizer.params, self.optimizer.offsets):
            out[by_id[id(p)]] = self.shadow[off:off + p.numel()].view(p.shape).cpu().clone()
        return out

    def state_dict(self, model):
        return {"schema": EMA_SCHEMA, "decay": self.decay, "num_updates": self.num_updates, "state": self.named(model)}

    def load_state_dict(self, state, model) -> None:
        if state.get("schema") != EMA_SCHEMA:
            raise BackendContractError("ema.pt has an unknown schema")
        by_id = {id(p): n for n, p in model.named_parameters()}
        for p, off in zip(self.optimizer.params, self.optimizer.offsets):
            src = state["state"][by_id[id(p)]]
            if tuple(src.shape) != tuple(p.shape) or src.dtype != torch.float32:
                raise BackendContractError(f"ema.pt entry {by_id[id(p)]} has another shape or dtype")
            self.shadow[off:off + p.numel()].copy_(src.reshape(-1))
        self.decay, self.num_updates = float(state["decay"]), int(state["num_updates"])


# ---------------------------------------------------------------------------------------------------------------------
# the runtime
# ---------------------------------------------------------------------------------------------------------------------
class H3TrainingRuntime:
    def __init__(self, config: Mapping[str, Any], *, model_config, load_released=None):
        self.config = config
        self.route = validate_route(config)
        train, data = config["train"], config["data"]
        dist_cfg = config.get("distributed", {}) or {}
        sp_size = int(dist_cfg.get("sequence_parallel_size", 1))
        self.ctx = dist_init.initialize(sp_size, device=str(config.get("runtime", {}).get("device", "auto")))
        topo = self.topology = self.ctx.topology
        declared = int(dist_cfg.get("world_size", topo.raw_world_size))
        if declared != topo.raw_world_size:
            raise BackendContractError(f"distributed.world_size={declared} but {topo.raw_world_size} ranks are running")
        dev = self.device = self.ctx.device
        self.seed = int(data.get("seed", 0))
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.model = H3DiT(model_config, device=dev, dtype=dtype, seed=model_init_seed("minimax_h3", self.seed) % (2 ** 31))
        if load_released is not None:
            load_released(self.model, config)
        from ..wan22.runtime import activation_and_sharding_options

        self.model.checkpointing = activation_and_sharding_options(train, 1)["checkpointing"]
        if self.ctx.sp is not None:
            self.model.sp, self.model.shard_rows = self.ctx.sp, True
        o = train.get("optimizer", {}) or {}
        self.clip = float(o.get("grad_clip", o.get("gradient_clip", 1.0)))
        self.optimizer = FP32MasterAdamW(self.model.trainable_parameters(), lr=float(o.get("lr", o.get("learning_rate", 1e-4))),
                                         betas=tuple(float(b) for b in o.get("betas", (0.9, 0.95))),
                                         eps=float(o.get("eps", o.get("epsilon", 1e-8))),
                                         weight_decay=float(o.get("weight_decay", 0.01)))
        self.max_steps = int(config.get("runtime", {}).get("max_steps_override") or train["max_steps"])
        self.scheduler = WarmupCosine(self.optimizer, warmup=int(o.get("warmup_steps", train.get("warmup_steps", 0))),
                                      total=self.max_steps, min_ratio=float(o.get("min_lr_ratio", 0.1)))
        e = train.get("ema", {}) or {}
        self.ema = AdapterEMA(self.optimizer, float(e.get("decay", 0.999))) if e.get("enabled", True) else None
        self.ema_start, self.ema_every = int(e.get("start_step", 0)), int(e.get("update_every_steps", 1))
        self.gen = torch.Generator(device=dev).manual_seed(objective_seed(self.seed, topo.dp_rank))
        self.silence = None
        if data.get("silence_latents_path"):
            from .silence import load_silence_latents, silence_rows

            self.silence = silence_rows(load_silence_latents(data["silence_latents_path"], pixel_frames=int(data.get("pixel_frames", 158))))
        self.core = None
        if self.route.stage == "stage1":
            # teacher forcing under the block-causal mask: one packed sample per replica, so data parallelism only
            if topo.sp_size > 1:
                raise BackendContractError("H3 Stage1 packs clean and noisy halves of one video per rank: "
                                           "sequence_parallel_size must be 1 (use data parallelism)")
            from .stage1 import H3Stage1Trainer

            causal = config["model"].get("causal", {}) or {}
            self.core = H3Stage1Trainer(model_config, dev, model=self.model, optimizer=self.optimizer, generator=self.gen,
                                        objective="anyflow" if self.route.objective.startswith("anyflow") else "tf_fm",
                                        chunk_latents=int(causal.get("chunk_latents", 5)),
                                        window_chunks=int(causal.get("window_chunks", 5)))
            self.core.silence = self.silence
        elif self.route.stage != "stage0p5":
            raise BackendContractError(f"no multi-rank H3 runtime for {self.route.stage}")
        self._global_step, self.batches_consumed = 0, 0
        self.checkpoint_id = "init:random"
        self.plan_fingerprint = f"h3-{self.route.stage}-seed{self.seed}-dp{topo.dp_size}"
        self._corpus = None
        if str(data.get("source", "synthetic")) == "index":
            from ..wan22.runtime import iter_encoded_samples

            self._corpus = iter_encoded_samples(data, topo.dp_rank, topo.dp_size)
        ck = config.get("checkpoint", {}) or {}
        if ck.get("mode") == "full_resume" and ck.get("resume_from"):
            self.load_checkpoint(str(ck["resume_from"]))

    # -- engine hooks -------------------------------------------------------------------------------------------------
    @property
    def global_step(self) -> int:
        return self._global_step

    def set_global_step(self, step: int) -> None:
        self._global_step = int(step)

    def zero_grad(self) -> None:
        self.optimizer.zero_grad()

    def _next_sample(self):
        """The next sample of this data-parallel replica (its SP peers read the same one)."""
        data, cfg = self.config["data"], self.model.cfg
        ordinal = self.batches_consumed * self.topology.dp_size + self.topology.dp_rank
        self.batches_consumed += 1
        if self._corpus is not None:
            row, enc = next(self._corpus)
            lat = enc["latents"]
            if lat.shape[0] < 2 or tuple(enc["text"].shape[1:]) != (cfg.text_dim,):
                raise BackendContractError(f"{row.sample_id}: needs >= 2 latent frames and text of width {cfg.text_dim}")
            s = {"target_latents": lat[1:].permute(1, 0, 2, 3).contiguous(),
                 "anchor_latents": lat[:1].permute(1, 0, 2, 3).contiguous(), "prompt_embeds": enc["text"]}
            ident = str(row.sample_id)
            if "camera_c2w" in enc:                 # absolute poses of the corpus -> world-to-camera relative to the anchor's camera
                from ...renderer.data import views_from_c2w

                s["camera_w2c"] = views_from_c2w(enc["camera_c2w"].float())
                return ident, ordinal, s
        else:
            from ...data.synthetic import h3_sample

            default_frames = 3 if self.core is None else 2 * self.core.chunk_latents
            s = h3_sample(latent_frames=int(data.get("latent_frames", default_frames)), height=int(data.get("latent_height", 8)),
                          width=int(data.get("latent_width", 8)), prompt_len=int(data.get("prompt_len", 8)),
                          text_dim=cfg.text_dim, seed=self.seed * 100003 + ordinal)
            ident = f"synthetic-{ordinal:08d}"
        s["camera_w2c"] = torch.eye(4).repeat(s["target_latents"].shape[1] + 1, 1, 1)
        return ident, ordinal, s

    def train_microbatch(self, micro_index: int, grad_accum: int) -> MicrobatchResult:
        ident, ordinal, sample = self._next_sample()
        if self.core is not None:
            objective = self.core.compute_loss(sample)
            (objective / grad_accum).backward()
            loss = float(objective.detach())
            if not math.isfinite(loss):
                raise BackendContractError(f"non-finite loss on {ident}")
            identity = BatchIdentity((ident,), (0,), (objective_seed(self.seed, self.topology.dp_rank) + ordinal,),
                                     self.checkpoint_id, self.plan_fingerprint)
            return MicrobatchResult(identity, {"loss": loss})
        u = torch.rand(1, generator=self.gen, device=self.device)
        share, tgt_numel = self._stage0p5_share(sample, float(1.0 - flow.shifted_sigma(u, flow.VIDEO_SHIFT)), self.gen)
        (share / grad_accum).backward()
        total = share.detach().clone()
        if self.topology.sp_size > 1:
            import torch.distributed as dist

            dist.all_reduce(total, group=self.ctx.sp_group)
        loss = float(total)
        if not math.isfinite(loss):
            raise BackendContractError(f"non-finite loss on {ident}")
        identity = BatchIdentity((ident,), (0,), (objective_seed(self.seed, self.topology.dp_rank) + ordinal,),
                                 self.checkpoint_id, self.plan_fingerprint)
        return MicrobatchResult(identity, {"loss": loss})

    def _stage0p5_share(self, sample, t_video: float, gen: torch.Generator):
        """This rank's share of the sample's mean-square flow-matching error at time ``t_video`` (all noise from ``gen``);
        summed over the SP group it is the sample's loss."""
        dev, dt = self.device, self.model.dtype
        lat, anchor = sample["target_latents"].to(dev), sample["anchor_latents"].to(dev)
        prompt = sample["prompt_embeds"].to(dev)
        C, F, H, W = lat.shape
        audio, t_audio = None, 0.5
        if self.silence is not None:                # the silent soundtrack: input rows at their own time, prediction ignored
            from .silence import noised_silence

            audio, t_audio = noised_silence(self.silence, gen, dev)
        layout = build_layout(n_text=prompt.shape[0], latent_frames=F, grid_hw=(H // 2, W // 2), t_video=t_video,
                              n_audio=0 if audio is None else audio.shape[0], t_audio=t_audio)
        noise = torch.randn(lat.shape, generator=gen, device=dev, dtype=torch.float32).to(lat.dtype)
        a_noise = torch.randn(anchor.shape, generator=gen, device=dev, dtype=torch.float32).to(lat.dtype)
        x_t, anchor_t = flow.interpolate(lat, noise, t_video), flow.interpolate(anchor, a_noise, 0.999)
        vid, _ = self.model(video_rows=patchify_latents(x_t).to(dt), text_rows=prompt.to(dt),
                            audio_rows=None if audio is None else audio.to(dt),
                            anchor_rows=patchify_latents(anchor_t).to(dt), timesteps=layout.timesteps,
                            t_index=layout.t_index.to(dev), tags=layout.tags.to(dev), position_ids=layout.position_ids,
                            viewmats=expand_cameras(layout, sample["camera_w2c"]))
        tgt = patchify_latents(flow.target(lat, noise).to(lat.dtype)).float()
        a, b = self.model.local_video_rows                      # this rank's share of the video rows
        return (vid.float() - tgt[a:b]).pow(2).sum() / tgt.numel(), tgt.numel()

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
        sync_adapter_gradients(self.optimizer.params, flat, sp_group=self.ctx.sp_group, sp_size=topo.sp_size,
                               dp_group=self.ctx.dp_group, dp_size=topo.dp_size)
        norm = float(self.optimizer.clip_(self.clip))
        return GradientStatus(finite=math.isfinite(norm), norm=norm)

    def optimizer_step(self) -> None:
        self.optimizer.step()

    def scheduler_step(self) -> None:
        self.scheduler.step()

    def ema_update(self, step: int) -> None:
        if self.ema is not None and step >= self.ema_start and step % max(1, self.ema_every) == 0:
            self.ema.update()

    # -- checkpoints --------------------------------------------------------------------------------------------------
    def _contract(self) -> CheckpointContract:
        r = self.route
        return CheckpointContract(family="minimax_h3", stage=r.stage, causal_mode=r.causal_mode, objective=r.objective,
                                  objective_variant=r.variant, camera_translation_transform="logd4",
                                  parameterization="lora", sp_size=self.topology.sp_size,
                                  data_generation=str(self.config["data"].get("source", "synthetic")))

    def _rank_state(self) -> dict:
        state = capture_rank_state(self.device)
        state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in state.items()}
        state["objective_gen"] = self.gen.get_state().cpu()
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
                adapter = {n: p.detach().cpu() for n, p in self.model.named_parameters() if p.requires_grad}
                torch.save({"schema": ADAPTER_SCHEMA, "state": adapter, "rank": self.model.cfg.lora_rank}, tx.path / "adapter.pt")
                torch.save(self.optimizer.state_dict(), tx.path / "optimizer.pt")
                torch.save(self.scheduler.state_dict(), tx.path / "scheduler.pt")
                torch.save(self.ema.state_dict(self.model) if self.ema is not None else {"schema": EMA_SCHEMA, "state": None},
                           tx.path / "ema.pt")
                torch.save({"ranks": states, "world_size": topo.raw_world_size, "sp_size": topo.sp_size}, tx.path / "rank-state.pt")
                torch.save({"global_step": int(step)}, tx.path / "runtime.pt")
                done = tx.commit(step=int(step), contract=self._contract(), required_components=list(COMPONENTS), metadata={})
            return done.manifest_digest

        ident = rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None,
                                                label="checkpoint commit")
        self.checkpoint_id = ident
        return ident

    def load_checkpoint(self, path: str) -> None:
        """Exact resume: adapters (through the optimizer's fp32 master), moments, schedule, EMA, step counter and
        this rank's random streams.  The saved topology must be the running one."""
        verified = verify_checkpoint(path)
        root = verified.path
        ranks = torch.load(root / "rank-state.pt", weights_only=True)
        topo = self.topology
        if int(ranks["world_size"]) != topo.raw_world_size or int(ranks["sp_size"]) != topo.sp_size:
            raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks (SP {ranks['sp_size']}); "
                                       f"{topo.raw_world_size} (SP {topo.sp_size}) are running")
        opt = torch.load(root / "optimizer.pt", weights_only=True)
        self.optimizer.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in opt.items()})
        self.optimizer.lr = float(opt["lr"])
        self.scheduler.load_state_dict(torch.load(root / "scheduler.pt", weights_only=True))
        ema = torch.load(root / "ema.pt", weights_only=True)
        if self.ema is not None:
            if ema.get("state") is None:
                raise BackendContractError("the checkpoint holds no EMA state and this run averages its adapters")
            self.ema.load_state_dict(ema, self.model)
        mine = ranks["ranks"][topo.raw_rank]
        restore_rank_state(mine, self.device)
        self.gen.set_state(mine["objective_gen"])
        self.batches_consumed = int(mine["batches_consumed"])
        if self._corpus is not None:
            for _ in range(self.batches_consumed):
                next(self._corpus)
        self._global_step = int(torch.load(root / "runtime.pt", weights_only=True)["global_step"])
        self.checkpoint_id = verified.manifest_digest

    def validate(self, step: int) -> Mapping[str, Any]:
        """The adapters' state at a validation boundary (norms of the live and the averaged weights) and, for Stage0.5
        with ``validation.index``, the loss on the run's fixed, source-balanced validation clips (``validation.py``)."""
        report = {"step": int(step), "adapter_norm": float(self.optimizer.master.norm())}
        if self.ema is not None:
            report["ema_norm"] = float(self.ema.shadow.norm())
        val = self.config.get("validation", {}) or {}
        if val.get("index") and self.core is None:
            report["validation"] = self._validation_loss(val)
        return report

    def _validation_loss(self, val: Mapping[str, Any]) -> Mapping[str, Any]:
        import torch.distributed as dist
        from pathlib import Path

        from ...data.index import read_index
        from ...preencode.shards import read_encoded_sample
        from .validation import IndexedValidation, score

        topo = self.topology
        if getattr(self, "_validation", None) is None:
            index = Path(str(val["index"]))
            root = Path(str(val.get("root") or index.parent))

            def read(row):
                enc = read_encoded_sample(root, row.values)
                lat = enc["latents"]
                if lat.shape[0] < 2:
                    raise BackendContractError(f"{row.sample_id}: needs at least two latent frames")
                return {"target_latents": lat[1:].permute(1, 0, 2, 3).contiguous(), "anchor_latents": lat[:1].permute(1, 0, 2, 3).contiguous(),
                        "prompt_embeds": enc["text"], "camera_w2c": torch.eye(4).repeat(lat.shape[0], 1, 1)}

            self._validation = IndexedValidation(read_index(index), read, sample_count=int(val.get("sample_count", 8)),
                                                 seed=int(val.get("seed", 42)), dp_rank=topo.dp_rank, dp_size=topo.dp_size,
                                                 balance=bool(val.get("balance_sources", True)),
                                                 freeze_path=output_root(self.config) / "validation-selection.json")
            self._validation.prepare(dist if topo.raw_world_size > 1 else None)

        def loss_at(sample, t, gen):
            share, _ = self._stage0p5_share(sample, t, gen)
            if topo.sp_size > 1:
                share = share.clone()
                dist.all_reduce(share, group=self.ctx.sp_group)
            return share

        was_training = self.model.training
        self.model.eval()
        try:
            return dict(score(self._validation, loss_at, device=self.device, dist=dist if topo.dp_size > 1 else None, group=self.ctx.dp_group))
        finally:
            self.model.train(was_training)

    def close(self) -> None:
        dist_init.shutdown(self.ctx)


def run_training(config: Mapping[str, Any], *, model_config, load_released=None) -> Mapping[str, Any]:
    runtime = H3TrainingRuntime(config, model_config=model_config, load_released=load_released)
    try:
        train, rt = config["train"], config.get("runtime", {})
        policy = StepPolicy(max_steps=runtime.max_steps,
                            grad_accum=int(train.get("grad_accum", train.get("gradient_accumulation_steps", 1))),
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
                "checkpoint": str(checkpoint_model_dir(output_root(config), final)),
                "native_launches": ops.total_launches()}
    finally:
        runtime.close()
