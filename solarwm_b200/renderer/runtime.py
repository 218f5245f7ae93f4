"""Config-driven renderer training: control (flow-matching) LoRAs behind the shared optimizer-step engine.

``RendererTrainingRuntime`` reads its clips from an ``OmniStream`` (data-parallel ownership, optional length buckets),
computes the plan-weighted flow-matching loss of ``core.OmniFlowTrainer`` per microbatch, averages the flat fp32 adapter
gradients over the replicas, and keeps warm-up + cosine schedule and adapter EMA.  Checkpoints hold ``adapter.pt``,
``optimizer.pt``, ``scheduler.pt``, ``ema.pt``, ``rank-state.pt`` (random streams AND each reader's epoch / cursor) and
``runtime.pt``; the contract records the data plan's fingerprint, the observation profile and the parents the adapters
started from, so a resume under another corpus, profile or parent is refused.  ``export_adapter`` turns a checkpoint
into a standalone adapter file (live or averaged weights).

Reference: RendererTrainingRuntime (solar/renderer/runtime.py:63-187), run_control_training
(solar/renderer/training.py:53-74), export (solar/renderer/export_lora.py).
"""
from __future__ import annotations

import hashlib
import math
from pathlib import Path
from typing import Any, Mapping, Optional

import torch

from .. import ops
from ..backends.minimax_h3.runtime import ADAPTER_SCHEMA, EMA_SCHEMA, AdapterEMA, WarmupCosine, sync_adapter_gradients
from ..checkpoint.store import CheckpointContract, CheckpointTransaction, verify_checkpoint
from ..engine.master_adamw import FP32MasterAdamW
from ..engine.train_engine import (BatchIdentity, GradientStatus, JsonlEventSink, MicrobatchResult, StepPolicy,
                                   TrainingEngine)
from ..errors import BackendContractError, ConfigurationError
from ..models.h3 import H3DiT, h3_preset
from ..parallel import dist_init
from ..runtime import distributed as rdist
from ..runtime.output_layout import checkpoint_model_dir, events_path, output_root
from ..runtime.randomness import model_init_seed, objective_seed
from ..runtime.safe_state import capture_rank_state, restore_rank_state
from .core import OmniFlowTrainer
from .data import MemberContract, OmniStream
from .known_degree import ObservationProfile

COMPONENTS = ("adapter.pt", "optimizer.pt", "scheduler.pt", "ema.pt", "rank-state.pt", "runtime.pt")


def validate_config(config: Mapping[str, Any]) -> None:
    """The renderer's own section contract (it does not go through the backend route table)."""
    for section in ("model", "data", "train", "runtime"):
        if not isinstance(config.get(section), Mapping):
            raise ConfigurationError(f"renderer config needs a {section} section")
    train, data = config["train"], config["data"]
    if train.get("objective", "flow_matching") not in ("flow_matching", "dmd"):
        raise ConfigurationError("train.objective is flow_matching (control) or dmd (few-step distillation)")
    if int(train.get("max_steps", 0)) < 1:
        raise ConfigurationError("train.max_steps must be positive")
    if int(train.get("gradient_accumulation_steps", 1)) < 1:
        raise ConfigurationError("train.gradient_accumulation_steps must be positive")
    for key in ("omni_root", "omni_index"):
        if not data.get(key):
            raise ConfigurationError(f"data.{key} is required")
    if int((config.get("distributed", {}) or {}).get("sequence_parallel_size", 1)) != 1:
        raise ConfigurationError("renderer training is data parallel: distributed.sequence_parallel_size must be 1")
    causal = train.get("causal_omni")
    if causal is not None:
        if not isinstance(causal, Mapping) or int(causal.get("chunk", 5)) < 1 or int(causal.get("window", 6)) < 1:
            raise ConfigurationError("train.causal_omni is a mapping with positive chunk and window")
    if not config["runtime"].get("output_dir"):
        raise ConfigurationError("runtime.output_dir is required")


def weight_identity(path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as fh:
        for block in iter(lambda: fh.read(1 << 20), b""):
            h.update(block)
    return f"sha256:{h.hexdigest()}"


def read_adapter(path) -> Mapping[str, torch.Tensor]:
    """An adapter file, or the ``adapter.pt`` of a verified checkpoint directory."""
    p = Path(path)
    if p.is_dir():
        p = verify_checkpoint(p).path / "adapter.pt"
    doc = torch.load(str(p), map_location="cpu", weights_only=True)
    if not isinstance(doc, dict) or doc.get("schema") != ADAPTER_SCHEMA or not isinstance(doc.get("state"), dict):
        raise BackendContractError(f"{p} is not an adapter file")
    return doc["state"]


class RendererTrainingRuntime:
    def __init__(self, config: Mapping[str, Any]):
        validate_config(config)
        self.config = config
        train, data, model_cfg = config["train"], config["data"], config["model"]
        self.ctx = dist_init.initialize(1, device=str(config["runtime"].get("device", "auto")))
        topo = self.topology = self.ctx.topology
        dev = self.device = self.ctx.device
        self.seed = int(data.get("seed", 42))
        cfg = h3_preset(str(model_cfg.get("architecture", "h3_33b")))
        cfg.lora_rank = int((model_cfg.get("adapter", {}) or {}).get("rank", cfg.lora_rank or 8))
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        self.model = H3DiT(cfg, device=dev, dtype=dtype, seed=model_init_seed("minimax_h3", self.seed) % (2 ** 31))
        o = train.get("optimizer", {}) or {}
        self.clip = float(o.get("grad_clip", 1.0))
        self.optimizer = FP32MasterAdamW(self.model.trainable_parameters(), lr=float(o.get("lr", o.get("learning_rate", 1e-4))),
                                         betas=tuple(float(b) for b in o.get("betas", (0.9, 0.95))),
                                         eps=float(o.get("eps", 1e-8)), weight_decay=float(o.get("weight_decay", 0.01)))
        self.max_steps = int(config["runtime"].get("max_steps_override") or train["max_steps"])
        self.scheduler = WarmupCosine(self.optimizer, warmup=int(o.get("warmup_steps", 0)), total=self.max_steps,
                                      min_ratio=float(o.get("min_lr_ratio", 0.1)))
        ck = self.ck = config.get("checkpoint", {}) or {}
        e = ck.get("ema", {}) or {}
        self.ema = AdapterEMA(self.optimizer, float(e.get("decay", 0.999))) if e.get("enabled", True) else None
        self.ema_start, self.ema_every = int(e.get("start_step", 0)), int(e.get("update_every_steps", 1))
        self.profile = ObservationProfile.from_config(train) or ObservationProfile()
        causal = train.get("causal_omni")
        if causal:
            from .causal import CausalOmniTrainer

            self.core = CausalOmniTrainer(self.model, self.optimizer, chunk=int(causal.get("chunk", 5)), window=int(causal.get("window", 6)),
                                          seed=objective_seed(self.seed, topo.dp_rank) % (2 ** 31))
        else:
            self.core = OmniFlowTrainer(cfg, dev, self.profile, model=self.model, optimizer=self.optimizer,
                                        seed=objective_seed(self.seed, topo.dp_rank) % (2 ** 31))
        c = data.get("member_contract", {}) or {}
        contract = MemberContract(latent_channels=int(c.get("latent_channels", 24)), text_dim=int(c.get("text_dim", cfg.text_dim)),
                                  grids=tuple(tuple(int(v) for v in g) for g in c.get("grids", ((48, 84), (84, 48)))),
                                  frames_period=int(c.get("frames_period", 5)), frames_offset=int(c.get("frames_offset", 2)))
        self.reader = OmniStream(root=data["omni_root"], index=data["omni_index"], dp_rank=topo.dp_rank, dp_size=topo.dp_size,
                                 seed=self.seed, shuffle=bool(data.get("shuffle", True)),
                                 length_buckets=bool(data.get("omni_length_buckets", True)), contract=contract)
        self.plan_fingerprint = self.reader.plan_fingerprint
        self.parents = {}
        init = (ck.get("initialization") or {}).get("student")
        if init:
            if init.get("weight_source", "live") != "live":
                raise BackendContractError("renderer initialization takes live adapter weights")
            self._adopt(read_adapter(init["path"]))
            target = Path(init["path"])
            self.parents["control_initialization"] = weight_identity(target / "adapter.pt" if target.is_dir() else target)
        self._global_step = 0
        self.checkpoint_id = "init:" + (self.parents.get("control_initialization") or "random")
        if ck.get("resume_from"):
            self.load_checkpoint(str(ck["resume_from"]))

    def _adopt(self, state: Mapping[str, torch.Tensor]) -> None:
        own = {n: p for n, p in self.model.named_parameters() if p.requires_grad}
        if set(own) != set(state):
            raise BackendContractError("the adapter file does not hold exactly this architecture's adapter tensors")
        with torch.no_grad():
            for n, p in own.items():
                if tuple(state[n].shape) != tuple(p.shape):
                    raise BackendContractError(f"{n}: adapter shape {tuple(state[n].shape)} does not fit {tuple(p.shape)}")
                p.copy_(state[n].to(p))
            self.optimizer.master.copy_(self.optimizer.live.float())
        if self.ema is not None:
            self.ema.shadow.copy_(self.optimizer.master)

    # -- engine hooks -------------------------------------------------------------------------------------------------------
    @property
    def global_step(self) -> int:
        return self._global_step

    def set_global_step(self, step: int) -> None:
        self._global_step = int(step)

    def zero_grad(self) -> None:
        self.optimizer.zero_grad()

    def _all_finite(self, finite: bool, message: str) -> None:
        if self.topology.dp_size > 1:
            import torch.distributed as dist

            flag = torch.tensor(int(finite), dtype=torch.int32, device=self.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            finite = bool(flag.item())
        if not finite:
            raise FloatingPointError(message)

    def train_microbatch(self, micro_index: int, grad_accum: int) -> MicrobatchResult:
        import torch.distributed as dist

        # a rank whose read fails takes the others down with it instead of leaving them in the next collective
        sample = rdist.collective_call(self.reader.next, dist=dist if self.topology.raw_world_size > 1 else None,
                                       label="renderer data read")
        loss = self.core.compute_loss(sample.as_training_sample())
        (loss / grad_accum).backward()
        value = float(loss.detach())
        self._all_finite(math.isfinite(value), f"non-finite renderer loss on {sample.sample_id}")
        plan = self.core.last_plan
        identity = BatchIdentity((sample.sample_id,), (0,), (objective_seed(self.seed, self.topology.dp_rank) + self._global_step,),
                                 self.checkpoint_id, self.plan_fingerprint)
        return MicrobatchResult(identity, {"loss": value, "generated_fraction": float(plan.generated_fraction)})

    def assert_sp_peer_identity(self, identity: BatchIdentity) -> None:
        return None                                 # no sequence parallelism here

    def prepare_optimizer_step(self) -> GradientStatus:
        flat = self.optimizer.gather_grads()
        sync_adapter_gradients(self.optimizer.params, flat, sp_group=None, sp_size=1, dp_group=self.ctx.dp_group,
                               dp_size=self.topology.dp_size)
        norm = float(self.optimizer.clip_(self.clip))
        return GradientStatus(finite=math.isfinite(norm), norm=norm)

    def optimizer_step(self) -> None:
        self.optimizer.step()

    def scheduler_step(self) -> None:
        self.scheduler.step()

    def ema_update(self, step: int) -> None:
        if self.ema is not None and step >= self.ema_start and step % self.ema_every == 0:
            self.ema.update()

    # -- checkpoints --------------------------------------------------------------------------------------------------------
    def _contract(self) -> CheckpointContract:
        train = self.config["train"]
        return CheckpointContract(family="minimax_h3_renderer", stage="control",
                                  causal_mode="block_causal" if train.get("causal_omni") else "bidirectional",
                                  objective=str(train.get("objective", "flow_matching")), objective_variant="data_ward_velocity",
                                  camera_translation_transform="logd4", parameterization=f"lora-r{self.model.cfg.lora_rank}",
                                  sp_size=1, data_generation="solarrenderer.omni.v1")

    def _metadata(self) -> dict:
        return {"observations": dict(self.profile.fingerprint()), "data_plan": self.plan_fingerprint, "parents": dict(self.parents),
                "causal_omni": dict(self.config["train"].get("causal_omni") or {})}

    def _rank_state(self) -> dict:
        state = {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in capture_rank_state(self.device).items()}
        state["objective_gen"] = self.core.gen.get_state().cpu()
        state["plan_rng"] = self.core.rng.bit_generator.state
        state["reader"] = self.reader.state_dict()
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
                torch.save({"ranks": states, "world_size": topo.raw_world_size}, tx.path / "rank-state.pt")
                torch.save({"global_step": int(step), **self._metadata()}, tx.path / "runtime.pt")
                done = tx.commit(step=int(step), contract=self._contract(), required_components=list(COMPONENTS),
                                 metadata=self._metadata())
            return done.manifest_digest

        self.checkpoint_id = rdist.collective_rank_zero_call(write, dist=dist if topo.raw_world_size > 1 else None,
                                                             label="checkpoint commit")
        return self.checkpoint_id

    def load_checkpoint(self, path: str) -> None:
        verified = verify_checkpoint(path)
        root, topo = verified.path, self.topology
        run = torch.load(root / "runtime.pt", weights_only=True)
        mine = self._metadata()
        for key, what in (("data_plan", "data plan"), ("observations", "observation profile"), ("parents", "parent adapters"),
                          ("causal_omni", "causal chunking")):
            if run.get(key) != mine[key]:
                raise BackendContractError(f"the checkpoint was trained under another {what}")
        ranks = torch.load(root / "rank-state.pt", weights_only=True)
        if int(ranks["world_size"]) != topo.raw_world_size:
            raise BackendContractError(f"checkpoint was written by {ranks['world_size']} ranks; {topo.raw_world_size} are running")
        opt = torch.load(root / "optimizer.pt", weights_only=True)
        self.optimizer.load_state_dict({k: (v.to(self.device) if torch.is_tensor(v) else v) for k, v in opt.items()})
        self.optimizer.lr = float(opt["lr"])
        self.scheduler.load_state_dict(torch.load(root / "scheduler.pt", weights_only=True))
        ema = torch.load(root / "ema.pt", weights_only=True)
        if self.ema is not None:
            if ema.get("state") is None:
                raise BackendContractError("the checkpoint holds no EMA state and this run averages its adapters")
            self.ema.load_state_dict(ema, self.model)
        state = ranks["ranks"][topo.raw_rank]
        restore_rank_state(state, self.device)
        self.core.gen.set_state(state["objective_gen"])
        self.core.rng.bit_generator.state = state["plan_rng"]
        self.reader.load_state_dict(state["reader"])
        self._global_step = int(run["global_step"])
        self.checkpoint_id = verified.manifest_digest

    def validate(self, step: int) -> Mapping[str, Any]:
        raise BackendContractError("renderer checkpoints are evaluated with the renderer's render command")

    def close(self) -> None:
        self.reader.close()
        dist_init.shutdown(self.ctx)


def run_control_training(config: Mapping[str, Any]) -> Mapping[str, Any]:
    runtime = RendererTrainingRuntime(config)
    try:
        train, ck = config["train"], config.get("checkpoint", {}) or {}
        policy = StepPolicy(max_steps=runtime.max_steps, grad_accum=int(train.get("gradient_accumulation_steps", 1)),
                            save_every=int(ck.get("save_every_steps", 0)),
                            save_steps=tuple(int(s) for s in ck.get("save_steps", ())) + (runtime.max_steps,))
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


def export_adapter(checkpoint, destination, *, weight_source: str = "live") -> Mapping[str, Any]:
    """A verified checkpoint's adapters as one standalone file: ``live`` = ``adapter.pt``, ``ema`` = the averaged weights
    (cast to the live dtype).  The file records where it came from."""
    if weight_source not in ("live", "ema"):
        raise ConfigurationError("weight_source is live or ema")
    verified = verify_checkpoint(checkpoint)
    live = torch.load(verified.path / "adapter.pt", map_location="cpu", weights_only=True)
    state = live["state"]
    if weight_source == "ema":
        ema = torch.load(verified.path / "ema.pt", map_location="cpu", weights_only=True)
        if ema.get("state") is None:
            raise BackendContractError("the checkpoint holds no averaged weights")
        if set(ema["state"]) != set(state):
            raise BackendContractError("the averaged weights do not cover the adapters")
        state = {n: ema["state"][n].to(state[n].dtype) for n in state}
    out = Path(destination)
    out.parent.mkdir(parents=True, exist_ok=True)
    doc = {"schema": ADAPTER_SCHEMA, "state": state, "rank": live.get("rank"), "weight_source": weight_source,
           "parent_checkpoint": verified.manifest_digest, "step": int(verified.step)}
    torch.save(doc, out)
    return {"path": str(out), "tensors": len(state), "weight_source": weight_source, "identity": weight_identity(out)}
