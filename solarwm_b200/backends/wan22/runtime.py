"""``TrainingRuntime`` implementation for the Wan Stage0.5 flow-matching route and the
``run_training`` entry the backend calls (reference: Wan5BStage0p5Runtime and
run_stage0p5_training, solar/backends/wan22/runtime/stage0p5.py:105-587)."""
from __future__ import annotations

import hashlib
from typing import Any, Iterator, Mapping

import torch

from ...config.routes import validate_route
from ...engine.schedule import WarmupCosine
from ...engine.train_engine import (BatchIdentity, GradientStatus, JsonlEventSink, MicrobatchResult, StepPolicy,
                                    TrainingEngine)
from ...errors import BackendContractError, ConfigurationError
from ...parallel import dist_init
from ...runtime import distributed as rdist
from ...runtime.output_layout import events_path, output_root
from ...runtime.randomness import model_init_seed, objective_seed
from ...runtime.safe_state import capture_rank_state
from . import checkpoint as ckpt
from .contracts import PROFILES, architecture, latent_frames
from .stage0p5 import Stage0p5Options, WanStage0p5Trainer


def synthetic_batches(config, arch, device) -> Iterator[dict]:
    data, family = config["data"], config["model"]["family"]
    prof = PROFILES[family]
    frames = latent_frames(int(data["pixel_frames"]), prof.vae_stride[0])
    h = int(data.get("latent_height", 16))
    w = int(data.get("latent_width", 16))
    micro = int(config["train"].get("micro_batch_size", 1))
    g = torch.Generator().manual_seed(int(data.get("seed", 0)))
    step = 0
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    ch = arch.out_dim
    while True:
        lat = torch.randn(micro, frames, ch, h, w, generator=g).to(dtype)
        txt = torch.randn(micro, arch.text_len, arch.text_dim, generator=g).to(dtype)
        batch = {"latents": lat, "text": txt, "sample_ids": [f"synthetic-{step}-{i}" for i in range(micro)],
                 "start_frames": [0] * micro}
        if data.get("cameras"):                     # a seeded dolly per clip for the camera-conditioned routes
            c2w = torch.eye(4).repeat(micro, frames, 1, 1)
            c2w[:, :, 2, 3] = torch.arange(frames) * 0.05 * (1.0 + torch.rand(micro, 1, generator=g))
            batch["camera_c2w"] = c2w
            batch["camera_K"] = torch.tensor([[0.505, 0.0, 0.5], [0.0, 0.898, 0.5], [0.0, 0.0, 1.0]]).repeat(micro, frames, 1, 1)
        if arch.in_dim > ch:
            batch["y"] = torch.randn(micro, frames, arch.in_dim - ch, h, w, generator=g).to(dtype)
        if device.type == "cuda":
            batch = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in batch.items()}
        step += 1
        yield batch


def iter_encoded_samples(data: Mapping[str, Any], dp_rank: int = 0, dp_size: int = 1):
    """``(index row, {name: tensor})`` pairs of a pre-encoded corpus, forever: ``data.index`` is the corpus index
    written by the pre-encoding run, shards sit under ``data.root`` (default: beside the index).  Every epoch is one
    seeded permutation of the rows; occurrence v of the permutation belongs to logical DP rank ``v % dp_size`` (SP
    peers read the same samples).  A pure function of (index, seed, rank): a resumed run that replays its consumed
    count reads on exactly where it stopped."""
    import json as _json
    from pathlib import Path

    import numpy as np

    from ...data.index import read_index
    from ...errors import DataContractError
    from ...preencode.contracts import EncoderContract
    from ...preencode.shards import read_encoded_sample

    index = Path(str(data["index"]))
    root = Path(str(data.get("root") or index.parent))
    rows = read_index(index)
    if not rows:
        raise DataContractError(f"{index} holds no samples")
    contract = None
    cpath = root / "encoder-contract.json"
    if cpath.exists():
        contract = EncoderContract.from_dict(_json.loads(cpath.read_text()))
    seed, epoch = int(data.get("seed", 0)), 0
    while True:
        order = np.random.default_rng([seed, epoch]).permutation(len(rows))
        mine = [rows[int(i)] for v, i in enumerate(order) if v % dp_size == dp_rank]
        if not mine:
            raise DataContractError(f"rank {dp_rank} of {dp_size} owns no sample of {index}")
        for row in mine:
            yield row, read_encoded_sample(root, row.values, contract)
        epoch += 1


def encoded_batches(config, arch, device, dp_rank: int = 0, dp_size: int = 1) -> Iterator[dict]:
    """Training batches out of a pre-encoded corpus (``data.source: index``): ``micro_batch_size`` consecutive samples of
    this rank's stream, checked against the architecture (latent channels, text geometry, enough latent frames)."""
    from ...errors import DataContractError

    data = config["data"]
    frames = latent_frames(int(data["pixel_frames"]), PROFILES[config["model"]["family"]].vae_stride[0])
    micro = int(config["train"].get("micro_batch_size", 1))
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    stream = iter_encoded_samples(data, dp_rank, dp_size)
    while True:
        group = [next(stream) for _ in range(micro)]
        for r, smp in group:
            lat, txt = smp["latents"], smp["text"]
            if lat.dim() != 4 or lat.shape[0] < frames or lat.shape[1] != arch.out_dim:
                raise DataContractError(f"{r.sample_id}: latents {tuple(lat.shape)} do not provide [{frames}+, {arch.out_dim}, h, w]")
            if tuple(txt.shape) != (arch.text_len, arch.text_dim):
                raise DataContractError(f"{r.sample_id}: text {tuple(txt.shape)} is not ({arch.text_len}, {arch.text_dim})")
        batch = {"latents": torch.stack([smp["latents"][:frames] for _, smp in group]).to(dtype),
                 "text": torch.stack([smp["text"] for _, smp in group]).to(dtype),
                 "sample_ids": [r.sample_id for r, _ in group], "start_frames": [0] * micro}
        if all("camera_c2w" in smp for _, smp in group):
            batch["camera_c2w"] = torch.stack([smp["camera_c2w"][:frames].float() for _, smp in group])
            batch["camera_K"] = torch.stack([smp["camera_K"][:frames].float() for _, smp in group])
        if device.type == "cuda":
            batch = {k: (v.pin_memory() if torch.is_tensor(v) else v) for k, v in batch.items()}
        yield batch


def camera_condition(batch: Mapping[str, Any], arch, transform: str, device):
    """The ``y_camera`` argument of the camera-conditioned models out of a batch's absolute poses: world-to-camera
    matrices relative to each clip's first camera, the normalised intrinsics, the translation compression.  ``None`` when
    the architecture has no camera path or the batch carries no cameras."""
    if getattr(arch, "camera_attention_mode", "none") == "none" or "camera_c2w" not in batch:
        return None
    c2w = batch["camera_c2w"].to(device=device, dtype=torch.float64)
    if c2w.dim() != 4 or tuple(c2w.shape[-2:]) != (4, 4) or not bool(torch.isfinite(c2w).all()):
        raise BackendContractError("camera_c2w must be finite [B, F, 4, 4]")
    rel = torch.linalg.inv(c2w[:, :1]) @ c2w
    rel[:, 0] = torch.eye(4, dtype=torch.float64, device=device)
    Ks = batch.get("camera_K")
    return {"viewmats": torch.linalg.inv(rel).float(), "Ks": None if Ks is None else Ks.to(device=device, dtype=torch.float32),
            "transform": str(transform)}


def build_online_codecs(config: Mapping[str, Any], device):
    """The text encoder and the video VAE of ``data.encoding: online`` training.  With ``model.base_path`` the published
    files are loaded strictly (``WanTextEncoder.from_released``; ``Wan5BVAE`` / ``WanA14BVAE.from_checkpoint``); without
    one, ``data.online_codecs`` (``{t5: T5Config fields, vae: {z_dim, base, temporal_ups}}``) builds seeded stand-ins so the
    path runs without any weight file (reference: build_online_codec_components,
    solar/backends/wan22/runtime/components.py:662-673)."""
    from ...models.t5 import T5Config, WanTextEncoder
    from ...models.vae import VAEConfig, VideoVAE
    from .codec import Wan5BVAE, WanA14BVAE, WanVideoCodec
    from .readiness import AssetLayout

    family = str(config["model"]["family"])
    layout = AssetLayout.from_config(config)
    if layout.base is not None:
        kind = {"wan22_ti2v_5b": Wan5BVAE, "wan22_i2v_a14b": WanA14BVAE}.get(family)
        if kind is None:
            raise BackendContractError(f"no online codec for family {family!r}")
        text = WanTextEncoder.from_released(layout.text_encoder, layout.tokenizer, device=device)
        return text, kind.from_checkpoint(layout.vae, device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    spec = config["data"].get("online_codecs") or {}
    tcfg = T5Config(**spec["t5"]) if "t5" in spec else T5Config.tiny()
    v = dict(spec.get("vae", {}))
    if "temporal_ups" in v:
        v["temporal_ups"] = tuple(bool(u) for u in v["temporal_ups"])
    vae = VideoVAE(VAEConfig(**v)).to(device=device, dtype=torch.float32).eval()
    return WanTextEncoder(tcfg, device=device, dtype=torch.float32), WanVideoCodec(vae)


def online_batches(config, arch, device, dp_rank: int = 0, dp_size: int = 1) -> Iterator[dict]:
    """Training batches encoded on the fly (``data.encoding: online``): raw clips and captions of this rank (the same
    reader the pre-encoder uses: synthetic clips, or tar shards of ``.npy`` / compressed video) go through the frozen VAE
    and text encoder right before the step, so no latent corpus has to exist.  The epoch repeats when the source ends."""
    from ...errors import DataContractError
    from .preencode import _clips

    text_encoder, codec = build_online_codecs(config, device)
    data = config["data"]
    micro = int(config["train"].get("micro_batch_size", 1))
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    source = dict(config, preencode={"source": str(data.get("raw_source", data.get("source", "synthetic"))).replace("raw", "index"),
                                      "raw_root": data.get("raw_root"), "raw_index": data.get("raw_index"),
                                      "num_samples": int(data.get("num_samples", 8))})
    while True:
        group = []
        for sample_id, clip, caption, *_ in _clips(source, dp_rank, dp_size):
            with torch.no_grad():
                z = codec.encode(clip.permute(1, 0, 2, 3).unsqueeze(0).to(device))[0]                 # [F, z, h, w]
                e = text_encoder([caption])[0]
            if z.shape[1] != arch.out_dim or tuple(e.shape) != (arch.text_len, arch.text_dim):
                raise DataContractError(f"{sample_id}: online codecs give latents {tuple(z.shape)} / text {tuple(e.shape)}; the model "
                                        f"takes {arch.out_dim} channels and text ({arch.text_len}, {arch.text_dim})")
            if not bool(torch.isfinite(z.float()).all()):
                raise DataContractError(f"{sample_id}: the VAE produced non-finite latents")
            group.append((sample_id, z, e))
            if len(group) == micro:
                yield {"latents": torch.stack([g[1] for g in group]).to(dtype), "text": torch.stack([g[2] for g in group]).to(dtype),
                       "sample_ids": [g[0] for g in group], "start_frames": [0] * micro}
                group = []
        if not group and micro > int(data.get("num_samples", 8)) and source["preencode"]["source"] == "synthetic":
            raise DataContractError("the online source holds fewer clips than one micro batch")


def activation_and_sharding_options(train: Mapping[str, Any], world_size: int) -> Mapping[str, Any]:
    """Trainer options out of the ``train`` section.

    ``fsdp.activation_checkpointing``: false / true ("full") / "none" | "full" | "selective";
    ``fsdp.saved_attention_blocks`` > 0 means "selective" (attention outputs are carried across the recompute);
    ``activation_memory.keep_blocks`` / ``.lean``: how many of the last blocks stay resident, and whether resident
    blocks rebuild their norm outputs and FFN hidden tensor in backward;
    optimizer sharding is on with ``zero.enabled`` or ``fsdp.enabled`` (more than one rank), its transport is
    ``zero.transport``: "collective" (NCCL) or "fused" (peer loads / stores over NVLink);
    ``fsdp.shard_parameters`` (fused transport only) also shards every block's parameters and gradient buffers with
    just-in-time gathers; ``cuda_graph`` captures the whole optimizer step once and replays it (fused transports or
    one rank, no gradient accumulation)."""
    fsdp = train.get("fsdp", {}) or {}
    ac = fsdp.get("activation_checkpointing", False)
    if isinstance(ac, str):
        mode = ac.strip().lower()
        if mode not in ("none", "full", "selective"):
            raise ConfigurationError("train.fsdp.activation_checkpointing must be a boolean or none / full / selective")
    else:
        mode = "full" if ac else "none"
    if int(fsdp.get("saved_attention_blocks", 0) or 0) > 0 and mode != "none":
        mode = "selective"
    mem = train.get("activation_memory", {}) or {}
    zero_cfg = train.get("zero", {}) or {}
    transport = str(zero_cfg.get("transport", "collective"))
    if transport not in ("collective", "fused"):
        raise ConfigurationError("train.zero.transport must be collective or fused")
    zero = bool(zero_cfg.get("enabled", fsdp.get("enabled", False))) and world_size > 1
    shard = bool(fsdp.get("shard_parameters", False)) and zero
    if shard and transport != "fused":
        raise ConfigurationError("train.fsdp.shard_parameters needs train.zero.transport: fused")
    return dict(checkpointing=mode, keep_blocks=int(mem.get("keep_blocks", 0)), lean_kept=bool(mem.get("lean", False)),
                zero=zero, zero_transport=transport, shard_params=shard, cuda_graph=bool(train.get("cuda_graph", False)))


class WanStage0p5Runtime:
    """Adapts ``WanStage0p5Trainer`` to the engine's 11-hook protocol."""

    def __init__(self, config: Mapping[str, Any], trainer_cls=WanStage0p5Trainer, options_cls=Stage0p5Options,
                 extra_options: Mapping[str, Any] = None):
        self.config = config
        self.route = validate_route(config)
        dist_cfg = config.get("distributed", {}) or {}
        self.ctx = dist_init.initialize(int(dist_cfg.get("sequence_parallel_size", 1)),
                                        device=str(config.get("runtime", {}).get("device", "auto")))
        topo = self.ctx.topology
        self.arch = architecture(config)
        train = config["train"]
        opt = train.get("optimizer", {}) or {}
        ema = train.get("ema", {}) or {}
        seed = int(config["data"].get("seed", 0))
        opts = options_cls(
            lr=float(opt.get("lr", 1e-4)), betas=tuple(opt.get("betas", (0.9, 0.999))), eps=float(opt.get("eps", 1e-8)),
            weight_decay=float(opt.get("weight_decay", 0.01)), max_grad_norm=float(opt.get("grad_clip", 1.0)),
            timestep_shift=float(config["model"].get("timestep_shift", 5.0)),
            sigma_sampling=str(train.get("sigma_sampling", "uniform_index")),
            image_dropout=float(train.get("i2v_image_condition_dropout", 0.0)),
            grad_accum=int(train.get("grad_accum", train.get("gradient_accumulation_steps", 1))),
            ema_decay=float(ema["decay"]) if ema.get("enabled") else None,
            seed=seed, **activation_and_sharding_options(train, topo.raw_world_size), **dict(extra_options or {}))
        dtype = torch.bfloat16 if self.ctx.device.type == "cuda" else torch.float32
        from ...models.wan import WanDiT

        model = WanDiT(self.arch, device=self.ctx.device, dtype=dtype,
                       seed=model_init_seed(self.route.family, seed), shard_pad=topo.raw_world_size)
        if bool(config["model"].get("nonzero_head_init", False)):
            with torch.no_grad():
                model.get_parameter("head.head.weight").normal_(0, 0.02)
        sp_ctx, heap = self._fused_transports(dist_cfg, opts, model)
        if trainer_cls is WanStage0p5Trainer:
            self.trainer = trainer_cls(self.arch, self.ctx.device, opts, sp=sp_ctx, dtype=dtype, model=model,
                                       dp_group=self.ctx.dp_group, dp_size=topo.dp_size, heap=heap)
        else:
            self.trainer = trainer_cls(self.arch, self.ctx.device, opts, sp=sp_ctx, model=model,
                                       dp_group=self.ctx.dp_group, dp_size=topo.dp_size, heap=heap)
        self.trainer.gen.manual_seed(objective_seed(seed, topo.dp_rank))
        self._graphed = bool(getattr(opts, "cuda_graph", False)) and self.ctx.device.type == "cuda"
        self.scheduler = WarmupCosine(self.trainer.optimizer, warmup_steps=int(train.get("warmup_steps", 0)),
                                      total_steps=int(train["max_steps"]),
                                      min_lr_ratio=float(opt.get("min_lr_ratio", 0.1)))
        if str(config["data"].get("encoding", "preencoded")) == "online":
            self.batches = online_batches(config, self.arch, self.ctx.device, topo.dp_rank, topo.dp_size)
        elif str(config["data"].get("source", "synthetic")) == "index":
            self.batches = encoded_batches(config, self.arch, self.ctx.device, topo.dp_rank, topo.dp_size)
        else:
            self.batches = synthetic_batches(config, self.arch, self.ctx.device)
        self.batches_consumed = 0
        self._step = 0
        self.checkpoint_id = "init:random"
        self.contract = ckpt.build_contract(config, self.route, topo.sp_size)
        self._resume()

    # -- checkpoint wiring ---------------------------------------------------------------
    def _resume(self) -> None:
        c = self.config.get("checkpoint", {}) or {}
        mode = str(c.get("mode", "none"))
        if mode == "none" or not c.get("resume_from"):
            return
        verified, payload = ckpt.load_checkpoint(
            c["resume_from"], model=self.trainer.model, optimizer=self.trainer.optimizer, scheduler=self.scheduler,
            mode=mode, expected=self.contract, weight_source=str(c.get("weight_source", "live")),
            map_location=self.ctx.device, ema_source=c.get("ema_source"))
        self.checkpoint_id = verified.manifest_digest
        if mode == "full_resume":
            self._step = int(payload["global_step"])
            self.trainer.global_step = self._step
            # exact resume: this rank's objective RNG stream and reader cursor
            states = payload.get("rank_runtime_state") or []
            rank = self.ctx.topology.raw_rank
            if rank < len(states) and states[rank] is not None:
                mine = states[rank]
                self.trainer.gen.set_state(mine["objective_gen"].cpu())
                for _ in range(int(mine["batches_consumed"])):
                    next(self.batches)
                self.batches_consumed = int(mine["batches_consumed"])

    # -- TrainingRuntime -----------------------------------------------------------------
    @property
    def global_step(self) -> int:
        return self._step

    def _fused_transports(self, dist_cfg, opts, model):
        """``distributed.sp_transport: fused`` and ``train.zero.transport: fused`` (both opt-in, CUDA, one node): the
        Ulysses exchanges ride on the producing kernels and the optimizer reduces / pushes over peer memory.  Every
        rank must be able to map every peer; the ranks agree on that before a symmetric buffer exists and fall back to
        the NCCL forms together."""
        sp_ctx, heap = self.ctx.sp, None
        topo = self.ctx.topology
        want_sp = str(dist_cfg.get("sp_transport", "nccl")) == "fused" and topo.sp_size > 1
        want_zero = opts.zero and opts.zero_transport == "fused"
        if not (want_sp or want_zero):
            return sp_ctx, heap
        if self.ctx.device.type != "cuda":
            raise ConfigurationError("the fused transports need CUDA devices")
        import torch.distributed as dist

        local, n = self.ctx.device.index, torch.cuda.device_count()
        can = n >= topo.raw_world_size and all(torch.cuda.can_device_access_peer(local, d) for d in range(topo.raw_world_size)
                                               if d != local)
        agree = torch.tensor([1 if can else 0], device=self.ctx.device)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            if want_zero:
                opts.zero_transport = "collective"
            return sp_ctx, heap
        if want_sp:
            from ...parallel.fused_ulysses import FusedUlysses

            data = self.config["data"]
            pt, ph, pw = self.arch.patch_size
            frames = latent_frames(int(data["pixel_frames"]), PROFILES[self.route.family].vae_stride[0]) \
                if "latent_frames" not in data else int(data["latent_frames"])
            tokens = (frames // pt) * (int(data["latent_height"]) // ph) * (int(data["latent_width"]) // pw)
            sp_ctx = FusedUlysses(self.ctx.sp_group, max_tokens=tokens, dim=self.arch.dim, num_heads=self.arch.num_heads)
        if want_zero:
            from ...parallel.symm import SymmetricHeap

            from ...parallel.zero import fused_heap_bytes

            sharded = [b.unit for b in model.blocks] if getattr(opts, "shard_params", False) else ()
            heap = SymmetricHeap(fused_heap_bytes(model.units(), topo.raw_world_size, sharded) + (1 << 16), None)
        return sp_ctx, heap

    def zero_grad(self) -> None:
        self.trainer.model.zero_grads()

    def train_microbatch(self, micro_index: int, grad_accum: int) -> MicrobatchResult:
        batch = next(self.batches)
        self.batches_consumed += 1
        dev = self.ctx.device
        seed_digest = hashlib.blake2s(self.trainer.gen.get_state().cpu().numpy().tobytes()).hexdigest()
        self.trainer.y_camera = camera_condition(batch, self.arch, str(self.config["model"].get("camera_translation_transform", "linear")), dev)
        if self._graphed and self.trainer.y_camera is not None:
            raise BackendContractError("camera-conditioned steps are not captured as a graph: set train.cuda_graph: false")
        if self._graphed:
            # ``train.cuda_graph``: the WHOLE optimizer step (this microbatch, the reduce-scatter, clipping and the
            # sharded AdamW with its device-side skip on a non-finite norm) is one replayed graph; the two optimizer
            # hooks that follow only report what it computed
            loss = self.trainer.train_step({k: batch[k] for k in ("latents", "text", "y") if k in batch})
        else:
            loss = self.trainer.microbatch(batch["latents"].to(dev, non_blocking=True),
                                           batch["text"].to(dev, non_blocking=True),
                                           None if "y" not in batch else batch["y"].to(dev, non_blocking=True))
        value = float(loss.item())
        if value != value or value in (float("inf"), float("-inf")):
            raise BackendContractError(f"non-finite Wan Stage0.5 loss: {value}")
        plan = repr((batch["sample_ids"], batch["start_frames"]))
        ident = BatchIdentity(tuple(batch["sample_ids"]), tuple(batch["start_frames"]),
                              tuple(int(seed_digest[:15], 16) + i for i in range(len(batch["sample_ids"]))),
                              self.checkpoint_id, hashlib.blake2s(plan.encode()).hexdigest())
        return MicrobatchResult(ident, {"flow_matching": value})

    def assert_sp_peer_identity(self, identity: BatchIdentity) -> None:
        rdist.gather_and_assert_sp_identity(
            {"sample_ids": identity.sample_ids, "start_frames": identity.start_frames,
             "noise_seeds": identity.noise_seeds, "plan_fingerprint": identity.plan_fingerprint},
            sp_size=self.ctx.topology.sp_size, group=self.ctx.sp_group)

    def prepare_optimizer_step(self) -> GradientStatus:
        tr = self.trainer
        if self._graphed:
            value = float(tr.last_grad_norm.item())
            self._check_device_waits(value)
            return GradientStatus(finite=value == value and value not in (float("inf"), float("-inf")), norm=value)
        tr.model.finalize_grads()
        if hasattr(tr.optimizer, "sharded_step"):
            norm = tr.optimizer.global_grad_norm(tr.optimizer.reduce_scatter_grads())
        else:
            flat = [g for u in tr.model.units() for g in (u.grad, u.grad_v)]
            if tr.sp is not None and tr.sp.size > 1:
                tr.sp.sum_gradients_(flat)
            if tr.dp_size > 1:
                import torch.distributed as dist

                for g in flat:
                    dist.all_reduce(g, op=dist.ReduceOp.SUM, group=tr.dp_group)
            norm = tr.optimizer.local_grad_sumsq().sqrt()
        tr.optimizer.set_clip(norm, tr.opts.max_grad_norm)
        value = float(norm.item())
        tr.last_grad_norm = norm
        self._check_device_waits(value)
        return GradientStatus(finite=value == value and value not in (float("inf"), float("-inf")), norm=value)

    def _check_device_waits(self, norm_value: float) -> None:
        """The fused transports' device-side waits are bounded: one that gives up sets a status word and lets the
        consumer kernels run on whatever had arrived.  The sharded optimizer folds a non-zero word of ANY rank into
        the gradient norm as infinity, so the common path costs nothing; on a non-finite norm every rank reads its own
        word and all ranks raise the same message together, before the update and before any checkpoint."""
        tr = self.trainer
        fused = getattr(tr.sp, "fused", False) or getattr(tr.optimizer, "transport", "") == "fused"
        if not fused or self.ctx.device.type != "cuda":
            return
        if norm_value == norm_value and norm_value not in (float("inf"), float("-inf")):
            return
        import torch.distributed as dist

        from ... import ops

        rdist.raise_if_device_wait_failed(ops.read_status(self.ctx.device),
                                          dist=dist if self.ctx.topology.raw_world_size > 1 else None)

    def optimizer_step(self) -> None:
        if not self._graphed:
            self.trainer.optimizer.step()

    def scheduler_step(self) -> None:
        self.scheduler.step()

    def ema_update(self, step: int) -> None:
        return None  # the EMA shadow is refreshed inside the fused AdamW kernel

    def set_global_step(self, step: int) -> None:
        self._step = int(step)
        self.trainer.global_step = int(step)

    def save_checkpoint(self, step: int) -> str:
        import torch.distributed as dist

        topo = self.ctx.topology
        state = capture_rank_state(self.ctx.device)
        state = {k: (v if not torch.is_tensor(v) else v.cpu()) for k, v in state.items()}
        state["objective_gen"] = self.trainer.gen.get_state().cpu()
        state["batches_consumed"] = int(self.batches_consumed)
        states = [state]
        if topo.raw_world_size > 1:
            states = [None] * topo.raw_world_size
            dist.all_gather_object(states, state)
        # the optimizer state is gathered into the un-sharded layout on every rank (a collective when the optimizer is
        # sharded); the EMA weights are named out of the same gathered tensors
        opt_state = self.trainer.optimizer.state_dict(keep=topo.is_main)
        ema_state = None
        if self.trainer.optimizer.ema_decay is not None and topo.is_main:
            from ...engine.ema import FlatEMAView

            ema_state = FlatEMAView(self.trainer.model, self.trainer.optimizer, gathered=opt_state).state_dict()
        weights = None
        provider = getattr(self.trainer.model, "param_provider", None)
        if provider is not None and topo.is_main:
            weights = provider.materialize(self.trainer.model)       # sharded blocks are gathered one by one
        if not topo.is_main:
            opt_state = ema_state = None

        def agree(ident):
            return rdist.collective_rank_zero_call(lambda: ident, dist=dist if topo.raw_world_size > 1 else None,
                                                   label="checkpoint commit")

        ident = ckpt.save_checkpoint(output_root(self.config), step, model=self.trainer.model,
                                     optimizer_state=opt_state, weights=weights, scheduler=self.scheduler,
                                     contract=self.contract, config=self.config, ema_state=ema_state,
                                     ema_num_updates=self.trainer.optimizer.step_count, rank_states=states,
                                     is_main=topo.is_main, barrier=agree)
        self.checkpoint_id = ident
        return ident

    def validate(self, step: int) -> Mapping[str, Any]:
        from .inference import run_inline_validation

        return run_inline_validation(self, step)

    def close(self) -> None:
        dist_init.shutdown(self.ctx)


class _TrainingRun:
    def __init__(self, config, **kw):
        self.config, self.kw = config, kw

    def run(self):
        return run_training(self.config, **self.kw)


def build_training_run(config: Mapping[str, Any], *, trainer_cls, options_cls, extra_options=None) -> _TrainingRun:
    """Stage1 / Stage2 reuse the Stage0.5 runtime shell (data, checkpoints, engine hooks) with their own
    trainer and option classes."""
    return _TrainingRun(config, trainer_cls=trainer_cls, options_cls=options_cls, extra_options=extra_options)


def run_training(config: Mapping[str, Any], **runtime_kw) -> Mapping[str, Any]:
    runtime = WanStage0p5Runtime(config, **runtime_kw)
    try:
        train, rt = config["train"], config.get("runtime", {})
        max_steps = int(rt.get("max_steps_override") or train["max_steps"])
        policy = StepPolicy(max_steps=max_steps,
                            grad_accum=int(train.get("grad_accum", train.get("gradient_accumulation_steps", 1))),
                            save_every=int(rt.get("save_every", 0)), validate_every=int(rt.get("validate_every", 0)))
        sink = JsonlEventSink(events_path(output_root(config), runtime.ctx.topology.raw_rank))
        final = TrainingEngine(runtime, policy, event_sink=sink).run()
        return {"final_step": final, "checkpoint_id": runtime.checkpoint_id,
                "native_launches": __import__("solarwm_b200.ops", fromlist=["x"]).total_launches()}
    finally:
        runtime.close()
