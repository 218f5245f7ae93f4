"""Wan Stage0.5: bidirectional flow-matching training step.

One call of ``train_step`` does what the reference's ``Wan5BStage0p5Runtime.train_microbatch`` +
``prepare_optimizer_step`` + ``optimizer_step`` do (solar/backends/wan22/runtime/stage0p5.py:148-383):
copy the batch from pinned host memory, sample per-video timesteps, broadcast the sampled
tensors inside the SP group, build ``x_t`` / velocity target with the fused scheduler kernel,
run the DiT forward and backward, sum gradients over the SP group, clip by global norm and
apply the sharded fused AdamW (+EMA) update.

TI2V semantics: frame 0 is a clean image condition (timestep 0, excluded from the loss) unless
the sample's image condition is dropped.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ... import ops
from ...engine.flow import FlowMatchScheduler, first_frame_loss_mask, logit_normal_sigmas
from ...engine.optim import FlatAdamW
from ...models.wan import WanConfig, WanDiT
from ...utils.trace import span


@dataclass
class Stage0p5Options:
    lr: float = 1e-4
    betas: tuple = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    max_grad_norm: Optional[float] = 1.0
    timestep_shift: float = 5.0
    sigma_sampling: str = "logit_normal"      # or "uniform_index" (reference randint over the 1000-grid)
    ti2v_first_frame_clean: bool = True
    image_dropout: float = 0.0
    grad_accum: int = 1
    ema_decay: Optional[float] = None
    checkpointing: str = "none"
    keep_blocks: int = 0
    lean_kept: bool = False          # resident blocks rebuild their norm outputs / FFN hidden in backward
    zero: bool = False                 # shard optimizer state + gradient reduction over all ranks (own FSDP)
    zero_transport: str = "collective"  # or "fused" (NVLink peer reduce / push; needs a symmetric heap)
    shard_params: bool = False         # fused sharded optimizer only: keep 1 / world of every block's parameters and
                                       # gather each block just in time (parallel/shard_params.py)
    cuda_graph: bool = False           # capture the whole step (forward, backward, optimizer) once and replay it; needs
                                       # the fused transports (no library collective inside the step) and grad_accum 1
    graph_warmup_steps: int = 2        # eager steps before the capture (lazy initialisation happens there)
    seed: int = 0


class WanStage0p5Trainer:
    def __init__(self, cfg: WanConfig, device, opts: Stage0p5Options = Stage0p5Options(), sp=None,
                 dtype=torch.bfloat16, model: Optional[WanDiT] = None, dp_group=None, dp_size: int = 1, heap=None):
        self.cfg, self.opts, self.device = cfg, opts, torch.device(device)
        self.sp = sp
        self.sp_size = 1 if sp is None else sp.size
        self.dp_group, self.dp_size = dp_group, int(dp_size)
        self.model = model or WanDiT(cfg, device=device, dtype=dtype, seed=opts.seed)
        if sp is not None:
            self.model.sp = sp
        self.model.checkpointing = opts.checkpointing
        self.model.keep_blocks = opts.keep_blocks
        self.model.lean_kept = bool(opts.lean_kept)
        if opts.shard_params:
            self.model.stem.ensure_grads()       # block gradients live in the shared slots of the parameter shards
        else:
            self.model.ensure_grads()
        okw = dict(lr=opts.lr, betas=opts.betas, eps=opts.eps, weight_decay=opts.weight_decay, ema_decay=opts.ema_decay)
        if opts.zero and self.sp_size * self.dp_size > 1:
            from ...parallel.zero import ZeroAdamW

            # gradients are SUMMED over every rank (SP partial sums and DP replicas alike; the loss carries
            # the 1 / (accum * sp * dp) factor), so the shard group is the whole job
            shards = None
            if opts.shard_params:
                if opts.zero_transport != "fused" or heap is None:
                    raise ValueError("shard_params needs the fused sharded optimizer (zero_transport='fused' and a heap)")
                if opts.grad_accum != 1:
                    raise ValueError("shard_params reduces every block's gradients inside backward: grad_accum must be 1")
                from ...parallel.shard_params import ShardedParameters

                shards = ShardedParameters([b.unit for b in self.model.blocks], heap)
                self.model.param_provider = shards
            self.optimizer = ZeroAdamW(self.model.units(), None, transport=opts.zero_transport, heap=heap,
                                       param_shards=shards, **okw)
        else:
            self.optimizer = FlatAdamW(self.model.units(), **okw)
        if hasattr(self.optimizer, "unit_ready") and opts.grad_accum == 1:
            # the sharded optimizer reduces a block's gradients as soon as the block's backward is done
            self.model.grad_ready_hook = self.optimizer.unit_ready
        self.scheduler = FlowMatchScheduler(shift=opts.timestep_shift)
        self.gen = torch.Generator(device=self.device).manual_seed(opts.seed * 100003)
        self.global_step = 0
        self.last_grad_norm = None

    # ------------------------------------------------------------------------------------
    def sample_timesteps(self, B: int) -> torch.Tensor:
        """One timestep per video on the 1000-step grid (values in [0, 1000])."""
        if self.opts.sigma_sampling == "uniform_index":
            idx = torch.randint(0, self.scheduler.num_train_timesteps, (B,), generator=self.gen, device=self.device)
            return self.scheduler._on("timesteps", self.device)[idx]      # the cached device copy (no host copy in a captured step)
        s = logit_normal_sigmas(B, self.opts.timestep_shift, generator=self.gen, device=self.device)
        return s * self.scheduler.num_train_timesteps

    def microbatch(self, latents: torch.Tensor, text: torch.Tensor, y: Optional[torch.Tensor] = None,
                   t_video: Optional[torch.Tensor] = None):
        """latents [B, F, C, H, W] (frame-major, as stored by the data plane); text [B, T, text_dim];
        ``t_video`` [B]: the per-video timesteps when the caller draws them (two-expert training picks the expert
        from them before the step), default: drawn here."""
        o = self.opts
        B, F = latents.shape[:2]
        t_video = self.sample_timesteps(B) if t_video is None else t_video.to(self.device, torch.float32)
        noise = torch.randn(latents.shape, generator=self.gen, device=self.device, dtype=torch.float32).to(latents.dtype)
        dropped = torch.rand(B, generator=self.gen, device=self.device) < o.image_dropout
        if self.sp is not None and self.sp.size > 1 and not getattr(self.sp, "fused", False):
            # SP peers must consume identical samples.  The collective transport broadcasts them; under the fused
            # transport the peers draw from identically seeded generators (``objective_seed`` depends on the DP rank
            # only) and the engine compares their identity fingerprints on the host, so the step needs no collective.
            d8 = dropped.to(torch.uint8)
            self.sp.broadcast_(t_video, noise, d8)
            dropped = d8.bool()
        t = t_video.view(B, 1).expand(B, F).clone()
        if o.ti2v_first_frame_clean and self.cfg.model_type == "ti2v":
            t[:, 0] = torch.where(dropped, t[:, 0], torch.zeros_like(t[:, 0]))
            mask = first_frame_loss_mask(B, F, dropped).to(self.device)
        else:
            mask = torch.ones((B, F), dtype=torch.bool, device=self.device)
        sigma = (t / self.scheduler.num_train_timesteps).float().reshape(B * F)
        x_t, target = ops.add_noise(latents.reshape(B * F, *latents.shape[2:]),
                                    noise.reshape(B * F, *latents.shape[2:]), sigma)
        x_in = x_t.view(B, F, *latents.shape[2:]).permute(0, 2, 1, 3, 4)
        y_in = None if y is None else y.permute(0, 2, 1, 3, 4)
        with span("forward"):
            pred = self.model(x_in, t, text, y=y_in, y_camera=getattr(self, "y_camera", None))      # [B, C, F, H, W]
            pred = pred.permute(0, 2, 1, 3, 4).reshape(B * F, *pred.shape[1:2], *pred.shape[3:]).contiguous()
            weight = self.scheduler.training_weight(t_video).view(B, 1).expand(B, F).reshape(B * F)
            loss = ops.weighted_masked_mse(pred, target[:, :pred.shape[1]], weight.float(),
                                           mask.reshape(B * F).float())
        with span("backward"):
            (loss / (o.grad_accum * self.sp_size * self.dp_size)).backward()
        return loss.detach()

    def optimizer_step(self) -> torch.Tensor:
        with span("optimizer"):
            return self._optimizer_step()

    def _optimizer_step(self) -> torch.Tensor:
        self.model.finalize_grads()
        opt = self.optimizer
        if hasattr(opt, "sharded_step"):
            norm = opt.sharded_step(self.opts.max_grad_norm)      # reduce-scatter, clip, AdamW, all-gather
        else:
            flat = [g for u in self.model.units() for g in (u.grad, u.grad_v)]
            if self.sp is not None and self.sp.size > 1:
                self.sp.sum_gradients_(flat)
            if self.dp_size > 1:
                import torch.distributed as dist

                for g in flat:
                    dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.dp_group)
            norm = opt.local_grad_sumsq().sqrt()
            opt.set_clip(norm, self.opts.max_grad_norm)
            opt.step()
        self.model.zero_grads()
        self.global_step += 1
        self.last_grad_norm = norm
        return norm

    def train_step(self, batch: dict) -> torch.Tensor:
        """batch: pinned host (or device) tensors ``latents`` [B,F,C,H,W], ``text`` [B,T,text_dim], optional ``y``."""
        if self.opts.cuda_graph and self.device.type == "cuda":
            return self._graphed_step(batch)
        dev = self.device
        lat = batch["latents"].to(dev, non_blocking=True)
        txt = batch["text"].to(dev, non_blocking=True)
        y = batch.get("y")
        y = None if y is None else y.to(dev, non_blocking=True)
        extra = {} if batch.get("t_video") is None else {"t_video": batch["t_video"]}
        loss = self.microbatch(lat, txt, y, **extra)        # (stage trainers that draw their own times take no t_video)
        self.optimizer_step()
        return loss

    # -- whole-step CUDA graph --------------------------------------------------------------------------------------
    def _graph_supported(self) -> Optional[str]:
        opt = self.optimizer
        if self.opts.grad_accum != 1:
            return "gradient accumulation"
        if self.sp_size * self.dp_size == 1:
            return "one rank (the unsharded optimizer passes its step-dependent scalars by value)"
        if self.sp_size * self.dp_size > 1:
            if not getattr(self.sp, "fused", False) or self.dp_size > 1:
                return "a library collective inside the step (needs the fused sequence-parallel transport, dp 1)"
            if not (hasattr(opt, "begin_step_host") and getattr(opt, "transport", "") == "fused"):
                return "a library collective inside the optimizer (needs the fused sharded optimizer)"
        return None

    def _graphed_step(self, batch: dict) -> torch.Tensor:
        """The step as ONE replayed CUDA graph: inputs are copied into fixed device buffers, the graph runs sampling,
        forward, backward, the overlapped reduce-scatter, clipping and the sharded AdamW, and the loss is read from a
        fixed device scalar.  The first ``graph_warmup_steps`` calls run eagerly; the capture happens on the next one.
        Learning rate and bias corrections reach the captured optimizer through pinned host memory."""
        why = self._graph_supported()
        if why is not None:
            raise RuntimeError(f"cuda_graph is not available with {why}")
        st = self.__dict__.setdefault("_graph_state", {"eager": 0, "graph": None})
        keys = [k for k in ("latents", "text", "y", "t_video") if batch.get(k) is not None]
        if st["graph"] is None and st["eager"] < int(self.opts.graph_warmup_steps):
            st["eager"] += 1
            dev = self.device
            loss = self.microbatch(batch["latents"].to(dev, non_blocking=True), batch["text"].to(dev, non_blocking=True),
                                   None if batch.get("y") is None else batch["y"].to(dev, non_blocking=True),
                                   **({} if batch.get("t_video") is None else {"t_video": batch["t_video"]}))
            self.optimizer_step()
            return loss
        opt = self.optimizer
        fused_opt = hasattr(opt, "begin_step_host") and getattr(opt, "transport", "") == "fused" and opt.world > 1
        if st["graph"] is None:
            st["inputs"] = {k: torch.empty(batch[k].shape, dtype=batch[k].dtype, device=self.device) for k in keys}
            for k in keys:
                st["inputs"][k].copy_(batch[k], non_blocking=True)
            torch.cuda.synchronize(self.device)
            if getattr(self.model, "param_provider", None) is not None:
                self.model.param_provider.reset_events()
            graph = torch.cuda.CUDAGraph()
            graph.register_generator_state(self.gen)
            if fused_opt:
                opt.begin_step_host()
                opt._host_prepared = True
            step_before = self.global_step
            counted = dict(ops.COUNTERS)
            # a trainer that never runs at the same time as this one (the other expert of a two-expert model) lends
            # its graph's memory pool: the two captured steps then reuse ONE set of activation buffers
            donor = getattr(self, "graph_pool_donor", None)
            lent = None if donor is None else (donor.__dict__.get("_graph_state") or {}).get("graph")
            with torch.cuda.graph(graph, pool=None if lent is None else lent.pool(), capture_error_mode="thread_local"):
                loss = self.microbatch(st["inputs"]["latents"], st["inputs"]["text"], st["inputs"].get("y"),
                                       **({} if "t_video" not in st["inputs"] else {"t_video": st["inputs"]["t_video"]}))
                norm = self.optimizer_step()
            self.global_step = step_before
            # the launch counters advanced while capturing although nothing ran: take that back, and add the same
            # amounts at every replay instead (a replay launches exactly the captured kernels)
            per_replay = {k: v - counted.get(k, 0) for k, v in ops.COUNTERS.items() if v != counted.get(k, 0)}
            for k, v in per_replay.items():
                ops.COUNTERS[k] -= v
            st.update(graph=graph, loss=loss, norm=norm, keys=keys, per_replay=per_replay)
        else:
            if keys != st["keys"] or any(batch[k].shape != st["inputs"][k].shape for k in keys):
                raise RuntimeError("a captured step replays one batch geometry; this batch differs")
            for k in keys:
                st["inputs"][k].copy_(batch[k], non_blocking=True)
            if fused_opt:
                opt.begin_step_host()
            elif hasattr(opt, "step_count"):
                opt.step_count += 1
        st["graph"].replay()
        for k, v in st["per_replay"].items():
            ops.count(k, v)
        self.global_step += 1
        self.last_grad_norm = st["norm"]
        return st["loss"]
