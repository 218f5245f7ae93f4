"""LTX backend boundary: Stage0.5 rectified-flow training (full parameters or with SP), 8-step
inference (reference: LTX25Backend, solar/backends/ltx25/backend.py:165-487)."""
from __future__ import annotations

import io
from typing import Any, Mapping

import torch

from ... import ops
from ...config.routes import validate_route
from ...engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from ...engine.optim import FlatAdamW
from ...errors import BackendContractError, ConfigurationError
from ...models.ltx import LTXDiT, ltx_preset
from ...runtime.output_layout import output_root
from .flow import masked_flow_loss, noisy_input_and_target, sample_sigmas


def _arch(config):
    arch = config["model"].get("architecture", "ltx_video_2b")
    return ltx_preset(arch) if isinstance(arch, str) else ltx_preset("tiny")


def load_base_weights(model, spec):
    """``spec``: None, a path, or ``{path, allow_unplaced: [...], allow_missing: [...]}``.  Returns the load report."""
    if not spec:
        return None
    from .loader import load_video_core

    spec = {"path": spec} if isinstance(spec, (str, bytes)) or hasattr(spec, "__fspath__") else dict(spec)
    return load_video_core(model, spec["path"], allow_unplaced=tuple(spec.get("allow_unplaced", ())),
                           allow_missing=tuple(spec.get("allow_missing", ())))


class LTXTrainer:
    """One rectified-flow step: sigma sampling, clean first frame, DiT, masked loss, fused AdamW."""

    def __init__(self, cfg, device, lr=1e-4, seed=0, sp=None, checkpointing="none", lora_rank=0, lora_alpha=None, base_weights=None):
        """``lora_rank > 0``: the base is frozen and low-rank adapters on the q / k / v / out projections of both
        attentions and on both FFN linears train instead (``models/lora.py``), under an fp32-master AdamW.
        ``base_weights``: ``model.base_weights`` of the run configuration (a released-layout checkpoint that replaces
        the seeded base before any adapter is attached)."""
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.model = LTXDiT(cfg, device=device, dtype=dtype, seed=seed)
        with torch.no_grad():                  # seeded by the run, not by the process-wide stream: a resumed run rebuilds the same base
            head = self.model.get_parameter("head.head.weight")
            head.copy_(torch.randn(head.shape, generator=torch.Generator().manual_seed(int(seed) * 7919 + 5)).mul_(0.02).to(head))
        self.base_report = load_base_weights(self.model, base_weights)
        if sp is not None:
            self.model.sp = sp
        self.sp = sp
        self.model.checkpointing = checkpointing
        self.lora = None
        if lora_rank:
            from ...engine.master_adamw import FP32MasterAdamW
            from ...models.lora import inject_lora

            self.lora = inject_lora(self.model, rank=int(lora_rank), alpha=lora_alpha, seed=seed + 1)
            self.lora.broadcast()
            self.opt = FP32MasterAdamW(self.lora.parameters, lr=lr, betas=(0.9, 0.95), weight_decay=0.0)
        else:
            self.model.ensure_grads()
            self.opt = FlatAdamW(self.model.units(), lr=lr)
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device).manual_seed(seed * 100003)

    def train_step(self, latents, text):
        """latents [B, C, F, H, W], text [B, T, text_dim]"""
        lat = latents.to(self.device, non_blocking=True).to(self.model.dtype)
        txt = text.to(self.device, non_blocking=True)
        B, C, F, H, W = lat.shape
        sigma = sample_sigmas(B, F * H * W, generator=self.gen, device=self.device)
        noise = torch.randn(lat.shape, generator=self.gen, device=self.device, dtype=torch.float32).to(lat.dtype)
        if self.sp is not None and self.sp.size > 1:
            self.sp.broadcast_(sigma, noise)
        x_t, target, per_frame = noisy_input_and_target(lat, noise, sigma)
        pred = self.model(x_t, per_frame * 1000.0, txt)
        loss = masked_flow_loss(pred, target)
        (loss / (1 if self.sp is None else self.sp.size)).backward()
        if self.lora is not None:
            flat = self.opt.gather_grads()
            if self.sp is not None and self.sp.size > 1:
                self.sp.sum_gradients_([flat])           # adapters are replicated: one fp32 all-reduce of the flat buffer
            self.opt.clip_(1.0)
            self.opt.step()
            self.opt.zero_grad()
            return loss.detach()
        self.model.finalize_grads()
        if self.sp is not None and self.sp.size > 1:
            self.sp.sum_gradients_([g for u in self.model.units() for g in (u.grad, u.grad_v)])
        norm = self.opt.local_grad_sumsq().sqrt()
        self.opt.set_clip(norm, 1.0)
        self.opt.step()
        self.model.zero_grads()
        return loss.detach()


class GraphedForward:
    """``model(x, t, text)`` as one replayed CUDA graph for a fixed clip geometry: the solver's evaluations all have
    the same shapes, so the network is captured once (after an eager warm-up evaluation on a side stream) and every
    later evaluation is a copy into the static inputs plus a replay -- no per-kernel launch cost on the host, which
    is what bounds a 2 B-parameter network on a few thousand tokens.  Works at SP > 1 when the model's exchanges are
    the fused ones (no library collective inside the forward); the caller keeps one instance per geometry."""

    def __init__(self, model, x, t, text):
        self.model = model
        self.x, self.t, self.text = x.clone(), t.clone(), text.clone()
        side = torch.cuda.Stream(device=x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side), torch.no_grad():
            model(self.x, self.t, self.text)
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"), torch.no_grad():
            self.out = model(self.x, self.t, self.text)

    def matches(self, x, t, text) -> bool:
        return x.shape == self.x.shape and t.shape == self.t.shape and text.shape == self.text.shape

    def __call__(self, x, t, text):
        self.x.copy_(x)
        self.t.copy_(t)
        if text.data_ptr() != self.text.data_ptr():
            self.text.copy_(text)
        self.graph.replay()
        return self.out


@torch.no_grad()
def sample(model, text, *, frames, height, width, steps=8, seed=0, first_frame=None, graph=None):
    """Euler sampler on the linear sigma grid 1 -> 0 (one-stage LTX sampler).  ``graph``: a dict the caller keeps
    between calls; when given (CUDA only) the network evaluation is captured once per geometry and replayed."""
    dev = next(model.parameters()).device
    g = torch.Generator(device=dev).manual_seed(int(seed))
    x = torch.randn(1, model.cfg.out_dim, frames, height, width, generator=g, device=dev).to(model.dtype)
    sig = torch.linspace(1.0, 0.0, steps + 1, device=dev)
    evaluate = model
    for i in range(steps):
        t = sig[i].expand(1, frames).clone()
        if first_frame is not None:
            x[:, :, 0] = first_frame
            t[:, 0] = 0.0
        if graph is not None and dev.type == "cuda" and not torch.is_grad_enabled():
            runner = graph.get("runner")
            if runner is None or not runner.matches(x, t, text):
                runner = graph["runner"] = GraphedForward(model, x, t * 1000.0, text)
            evaluate = runner
        v = evaluate(x, t * 1000.0, text)
        x = (x.float() + (sig[i + 1] - sig[i]) * v.float()).to(x.dtype)
    if first_frame is not None:
        x[:, :, 0] = first_frame
    return x


def guided_x0(cond, uncond, perturbed, *, cfg_scale: float = 1.0, stg_scale: float = 0.0, rescale: float = 0.0):
    """x0 = cond + (cfg - 1)(cond - uncond) + stg (cond - perturbed), optionally pulled back towards the
    conditional prediction's spread: factor = rescale * std(cond) / std(x0) + 1 - rescale
    (reference: _guided_x0, solar/backends/ltx25/torch_inference.py:197-218)."""
    c = cond.float()
    x0 = c + (cfg_scale - 1.0) * (c - uncond.float()) + stg_scale * (c - perturbed.float())
    if rescale != 0.0:
        std = x0.std()
        if not bool(torch.isfinite(std)) or float(std) <= 0:
            raise BackendContractError("LTX guidance prediction has invalid variance")
        x0 = x0 * (rescale * c.std() / std + 1.0 - rescale)
    return x0


@torch.no_grad()
def sample_guided(model, text, negative_text, *, frames, height, width, steps=8, seed=0, first_frame=None,
                  cfg_scale=3.0, stg_scale=1.0, rescale=0.7, stg_blocks=(1,)):
    """The guided one-stage sampler ("stg-euler"): per step a conditional, an unconditional and a perturbed
    evaluation (self-attention skipped in ``stg_blocks``), combined on the x0 side, then an Euler move
    towards the guided x0."""
    dev = next(model.parameters()).device
    g = torch.Generator(device=dev).manual_seed(int(seed))
    x = torch.randn(1, model.cfg.out_dim, frames, height, width, generator=g, device=dev).to(model.dtype)
    sig = torch.linspace(1.0, 0.0, steps + 1, device=dev)
    for i in range(steps):
        t = sig[i].expand(1, frames).clone()
        if first_frame is not None:
            x[:, :, 0] = first_frame
            t[:, 0] = 0.0
        s = float(sig[i])
        x0 = lambda v: x.float() - s * v.float()   # noqa: E731
        cond = x0(model(x, t * 1000.0, text))
        unc = x0(model(x, t * 1000.0, negative_text)) if cfg_scale != 1.0 else cond
        per = x0(model(x, t * 1000.0, text, perturb_blocks=stg_blocks)) if stg_scale != 0.0 else cond
        target = guided_x0(cond, unc, per, cfg_scale=cfg_scale, stg_scale=stg_scale, rescale=rescale)
        v = (x.float() - target) / max(s, 1e-6)
        x = (x.float() + (float(sig[i + 1]) - s) * v).to(x.dtype)
    if first_frame is not None:
        x[:, :, 0] = first_frame
    return x


class RuntimeProvider:
    """What the backend boundary needs from a heavy runtime, resolved lazily so that configuration checks,
    readiness probes and the CLI never import or allocate a model: ``readiness()`` (dependency / device /
    asset report), ``training()``, ``inference()`` and ``preencode()`` bundles
    (reference: LTX25RuntimeProvider, solar/backends/ltx25/runtime.py:119-140)."""

    def __init__(self, config: Mapping[str, Any]):
        self.config = config

    def readiness(self) -> Mapping[str, Any]:
        from ...ops import _lib

        report = {"torch": torch.__version__, "cuda": torch.cuda.is_available(), "native_library": False, "problems": []}
        try:
            _lib.load()
            report["native_library"] = True
        except Exception as exc:  # noqa: BLE001 - reported, not raised
            report["problems"].append(f"native library: {exc}")
        import os

        assets = (self.config.get("model", {}) or {}).get("assets", {}) or {}
        for name, path in assets.items():
            if not os.path.exists(str(path)):
                report["problems"].append(f"asset {name} missing: {path}")
        base = assets.get("base_checkpoint")
        if base and os.path.isfile(str(base)) and str(base).endswith(".safetensors"):
            # header-only: tensor families, counts, dtype policy and layout digest, before any weight byte is read
            from ...errors import BackendContractError
            from .checkpoint import inspect_base_checkpoint

            try:
                report["base_checkpoint"] = inspect_base_checkpoint(base).as_dict()
            except BackendContractError as exc:
                report["problems"].append(f"base checkpoint: {exc}")
        report["ready"] = not report["problems"]
        return report

    def _device(self):
        return "cuda" if torch.cuda.is_available() and self.config.get("runtime", {}).get("device") != "cpu" else "cpu"

    def training(self) -> "LTXTrainer":
        return LTXTrainer(_arch(self.config), self._device(),
                          lr=float(self.config.get("train", {}).get("optimizer", {}).get("lr", 1e-4)),
                          seed=int(self.config.get("data", {}).get("seed", 0)))

    def inference(self) -> LTXDiT:
        dev = self._device()
        return LTXDiT(_arch(self.config), device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)

    def preencode(self) -> Mapping[str, Any]:
        """Run the pre-encoding described by ``config['preencode']`` (128-channel latents, 8 x 32 x 32 geometry)."""
        from ..wan22.preencode import run_preencode

        return run_preencode(self.config, "ltx25_video", latent_channels=128, temporal_ups=(True, True, True, False, False))


class _Adapter:
    family = "ltx25_video"

    def __init__(self, model, config):
        self.model, self.config = model, config

    def generate(self, case: InferenceCase, *, weights_id: str) -> GeneratedSample:
        inf = self.config.get("inference", {}) or {}
        cfg = self.model.cfg
        dev = next(self.model.parameters()).device
        g = torch.Generator().manual_seed(case.noise_seed)
        text = torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).to(dev, self.model.dtype)
        geo = dict(frames=int(inf.get("latent_frames", 4)), height=int(inf.get("latent_height", 8)),
                   width=int(inf.get("latent_width", 8)), steps=int(inf.get("steps", 8)), seed=case.noise_seed)
        gd = inf.get("guidance")
        if gd:
            lat = sample_guided(self.model, text, torch.zeros_like(text), cfg_scale=float(gd.get("cfg_scale", 3.0)),
                                stg_scale=float(gd.get("stg_scale", 1.0)), rescale=float(gd.get("rescale_scale", 0.7)),
                                stg_blocks=tuple(gd.get("stg_blocks", (1,))), **geo)
        else:
            lat = sample(self.model, text, **geo)
        buf = io.BytesIO()
        torch.save(lat.float().cpu(), buf)
        return GeneratedSample({"latents.pt": buf.getvalue()}, tuple(lat.shape), "bfloat16",
                               provenance={"sampler": "stg-euler" if gd else "euler", "steps": int(inf.get("steps", 8))})


class LTX25Backend:
    def __init__(self, family: str):
        if family != "ltx25_video":
            raise BackendContractError(f"not the LTX family: {family!r}")
        self.family = family

    def validate_config(self, config: Mapping[str, Any]) -> None:
        if not config.get("runtime", {}).get("output_dir"):
            raise ConfigurationError("runtime.output_dir is required")
        sp = int((config.get("distributed", {}) or {}).get("sequence_parallel_size", 1))
        if _arch(config).num_heads % sp:
            raise ConfigurationError("sequence_parallel_size must divide the head count")

    def train(self, config):
        validate_route(config)
        if int((config["model"].get("adapter") or {}).get("rank", 0)) > 0:
            # adapter training: any SP x DP layout behind the shared engine, with schedule, average and exact resume
            from .runtime import run_training

            return run_training(config)
        dev = "cuda" if torch.cuda.is_available() and config.get("runtime", {}).get("device") != "cpu" else "cpu"
        cfg = _arch(config)
        adapter = (config["model"].get("adapter") or {})
        tr = LTXTrainer(cfg, dev, lr=float(config["train"].get("optimizer", {}).get("lr", 1e-4)),
                        seed=int(config["data"].get("seed", 0)), lora_rank=int(adapter.get("rank", 0)),
                        lora_alpha=adapter.get("alpha"))
        data = config["data"]
        g = torch.Generator().manual_seed(int(data.get("seed", 0)))
        shape = (1, cfg.in_dim, int(data.get("latent_frames", 4)), int(data.get("latent_height", 8)), int(data.get("latent_width", 8)))
        losses = []
        corpus = None
        if str(data.get("source", "synthetic")) == "index":         # a pre-encoded corpus written by ``preencode``
            from ..wan22.runtime import iter_encoded_samples

            corpus = iter_encoded_samples(data)
        for _ in range(int(config["train"]["max_steps"])):
            if corpus is not None:
                row, enc = next(corpus)
                if enc["latents"].shape[1] != cfg.in_dim or tuple(enc["text"].shape) != (cfg.text_len, cfg.text_dim):
                    raise BackendContractError(f"{row.sample_id}: latents / text do not match the architecture")
                lat, txt = enc["latents"].permute(1, 0, 2, 3).unsqueeze(0).float(), enc["text"].unsqueeze(0).float()
            else:
                lat, txt = torch.randn(shape, generator=g), torch.randn(1, cfg.text_len, cfg.text_dim, generator=g)
            losses.append(float(tr.train_step(lat, txt).item()))
        out = {"final_step": len(losses), "last_loss": losses[-1], "native_launches": ops.total_launches()}
        if tr.lora is not None:
            out["checkpoint"] = str(self._save_adapter(config, tr, len(losses)))
        return out

    @staticmethod
    def _save_adapter(config, tr, step: int):
        """``adapter.pt`` (state under the released key inventory + its metadata record), ``optimizer.pt`` and
        ``runtime.pt`` through the transactional store; the frozen base is never written."""
        from ...checkpoint.store import CheckpointContract, CheckpointTransaction
        from ...runtime.output_layout import checkpoint_model_dir

        route = validate_route(config)
        target = checkpoint_model_dir(output_root(config), step)
        with CheckpointTransaction(target) as tx:
            torch.save({"metadata": tr.lora.metadata(), "state": {k: v.cpu() for k, v in tr.lora.state_dict().items()}},
                       tx.path / "adapter.pt")
            torch.save(tr.opt.state_dict(), tx.path / "optimizer.pt")
            torch.save({"global_step": int(step)}, tx.path / "runtime.pt")
            tx.commit(step=int(step), contract=CheckpointContract(
                family="ltx25_video", stage=route.stage, causal_mode=route.causal_mode, objective=route.objective,
                objective_variant=route.variant, camera_translation_transform=str(config["model"].get("camera_translation_transform", "linear")),
                parameterization="lora", sp_size=1, data_generation=str(config["data"].get("source", "synthetic"))),
                required_components=["adapter.pt", "optimizer.pt", "runtime.pt"], metadata={})
        return target

    def infer(self, config):
        dev = "cuda" if torch.cuda.is_available() and config.get("runtime", {}).get("device") != "cpu" else "cpu"
        trainer_seed = int((config.get("data", {}) or {}).get("seed", 0))
        ck = config.get("checkpoint", {}) or {}
        weights_id = "init:random"
        if ck.get("resume_from"):
            # the base the adapters were trained on is rebuilt from the run's seed; the adapters (live or averaged) are
            # installed under the released key inventory and folded into the base weights for sampling
            from ...models.lora import inject_lora
            from .runtime import adapter_weights

            meta, state, verified = adapter_weights(ck["resume_from"], str(ck.get("weight_source", "ema")))
            model = LTXTrainer(_arch(config), dev, seed=trainer_seed, base_weights=config["model"].get("base_weights")).model
            lora = inject_lora(model, rank=int(meta["rank"]), alpha=float(meta["alpha"]))
            lora.load_state_dict({k: v.to(dev) for k, v in state.items()}, broadcast=False)
            lora.merge_()
            weights_id = verified.manifest_digest
        else:
            model = LTXDiT(_arch(config), device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
            report = load_base_weights(model, config["model"].get("base_weights"))
            if report is not None:
                weights_id = "released:" + report.header_digest
        cases = [InferenceCase(i, f"case-{i}", "synthetic", 0, 1000 + i, "none") for i in range(int(config.get("inference", {}).get("cases", 1)))]
        s = InferenceEngine(_Adapter(model, config)).run(cases, weights_id=weights_id, output_dir=output_root(config) / "generate")
        return {"output_dir": str(s.output_dir), "cases": s.cases, "weights_id": weights_id}

    def preencode(self, config):
        """Raw clips + captions -> 128-channel latent / text shards (8 x 32 x 32 codec geometry; random-init codecs
        unless ``preencode.codecs`` names checkpoints) through the shared commit-last corpus assembly."""
        from ..wan22.preencode import run_preencode

        return run_preencode(config, "ltx25_video", latent_channels=128, temporal_ups=(True, True, True, False, False))
