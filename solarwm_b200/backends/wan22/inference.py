"""Wan generation: bidirectional Euler flow sampling through the inference engine's create-only
publication (reference: CudaWanGenerationAdapter, solar/backends/wan22/runtime/inference.py:970-3040).
Artifacts are the generated latents (``latents.pt``) and the sigma schedule (``schedule.json``); pixel
decoding and MP4 muxing need VAE weights / an ffmpeg binary and are applied when present."""
from __future__ import annotations

import io
import json
from typing import Any, Mapping

import torch

from ... import ops
from ...engine.flow import FlowMatchScheduler
from ...errors import BackendContractError
from ...engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from ...runtime.output_layout import output_root, public_validation_dir
from ...runtime.randomness import stable_validation_seed


@torch.no_grad()
def sample_bidirectional(model, text, *, frames, height, width, steps=8, shift=5.0, seed=0, first_frame=None):
    dev = next(model.parameters()).device
    cfg = model.cfg
    sched = FlowMatchScheduler(shift=shift)
    sched.set_timesteps(steps)
    sig = torch.cat([sched.sigmas, torch.zeros(1)]).to(dev)
    g = torch.Generator(device=dev).manual_seed(int(seed))
    x = torch.randn(1, frames, cfg.out_dim, height, width, generator=g, device=dev).to(model.dtype)
    for i in range(steps):
        s = sig[i].expand(frames).clone()
        s_next = sig[i + 1].expand(frames).clone()
        t = (s * 1000.0).view(1, frames).clone()
        if first_frame is not None:
            x[:, 0] = first_frame
            t[:, 0] = 0.0
        v = model(x.permute(0, 2, 1, 3, 4), t, text).permute(0, 2, 1, 3, 4).contiguous()
        x = ops.euler_step(x.reshape(frames, -1), v.reshape(frames, -1), s.float(), s_next.float()).view_as(x)
    if first_frame is not None:
        x[:, 0] = first_frame
    return x, [float(v) for v in sig.tolist()]


class WanLatentAdapter:
    def __init__(self, family: str, model, config: Mapping[str, Any]):
        self.family, self.model, self.config = family, model, config
        self._text_encoder = None

    def _decode(self, latents):
        """``inference.vae`` (``{z_dim, base, temporal_ups, checkpoint?, fps?, chunk_latent_frames?}``) turns the sampled latents
        [1, F, C, H, W] into an MP4 (streaming chunk decode through the codec adapter, OpenCV's encoder)."""
        spec = (self.config.get("inference", {}) or {}).get("vae")
        if not spec:
            return None
        import os
        import tempfile

        import cv2

        from ...models.vae import VAEConfig, VideoVAE
        from .codec import WanVideoCodec

        if getattr(self, "_codec", None) is None:
            spec = dict(spec)
            ckpt, self._fps = spec.pop("checkpoint", None), float(spec.pop("fps", 16.0))
            self._chunk = int(spec.pop("chunk_latent_frames", 8))
            if "temporal_ups" in spec:
                spec["temporal_ups"] = tuple(bool(u) for u in spec["temporal_ups"])
            vae = VideoVAE(VAEConfig(**spec)).to(latents.device, latents.dtype)
            if ckpt:
                vae.load_state_dict(torch.load(ckpt, map_location=latents.device, weights_only=True))
            self._codec = WanVideoCodec(vae)
        fd, path = tempfile.mkstemp(suffix=".mp4")
        os.close(fd)
        writer = None
        try:
            for piece in self._codec.decode_streaming_chunks(latents, chunk_latent_frames=self._chunk):
                rgb = ((piece[0].permute(0, 2, 3, 1) * 0.5 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).numpy()   # [T, H, W, 3]
                if writer is None:
                    writer = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), self._fps, (rgb.shape[2], rgb.shape[1]))
                    if not writer.isOpened():
                        raise BackendContractError("the video encoder could not be opened")
                for frame in rgb:
                    writer.write(cv2.cvtColor(frame, cv2.COLOR_RGB2BGR))
            if writer is not None:
                writer.release()
            with open(path, "rb") as fh:
                return fh.read()
        finally:
            os.unlink(path)

    def _embed(self, case: InferenceCase, dev):
        """The prompt's embedding: through the configured text encoder (``inference.text_encoder``: a ``T5Config``
        mapping, optionally with ``checkpoint``), else a seeded stand-in of the right shape (synthetic runs)."""
        cfg = self.model.cfg
        spec = (self.config.get("inference", {}) or {}).get("text_encoder")
        if spec:
            if self._text_encoder is None:
                from ...models.t5 import T5Config, WanTextEncoder

                spec = dict(spec)
                ckpt = spec.pop("checkpoint", None)
                enc = WanTextEncoder(T5Config(**spec), device=dev, dtype=torch.float32)
                if ckpt:
                    enc.model.load_state_dict(torch.load(ckpt, map_location=dev, weights_only=True))
                self._text_encoder = enc
            text = self._text_encoder([case.prompt])
            if tuple(text.shape[1:]) != (cfg.text_len, cfg.text_dim):
                raise BackendContractError(f"the text encoder yields {tuple(text.shape[1:])}, the model takes "
                                           f"({cfg.text_len}, {cfg.text_dim})")
            return text.to(dev, self.model.dtype)
        g = torch.Generator().manual_seed(stable_validation_seed("prompt", case.prompt, case.sample_id) % (2 ** 31))
        return torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).to(dev, self.model.dtype)

    def generate(self, case: InferenceCase, *, weights_id: str) -> GeneratedSample:
        inf = self.config.get("inference", {}) or {}
        cfg = self.model.cfg
        dev = next(self.model.parameters()).device
        text = self._embed(case, dev)
        lat, sigmas = sample_bidirectional(
            self.model, text, frames=int(inf.get("latent_frames", 5)), height=int(inf.get("latent_height", 16)),
            width=int(inf.get("latent_width", 16)), steps=int(inf.get("steps", 8)),
            shift=float(self.config["model"].get("timestep_shift", 5.0)), seed=case.noise_seed)
        buf = io.BytesIO()
        torch.save(lat.float().cpu(), buf)
        artifacts = {"latents.pt": buf.getvalue(), "schedule.json": json.dumps({"sigmas": sigmas}).encode()}
        video = self._decode(lat)
        if video is not None:
            artifacts["video.mp4"] = video
        return GeneratedSample(artifacts,
                               tuple(lat.shape), str(lat.dtype).replace("torch.", ""),
                               metrics={"latent_abs_mean": float(lat.float().abs().mean())},
                               provenance={"sampler": "euler-flow", "steps": len(sigmas) - 1})


def _cases(config, count):
    seed = int((config.get("validation", {}) or {}).get("noise_seed", 42))
    prompts = (config.get("inference", {}) or {}).get("prompts")
    if prompts:                                   # one case per given prompt
        if not all(isinstance(p, str) and p.strip() for p in prompts):
            raise BackendContractError("inference.prompts must be non-empty strings")
        return [InferenceCase(slot=i, sample_id=f"case-{i:04d}", prompt=p.strip(), start_frame=0,
                              noise_seed=stable_validation_seed(seed, i) % (2 ** 31), camera_fingerprint="none")
                for i, p in enumerate(prompts)]
    return [InferenceCase(slot=i, sample_id=f"case-{i:04d}", prompt=f"synthetic prompt {i}", start_frame=0,
                          noise_seed=stable_validation_seed(seed, i) % (2 ** 31), camera_fingerprint="none")
            for i in range(count)]


def run_inference(config: Mapping[str, Any], family: str) -> Mapping[str, Any]:
    from ...models.wan import WanDiT
    from ...parallel import dist_init
    from ...runtime.randomness import model_init_seed
    from .checkpoint import load_checkpoint
    from .contracts import architecture

    ctx = dist_init.initialize(1, device=str(config.get("runtime", {}).get("device", "auto")))
    try:
        dtype = torch.bfloat16 if ctx.device.type == "cuda" else torch.float32
        model = WanDiT(architecture(config), device=ctx.device, dtype=dtype,
                       seed=model_init_seed(family, int(config["data"].get("seed", 0))))
        weights_id = "init:random"
        c = config.get("checkpoint", {}) or {}
        if c.get("resume_from"):
            source = c.get("weight_source")
            if source in (None, "release"):          # a released package names its own default role
                from ...checkpoint.release import NAME, resolve_default_weights
                from pathlib import Path as _P

                has_manifest = (_P(c["resume_from"]) / NAME).exists()
                if source == "release" or has_manifest:
                    source = resolve_default_weights(c["resume_from"])
            verified, _ = load_checkpoint(c["resume_from"], model=model, mode="weights_only",
                                          weight_source=str(source or "ema"), map_location=ctx.device)
            weights_id = verified.manifest_digest
        inf = config.get("inference", {}) or {}
        cases = _cases(config, int(inf.get("cases", 1)))
        target = output_root(config) / str(inf.get("output_name", "generate"))
        summary = InferenceEngine(WanLatentAdapter(family, model, config)).run(cases, weights_id=weights_id,
                                                                             output_dir=target)
        return {"output_dir": str(summary.output_dir), "cases": summary.cases,
                "ordered_manifest_digest": summary.ordered_manifest_digest, "weights_id": weights_id}
    finally:
        dist_init.shutdown(ctx)


def run_inline_validation(runtime, step: int) -> Mapping[str, Any]:
    cfg = runtime.config
    val = cfg.get("validation", {}) or {}
    count = int(val.get("sample_count", 1))
    target = public_validation_dir(output_root(cfg), step, str(val.get("pass_name", "live")))
    if not runtime.ctx.topology.is_main:
        return {"skipped": True}
    adapter = WanLatentAdapter(runtime.route.family, runtime.trainer.model, cfg)
    summary = InferenceEngine(adapter).run(_cases(cfg, count), weights_id=runtime.checkpoint_id, output_dir=target)
    return {"output_dir": str(summary.output_dir), "cases": summary.cases}
