"""H3 generation through the shared inference engine: one published directory of cases, whatever the stage.

  sampler      the route's stage decides: Stage0.5 weights are bidirectional and are sampled by data-ward Euler steps over
               the shifted grid on the whole packed document (``renderer.core.render`` without a structure stream);
               Stage1 / Stage2 weights are block-causal and are rolled out chunk by chunk by the streaming generator with
               the few-step schedule, every chunk carrying its cameras.
  conditions   one mapping per slot: ``prompt_embeds``, ``anchor_latents`` [C, 1, H, W], ``camera_w2c`` [1 + F, 4, 4]
               (first-frame relative), optionally ``camera_K``; from a pre-encoded corpus, a ``.pt`` list, or seeded.
  identity     a case carries the fingerprint of its cameras (view matrices and intrinsics, bytes as stored), so a re-run
               against another trajectory is another case.
  package      ``latents.pt`` plus finite-value metrics; decoded pixels when a streaming decoder is configured:
               ``5 n + 2`` latent frames decode to ``17 n + 5`` pixel frames, anything else is refused.

Reference: H3InferenceAdapter, camera_fingerprint, decoded_pixel_frames, package_generated
(solar/backends/minimax_h3/inference.py:17-231), generate_stage1 (stage1_sampling.py:15-105).
"""
from __future__ import annotations

import hashlib
import io
from typing import Any, Mapping, Optional, Sequence

import torch

from ...engine.inference_engine import GeneratedSample, InferenceCase
from ...errors import BackendContractError


def camera_fingerprint(viewmats: torch.Tensor, intrinsics: Optional[torch.Tensor] = None) -> str:
    h = hashlib.blake2s()
    h.update(viewmats.detach().cpu().contiguous().numpy().tobytes())
    if intrinsics is not None:
        h.update(intrinsics.detach().cpu().contiguous().numpy().tobytes())
    return h.hexdigest()


def decoded_pixel_frames(latent_frames: int) -> int:
    if latent_frames < 2 or (latent_frames - 2) % 5:
        raise BackendContractError(f"H3 latents hold {latent_frames} frames, which is not 5 n + 2")
    return 17 * ((latent_frames - 2) // 5) + 5


def build_cases(conditions: Sequence[Mapping[str, Any]], *, noise_seed: int = 42) -> list:
    from ...runtime.randomness import stable_validation_seed

    cases = []
    for slot, cond in enumerate(conditions):
        sid = str(cond.get("sample_id", f"case-{slot:04d}"))
        cases.append(InferenceCase(slot=slot, sample_id=sid, prompt=str(cond.get("prompt", "")), start_frame=int(cond.get("start_frame", 0)),
                                   noise_seed=stable_validation_seed("h3-infer", sid, str(noise_seed)) % (2 ** 31),
                                   camera_fingerprint=camera_fingerprint(cond["camera_w2c"], cond.get("camera_K"))))
    return cases


class H3InferenceAdapter:
    family = "minimax_h3"

    def __init__(self, model, conditions: Sequence[Mapping[str, Any]], *, stage: str, steps: int = 8, stream_cfg=None, decoder_factory=None):
        if stage not in ("stage0p5", "stage1", "stage2"):
            raise BackendContractError(f"no H3 sampler for stage {stage!r}")
        if stage != "stage0p5" and stream_cfg is None:
            raise BackendContractError("block-causal weights need a stream configuration")
        self.model, self.conditions, self.stage, self.steps = model, list(conditions), stage, int(steps)
        self.stream_cfg, self.decoder_factory = stream_cfg, decoder_factory

    def _bidirectional(self, cond, seed: int) -> torch.Tensor:
        from ...renderer.core import render

        C, _, H, W = cond["anchor_latents"].shape
        frames = cond["camera_w2c"].shape[0] - 1
        sample = {"prompt_embeds": cond["prompt_embeds"], "anchor_latents": cond["anchor_latents"], "camera_w2c": cond["camera_w2c"],
                  "shape": (C, frames, H, W)}
        return render(self.model, sample, steps=self.steps, seed=seed)

    def _rollout(self, cond, seed: int) -> torch.Tensor:
        from ...serve.h3_stream import H3StreamingGenerator

        cfg = self.stream_cfg.__class__(**{**self.stream_cfg.__dict__, "seed": int(seed)})
        k = cfg.chunk_latents
        views = cond["camera_w2c"]
        frames = views.shape[0] - 1
        if frames < k or frames % k:
            raise BackendContractError(f"a rollout of {frames} latents is not whole chunks of {k}")
        gen = H3StreamingGenerator(self.model, cfg)
        gen.start(cond["prompt_embeds"], cond["anchor_latents"], views[0])
        return torch.cat([gen.next_chunk(views[1 + i * k:1 + (i + 1) * k]) for i in range(frames // k)], dim=1)

    def generate(self, case: InferenceCase, *, weights_id: str) -> GeneratedSample:
        cond = self.conditions[case.slot]
        if camera_fingerprint(cond["camera_w2c"], cond.get("camera_K")) != case.camera_fingerprint:
            raise BackendContractError(f"{case.sample_id}: the cameras differ from the case's fingerprint")
        with torch.no_grad():
            lat = self._bidirectional(cond, case.noise_seed) if self.stage == "stage0p5" else self._rollout(cond, case.noise_seed)
        if not bool(torch.isfinite(lat.float()).all()):
            raise BackendContractError(f"{case.sample_id}: generation produced non-finite latents")
        buf = io.BytesIO()
        torch.save(lat.float().cpu(), buf)
        artifacts = {"latents.pt": buf.getvalue()}
        metrics = {"latent_abs_mean": float(lat.float().abs().mean()), "latent_abs_max": float(lat.float().abs().max())}
        provenance = {"sampler": "bidirectional-euler" if self.stage == "stage0p5" else "few-step-rollout", "stage": self.stage,
                      "steps": self.steps if self.stage == "stage0p5" else int(self.stream_cfg.denoise_steps), "weights_id": weights_id}
        if self.decoder_factory is not None:
            dec, frames = self.decoder_factory(), []
            for i in range(lat.shape[1]):
                out = dec.push(lat[:, i])
                if out is not None:
                    frames.append(out.float().cpu())
            video = torch.cat(frames, dim=1) if frames else None
            if video is not None:
                if (lat.shape[1] - 2) % 5 == 0 and lat.shape[1] >= 2 and video.shape[1] != decoded_pixel_frames(lat.shape[1]):
                    raise BackendContractError(f"{case.sample_id}: {video.shape[1]} decoded frames for {lat.shape[1]} latents")
                vb = io.BytesIO()
                torch.save(((video.clamp(-1, 1) * 0.5 + 0.5) * 255).round().to(torch.uint8), vb)
                artifacts["frames.pt"] = vb.getvalue()
                metrics["decoded_frames"] = float(video.shape[1])
        return GeneratedSample(artifacts, tuple(lat.shape), str(lat.dtype).replace("torch.", ""), metrics=metrics, provenance=provenance)
