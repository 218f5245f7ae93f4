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


def _velocity(model, x, timestep: float, text, anchor, y_camera=None):
    """One network evaluation at a uniform noise level; with an anchor, frame 0 is clean (timestep 0, the given
    latent) and its velocity is dropped."""
    frames = x.shape[1]
    t = torch.full((1, frames), float(timestep), device=x.device, dtype=torch.float32)
    if anchor is not None:
        x[:, 0] = anchor
        t[:, 0] = 0.0
    v = model(x.permute(0, 2, 1, 3, 4), t, text, y_camera=y_camera).permute(0, 2, 1, 3, 4).contiguous()
    if anchor is not None:
        v[:, 0] = 0
    return v


@torch.no_grad()
def sample_bidirectional(model, text, *, frames, height, width, steps=50, shift=5.0, seed=0, first_frame=None,
                         solver="unipc", y_camera=None):
    """Denoise ``[1, frames, C, height, width]`` latents from seeded noise.  ``solver`` is ``"unipc"`` (the second-order
    multistep predictor-corrector on the pinned shifted grid, the validation default at 50 steps) or ``"euler"``
    (first-order flow steps through the fused update kernel).  ``y_camera`` conditions every evaluation on a camera path.
    ``first_frame`` anchors latent frame 0 (text+image
    conditioning of the 5B family): it enters every evaluation clean and is restored after every step (reference:
    CudaWanGenerationAdapter._bidirectional, solar/backends/wan22/runtime/inference.py:1647-1712)."""
    dev = next(model.parameters()).device
    cfg = model.cfg
    g = torch.Generator(device=dev).manual_seed(int(seed))
    x = torch.randn(1, frames, cfg.out_dim, height, width, generator=g, device=dev).to(model.dtype)
    anchor = None if first_frame is None else first_frame.to(dev, model.dtype)
    if solver == "unipc":
        from ...engine.unipc import FlowUniPC

        unipc = FlowUniPC(int(steps), float(shift))
        for i in range(int(steps)):
            v = _velocity(model, x, float(unipc.timesteps[i]), text, anchor, y_camera)
            x = unipc.step(v.float(), x.float()).to(model.dtype)
        sigmas = [float(s) for s in unipc.sigmas.tolist()]
    elif solver == "euler":
        sched = FlowMatchScheduler(shift=shift)
        sched.set_timesteps(steps)
        sig = torch.cat([sched.sigmas, torch.zeros(1)]).to(dev)
        for i in range(steps):
            v = _velocity(model, x, float(sig[i]) * 1000.0, text, anchor, y_camera)
            s, s_next = sig[i].expand(frames).clone(), sig[i + 1].expand(frames).clone()
            x = ops.euler_step(x.reshape(frames, -1), v.reshape(frames, -1), s.float(), s_next.float()).view_as(x)
        sigmas = [float(s) for s in sig.tolist()]
    else:
        raise BackendContractError(f"inference.solver must be unipc or euler, not {solver!r}")
    if anchor is not None:
        x[:, 0] = anchor
    return x, sigmas


def partition_cases(cases, dp_rank: int, dp_world: int):
    """The cases of one data-parallel replica: ordinal ``i`` goes to replica ``i % dp_world``, so replicas differ by
    at most one case and sequence-parallel peers of a replica hold the same list (reference:
    _partition_generation_cases, solar/backends/wan22/runtime/inference.py:2259-2272)."""
    if dp_world < 1 or not 0 <= dp_rank < dp_world:
        raise BackendContractError(f"data-parallel identity {dp_rank}/{dp_world} is invalid")
    if len({int(c.slot) for c in cases}) != len(cases):
        raise BackendContractError("generation cases contain duplicate slots")
    return tuple(c for i, c in enumerate(cases) if i % dp_world == dp_rank)


def merge_partitions(parts, target, *, family: str, weights_id: str, expected_cases: int):
    """Join the sealed per-replica publications ``parts`` into ``target`` (create-only): slot folders move over, the
    ordered manifest is rebuilt in slot order and sealed with one COMPLETE record.  Every slot must appear exactly
    once (reference: _merge_generation_partitions, solar/backends/wan22/runtime/inference.py:2298-2370)."""
    import hashlib
    import os
    import uuid
    from pathlib import Path

    from ...engine.inference_engine import COMPLETE_SCHEMA, _create
    from ...config.loader import canonical_json
    from ...runtime.create_only import publish_directory_no_replace

    target = Path(target)
    if target.exists():
        raise BackendContractError(f"inference output already exists: {target}")
    staging = target.with_name(f".{target.name}.{uuid.uuid4().hex}.merge")
    staging.mkdir(parents=True)
    by_slot = {}
    for part in map(Path, parts):
        seal = json.loads((part / "COMPLETE.json").read_text())
        if seal.get("weights_id") != weights_id or seal.get("family") != family:
            raise BackendContractError(f"partition {part} was generated by other weights or another family")
        lines = [ln for ln in (part / "ordered-manifest.jsonl").read_bytes().split(b"\n") if ln.strip()]
        if len(lines) != int(seal["cases"]):
            raise BackendContractError(f"partition {part} lists {len(lines)} cases, its seal says {seal['cases']}")
        for ln in lines:
            m = json.loads(ln)
            slot = int(m["case"]["slot"])
            if slot in by_slot:
                raise BackendContractError(f"slot {slot} was generated by two replicas")
            by_slot[slot] = (part, m)
    if len(by_slot) != int(expected_cases):
        raise BackendContractError(f"merged publication has {len(by_slot)} cases, the plan has {expected_cases}")
    ordered = []
    for slot in sorted(by_slot):
        part, m = by_slot[slot]
        name = f"slot-{slot:06d}"
        os.replace(part / name, staging / name)
        ordered.append(m)
    blob = b"".join(canonical_json(m) for m in ordered)
    digest = hashlib.blake2s(blob).hexdigest()
    _create(staging / "ordered-manifest.jsonl", blob)
    _create(staging / "COMPLETE.json", canonical_json({
        "schema": COMPLETE_SCHEMA, "family": family, "weights_id": weights_id, "cases": len(ordered),
        "ordered_manifest_digest": digest}))
    publish_directory_no_replace(staging, target)
    return digest


class WanLatentAdapter:
    def __init__(self, family: str, model, config: Mapping[str, Any]):
        self.family, self.model, self.config = family, model, config
        self._text_encoder = None

    def _pixels(self, latents):
        """``inference.vae`` (``{z_dim, base, temporal_ups, checkpoint?, released?, fps?, chunk_latent_frames?}``): the sampled latents
        [1, F, C, H, W] decoded chunk by chunk through the codec adapter, as pieces ``[T, 3, H, W]`` in [-1, 1]."""
        spec = (self.config.get("inference", {}) or {}).get("vae")
        if not spec:
            return None
        from ...models.vae import VAEConfig, VideoVAE
        from .codec import WanVideoCodec

        if getattr(self, "_codec", None) is None:
            spec = dict(spec)
            ckpt, self._fps = spec.pop("checkpoint", None), float(spec.pop("fps", 16.0))
            self._chunk = int(spec.pop("chunk_latent_frames", 8))
            released = spec.pop("released", None)       # "wan2.2" / "wan2.1": the published topology + weight file
            if released:
                from .codec import Wan5BVAE, WanA14BVAE

                kind = {"wan2.2": Wan5BVAE, "wan2.1": WanA14BVAE}.get(str(released))
                if kind is None or not ckpt:
                    raise BackendContractError("inference.vae.released is 'wan2.2' or 'wan2.1' and needs a checkpoint")
                self._codec = kind.from_checkpoint(ckpt, device=latents.device, dtype=latents.dtype)
                return (piece[0] for piece in self._codec.decode_streaming_chunks(latents, chunk_latent_frames=self._chunk))
            if "temporal_ups" in spec:
                spec["temporal_ups"] = tuple(bool(u) for u in spec["temporal_ups"])
            vae = VideoVAE(VAEConfig(**spec)).to(latents.device, latents.dtype)
            if ckpt:
                vae.load_state_dict(torch.load(ckpt, map_location=latents.device, weights_only=True))
            self._codec = WanVideoCodec(vae)
        return (piece[0] for piece in self._codec.decode_streaming_chunks(latents, chunk_latent_frames=self._chunk))

    def _encode_mp4(self, pieces) -> bytes:
        """Pieces ``[T, 3, H, W]`` in [-1, 1] -> MP4 bytes (OpenCV's encoder through a temporary file)."""
        import os
        import tempfile

        import cv2

        fd, path = tempfile.mkstemp(suffix=".mp4")
        os.close(fd)
        writer = None
        try:
            for piece in pieces:
                rgb = ((piece.float().permute(0, 2, 3, 1) * 0.5 + 0.5).clamp(0, 1) * 255).round().to(torch.uint8).cpu().numpy()
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

    def _decode(self, latents):
        pieces = self._pixels(latents)
        return None if pieces is None else self._encode_mp4(pieces)

    def _source_latents(self, case: InferenceCase, like):
        """The clip a generated sample is compared with: ``inference.compare_source`` names a ``.pt`` file holding
        ``[F, C, H, W]`` or ``[cases, F, C, H, W]`` latents, or ``"seeded"`` (a seeded stand-in, synthetic runs)."""
        spec = (self.config.get("inference", {}) or {}).get("compare_source")
        if not spec:
            return None
        if spec == "seeded":
            g = torch.Generator().manual_seed(stable_validation_seed("source", case.sample_id) % (2 ** 31))
            return torch.randn(like.shape, generator=g).to(like.device, like.dtype)
        value = torch.load(str(spec), map_location="cpu", weights_only=True)
        if value.dim() == like.dim():
            value = value[case.slot]
        if tuple(value.shape) != tuple(like.shape[1:]):
            raise BackendContractError(f"inference.compare_source holds {tuple(value.shape)}, the sample is {tuple(like.shape[1:])}")
        return value.unsqueeze(0).to(like.device, like.dtype)

    def _compare(self, case: InferenceCase, latents):
        """``compare.mp4``: the generated clip beside its source, both through the same decoder."""
        source = self._source_latents(case, latents)
        if source is None:
            return None
        gen, src = self._pixels(latents), self._pixels(source)
        if gen is None:
            raise BackendContractError("inference.compare_source needs inference.vae (both clips are decoded)")
        from ...engine.comparison import side_by_side

        view = side_by_side(torch.cat(list(gen), 0), torch.cat(list(src), 0))
        return self._encode_mp4([view])

    def _embed(self, case: InferenceCase, dev):
        """The prompt's embedding: through the configured text encoder (``inference.text_encoder``: a ``T5Config``
        mapping, optionally with ``checkpoint``), else a seeded stand-in of the right shape (synthetic runs)."""
        cfg = self.model.cfg
        spec = (self.config.get("inference", {}) or {}).get("text_encoder")
        if spec:
            if self._text_encoder is None:
                from ...models.t5 import T5Config, WanTextEncoder

                spec = dict(spec)
                ckpt, tokenizer = spec.pop("checkpoint", None), spec.pop("tokenizer", None)
                if ckpt and tokenizer:                  # the published encoder file + tokenizer directory
                    enc = WanTextEncoder.from_released(ckpt, tokenizer, cfg=T5Config(**spec), device=dev)
                else:
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

    def _first_frame(self, case: InferenceCase, shape, dev):
        """The anchor latent of text+image generation: ``inference.first_frame`` names a ``.pt`` file holding
        ``[C, H, W]`` (one for every case) or ``[cases, C, H, W]`` (indexed by slot); ``"seeded"`` draws one from the
        case's seed (synthetic runs).  Absent: no anchor."""
        spec = (self.config.get("inference", {}) or {}).get("first_frame")
        if not spec:
            return None
        if spec == "seeded":
            g = torch.Generator().manual_seed(stable_validation_seed("first-frame", case.sample_id) % (2 ** 31))
            return torch.randn(*shape, generator=g).to(dev, self.model.dtype)
        value = torch.load(str(spec), map_location="cpu", weights_only=True)
        if value.dim() == len(shape) + 1:
            value = value[case.slot]
        if tuple(value.shape) != tuple(shape):
            raise BackendContractError(f"inference.first_frame holds {tuple(value.shape)}, the model takes {tuple(shape)}")
        return value.to(dev, self.model.dtype)

    @property
    def autoregressive(self) -> bool:
        """Causal checkpoints (teacher forcing, self-gradient forcing) are sampled chunk by chunk with the rolling KV
        cache and the few-step schedule they were trained for; ``inference.mode`` overrides the route's choice."""
        mode = (self.config.get("inference", {}) or {}).get("mode")
        if mode is not None:
            if mode not in ("bidirectional", "autoregressive"):
                raise BackendContractError("inference.mode is bidirectional or autoregressive")
            return mode == "autoregressive"
        return str((self.config.get("train", {}) or {}).get("causal_mode", "bidirectional")) in ("teacher_forcing", "self_gradient_forcing")

    def _rollout(self, case: InferenceCase, text, frames: int, h: int, w: int, first, dev):
        """Chunked rollout of ``frames`` latent frames.  With ``inference.cameras`` (a ``.pt`` holding ``viewmats``
        ``[cases?, F, 4, 4]`` first-frame-relative world-to-camera and optional ``Ks``) every chunk carries its cameras and
        the clip is as long as the camera path; otherwise the generator runs ``frames / chunk_frames`` chunks."""
        from ...serve.streaming import StreamingConfig, StreamingGenerator, camera_rollout

        inf, model_cfg = self.config.get("inference", {}) or {}, self.config["model"]
        causal = model_cfg.get("causal", {}) or {}
        k = int(causal.get("chunk_frames", 3))
        window = int(causal.get("window_chunks", 6)) * k
        steps = tuple(float(t) for t in inf.get("denoising_steps", (self.config.get("train", {}) or {}).get("denoising_steps", (1000.0, 750.0, 500.0, 250.0))))
        scfg = StreamingConfig(chunk_frames=k, denoise_timesteps=steps, timestep_shift=float(model_cfg.get("timestep_shift", 5.0)),
                               window_frames=window, sink_frames=int(causal.get("sink_frames", 0)),
                               use_cuda_graphs=bool(inf.get("cuda_graphs", dev.type == "cuda")), seed=int(case.noise_seed))
        ph, pw = self.model.cfg.patch_size[1], self.model.cfg.patch_size[2]
        grid = (h // ph, w // pw)
        anchor = None if first is None else first.unsqueeze(0).unsqueeze(2)           # [1, C, 1, H, W]
        cams = inf.get("cameras")
        if cams:
            doc = torch.load(str(cams), map_location="cpu", weights_only=True)
            views = doc["viewmats"]
            views = views[case.slot] if views.dim() == 4 else views
            Ks = doc.get("Ks")
            Ks = None if Ks is None else (Ks[case.slot] if Ks.dim() == 4 else Ks)
            if views.shape[0] < 1 or tuple(views.shape[1:]) != (4, 4):
                raise BackendContractError("inference.cameras holds viewmats [F, 4, 4] (or one set per case)")
            lat = camera_rollout(self.model, text, grid, views.unsqueeze(0).to(dev), None if Ks is None else Ks.unsqueeze(0).to(dev),
                                 cfg=scfg, first_frame=anchor, transform=str(model_cfg.get("camera_translation_transform", "linear")),
                                 sp=getattr(self.model, "sp", None))
            extra = {"mode": "autoregressive", "camera_frames": int(views.shape[0]), "chunk_frames": k}
        else:
            body = frames - (0 if anchor is None else 1)
            if body < 1 or body % k:
                raise BackendContractError(f"inference.latent_frames leaves {body} frames to generate; chunks hold {k}")
            gen = StreamingGenerator(self.model, scfg, sp=getattr(self.model, "sp", None))
            gen.start(text, grid, first_frame=anchor)
            parts = ([] if anchor is None else [anchor.to(dev, self.model.dtype)]) + [gen.next_chunk() for _ in range(body // k)]
            lat = torch.cat(parts, dim=2)
            extra = {"mode": "autoregressive", "chunks": body // k, "chunk_frames": k,
                     "graph_chunks": sum(1 for st in gen.stats if st.graph)}
        sigmas = [float(t) / 1000.0 for t in steps] + [0.0]
        return lat.permute(0, 2, 1, 3, 4).contiguous(), sigmas, extra        # [1, F, C, H, W] like the bidirectional sampler

    def generate(self, case: InferenceCase, *, weights_id: str) -> GeneratedSample:
        inf = self.config.get("inference", {}) or {}
        cfg = self.model.cfg
        dev = next(self.model.parameters()).device
        text = self._embed(case, dev)
        solver = str(inf.get("solver", "unipc"))
        frames, h, w = int(inf.get("latent_frames", 5)), int(inf.get("latent_height", 16)), int(inf.get("latent_width", 16))
        first = self._first_frame(case, (cfg.out_dim, h, w), dev)
        if self.autoregressive:
            lat, sigmas, extra = self._rollout(case, text, frames, h, w, first, dev)
            solver = "few-step-rollout"
        else:
            y_camera, extra = None, {}
            if inf.get("cameras"):
                doc = torch.load(str(inf["cameras"]), map_location="cpu", weights_only=True)
                views = doc["viewmats"]
                views = views[case.slot] if views.dim() == 4 else views
                if tuple(views.shape) != (frames, 4, 4):
                    raise BackendContractError(f"inference.cameras holds {tuple(views.shape)} for {frames} latent frames")
                Ks = doc.get("Ks")
                Ks = None if Ks is None else (Ks[case.slot] if Ks.dim() == 4 else Ks)
                y_camera = {"viewmats": views.unsqueeze(0).to(dev), "Ks": None if Ks is None else Ks.unsqueeze(0).to(dev),
                            "transform": str(self.config["model"].get("camera_translation_transform", "linear"))}
                extra = {"camera_frames": int(frames)}
            lat, sigmas = sample_bidirectional(
                self.model, text, frames=frames, height=h, width=w, steps=int(inf.get("steps", 50)),
                shift=float(self.config["model"].get("timestep_shift", 5.0)), seed=case.noise_seed, solver=solver,
                first_frame=first, y_camera=y_camera)
        buf = io.BytesIO()
        torch.save(lat.float().cpu(), buf)
        artifacts = {"latents.pt": buf.getvalue(), "schedule.json": json.dumps({"sigmas": sigmas}).encode()}
        video = self._decode(lat)
        if video is not None:
            artifacts["video.mp4"] = video
        compare = self._compare(case, lat)
        if compare is not None:
            artifacts["compare.mp4"] = compare
        return GeneratedSample(artifacts,
                               tuple(lat.shape), str(lat.dtype).replace("torch.", ""),
                               metrics={"latent_abs_mean": float(lat.float().abs().mean())},
                               provenance={"sampler": {"unipc": "unipc-flow", "euler": "euler-flow"}.get(solver, solver),
                                           "steps": len(sigmas) - 1, "anchored_first_frame": bool(inf.get("first_frame")), **extra})


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


def _fail_together(error, label):
    """Every rank learns whether any rank failed the phase ``label`` (an object all-gather of the error texts)."""
    import torch.distributed as dist

    texts = [None] * dist.get_world_size()
    dist.all_gather_object(texts, error)
    failed = [(r, t) for r, t in enumerate(texts) if t is not None]
    if failed and error is None:
        raise BackendContractError(f"inference {label} failed on rank {failed[0][0]}: {failed[0][1]}")


def _run_partitioned(adapter, cases, target, weights_id, topo):
    """Data-parallel generation: every replica generates its share of the cases into a private partition next to the
    target, all ranks walk the same number of case waves (a replica short of a case idles through the last one) and
    report failures to each other after each, then the main rank joins the partitions into the public directory."""
    import shutil
    import torch.distributed as dist

    mine = partition_cases(cases, topo.dp_rank, topo.dp_size)
    waves = (len(cases) + topo.dp_size - 1) // topo.dp_size
    parts_root = target.with_name(f".{target.name}.parts")
    part = parts_root / f"replica-{topo.dp_rank:04d}"
    writer = topo.sp_rank == 0                              # sequence-parallel peers compute, one of them writes
    engine = InferenceEngine(adapter)
    if writer:
        engine.run(mine, weights_id=weights_id, output_dir=part, collective_error=_fail_together,
                   collective_case_waves=waves)
    else:
        _PeerOnly(adapter).run(mine, weights_id, waves)
    dist.barrier()
    digest = None
    if topo.is_main:
        digest = merge_partitions([parts_root / f"replica-{d:04d}" for d in range(topo.dp_size)], target,
                                  family=adapter.family, weights_id=weights_id, expected_cases=len(cases))
        shutil.rmtree(parts_root, ignore_errors=True)
    box = [digest]
    dist.broadcast_object_list(box, src=0)
    return box[0], len(cases)


class _PeerOnly:
    """A sequence-parallel peer of a writing rank: it takes part in every network evaluation and every failure
    exchange of the writer's phases, and publishes nothing."""

    def __init__(self, adapter):
        self.adapter = adapter

    def run(self, cases, weights_id, waves):
        _fail_together(None, "output setup")
        for wave in range(waves):
            error = None
            if wave < len(cases):
                try:
                    self.adapter.generate(cases[wave], weights_id=weights_id)
                except Exception as exc:  # noqa: BLE001 - only the text crosses ranks
                    error = f"{type(exc).__name__}: {exc}"
            _fail_together(error, f"case wave {wave}")
            if error is not None:
                raise BackendContractError(f"inference case wave {wave} failed: {error}")
        _fail_together(None, "partition commit")


def run_inference(config: Mapping[str, Any], family: str) -> Mapping[str, Any]:
    from ...models.wan import WanDiT
    from ...parallel import dist_init
    from ...runtime.randomness import model_init_seed
    from .checkpoint import load_checkpoint
    from .contracts import architecture

    sp_size = int((config.get("inference", {}) or {}).get("sequence_parallel_size", 1))
    ctx = dist_init.initialize(sp_size, device=str(config.get("runtime", {}).get("device", "auto")))
    try:
        dtype = torch.bfloat16 if ctx.device.type == "cuda" else torch.float32
        model = WanDiT(architecture(config), device=ctx.device, dtype=dtype,
                       seed=model_init_seed(family, int(config["data"].get("seed", 0))))
        if bool(config["model"].get("nonzero_head_init", False)):      # synthetic runs: a head that predicts something
            g = torch.Generator().manual_seed(model_init_seed(family, int(config["data"].get("seed", 0))) + 1)
            w = model.get_parameter("head.head.weight")
            with torch.no_grad():
                w.copy_(torch.randn(w.shape, generator=g).mul_(0.02))
        if ctx.sp is not None:
            model.sp = ctx.sp
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
        adapter = WanLatentAdapter(family, model, config)
        topo = ctx.topology
        if topo.raw_world_size == 1:
            summary = InferenceEngine(adapter).run(cases, weights_id=weights_id, output_dir=target)
            digest, count = summary.ordered_manifest_digest, summary.cases
        else:
            digest, count = _run_partitioned(adapter, cases, target, weights_id, topo)
        return {"output_dir": str(target), "cases": count, "ordered_manifest_digest": digest, "weights_id": weights_id}
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
    report = {"output_dir": str(summary.output_dir), "cases": summary.cases}
    if (cfg.get("inference", {}) or {}).get("compare_source"):
        # the browsable comparison view of this pass, next to the publication it links into
        from ...engine.comparison import publish_comparison_view, seal_comparison_view

        name = str(val.get("pass_name", "live"))
        view = target.with_name(f"{target.name}_compare")
        publish_comparison_view(target, view, step=step, pass_name=name, cases=summary.cases, dp_world_size=1,
                                sp_size=runtime.ctx.topology.sp_size, run_root=output_root(cfg))
        seal_comparison_view(view, step=step, pass_name=name, cases=summary.cases)
        report["comparison_view"] = str(view)
    return report
