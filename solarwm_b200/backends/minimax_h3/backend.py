"""H3 backend boundary (reference: MiniMaxH3Backend solar/backends/minimax_h3/backend.py:15-44, H3Stage0p5Core
stage0p5.py:37-300).  Stage0.5 and Stage1 adapter training run through ``runtime.H3TrainingRuntime`` (any SP x DP layout for Stage0.5),
Stage2 through ``stage2_runtime.H3SGFRuntime`` (three roles over one base, data parallel); the
frozen bf16 base is never saved, the checkpoint holds ``adapter.pt`` (schema solarwm.minimax-h3-lora.v1),
``optimizer.pt``, ``scheduler.pt``, ``ema.pt``, ``rank-state.pt`` and ``runtime.pt``.  ``H3Stage0p5Trainer`` is the
single-process step the benchmarks and unit tests drive directly."""
from __future__ import annotations

import time
from typing import Any, Mapping

import torch

from ... import ops
from ...config.routes import validate_route
from ...engine.master_adamw import FP32MasterAdamW
from ...errors import BackendContractError, ConfigurationError
from ...models.h3 import H3DiT, h3_preset
from ...runtime.output_layout import output_root
from . import flow
from .layout import build_layout, expand_cameras, patchify_latents


class H3Stage0p5Trainer:
    def __init__(self, cfg, device, lr=1e-4, seed=0):
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.model = H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        self.opt = FP32MasterAdamW(self.model.trainable_parameters(), lr=lr)
        self.device = torch.device(device)
        self.gen = torch.Generator(device=self.device).manual_seed(seed * 100003)

    def train_step(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        dev, dt = self.device, self.model.dtype
        lat = sample["target_latents"].to(dev)                   # [C, F, H, W]
        anchor = sample["anchor_latents"].to(dev)
        prompt = sample["prompt_embeds"].to(dev)
        C, F, H, W = lat.shape
        u = torch.rand(1, generator=self.gen, device=dev)
        t_video = float(1.0 - flow.shifted_sigma(u, flow.VIDEO_SHIFT))
        layout = build_layout(n_text=prompt.shape[0], latent_frames=F, grid_hw=(H // 2, W // 2), t_video=t_video)
        noise = torch.randn(lat.shape, generator=self.gen, device=dev, dtype=torch.float32).to(lat.dtype)
        x_t = flow.interpolate(lat, noise, t_video)
        a_noise = torch.randn(anchor.shape, generator=self.gen, device=dev, dtype=torch.float32).to(lat.dtype)
        anchor_t = flow.interpolate(anchor, a_noise, 0.999)
        cams = sample.get("camera_w2c")
        view = None if cams is None else expand_cameras(layout, cams)
        vid, _ = self.model(video_rows=patchify_latents(x_t).to(dt), text_rows=prompt.to(dt),
                            anchor_rows=patchify_latents(anchor_t).to(dt), timesteps=layout.timesteps,
                            t_index=layout.t_index.to(dev), tags=layout.tags.to(dev),
                            position_ids=layout.position_ids, viewmats=view)
        tgt = patchify_latents(flow.target(lat, noise).to(lat.dtype)).float()
        loss = (vid.float() - tgt).pow(2).mean()
        loss.backward()
        self.opt.gather_grads()
        self.opt.clip_(1.0)
        self.opt.step()
        self.opt.zero_grad()
        return loss.detach()


class MiniMaxH3Backend:
    def __init__(self, family: str):
        if family != "minimax_h3":
            raise BackendContractError(f"not the H3 family: {family!r}")
        self.family = family

    def validate_config(self, config: Mapping[str, Any]) -> None:
        if str(config["model"].get("camera_translation_transform", "")) != "logd4":
            raise ConfigurationError("MiniMax-H3 requires camera_translation_transform: logd4")
        if not config.get("runtime", {}).get("output_dir"):
            raise ConfigurationError("runtime.output_dir is required")
        d = config.get("distributed", {}) or {}
        if int(d.get("context_parallel_size", 1)) != 1:
            raise ConfigurationError("context_parallel_size must be 1 (sequence scaling is Ulysses SP)")

    def _cfg(self, config):
        arch = config["model"].get("architecture", "h3_33b")
        cfg = h3_preset(arch)
        cfg.lora_rank = int((config["model"].get("adapter", {}) or {}).get("rank", 8 if arch == "tiny" else 384))
        return cfg

    @staticmethod
    def _load_released(model, config) -> None:
        """``model.weights_dir`` (safetensors shards in the released layout) is loaded strictly before anything runs;
        ``model.weight_rules`` ([[pattern, target], ...]) replaces the default naming table."""
        directory = config["model"].get("weights_dir")
        if not directory:
            return
        from .loader import DEFAULT_RULES, strict_load_mapped

        rules = config["model"].get("weight_rules")
        strict_load_mapped(model, directory, DEFAULT_RULES if not rules else [tuple(r) for r in rules])

    def _inference_model(self, config, dev):
        """The model an ``infer`` run samples with.  With ``checkpoint.resume_from`` the adapters of that (verified)
        training checkpoint -- ``checkpoint.weight_source``: ``ema`` (default when the checkpoint holds an average) or
        ``live`` -- are installed and folded into the base weights, so sampling runs adapter-free GEMMs; the manifest
        digest becomes the run's weights identity.  Without one the released / seeded base alone is used."""
        inf = config.get("inference", {}) or {}
        ck = config.get("checkpoint", {}) or {}
        cfg = self._cfg(config)
        dtype = torch.bfloat16 if dev == "cuda" else torch.float32
        if not ck.get("resume_from"):
            cfg.lora_rank = 0 if inf.get("merged_weights", True) else cfg.lora_rank
            model = H3DiT(cfg, device=dev, dtype=dtype, seed=int(inf.get("seed", 0)))
            self._load_released(model, config)
            return model, "init:random" if not config["model"].get("weights_dir") else "released"
        from ...checkpoint.store import verify_checkpoint
        from ...runtime.randomness import model_init_seed
        from .runtime import ADAPTER_SCHEMA

        verified = verify_checkpoint(ck["resume_from"])
        doc = torch.load(verified.path / "adapter.pt", map_location="cpu", weights_only=True)
        if doc.get("schema") != ADAPTER_SCHEMA:
            raise BackendContractError(f"{verified.path / 'adapter.pt'} is not an H3 adapter file")
        state, source = doc["state"], str(ck.get("weight_source", "") or "")
        ema = torch.load(verified.path / "ema.pt", map_location="cpu", weights_only=True) if (verified.path / "ema.pt").is_file() else {}
        if source not in ("", "live", "ema"):
            raise BackendContractError("checkpoint.weight_source is live or ema")
        if source == "ema" or (source == "" and ema.get("state") is not None):
            if ema.get("state") is None:
                raise BackendContractError("the checkpoint holds no averaged adapters")
            state, source = ema["state"], "ema"
        cfg.lora_rank = int(doc.get("rank") or cfg.lora_rank)
        # the base the adapters were trained on: the released weights, or the seeded stand-in of the training run
        seed = model_init_seed("minimax_h3", int((config.get("data", {}) or {}).get("seed", 0))) % (2 ** 31)
        model = H3DiT(cfg, device=dev, dtype=dtype, seed=seed)
        self._load_released(model, config)
        own = {n: p for n, p in model.named_parameters() if p.requires_grad}
        if set(own) != set(state):
            raise BackendContractError("the checkpoint's adapters do not fit this architecture")
        from ...models.h3 import LoRALinear

        with torch.no_grad():
            for n, p in own.items():
                p.copy_(state[n].to(p))
            for mod in model.modules():
                if isinstance(mod, LoRALinear):
                    mod.merge_()
                    mod.rank = 0
        model.requires_grad_(False)
        return model, f"{verified.manifest_digest}:{source or 'live'}"

    def train(self, config):
        route = validate_route(config)
        if route.stage == "stage2":
            from .stage2_runtime import run_sgf_training

            return run_sgf_training(config, model_config=self._cfg(config), load_released=self._load_released)
        from .runtime import run_training

        return run_training(config, model_config=self._cfg(config), load_released=self._load_released)

    def infer(self, config):
        """Camera-length generation: chunk-by-chunk streaming over the camera path with the latent memory bank
        optional (``inference.memory``) and the manifest written under ``<output>/generate``.  Conditions come from
        ``inference.conditions`` (a ``.pt`` with ``text``, ``anchor_latent``, ``c2w``, ``intrinsics``) or, with
        ``inference.source: synthetic``, from seeded random tensors of the configured geometry."""
        from ...serve.h3_full_inference import generate_full_length
        from ...serve.h3_stream import H3StreamConfig

        inf = config.get("inference", {}) or {}
        if inf.get("length_policy") == "source":
            return self._infer_source_length(config)
        if inf.get("cases") is not None or inf.get("case_conditions"):
            return self._infer_cases(config)
        dev = "cuda" if torch.cuda.is_available() and config.get("runtime", {}).get("device") != "cpu" else "cpu"
        model, weights_id = self._inference_model(config, dev)
        cfg = model.cfg
        gh, gw = (int(v) for v in inf.get("grid_hw", (4, 6)))
        k, chunks = int(inf.get("chunk_latents", 2)), int(inf.get("chunks", 2))
        use_memory = bool(inf.get("memory", False))
        scfg = H3StreamConfig(grid_hw=(gh, gw), chunk_latents=k, window_chunks=int(inf.get("window_chunks", 2)),
                              denoise_steps=int(inf.get("denoise_steps", 4)), use_cuda_graph=dev == "cuda",
                              memory_latents=int(inf.get("top_k", 2)) if use_memory else 0, seed=int(inf.get("seed", 0)))
        if inf.get("conditions"):
            cond = torch.load(inf["conditions"], map_location="cpu", weights_only=True)
        elif str(inf.get("source", "synthetic")) == "index":
            # prompt and anchor frame of a pre-encoded sample (``inference.sample``: its position in the corpus index),
            # a straight dolly path unless ``inference.cameras`` (.pt with c2w / intrinsics) is given
            from ...data.index import read_index
            from ...preencode.shards import read_encoded_sample
            from pathlib import Path as _P

            index = _P(str(config["data"]["index"]))
            rows = read_index(index)
            row = rows[int(inf.get("sample", 0)) % len(rows)]
            enc = read_encoded_sample(_P(str(config["data"].get("root") or index.parent)), row.values)
            anchor = enc["latents"][:1].permute(1, 0, 2, 3).contiguous()             # [C, 1, H, W]
            if tuple(anchor.shape) != (scfg.latent_channels, 1, 2 * gh, 2 * gw):
                raise BackendContractError(f"{row.sample_id}: anchor latent {tuple(anchor.shape)} does not fit grid_hw {(gh, gw)}")
            n = 1 + k * chunks
            if inf.get("cameras"):
                cams = torch.load(inf["cameras"], map_location="cpu", weights_only=True)
                c2w, K = cams["c2w"][:n], cams["intrinsics"][:n]
            else:
                c2w = torch.eye(4).repeat(n, 1, 1)
                c2w[:, 2, 3] = torch.arange(n) * 0.05
                K = torch.tensor([[0.505, 0.0, 0.5], [0.0, 0.898, 0.5], [0.0, 0.0, 1.0]]).repeat(n, 1, 1)
            cond = {"text": enc["text"], "anchor_latent": anchor, "c2w": c2w, "intrinsics": K}
        elif str(inf.get("source", "synthetic")) == "synthetic":
            g = torch.Generator().manual_seed(int(inf.get("seed", 0)) + 17)
            n = 1 + k * chunks
            c2w = torch.eye(4).repeat(n, 1, 1)
            c2w[:, 2, 3] = torch.arange(n) * 0.05
            K = torch.tensor([[cfg.fx if hasattr(cfg, "fx") else 0.505, 0.0, 0.5], [0.0, 0.898, 0.5], [0.0, 0.0, 1.0]])
            cond = {"text": torch.randn(int(inf.get("prompt_len", 8)), cfg.text_dim, generator=g),
                    "anchor_latent": torch.randn(scfg.latent_channels, 1, 2 * gh, 2 * gw, generator=g),
                    "c2w": c2w, "intrinsics": K.repeat(n, 1, 1)}
        else:
            raise BackendContractError("inference.conditions (a .pt file) is required unless inference.source is synthetic")
        out_dir = output_root(config) / "generate"
        out_dir.mkdir(parents=True, exist_ok=True)
        decoder = sink = None
        if inf.get("decoder"):                      # ``inference.decoder``: a ``ViTDecoderConfig`` mapping (+ ``checkpoint``)
            from ...models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
            from ...serve.media import SIGNED_UNIT, FrameSink

            spec = dict(inf["decoder"])
            ckpt = spec.pop("checkpoint", None)
            vcfg = ViTDecoderConfig(latent_channels=scfg.latent_channels, **spec)
            vit = ViTVideoDecoder(vcfg, device=dev, dtype=model.dtype, seed=0)
            if ckpt:
                vit.load_state_dict(torch.load(ckpt, map_location=dev, weights_only=True))
            decoder = StreamingViTDecoder(vit, (2 * gh, 2 * gw))
            frame_sink = FrameSink(out_dir / "frames", 2 * gw * vcfg.patch, 2 * gh * vcfg.patch, use_ffmpeg=False,
                                   normalization=SIGNED_UNIT)

            def sink(frames):                       # [3, F, H, W] in [-1, 1] -> one RGB8 frame at a time
                for f in range(frames.shape[1]):
                    frame_sink.push(frames[:, f])
        manifest = generate_full_length(model, text=cond["text"], anchor_latent=cond["anchor_latent"], c2w=cond["c2w"],
                                        intrinsics=cond["intrinsics"], stream_cfg=scfg, use_memory=use_memory,
                                        top_k=int(inf.get("top_k", 2)), out_dir=out_dir, decoder=decoder, frame_sink=sink)
        if decoder is not None:
            manifest = dict(manifest, video=frame_sink.close())
        return {"output_dir": str(out_dir), "chunks": manifest.get("chunks"), "frames": manifest.get("frames"),
                "video": manifest.get("video"), "weights_id": weights_id,
                "native_launches": ops.total_launches()}

    def _infer_cases(self, config):
        """``inference.cases: N`` (seeded conditions) or ``inference.case_conditions`` (a ``.pt`` list of condition
        mappings): N published cases through the shared inference engine, sampled the way the route's stage asks
        (``inference.py``: bidirectional Euler for Stage0.5 weights, the few-step rollout for block-causal ones)."""
        from ...engine.inference_engine import InferenceEngine
        from ...serve.h3_stream import H3StreamConfig
        from .inference import H3InferenceAdapter, build_cases

        inf = config["inference"]
        dev = "cuda" if torch.cuda.is_available() and config.get("runtime", {}).get("device") != "cpu" else "cpu"
        model, weights_id = self._inference_model(config, dev)
        cfg = model.cfg
        gh, gw = (int(v) for v in inf.get("grid_hw", (4, 6)))
        k = int(inf.get("chunk_latents", 5))
        frames = int(inf.get("latent_frames", 2 * k))
        if inf.get("case_conditions"):
            conditions = torch.load(str(inf["case_conditions"]), map_location="cpu", weights_only=True)
        else:
            conditions = []
            for i in range(int(inf["cases"])):
                g = torch.Generator().manual_seed(int(inf.get("seed", 0)) * 1009 + i)
                views = torch.eye(4).repeat(frames + 1, 1, 1)
                views[:, 2, 3] = -torch.arange(frames + 1) * 0.05
                conditions.append({"sample_id": f"synthetic-{i:04d}", "prompt_embeds": torch.randn(int(inf.get("prompt_len", 8)), cfg.text_dim, generator=g),
                                   "anchor_latents": torch.randn(cfg.latent_row_dim // 4, 1, 2 * gh, 2 * gw, generator=g), "camera_w2c": views})
        stage = str((config.get("train", {}) or {}).get("stage", "stage0p5"))
        scfg = H3StreamConfig(grid_hw=(gh, gw), latent_channels=cfg.latent_row_dim // 4, chunk_latents=k,
                              window_chunks=int(inf.get("window_chunks", 5)), denoise_steps=int(inf.get("denoise_steps", 4)),
                              use_cuda_graph=dev == "cuda")
        adapter = H3InferenceAdapter(model, conditions, stage=stage, steps=int(inf.get("steps", 8)), stream_cfg=scfg)
        summary = InferenceEngine(adapter).run(build_cases(conditions, noise_seed=int(inf.get("seed", 0))), weights_id=weights_id,
                                               output_dir=output_root(config) / str(inf.get("output_name", "generate")))
        return {"output_dir": str(summary.output_dir), "cases": summary.cases, "ordered_manifest_digest": summary.ordered_manifest_digest,
                "weights_id": weights_id, "native_launches": ops.total_launches()}

    def _infer_source_length(self, config):
        """``inference.length_policy: source``: every row of ``inference.plan`` is prepared once (cameras at the clip's
        latent cadence, prompt and anchor from ``<inference.sources>/<key>.pt`` holding ``text``, ``anchor_latent``,
        ``c2w`` [F, 4, 4], ``intrinsics`` [F, 3, 3]) and generated at the clip's own length; ranks split the plan, finished
        cases are verified and skipped (``serve/h3_source_length.py``)."""
        import os
        from pathlib import Path

        from ...serve.h3_source_length import load_plan, prepare_case, run_plan
        from ...serve.h3_stream import H3StreamConfig

        inf = config["inference"]
        dev = "cuda" if torch.cuda.is_available() and config.get("runtime", {}).get("device") != "cpu" else "cpu"
        model, weights_id = self._inference_model(config, dev)
        cfg = model.cfg
        gh, gw = (int(v) for v in inf.get("grid_hw", (24, 42)))
        use_memory = bool(inf.get("memory", False))
        top_k = int(inf.get("top_k", 5))
        scfg = H3StreamConfig(grid_hw=(gh, gw), chunk_latents=5, window_chunks=int(inf.get("window_chunks", 5)),
                              denoise_steps=int(inf.get("denoise_steps", 4)), use_cuda_graph=dev == "cuda",
                              memory_latents=top_k if use_memory else 0)
        fps_policy = str(inf.get("fps_policy", "source"))
        rows = load_plan(inf["plan"], stream_decode=bool(inf.get("stream_decode", False)), fps_policy=fps_policy)
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        work = Path(str(inf.get("work_dir") or (output_root(config) / "work")))
        sources = Path(str(inf["sources"]))
        prep_identity = {"sources": str(sources), "grid_hw": [gh, gw], "text_dim": cfg.text_dim}
        for row in rows[rank::world]:
            src = torch.load(sources / f"{row['key']}.pt", map_location="cpu", weights_only=True)
            prepare_case(work, row, c2w=src["c2w"], intrinsics=src["intrinsics"], encode_prompt=lambda _t, s=src: s["text"],
                         encode_anchor=lambda s=src: s["anchor_latent"], identity=prep_identity)
        decoder_factory = writer_factory = None
        if inf.get("decoder"):
            from ...models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
            from ...serve.media import SIGNED_UNIT, FrameSink

            spec = dict(inf["decoder"])
            ckpt = spec.pop("checkpoint", None)
            vcfg = ViTDecoderConfig(latent_channels=scfg.latent_channels, **spec)
            vit = ViTVideoDecoder(vcfg, device=dev, dtype=model.dtype, seed=0)
            if ckpt:
                vit.load_state_dict(torch.load(ckpt, map_location=dev, weights_only=True))
            decoder_factory = lambda: StreamingViTDecoder(vit, (2 * gh, 2 * gw))      # noqa: E731

            class _Writer:
                def __init__(self, path, fps):
                    self.path = Path(path)
                    self.sink = FrameSink(self.path.with_suffix(""), 2 * gw * vcfg.patch, 2 * gh * vcfg.patch, fps=fps,
                                          use_ffmpeg=inf.get("use_ffmpeg"), normalization=SIGNED_UNIT)

                def push(self, frames):
                    for f in range(frames.shape[1]):
                        self.sink.push(frames[:, f])

                def close(self):
                    info = self.sink.close()
                    self.path.write_text(json.dumps(dict(info), sort_keys=True, default=str))

            import json

            writer_factory = _Writer
        summary = run_plan(model, rows, work_dir=work, out_dir=output_root(config) / "generate", stream_cfg=scfg,
                           identity={"weights": weights_id,
                                     "denoise_steps": scfg.denoise_steps, "window_chunks": scfg.window_chunks},
                           rank=rank, world=world, noise_seed=int(inf.get("seed", 0)), decoder_factory=decoder_factory,
                           writer_factory=writer_factory, use_memory=use_memory, top_k=top_k, fps_policy=fps_policy,
                           save_latents=bool(inf.get("save_latents", False)))
        return {"output_dir": str(output_root(config) / "generate"), **summary, "native_launches": ops.total_launches()}

    def preencode(self, config):
        """Raw clips + captions -> 24-channel latent / text shards (4 x 16 x 16 codec geometry; random-init codecs
        unless ``preencode.codecs`` names checkpoints) through the shared commit-last corpus assembly."""
        from ..wan22.preencode import run_preencode

        return run_preencode(config, "minimax_h3", latent_channels=24, temporal_ups=(True, True, False, False))
