"""``solar-renderer``: train / distill / render on the configured (or synthetic) data.

    python -m solarwm_b200.renderer.cli train   --config FILE [--set KEY=VALUE ...] [--resolve]     (corpus-driven)
    python -m solarwm_b200.renderer.cli preencode --input rows.jsonl --out DIR --media-root DIR --codecs pkg.mod:factory
                                                  [--shard I --shards N] | --out DIR --merge
    python -m solarwm_b200.renderer.cli export  --checkpoint DIR --out FILE [--weight-source live|ema]
    python -m solarwm_b200.renderer.cli train   --steps N [--arch tiny] [--patterns shared=1,known_frames=1]     (synthetic)
    python -m solarwm_b200.renderer.cli distill --steps N
    python -m solarwm_b200.renderer.cli render  --out DIR [--steps 8] [--causal --frames F --chunk 5 --window 6]

(reference: solar/renderer/__main__.py, render.py)."""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..data.synthetic import h3_sample
from ..models.h3 import h3_preset
from .core import OmniFlowTrainer, render
from .dmd import RendererDMDTrainer
from .known_degree import ObservationProfile


def _sample(cfg, seed, frames=4, size=8):
    s = h3_sample(latent_frames=frames, height=size, width=size, prompt_len=8, text_dim=cfg.text_dim, seed=seed)
    s["structure_latents"] = torch.randn(s["target_latents"].shape, generator=torch.Generator().manual_seed(seed + 7))
    s["camera_w2c"] = torch.eye(4).repeat(frames + 1, 1, 1)
    s["shape"] = tuple(s["target_latents"].shape)
    return s


def _render_media(args, model) -> int:
    """``render --structure VIDEO --prompt TEXT --codecs pkg.mod:factory``: the structure video (and the optional first
    frame) are fitted onto the canvas and encoded by the factory's codecs (``renderer.preencode.Codecs``: ``video`` takes
    RGB8 frames, ``text`` a prompt), the clip is rendered in one pass or, with ``--causal``, chunk by chunk, and the latents
    are saved with a record of what produced them (reference: solar/renderer/render.py)."""
    import importlib

    import numpy as np

    from .comfy_nodes import snap_frames
    from .preencode import fit, on_grid, read_media, usable_frames

    if not (args.codecs and ":" in args.codecs and args.prompt.strip() and args.out):
        raise SystemExit("render --structure needs --prompt, --out and --codecs package.module:factory")
    module, _, factory = args.codecs.partition(":")
    codecs = getattr(importlib.import_module(module), factory)()
    H, W = (int(v) for v in args.canvas.lower().split("x"))
    frames, fps = read_media(args.structure)
    frames = on_grid(frames, fps) if len(frames) > 1 else np.repeat(frames, 22, axis=0)
    keep = snap_frames(len(frames), args.length)
    structure = codecs.video(fit(frames[:keep], (H, W)))
    C, F, h2, w2 = structure.shape
    if args.first_frame:
        still, _ = read_media(args.first_frame)
        anchor = codecs.video(np.repeat(fit(still[:1], (H, W)), usable_frames(22), axis=0))[:, :1]
    else:
        anchor = torch.zeros(C, 1, h2, w2)
    text, _tags = codecs.text(args.prompt)
    dev, dt = model.proj_in.device, model.dtype
    if args.adapter:
        from .runtime import read_adapter

        state = read_adapter(args.adapter)
        own = {n: p for n, p in model.named_parameters() if "lora_" in n}
        if set(own) != set(state):
            raise SystemExit("the adapter file does not fit this model's adapters")
        with torch.no_grad():
            for n, p in own.items():
                p.copy_(state[n].to(p))
    sample = {"prompt_embeds": text.to(dev, dt), "anchor_latents": anchor.to(dev, dt), "structure_latents": structure.to(dev, dt), "shape": (C, F, h2, w2)}
    if args.causal:
        from .causal import CausalRenderer

        lat = CausalRenderer(model, chunk=args.chunk, window=args.window, steps=max(args.steps, 2)).render(sample, seed=args.seed)
    else:
        lat = render(model, sample, steps=max(args.steps, 2), seed=args.seed)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    torch.save(lat.float().cpu(), out / "latents.pt")
    record = {"structure": str(args.structure), "first_frame": args.first_frame, "prompt": args.prompt, "pixel_frames": int(keep), "latents": list(lat.shape),
              "canvas": [H, W], "mode": "causal" if args.causal else "bidirectional", "steps": max(args.steps, 2), "seed": args.seed,
              "adapter": args.adapter, "finite": bool(torch.isfinite(lat.float()).all())}
    (out / "render.json").write_text(json.dumps(record, indent=1, sort_keys=True))
    print(json.dumps(record, sort_keys=True))
    return 0 if record["finite"] else 5


def _train_from_config(args) -> int:
    import os

    from ..config.loader import load_config
    from ..runtime.provenance import reject_inline_secrets
    from .runtime import run_control_training, validate_config

    resolved = load_config(args.config, args.set, route_validator=validate_config)
    reject_inline_secrets(resolved.values)
    config = resolved.mutable_copy()
    config["runtime"]["output_dir"] = str(Path(config["runtime"]["output_dir"]).expanduser().resolve())
    if args.resolve:
        print(json.dumps(config, indent=2, sort_keys=True))
        return 0
    out = Path(config["runtime"]["output_dir"])
    if int(os.environ.get("RANK", "0")) == 0:
        out.mkdir(parents=True, exist_ok=True)
        (out / "runtime-config.json").write_text(json.dumps(config, indent=2, sort_keys=True) + "\n")
    if config["train"].get("objective", "flow_matching") == "dmd":
        from .dmd_runtime import run_dmd_training

        print(json.dumps(run_dmd_training(config), sort_keys=True, default=str))
        return 0
    print(json.dumps(run_control_training(config), sort_keys=True, default=str))
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="solar-renderer")
    ap.add_argument("command", choices=["train", "distill", "render", "export", "preencode"])
    ap.add_argument("--input", default=None, help="preencode: JSON lines of media rows")
    ap.add_argument("--media-root", default=".")
    ap.add_argument("--codecs", default=None, help="preencode: 'package.module:factory' returning renderer.preencode.Codecs "
                                                   "(the released H3 front end is external to this package)")
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--shards", type=int, default=1)
    ap.add_argument("--merge", action="store_true", help="preencode: only merge the shard indexes into index.jsonl")
    ap.add_argument("--config", default=None, help="a renderer training config (YAML); trains on its omni corpus")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    ap.add_argument("--resolve", action="store_true", help="validate and print the configuration")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--weight-source", default="live")
    ap.add_argument("--arch", default="tiny")
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--lora-rank", type=int, default=4)
    ap.add_argument("--patterns", default="shared=1,known_frames=1,known_region=1,confidence_map=1,ramp=1")
    ap.add_argument("--out", default=None)
    ap.add_argument("--structure", default=None, help="render: a structure video (mp4 / image); needs --prompt and --codecs")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--first-frame", default=None, help="render: an image in the look of the shot")
    ap.add_argument("--canvas", default="768x1344", help="render: HEIGHTxWIDTH of the render")
    ap.add_argument("--length", type=int, default=158, help="render: frames, snapped down to 17 n + 5 and to the structure video")
    ap.add_argument("--adapter", default=None, help="render: an exported adapter file to load into the model")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--causal", action="store_true", help="render: chunk by chunk with a key / value window (clips of any length)")
    ap.add_argument("--frames", type=int, default=4, help="render: latent frames of the synthetic sample")
    ap.add_argument("--chunk", type=int, default=5)
    ap.add_argument("--window", type=int, default=6)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    if args.command == "export":
        from .runtime import export_adapter

        print(json.dumps(export_adapter(args.checkpoint, args.out, weight_source=args.weight_source), sort_keys=True))
        return 0
    if args.command == "train" and args.config:
        return _train_from_config(args)
    if args.command == "preencode":
        import importlib

        from .preencode import merge_indexes, run_shard

        if args.merge:
            print(json.dumps({"samples": merge_indexes(args.out)}))
            return 0
        if not (args.input and args.out and args.codecs and ":" in args.codecs):
            raise SystemExit("preencode needs --input, --out and --codecs package.module:factory")
        module, _, factory = args.codecs.partition(":")
        codecs = getattr(importlib.import_module(module), factory)()
        rows = [json.loads(line) for line in Path(args.input).read_text().splitlines() if line.strip()]
        report = run_shard(rows, out=args.out, media_root=args.media_root, codecs=codecs, shard=args.shard, shards=args.shards)
        print(json.dumps(report, sort_keys=True))
        return 0 if not report["pending"] else 4
    cfg = h3_preset(args.arch)
    cfg.lora_rank = args.lora_rank
    if args.command == "train":
        prof = ObservationProfile(patterns=tuple((k, float(v)) for k, v in (p.split("=") for p in args.patterns.split(","))))
        tr = OmniFlowTrainer(cfg, args.device, prof, lr=1e-3)
        for i in range(args.steps):
            loss = tr.train_step(_sample(cfg, i))
            print(json.dumps({"step": i + 1, "loss": float(loss), "pattern": tr.last_plan.pattern,
                              "generated_fraction": tr.last_plan.generated_fraction}))
    elif args.command == "distill":
        tr = RendererDMDTrainer(cfg, args.device, critic_updates_per_student=2, lr_student=1e-3, lr_critic=1e-3)
        for i in range(args.steps):
            print(json.dumps({"step": i + 1, **tr.train_outer_step(_sample(cfg, i))}))
    else:
        from ..models.h3 import H3DiT

        model = H3DiT(cfg, device=args.device, dtype=torch.bfloat16 if args.device == "cuda" else torch.float32)
        if args.structure:
            return _render_media(args, model)
        if args.causal:
            from .causal import CausalRenderer

            lat = CausalRenderer(model, chunk=args.chunk, window=args.window, steps=max(args.steps, 2)).render(_sample(cfg, 0, frames=args.frames))
        else:
            lat = render(model, _sample(cfg, 0, frames=args.frames), steps=max(args.steps, 2))
        if args.out:
            Path(args.out).mkdir(parents=True, exist_ok=True)
            torch.save(lat.cpu(), Path(args.out) / "latents.pt")
        print(json.dumps({"latents": list(lat.shape), "finite": bool(torch.isfinite(lat.float()).all())}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
