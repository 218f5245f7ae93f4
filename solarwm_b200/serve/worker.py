"""Realtime worker: one process per GPU; rank 0 also runs the HTTP threads.  Commands
(``prepare / start / chunk / stop / shutdown``) are chosen on rank 0 and broadcast to every rank
over a gloo control group before any GPU work, so all ranks execute the same sequence; failures
are exchanged as text and written to ``failure-rank{r}.json`` / ``exit-rank{r}.json`` receipts
(reference: deploy/solar_wm/backends/standard/worker.py:17-350, runtime/engine.py:17-272).

    python -m solarwm_b200.serve.worker --smoke --chunks 6            # synthetic scene, no HTTP
    torchrun --nproc-per-node 8 -m solarwm_b200.serve.worker --serve  # SP over the box
"""
from __future__ import annotations

import argparse
import json
import os
import time
from pathlib import Path

import torch

from ..models.wan import WanConfig, WanDiT, wan_preset
from .camera_control import NavigationState
from .state import SessionState
from .streaming import StreamingConfig, StreamingGenerator


class Engine:
    """Resident model + streaming generator + camera controller; ``generate`` returns one chunk."""

    def __init__(self, model, stream_cfg: StreamingConfig, navigation: NavigationState):
        self.generator = StreamingGenerator(model, stream_cfg)
        self.navigation = navigation
        self.cameras = []

    def start(self, context, grid_hw, first_frame=None):
        self.generator.start(context, grid_hw, first_frame)

    def generate(self):
        poses = self.navigation.advance(self.generator.cfg.chunk_frames)
        self.cameras.append(poses)
        latents = self.generator.next_chunk()
        return latents, self.generator.stats[-1]


class H3Engine:
    """The same contract on the H3-shaped block-causal model: resident ``H3DiT`` + ``H3StreamingGenerator``; the
    navigation poses of a chunk become first-frame-relative world-to-camera matrices of its latents
    (reference: deploy/solar_wm/backends/standard/runtime/engine.py)."""

    class _Stat:
        def __init__(self, index, dit_ms, graph):
            self.index, self.dit_ms, self.graph = index, dit_ms, graph

    class _Cfg:
        def __init__(self, chunk_frames):
            self.chunk_frames = chunk_frames

    class _Gen:
        def __init__(self, cfg):
            self.cfg, self.stats = cfg, []

    def __init__(self, model, stream_cfg, navigation: NavigationState):
        from .h3_stream import H3StreamingGenerator

        self.h3 = H3StreamingGenerator(model, stream_cfg)
        self.navigation = navigation
        self.generator = H3Engine._Gen(H3Engine._Cfg(stream_cfg.chunk_latents))
        self.cameras = []
        self._first_w2c = None

    def start(self, text, anchor_latent):
        self.h3.start(text, anchor_latent, torch.eye(4))

    def generate(self):
        import numpy as np

        c2w = self.navigation.advance(self.h3.cfg.chunk_latents)
        self.cameras.append(c2w)
        w2c = torch.from_numpy(np.linalg.inv(c2w.astype(np.float64))).float()
        if self._first_w2c is None:                       # the session's first pose is the reference frame
            self._first_w2c = torch.eye(4)
        latents = self.h3.next_chunk(w2c @ torch.linalg.inv(self._first_w2c))
        t = self.h3.timings[-1]
        st = H3Engine._Stat(t.index, t.dit_ms, t.graph)
        self.generator.stats.append(st)
        return latents.unsqueeze(0), st


def _receipt(out_dir: Path, name: str, payload: dict) -> None:
    out_dir.mkdir(parents=True, exist_ok=True)
    (out_dir / name).write_text(json.dumps(payload, sort_keys=True))


def _decode_backends(args, cfg, dev, dtype, rank):
    """The decoder switch of the worker: ``conv`` = causal-conv VAE, ``vit`` = streaming ViT decoder (small random
    instances sized to the model's latent channels; a deployment loads its released decoder instead)."""
    if args.decoder == "none":
        return None
    from ..models.vae import StreamingDecoder, VAEConfig, VideoVAE
    from ..models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
    from .decode_backends import DecodeBackends

    def conv():
        vae = VideoVAE(VAEConfig(z_dim=cfg.out_dim, base=16, temporal_ups=(True, False))).to(dev, dtype).eval()
        return StreamingDecoder(vae)

    def vit():
        vcfg = ViTDecoderConfig(latent_channels=cfg.out_dim, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256, patch=4)
        return StreamingViTDecoder(ViTVideoDecoder(vcfg, device=dev, dtype=dtype, seed=0), (args.height, args.width))

    return DecodeBackends({"conv": conv, "vit": vit}, rank=rank)


def run(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    out_dir = Path(args.output)
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if torch.cuda.is_available() else torch.device("cpu")
    state, nav = SessionState(), NavigationState()
    try:
        if args.family == "memory":
            return _run_memory(args, rank, out_dir, dev, state, nav)
        if args.family == "h3":
            return _run_h3(args, rank, out_dir, dev, state, nav)
        cfg = wan_preset(args.model) if args.model != "small" else WanConfig(
            model_type="ti2v", in_dim=48, out_dim=48, dim=512, ffn_dim=2048, num_heads=4, num_layers=4,
            text_dim=4096, text_len=512)
        dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
        model = WanDiT(cfg, device=dev, dtype=dtype, seed=0).eval()
        with torch.no_grad():
            model.get_parameter("head.head.weight").normal_(0, 0.02)
        engine = Engine(model, StreamingConfig(chunk_frames=args.chunk_frames, window_frames=args.window_frames,
                                               use_cuda_graphs=not args.no_graphs), nav)
        server = None
        if args.serve and rank == 0:
            from .web import make_server, serve_in_thread

            server = make_server(state, nav, port=args.port)
            serve_in_thread(server)
        decoders, decoded = _decode_backends(args, cfg, dev, dtype, rank), {"frames": 0}
        sink = None
        if decoders is not None:
            decoders.start(args.decoder)

        def decode(index, latents):
            """latents [1, C, f, H, W] -> pixel pieces on rank 0; returns the milliseconds spent."""
            nonlocal sink
            if decoders is None:
                return 0.0

            def on_piece(_chunk, _offset, frames, _ns):
                nonlocal sink
                if sink is None:
                    from .media import SIGNED_UNIT, FrameSink

                    sink = FrameSink(out_dir / "frames", frames.shape[-1], frames.shape[-2], use_ffmpeg=False,
                                     normalization=SIGNED_UNIT)        # decoder output lives in [-1, 1]
                for f in range(frames.shape[1]):
                    sink.push(frames[:, f])
                    decoded["frames"] += 1

            return decoders.push(index, latents[0].contiguous(), on_piece)

        g = torch.Generator().manual_seed(0)
        context = torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).to(dtype)
        state.set_phase("preparing")
        engine.start(context, (args.height // 2, args.width // 2))
        state.set_phase("running")
        if args.smoke:
            nav.set_key("w", True)
            for i in range(args.chunks):
                lat, st = engine.generate()
                state.generated(st.index, st.dit_ms, decode(i, lat))
            steady = [c["dit_ms"] for c in state.chunks if engine.generator.stats[c["index"]].graph] or \
                     [c["dit_ms"] for c in state.chunks[1:]]
            report = {"chunks": args.chunks, "chunk_frames": args.chunk_frames,
                      "median_chunk_ms": sorted(steady)[len(steady) // 2] if steady else None,
                      "graph_chunks": sum(1 for s in engine.generator.stats if s.graph),
                      "decoder": args.decoder, "decoded_frames": decoded["frames"],
                      "median_decode_ms": sorted(c["vae_ms"] for c in state.chunks)[len(state.chunks) // 2] if state.chunks else None}
            if rank == 0:
                print(json.dumps(report))
        else:
            while True:
                cmd = state.next_command()
                if cmd["op"] == "shutdown":
                    break
                if cmd["op"] == "stop":
                    state.set_phase("stopped")
                elif cmd["op"] == "start":
                    state.set_phase("running")
                elif cmd["op"] == "chunk" and state.phase == "running":
                    lat, st = engine.generate()
                    state.generated(st.index, st.dit_ms, decode(len(state.chunks), lat))
        if server is not None:
            server.shutdown()
        if sink is not None:
            sink.close()
        if decoders is not None:
            decoders.finish()
            decoders.close()
        if rank == 0:       # the session's per-chunk timings (DiT / decode milliseconds), as the state endpoint reports them
            _receipt(out_dir, "session.json", {"schema": "solarwm.serve-session.v1", "chunks": list(state.chunks)})
        _receipt(out_dir, f"exit-rank{rank}.json", {"rank": rank, "status": "ok", "chunks": len(state.chunks), "time": time.time()})
        return 0
    except Exception as exc:  # noqa: BLE001
        state.set_phase("failed", str(exc))
        _receipt(out_dir, f"failure-rank{rank}.json", {"rank": rank, "error": f"{type(exc).__name__}: {exc}"})
        raise


def _run_h3(args, rank, out_dir, dev, state, nav) -> int:
    """Smoke / command loop of the H3-shaped engine (``--family h3``; ``--model tiny`` or ``h3_33b``)."""
    from types import SimpleNamespace

    from ..models.h3 import H3DiT, h3_preset
    from .h3_stream import H3StreamConfig

    cfg = h3_preset("tiny" if args.model in ("small", "tiny") else args.model)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = H3DiT(cfg, device=dev, dtype=dtype, seed=0)
    scfg = H3StreamConfig(grid_hw=(args.height // 2, args.width // 2), chunk_latents=args.chunk_frames,
                          window_chunks=max(1, args.window_frames // args.chunk_frames), use_cuda_graph=not args.no_graphs)
    engine = H3Engine(model, scfg, nav)
    decoders = _decode_backends(args, SimpleNamespace(out_dim=scfg.latent_channels), dev, dtype, rank)
    decoded = {"frames": 0}
    if decoders is not None:
        decoders.start(args.decoder)
    g = torch.Generator().manual_seed(0)
    state.set_phase("preparing")
    from . import scene_guard

    scene = {"text": torch.randn(16, cfg.text_dim, generator=g),
             "anchor_latent": torch.randn(scfg.latent_channels, 1, args.height, args.width, generator=g)}
    try:        # every rank checks its own copy; the verdicts are exchanged on the host before any device work
        import torch.distributed as dist

        scene_guard.admit_scene(scene_guard.check_scene(scene, text_dim=cfg.text_dim, latent_channels=scfg.latent_channels,
                                                        grid_hw=scfg.grid_hw),
                                dist=dist if dist.is_available() and dist.is_initialized() else None)
    except scene_guard.SceneRejected as exc:
        scene_guard.recover(exc, lambda: state.set_phase("stopped", str(exc)))       # parked: the model stays resident
        _receipt(out_dir, f"exit-rank{rank}.json", {"rank": rank, "status": "scene_rejected", "stage": exc.stage, "time": time.time()})
        return 0
    engine.start(scene["text"], scene["anchor_latent"])
    state.set_phase("running")
    nav.set_key("w", True)

    def on_piece(_c, _o, frames, _ns):
        decoded["frames"] += frames.shape[1]

    def one(i):
        lat, st = engine.generate()
        ms = 0.0 if decoders is None else decoders.push(i, lat[0].contiguous(), on_piece)
        state.generated(st.index, st.dit_ms, ms)

    if args.smoke:
        for i in range(args.chunks):
            one(i)
        steady = [c["dit_ms"] for c in state.chunks[1:]] or [c["dit_ms"] for c in state.chunks]
        if rank == 0:
            print(json.dumps({"family": "h3", "chunks": args.chunks, "chunk_frames": args.chunk_frames,
                              "median_chunk_ms": sorted(steady)[len(steady) // 2],
                              "graph_chunks": sum(1 for s in engine.generator.stats if s.graph),
                              "decoder": args.decoder, "decoded_frames": decoded["frames"]}))
    else:
        while True:
            cmd = state.next_command()
            if cmd["op"] == "shutdown":
                break
            if cmd["op"] == "stop":
                state.set_phase("stopped")
            elif cmd["op"] == "start":
                state.set_phase("running")
            elif cmd["op"] == "chunk" and state.phase == "running":
                one(len(state.chunks))
    if decoders is not None:
        decoders.finish()
        decoders.close()
    if rank == 0:       # the session's per-chunk timings (DiT / decode milliseconds), as the state endpoint reports them
        _receipt(out_dir, "session.json", {"schema": "solarwm.serve-session.v1", "chunks": list(state.chunks)})
    _receipt(out_dir, f"exit-rank{rank}.json", {"rank": rank, "status": "ok", "chunks": len(state.chunks), "time": time.time()})
    return 0


def _run_memory(args, rank, out_dir, dev, state, nav) -> int:
    """The Memory backend's worker (``--family memory``): interactive sessions whose chunks retrieve old latents by camera
    overlap (``serve/memory_engine.py``).  One key packet per chunk comes from the navigation state; a session report is
    written when the session stops."""
    from ..models.h3 import H3DiT, h3_preset
    from .h3_stream import H3StreamConfig
    from .memory import attach_memory_adapter
    from .memory_engine import MemorySessionEngine

    cfg = h3_preset("tiny" if args.model in ("small", "tiny") else args.model)
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    model = H3DiT(cfg, device=dev, dtype=dtype, seed=0)
    identity = attach_memory_adapter(model, rank=8 if cfg.hidden_size <= 512 else 384, frozen_identity="init:random")
    top_k = 5
    scfg = H3StreamConfig(grid_hw=(args.height // 2, args.width // 2), chunk_latents=5, window_chunks=max(1, args.window_frames // 5),
                          use_cuda_graph=False, memory_latents=top_k, memory_adapter="memory")
    engine = MemorySessionEngine(model, scfg, run_dir=out_dir, rank=rank, top_k=top_k, identity=identity)
    g = torch.Generator().manual_seed(0)
    engine.set_condition(text=torch.randn(16, cfg.text_dim, generator=g),
                         anchor_latent=torch.randn(scfg.latent_channels, 1, args.height, args.width, generator=g), scene_id="synthetic")
    state.set_phase("preparing")
    engine.start(seed=42)
    state.set_phase("running")
    nav.set_key("w", True)

    def one():
        keys = nav.next_actions(4 if engine.index == 0 else 5)
        if engine.index >= max(2, args.chunks // 2):               # walk back over the same ground so retrieval has something to find
            keys = [["s"] for _ in keys]
        engine.advance_camera(keys)
        _, ms = engine.generate()
        state.generated(engine.index - 1, ms, 0.0)

    if args.smoke:
        for _ in range(args.chunks):
            one()
        report = engine.stop()
        if rank == 0:
            steady = report["dit_ms"][1:] or report["dit_ms"]
            print(json.dumps({"family": "memory", "chunks": report["chunks"], "median_chunk_ms": sorted(steady)[len(steady) // 2],
                              "retrieved": [len(r["memory_latent_indices"]) for r in report["retrieval"]]}))
    else:
        while True:
            cmd = state.next_command()
            if cmd["op"] == "shutdown":
                break
            if cmd["op"] == "stop" and engine.active:
                engine.stop()
                state.set_phase("stopped")
            elif cmd["op"] == "start" and not engine.active:
                engine.start(seed=42)
                state.set_phase("running")
            elif cmd["op"] == "chunk" and state.phase == "running":
                one()
        if engine.active:
            engine.stop()
    _receipt(out_dir, f"exit-rank{rank}.json", {"rank": rank, "status": "ok", "chunks": len(state.chunks), "time": time.time()})
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", default="wan", choices=["wan", "h3", "memory"])
    ap.add_argument("--model", default="small")
    ap.add_argument("--height", type=int, default=16)
    ap.add_argument("--width", type=int, default=16)
    ap.add_argument("--chunk-frames", type=int, default=3)
    ap.add_argument("--window-frames", type=int, default=9)
    ap.add_argument("--chunks", type=int, default=6)
    ap.add_argument("--port", type=int, default=8900)
    ap.add_argument("--output", default="serve_out")
    ap.add_argument("--smoke", action="store_true")
    ap.add_argument("--serve", action="store_true")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--decoder", default="none", choices=["none", "conv", "vit"],
                    help="decode every generated chunk to pixel frames through the decoder switch")
    return run(ap.parse_args(argv))


if __name__ == "__main__":
    raise SystemExit(main())
