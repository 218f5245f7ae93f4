"""Source-length H3 generation: chunked rollout of arbitrary length with bounded memory.

For every chunk: (optionally) retrieve the past latents whose cameras overlap the chunk's query camera
and install them as memory rows, generate the chunk with the streaming generator, commit it to the
latent bank, and push its latents one by one through the streaming video decoder, whose frames go
straight to the frame sink -- neither the latent history nor the decoded video is ever held on the
device beyond the window.  A manifest records per-chunk seconds, generation / decode totals, frames
per second and peak device memory (reference: solar/backends/minimax_h3/full_inference.py:278-645,
stream_decode.py:11-79, memory_inference.py:126).
"""
from __future__ import annotations

import json
import time
from pathlib import Path
from typing import Callable, Mapping, Optional

import torch

from .h3_stream import H3StreamConfig, H3StreamingGenerator
from .memory import LatentMemoryBank, RetrievalCameras


def _w2c(c2w: torch.Tensor) -> torch.Tensor:
    R, t = c2w[..., :3, :3], c2w[..., :3, 3:]
    out = torch.zeros_like(c2w)
    out[..., :3, :3] = R.transpose(-1, -2)
    out[..., :3, 3:] = -R.transpose(-1, -2) @ t
    out[..., 3, 3] = 1.0
    return out


def generate_full_length(model, *, text: torch.Tensor, anchor_latent: torch.Tensor, c2w: torch.Tensor,
                         intrinsics: torch.Tensor, stream_cfg: H3StreamConfig = H3StreamConfig(), sp=None,
                         decoder=None, frame_sink: Optional[Callable[[torch.Tensor], None]] = None,
                         use_memory: bool = False, top_k: int = 5, out_dir=None, decode_latents: Optional[int] = None,
                         max_frames: Optional[int] = None, progress: Optional[Callable[[int, int], None]] = None,
                         keep_latents: bool = False) -> Mapping[str, object]:
    """c2w [1 + n_latents, 4, 4] (anchor first), intrinsics [1 + n_latents, 3, 3] normalised.  ``decoder`` is a
    ``StreamingViTDecoder``-like object with ``push(latent [C, h, w]) -> frames or None``; ``frame_sink`` receives
    every emitted frame block [3, F, H, W].  ``decode_latents`` stops decoding after that many generated latents (a
    rollout is whole chunks, the clip may end inside the last one) and ``max_frames`` caps the frames handed to the
    sink; ``progress(chunk, chunks)`` is called after every chunk; ``keep_latents`` returns the generated latents on
    the host under ``"latents"`` (not written to the manifest file).  Returns the manifest (also written to
    ``out_dir``)."""
    cfg = stream_cfg
    k = cfg.chunk_latents
    n_lat = c2w.shape[0] - 1
    n_chunks = n_lat // k
    if n_chunks < 1:
        raise ValueError("the camera path is shorter than one chunk")
    if use_memory and cfg.memory_latents < top_k:
        raise ValueError("stream_cfg.memory_latents must cover top_k retrieved latents")
    gen = H3StreamingGenerator(model, cfg, sp=sp)
    first_w2c = _w2c(c2w[0].float())
    rel = lambda m: _w2c(m.float()) @ torch.linalg.inv(first_w2c)          # first-frame-relative world-to-camera  # noqa: E731
    gen.start(text, anchor_latent, torch.eye(4))
    bank, cams = LatentMemoryBank(chunk_latents=k), RetrievalCameras()
    dev = gen.device
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    chunk_s, decode_s, frames_out, retrieved, decoded, kept = [], 0.0, 0, [], 0, []
    for ci in range(n_chunks):
        t0 = time.perf_counter()
        sl = slice(1 + ci * k, 1 + (ci + 1) * k)
        for j in range(sl.start, sl.stop):
            cams.append(c2w[j].double().numpy(), intrinsics[j].double().numpy())
        if use_memory:
            idx, _ = cams.select(ci, chunk_latents=k, top_k=top_k)
            retrieved.append([int(i) for i in idx])
            if len(idx):
                mem = bank.gather(idx, anchor_latent.unsqueeze(0))[0]                     # [C, n, H, W]
                gen.set_memory(mem, torch.stack([rel(c2w[1 + int(i)]) for i in idx]))
            else:
                gen.set_memory(None)
        chunk = gen.next_chunk(torch.stack([rel(c2w[j]) for j in range(sl.start, sl.stop)]))
        bank.commit(chunk.unsqueeze(0), ci)
        if dev.type == "cuda":
            torch.cuda.synchronize(dev)
        chunk_s.append(time.perf_counter() - t0)
        if decoder is not None:
            t1 = time.perf_counter()
            for li in range(k):
                if decode_latents is not None and decoded >= decode_latents:
                    break
                frames = decoder.push(chunk[:, li].float() if dev.type == "cpu" else chunk[:, li])
                decoded += 1
                if frames is not None:
                    if max_frames is not None:
                        frames = frames[:, :max(0, max_frames - frames_out)]
                    if frames.shape[1]:
                        frames_out += frames.shape[1]
                        if frame_sink is not None:
                            frame_sink(frames)
            if dev.type == "cuda":
                torch.cuda.synchronize(dev)
            decode_s += time.perf_counter() - t1
        if keep_latents:
            kept.append(chunk.detach().to("cpu"))
        if progress is not None:
            progress(ci + 1, n_chunks)
    total = sum(chunk_s) + decode_s
    manifest = {"schema": "solarwm.h3-full-inference.v1", "chunks": n_chunks, "latents": n_chunks * k,
                "chunk_seconds": [round(s, 4) for s in chunk_s], "generation_seconds": round(sum(chunk_s), 4),
                "decode_seconds": round(decode_s, 4), "frames": frames_out,
                "fps": (frames_out / total) if (frames_out and total > 0) else None,
                "gpu_peak_memory_gib": (torch.cuda.max_memory_allocated(dev) / 2 ** 30) if dev.type == "cuda" else None,
                "memory": {"enabled": use_memory, "top_k": top_k, "retrieved": retrieved}}
    if out_dir is not None:
        Path(out_dir).mkdir(parents=True, exist_ok=True)
        (Path(out_dir) / "manifest.json").write_text(json.dumps(manifest, sort_keys=True, indent=1))
    if keep_latents:
        manifest = dict(manifest, latents_tensor=torch.cat(kept, dim=1))
    return manifest
