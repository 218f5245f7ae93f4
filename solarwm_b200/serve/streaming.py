"""Block-causal streaming generation: chunks of latent frames, a few denoising evaluations per chunk
against the rolling KV cache, one clean "commit" forward that appends the chunk to the cache.

Per chunk (reference: _stage2_self_forcing_latents, solar/backends/wan22/runtime/stage2.py:627-771;
engine.generate, deploy/solar_wm/backends/standard/runtime/engine.py:153-199):

    x <- noise
    for t_k in denoising timesteps (default 1000, 750, 500, 250):
        v  = DiT(x, t_k | cache)                      cache untouched
        x0 = x - sigma_k v
        x  = (1 - sigma_{k+1}) x0 + sigma_{k+1} eps   fresh noise, except after the last step
    DiT(x0, t = 0 | cache, commit)                   K/V of the clean chunk enter the cache

Once the window is full every chunk has the same shapes, so the denoise evaluation and the commit
forward are captured into two CUDA graphs and replayed (graph inputs live in pointer-stable
buffers); the first chunks run eagerly.  Per-chunk latency is measured with CUDA events.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..engine.flow import apply_timestep_shift
from ..models.wan_causal import CausalWanRunner, KVCache, allocate_kv_cache


@dataclass
class ChunkStats:
    index: int
    dit_ms: float
    graph: bool


@dataclass
class StreamingConfig:
    chunk_frames: int = 3
    denoise_timesteps: Sequence[float] = (1000.0, 750.0, 500.0, 250.0)
    timestep_shift: float = 5.0
    window_frames: Optional[int] = None
    sink_frames: Optional[int] = None
    use_cuda_graphs: bool = True
    seed: int = 0


class StreamingGenerator:
    def __init__(self, model, cfg: StreamingConfig = StreamingConfig(), sp=None):
        self.model, self.cfg = model, cfg
        self.runner = CausalWanRunner(model, sp=sp)
        self.device = next(model.parameters()).device
        self.cache: Optional[KVCache] = None
        self.stats: List[ChunkStats] = []
        self._graphs = None
        steps = torch.tensor(list(cfg.denoise_timesteps), dtype=torch.float32) / 1000.0
        self.sigmas = apply_timestep_shift(steps, cfg.timestep_shift).tolist() + [0.0]
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed)

    # -------------------------------------------------------------------------------------
    def start(self, context: torch.Tensor, grid_hw, first_frame: Optional[torch.Tensor] = None) -> None:
        """context [1, T, text_dim]; optional clean first latent frame [1, C, 1, H, W] (image condition)."""
        c = self.cfg
        self.cache = allocate_kv_cache(self.model, grid_hw=grid_hw, chunk_frames=c.chunk_frames,
                                       window_frames=c.window_frames, sink_frames=c.sink_frames)
        self.runner.encode_text(self.cache, context.to(self.device))
        self.stats, self._graphs, self.index = [], None, 0
        self.latent_hw = (grid_hw[0] * self.model.cfg.patch_size[1], grid_hw[1] * self.model.cfg.patch_size[2])
        if first_frame is not None:
            t0 = torch.zeros(1, 1, device=self.device)
            self.runner.forward_chunk(self.cache, first_frame.to(self.device), t0, commit=True)

    def _noise(self, f):
        C = self.model.cfg.out_dim
        H, W = self.latent_hw
        return torch.randn(1, C, f, H, W, generator=self.gen, device=self.device, dtype=torch.float32).to(self.model.dtype)

    def _denoise_eager(self, x, sigma):
        f = x.shape[2]
        t = torch.full((1, f), sigma * 1000.0, device=self.device)
        return self.runner.forward_chunk(self.cache, x, t, commit=False)

    def _chunk_eager(self, f):
        x = self._noise(f)
        x0 = x
        for k in range(len(self.sigmas) - 1):
            s, s_next = self.sigmas[k], self.sigmas[k + 1]
            v = self._denoise_eager(x, s)
            x0 = (x.float() - s * v.float()).to(x.dtype)
            if s_next > 0:
                x = ((1 - s_next) * x0.float() + s_next * self._noise(f).float()).to(x.dtype)
        self.runner.forward_chunk(self.cache, x0, torch.zeros(1, f, device=self.device), commit=True)
        return x0

    # -- CUDA graphs (steady state: window full, static shapes) -------------------------------
    def _capture(self, f):
        C = self.model.cfg.out_dim
        H, W = self.latent_hw
        g = {"x": torch.zeros(1, C, f, H, W, device=self.device, dtype=self.model.dtype),
             "t": torch.zeros(1, f, device=self.device)}
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):        # warm-up on a side stream, as graph capture requires
            self.runner.forward_chunk(self.cache, g["x"], g["t"], commit=False)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g["denoise"] = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g["denoise"]):
            g["v"] = self.runner.forward_chunk(self.cache, g["x"], g["t"], commit=False)
        frames_before = (self.cache.committed_frames, self.cache.total_frames, self.cache.newest_pos)
        g["commit"] = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g["commit"]):
            self.runner.forward_chunk(self.cache, g["x"], g["t"], commit=True)
        # capture ran the host-side bookkeeping once without running the kernels: undo it
        self.cache.committed_frames, self.cache.total_frames, self.cache.newest_pos = frames_before
        return g

    def _chunk_graph(self, f):
        g = self._graphs
        x = self._noise(f)
        x0 = x
        for k in range(len(self.sigmas) - 1):
            s, s_next = self.sigmas[k], self.sigmas[k + 1]
            g["x"].copy_(x)
            g["t"].fill_(s * 1000.0)
            g["denoise"].replay()
            x0 = (x.float() - s * g["v"].float()).to(x.dtype)
            if s_next > 0:
                x = ((1 - s_next) * x0.float() + s_next * self._noise(f).float()).to(x.dtype)
        g["x"].copy_(x0)
        g["t"].zero_()
        g["commit"].replay()
        self.cache.total_frames += f           # the committed length stays at the window limit
        return x0

    def next_chunk(self) -> torch.Tensor:
        """Generate the next chunk of clean latents [1, C, f, H, W]."""
        c, cache = self.cfg, self.cache
        f = c.chunk_frames
        # graphs are captured once the window is full AND the position rule has reached its cap: only then does
        # every chunk run the same program (same shapes, same re-basing rotation at commit)
        full = cache.committed_frames == cache.sink_frames + cache.window_frames and cache.positions_saturated
        use_graph = c.use_cuda_graphs and self.device.type == "cuda" and full
        if use_graph and self._graphs is None:
            self._graphs = self._capture(f)
        if self.device.type == "cuda":
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
        import time

        t0 = time.perf_counter()
        out = self._chunk_graph(f) if use_graph else self._chunk_eager(f)
        if self.device.type == "cuda":
            b.record()
            b.synchronize()
            ms = a.elapsed_time(b)
        else:
            ms = (time.perf_counter() - t0) * 1e3              # host clock on CPU
        self.stats.append(ChunkStats(self.index, ms, use_graph))
        self.index += 1
        return out


@torch.no_grad()
def camera_rollout(model, context: torch.Tensor, grid_hw, viewmats: torch.Tensor, Ks: Optional[torch.Tensor] = None, *,
                   cfg: StreamingConfig = StreamingConfig(), first_frame: Optional[torch.Tensor] = None,
                   transform: str = "linear", sp=None) -> torch.Tensor:
    """Camera-length rollout: as many chunks as the camera path has frames.  ``viewmats`` [1, F, 4, 4]
    (first-frame-relative world-to-camera), ``Ks`` [1, F, 3, 3] or None.  Every evaluation of a chunk carries
    the chunk's cameras (queries) while cached keys / values keep the cameras of their own frames.
    Returns the latents [1, C, F, H, W] (reference: camera-length rollout of the inference adapter,
    solar/backends/wan22/runtime/inference.py:1647-1714)."""
    gen = StreamingGenerator(model, cfg, sp=sp)
    gen.start(context, grid_hw, first_frame=None)
    F_total = viewmats.shape[1]
    f0 = 0
    outs = []

    def cams(a, b):
        return {"viewmats": viewmats[:, a:b], "Ks": None if Ks is None else Ks[:, a:b], "transform": transform}

    if first_frame is not None:
        t0 = torch.zeros(1, 1, device=gen.device)
        gen.runner.forward_chunk(gen.cache, first_frame.to(gen.device), t0, commit=True, y_camera=cams(0, 1))
        outs.append(first_frame.to(gen.device, model.dtype))
        f0 = 1
    while f0 < F_total:
        f = min(cfg.chunk_frames, F_total - f0)
        cam = cams(f0, f0 + f)
        x = gen._noise(f)
        x0 = x
        for k in range(len(gen.sigmas) - 1):
            s, s_next = gen.sigmas[k], gen.sigmas[k + 1]
            t = torch.full((1, f), s * 1000.0, device=gen.device)
            v = gen.runner.forward_chunk(gen.cache, x, t, commit=False, y_camera=cam)
            x0 = (x.float() - s * v.float()).to(x.dtype)
            if s_next > 0:
                x = ((1 - s_next) * x0.float() + s_next * gen._noise(f).float()).to(x.dtype)
        gen.runner.forward_chunk(gen.cache, x0, torch.zeros(1, f, device=gen.device), commit=True, y_camera=cam)
        outs.append(x0)
        f0 += f
    return torch.cat(outs, dim=2)
