"""Block-causal realtime streaming of the H3-shaped DiT: chunked rollout against a windowed KV cache.

One chunk of ``chunk_latents`` latent frames is produced by ``denoise_steps`` network evaluations
on the noisy chunk plus one *commit* evaluation of the clean result (t = 1) that writes the chunk's
keys / values into the cache.  Queries are the chunk rows only; keys are
``[condition rows (refined text + anchor frame) | up to window_chunks committed chunks | chunk]``.

Cache design (per layer, per SP rank: the rank's head shard after the Ulysses exchange):

* keys are stored *after* per-head RMSNorm, MM-RoPE and the PRoPE camera transform, values after the
  camera transform -- exactly what the attention kernel consumes, so a denoise step touches the
  history with no extra pass;
* video rows use window-local temporal positions.  When the window is full and slides by one chunk
  the history keys are re-based with one *delta rotation* (RoPE rotations compose, and only the
  temporal frequencies move), once per chunk instead of re-rotating raw keys on every evaluation as
  the reference does (H3RawKVCache + prepare_sgf_rotaries, solar/backends/minimax_h3/sgf_attention.py:40-149);
* all buffers are allocated once; once the window is full every evaluation has static shapes and the
  denoise / commit evaluations are captured in two CUDA graphs that are replayed per chunk
  (reference: deploy/solar_wm/.../acceleration/graph/{denoise,refresh}.py, engine.py:17-272).

Flow convention: ``x_t = t x0 + (1 - t) n``; the network predicts ``x0 - n``; ``x0 = x_t + (1 - t) v``
(solar/backends/minimax_h3/sgf_rollout.py:147-270).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional

import torch

from .. import ops
from ..backends.minimax_h3.flow import rollout_times
from ..backends.minimax_h3.layout import TAG_TEXT, TAG_VIDEO, spatial_axis, temporal_positions
from ..models.h3 import H3DiT, mm_rope_tables
from ..ops import functional as F_
from ..parallel.ulysses import balanced_lengths


@dataclass
class H3StreamConfig:
    grid_hw: tuple = (24, 42)          # token grid of one latent frame (latent 48 x 84, patch 2 x 2)
    latent_channels: int = 24
    chunk_latents: int = 5
    window_chunks: int = 5             # committed chunks kept as history
    denoise_steps: int = 4
    shift: float = 12.0
    fx: float = 0.505
    fy: float = 0.898
    use_cuda_graph: bool = True
    memory_latents: int = 0            # capacity of the retrieved-memory segment (0 = no memory rows)
    memory_adapter: Optional[str] = None   # adapter bank active while memory rows are installed (fill and query
                                       # evaluations); without memory rows the primary adapter serves
    sp_exchange: str = "fused"         # SP > 1 on CUDA: "fused" = this library's NVLink kernels (k / v rows are stored
                                       # straight into the peers' KV caches, the evaluation is graph-capturable);
                                       # "collective" = NCCL all-to-alls (the baseline arm; runs eagerly)
    max_text_tokens: int = 1536        # sizes the exchange buffers of the fused transport
    fuse_qkv: bool = True              # run q | k | v of adapter-free blocks as one GEMM (``H3DiT.fuse_qkv_``)
    seed: int = 0


@dataclass
class ChunkTiming:
    index: int
    dit_ms: float
    graph: bool


@dataclass
class _LayerKV:
    k: torch.Tensor          # [capacity_rows, local_heads * head_dim]
    v: torch.Tensor


class H3StreamingGenerator:
    def __init__(self, model: H3DiT, cfg: H3StreamConfig = H3StreamConfig(), sp=None):
        self.model, self.cfg, self.sp = model, cfg, sp
        self.P = 1 if sp is None else sp.size
        mc = model.cfg
        assert mc.num_attention_heads % self.P == 0, "SP size must divide the head count"
        self.heads_local = mc.num_attention_heads // self.P
        self.rows_per_latent = cfg.grid_hw[0] * cfg.grid_hw[1]
        self.chunk_rows = cfg.chunk_latents * self.rows_per_latent
        assert self.chunk_rows >= self.P, "every SP rank needs at least one row of a chunk"
        self.device = model.proj_in.device
        if cfg.fuse_qkv:
            model.fuse_qkv_()
        self.gen = torch.Generator(device=self.device).manual_seed(cfg.seed)
        self.times = rollout_times(cfg.denoise_steps, cfg.shift)[:cfg.denoise_steps]
        self.timings: List[ChunkTiming] = []
        self._graphs = None
        self.fx = None                     # parallel.fused_stream.FusedHeadExchange when the fused transport is on

    # ------------------------------------------------------------------------------------ scene
    @torch.no_grad()
    def start(self, text: torch.Tensor, anchor_latent: torch.Tensor, anchor_w2c: Optional[torch.Tensor] = None) -> None:
        """text [n_text, text_dim]; anchor_latent [C, 1, H, W] (the conditioning image latent)."""
        from ..backends.minimax_h3.layout import patchify_latents

        m, mc, cfg = self.model, self.model.cfg, self.cfg
        dev, dt = self.device, m.dtype
        self.n_text = text.shape[0]
        h, w = cfg.grid_hw
        rows = self.rows_per_latent
        # ---- positions: text (i, 0, 0); anchor at the temporal origin; video frames window-local
        ys, xs = spatial_axis(h, w), spatial_axis(w, h)
        import numpy as np

        grid = torch.from_numpy(np.stack(np.meshgrid(ys, xs, indexing="ij"), -1).reshape(rows, 2))
        win_frames = (cfg.window_chunks + 1) * cfg.chunk_latents
        tpos = torch.from_numpy(temporal_positions(1 + win_frames, origin=float(self.n_text)))
        self._grid, self._tpos = grid, tpos

        def frame_pos(t_values):
            p = torch.zeros(len(t_values) * rows, 3, dtype=torch.float64)
            p[:, 0] = torch.as_tensor(t_values, dtype=torch.float64).repeat_interleave(rows)
            p[:, 1:] = grid.repeat(len(t_values), 1)
            return p

        self._frame_pos = frame_pos
        pos_text = torch.zeros(self.n_text, 3, dtype=torch.float64)
        pos_text[:, 0] = torch.arange(self.n_text)
        # ---- condition rows through the network once: refined text + anchor frame at t ~ 1
        txt = F_.linear(text.to(dev, dt), m.context_embedder)
        cos_t, sin_t = mm_rope_tables(pos_text.to(dev), mc.rot_dims, mc.rope_sections)
        for blk in m.refiner:
            txt = blk(txt, None, None, cos_t, sin_t, None, None, None)
        anchor_rows = F_.linear(patchify_latents(anchor_latent.to(dev, dt)), m.proj_in)
        self.n_cond = self.n_text + rows
        self.cond_x = torch.cat([txt, anchor_rows], 0)
        self.cond_pos = torch.cat([pos_text, frame_pos([float(tpos[0])])], 0)
        self.cond_tags = torch.cat([torch.full((self.n_text,), TAG_TEXT), torch.full((rows,), TAG_VIDEO)]).to(dev, torch.int32)
        view = torch.eye(4).repeat(self.n_cond, 1, 1)
        if anchor_w2c is not None:
            view[self.n_text:] = anchor_w2c.float()
        self.cond_view = view
        # ---- caches
        # cache rows: [memory segment | condition | history chunks | current chunk]; the memory segment is filled
        # from its END backwards, so the live rows always form one contiguous range
        self.o_cond = cfg.memory_latents * rows
        self.mem_rows = 0
        cap = self.o_cond + self.n_cond + (cfg.window_chunks + 1) * self.chunk_rows
        a_local = self.heads_local * mc.attention_head_dim
        if self.P > 1 and cfg.sp_exchange == "fused" and dev.type == "cuda":
            if self.n_text > cfg.max_text_tokens:
                raise ValueError(f"{self.n_text} text rows exceed max_text_tokens={cfg.max_text_tokens}")
            if self.fx is None:
                from ..parallel.fused_stream import FusedHeadExchange

                cap_max = self.o_cond + cfg.max_text_tokens + rows + (cfg.window_chunks + 1) * self.chunk_rows
                self.fx = FusedHeadExchange(self.sp.group, heads=mc.num_attention_heads, head_dim=mc.attention_head_dim,
                                            layers=len(m.blocks), cache_rows=cap_max,
                                            max_rows=max(self.chunk_rows, cfg.max_text_tokens + rows, self.o_cond),
                                            out_width=mc.latent_row_dim, dtype=dt)
            # the KV caches are the exchange's symmetric buffers: peers append their rows in place
            self.kv = [_LayerKV(k[:cap], v[:cap]) for k, v in zip(self.fx.k_cache, self.fx.v_cache)]
            for kv in self.kv:
                kv.k.zero_()
                kv.v.zero_()
            self.fx.barrier()
        else:
            self.kv = [_LayerKV(torch.zeros(cap, a_local, dtype=dt, device=dev), torch.zeros(cap, a_local, dtype=dt, device=dev))
                       for _ in m.blocks]
        self.hist_chunks = 0
        self.chunk_index = 0
        self._graphs = None
        # delta rotation that moves a cached key one chunk towards the past (temporal axis only)
        span = float(tpos[1 + cfg.chunk_latents] - tpos[1])
        dpos = torch.zeros(cfg.window_chunks * self.chunk_rows, 3, dtype=torch.float64)
        dpos[:, 0] = -span
        self._delta_cos, self._delta_sin = mm_rope_tables(dpos.to(dev), mc.rot_dims, mc.rope_sections)
        self.cond_tags = self.cond_tags.contiguous()
        # static input slots (pointer-stable for graph replay)
        self._x_in = torch.zeros(self.chunk_rows, mc.latent_row_dim, dtype=dt, device=dev)
        self._t_in = torch.ones(1, dtype=torch.float32, device=dev)
        self._t_host, self._table_cache = None, {}
        self._view_in = torch.eye(4, device=dev).repeat(self.chunk_rows, 1, 1)
        self._out = torch.zeros(self.chunk_rows, mc.latent_row_dim, dtype=dt, device=dev)
        self._video_tags = torch.full((self.chunk_rows,), TAG_VIDEO, dtype=torch.int32, device=dev)
        self._pos_cache = {}
        self._lift = torch.tensor([cfg.fx, cfg.fy, 1.0, 1.0], device=dev)
        self._commit_condition()

    def _local(self, n_rows: int):
        """Row slice of this SP rank for a segment of ``n_rows`` rows."""
        if self.P == 1:
            return slice(0, n_rows)
        from ..parallel.ulysses import balanced_bounds

        return slice(*balanced_bounds(n_rows, self.P, self.sp.rank))    # balanced, descending; need not be even

    # ------------------------------------------------------------------------------------ network
    def _evaluate(self, x_rows, t_scalar, pos, tags, view, key_base: int, n_rows: int, write_only: bool = False,
                  key_lo: int = None, key_hi: int = None, tables=None):
        """Run the 50 blocks on ``n_rows`` new rows (sharded over SP) whose keys / values are written at
        cache rows ``[key_base, key_base + n_rows)`` and which attend to cache rows ``[key_lo, key_hi)``
        (default: everything from the first live row up to and including the new rows).
        Returns the output rows of this rank (or None with ``write_only``, used for condition / memory rows)."""
        key_lo = self.o_cond - self.mem_rows if key_lo is None else key_lo
        key_hi = key_base + n_rows if key_hi is None else key_hi
        m, mc = self.model, self.model.cfg
        H, hd, hl = mc.num_attention_heads, mc.attention_head_dim, self.heads_local
        loc = self._local(n_rows)
        x = x_rows[loc]
        cos, sin = pos                                                   # tables of this rank's rows (device)
        cam_q, cam_kv, cam_o = self._camera_mats(view[loc])
        temb = None if tables is not None else m.time_embed(t_scalar.view(1))
        idx = (tags[loc].to(torch.int32)).contiguous()                 # one timestep group: row = 0 * 3 + tag
        kw = dict(rot_dims=mc.rot_dims, sections=mc.rope_sections, eps=mc.eps)
        S = x.shape[0]
        for bi, (blk, kv) in enumerate(zip(m.blocks, self.kv)):
            table = tables[bi] if tables is not None else blk.tables(temb)
            xm = F_.norm_modulate(x, table[:, 0], table[:, 1], mode=1, w=blk.norm1, eps=mc.eps, table=idx)
            fused_w = getattr(blk, "qkv_weight", None) if blk.to_q._bank is None else None
            if fused_w is not None:                                      # one GEMM for the three projections
                qkv = F_.linear(xm, fused_w)
                a_ = H * hd
                q_in, k_in, v_in = qkv[:, :a_], qkv[:, a_:2 * a_], qkv[:, 2 * a_:]
            else:
                q_in, k_in, v_in = blk.to_q(xm), blk.to_k(xm), blk.to_v(xm)
            q = ops.head_norm_rope_prope(q_in, blk.norm_q, cos, sin, cam_q, heads=H, **kw)
            k = ops.head_norm_rope_prope(k_in, blk.norm_k, cos, sin, cam_kv, heads=H, **kw)
            v = ops.head_norm_rope_prope(v_in, None, None, None, cam_kv, heads=H, **kw)
            if self.fx is not None:
                # fused transport: one launch stores q into the exchange buffer and k / v straight into every peer's
                # cache rows; the attention epilogue returns the output rows to their owners
                fx = self.fx
                fx.set_rows(n_rows)
                par = fx.next_parity()
                qh = fx.exchange_qkv(q, k, v, bi, key_base, par)
                o = fx.attention(qh, bi, key_lo, key_hi, 1.0 / (hd ** 0.5), par)
            else:
                q, k, v = (t.view(1, S, H, hd) for t in (q, k, v))
                if self.P > 1:
                    self.sp.set_layout_rows(1, balanced_lengths(n_rows, self.P))
                    q, k, v = self.sp.scatter_heads(q, k, v, contiguous=False)      # strided views of the exchange buffer
                kv.k[key_base:key_base + n_rows].view(1, n_rows, hl, hd).copy_(k)     # one strided copy each
                kv.v[key_base:key_base + n_rows].view(1, n_rows, hl, hd).copy_(v)
                n_keys = key_hi - key_lo
                o = ops.attention(q.reshape(1, n_rows, hl, hd), kv.k[key_lo:key_hi].view(1, n_keys, hl, hd),
                                  kv.v[key_lo:key_hi].view(1, n_keys, hl, hd))
                if self.P > 1:
                    o = self.sp.gather_heads(o)
            o = ops.head_norm_rope_prope(o.reshape(S, H * hd), None, None, None, cam_o, heads=H, **kw)
            x = F_.gated_residual(x, blk.to_out(o), table[:, 2], table=idx)
            xm = F_.norm_modulate(x, table[:, 3], table[:, 4], mode=1, w=blk.norm2, eps=mc.eps, table=idx)
            x = F_.gated_residual(x, blk.ffn_down(F_.swiglu(blk.ffn_gate_up(xm))), table[:, 5], table=idx)
        if write_only:
            return None
        xn = F_.norm_modulate(x, mode=1, w=m.norm_out, eps=mc.eps)
        return F_.linear(xn, m.proj_out)

    def _camera_mats(self, view: torch.Tensor):
        """Rigid view matrices [S, 4, 4] -> (P^T, P^-1, P) with P = diag(fx, fy, 1, 1) @ view, in closed form
        (R^T, -R^T t) so that the computation is plain device arithmetic and can sit inside a CUDA graph."""
        v = view.to(self.device, torch.float32)
        lift = self._lift
        P = v * lift.view(1, 4, 1)
        R, t = v[:, :3, :3], v[:, :3, 3:]
        inv = torch.zeros_like(v)
        inv[:, :3, :3] = R.transpose(1, 2)
        inv[:, :3, 3:] = -R.transpose(1, 2) @ t
        inv[:, 3, 3] = 1.0
        Pinv = inv / lift.view(1, 1, 4)
        return P.transpose(1, 2).contiguous(), Pinv.contiguous(), P.contiguous()

    def _tables(self, pos64: torch.Tensor, n_rows: int):
        mc = self.model.cfg
        return mm_rope_tables(pos64[self._local(n_rows)].to(self.device), mc.rot_dims, mc.rope_sections)

    def _commit_condition(self) -> None:
        """Text + anchor rows attend among themselves; their keys / values head the cache for good."""
        self._evaluate(self.cond_x, torch.tensor([0.999], device=self.device), self._tables(self.cond_pos, self.n_cond),
                       self.cond_tags, self.cond_view, key_base=self.o_cond, n_rows=self.n_cond, write_only=True,
                       key_lo=self.o_cond)

    def _chunk_eval(self) -> None:
        """Evaluate the chunk in the static input slots against the current window -> ``self._out``."""
        cfg = self.cfg
        base = self.o_cond + self.n_cond + self.hist_chunks * self.chunk_rows
        first = 1 + self.hist_chunks * cfg.chunk_latents
        if first not in self._pos_cache:                               # built outside any graph capture
            pos = self._frame_pos([float(self._tpos[first + i]) for i in range(cfg.chunk_latents)])
            self._pos_cache[first] = self._tables(pos, self.chunk_rows)
        x = F_.linear(self._x_in, self.model.proj_in)
        out = self._evaluate(x, self._t_in, self._pos_cache[first], self._video_tags, self._view_in, key_base=base,
                             n_rows=self.chunk_rows, tables=self._step_tables())
        if self.fx is not None:
            self.fx.set_rows(self.chunk_rows)
            out = self.fx.gather_rows(out)
        elif self.P > 1:
            self.sp.set_layout_rows(1, balanced_lengths(self.chunk_rows, self.P))
            out = self.sp.gather_sequence(out, 1)
        self._out.copy_(out)

    def _step_tables(self):
        """Per-block adaLN tables of the current denoise level, kept per level: the schedule has ``denoise_steps``
        + 1 distinct times, so the eager path (one launch per kernel) skips the time MLP and 50 small projection
        GEMMs in every evaluation.  Inside a graph capture the tables are computed from the device scalar instead,
        so that one captured graph serves every level."""
        t = self._t_host
        if t is None or (self.device.type == "cuda" and torch.cuda.is_current_stream_capturing()):
            return None
        if t not in self._table_cache:
            temb = self.model.time_embed(torch.full((1,), t, dtype=torch.float32, device=self.device))
            self._table_cache[t] = [blk.tables(temb) for blk in self.model.blocks]
        return self._table_cache[t]

    def _slide(self) -> None:
        """Commit bookkeeping: keep the chunk just written; with a full window drop the oldest chunk and
        re-base the surviving keys by one chunk (delta rotation on the temporal frequencies)."""
        cfg, mc = self.cfg, self.model.cfg
        if self.hist_chunks < cfg.window_chunks:
            self.hist_chunks += 1
            if self.fx is not None:
                self.fx.barrier()
            return
        a, n = self.o_cond + self.n_cond, cfg.window_chunks * self.chunk_rows
        for kv in self.kv:
            kv.k[a:a + n] = kv.k[a + self.chunk_rows:a + self.chunk_rows + n].clone()
            kv.v[a:a + n] = kv.v[a + self.chunk_rows:a + self.chunk_rows + n].clone()
            kv.k[a:a + n] = ops.head_norm_rope_prope(kv.k[a:a + n], None, self._delta_cos, self._delta_sin, None,
                                                     heads=self.heads_local, rot_dims=mc.rot_dims,
                                                     sections=mc.rope_sections, eps=mc.eps)
        if self.fx is not None:
            self.fx.barrier()          # peers append the next chunk's rows into this cache: not before the slide is done

    # ------------------------------------------------------------------------------------ memory
    @torch.no_grad()
    def set_memory(self, latents: Optional[torch.Tensor], w2c: Optional[torch.Tensor] = None) -> None:
        """Install retrieved latents [C, k, H, W] (k <= memory_latents) with their cameras [k, 4, 4] as extra
        key rows for the following chunks.  The memory rows run through the network once as clean rows that
        see the condition rows and one another; they sit temporally before the anchor frame.  ``None`` clears
        the segment (reference: memory-bank rows of the packed document, memory_inference.py:126)."""
        from ..backends.minimax_h3.layout import patchify_latents

        cfg, m = self.cfg, self.model
        rows = self.rows_per_latent
        k = 0 if latents is None else latents.shape[1]
        if k > cfg.memory_latents:
            raise ValueError(f"{k} memory latents exceed the configured capacity {cfg.memory_latents}")
        if k * rows != self.mem_rows:
            self._graphs = None                 # the key range changes: a captured graph no longer applies
        if cfg.memory_adapter is not None:
            want = cfg.memory_adapter if k > 0 else None
            if getattr(m, "active_adapter", None) != want:
                m.set_adapter(want)             # other weights: a captured graph no longer applies either
                self._graphs = None
        self.mem_rows = k * rows
        if k == 0:
            return
        span = float(self._tpos[2] - self._tpos[1])
        t_mem = [float(self._tpos[0]) - (k - i) * span for i in range(k)]
        pos = self._tables(self._frame_pos(t_mem), k * rows)
        x = F_.linear(patchify_latents(latents.to(self.device, m.dtype)), m.proj_in)
        view = torch.eye(4).repeat(k * rows, 1, 1) if w2c is None else w2c.float().repeat_interleave(rows, dim=0)
        tags = torch.full((k * rows,), TAG_VIDEO, dtype=torch.int32, device=self.device)
        lo = self.o_cond - k * rows
        self._evaluate(x, torch.ones(1, device=self.device), pos, tags, view, key_base=lo, n_rows=k * rows,
                       write_only=True, key_lo=lo, key_hi=self.o_cond + self.n_cond)

    # ------------------------------------------------------------------------------------ rollout
    def _noise(self):
        return torch.randn(self._x_in.shape, generator=self.gen, device=self.device, dtype=torch.float32)

    def _denoise_chunk(self, eval_fn) -> torch.Tensor:
        """4 evaluations with re-noising between them; returns the clean chunk rows (fp32)."""
        x = self._noise()
        x0 = x
        for i, t in enumerate(self.times):
            self._x_in.copy_(x.to(self._x_in.dtype))
            self._t_in.fill_(float(t))
            self._t_host = float(t)
            eval_fn()
            x0 = x + (1.0 - float(t)) * self._out.float()
            if i + 1 < len(self.times):
                tn = float(self.times[i + 1])
                x = tn * x0 + (1.0 - tn) * self._noise()
        return x0

    @torch.no_grad()
    def next_chunk(self, w2c_per_latent: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Generate one chunk; ``w2c_per_latent`` [chunk_latents, 4, 4] are the cameras of its frames.
        Returns the latent chunk ``[C, chunk_latents, H, W]`` (bf16)."""
        from ..backends.minimax_h3.layout import unpatchify_rows

        cfg = self.cfg
        if w2c_per_latent is not None:
            self._view_in.copy_(w2c_per_latent.to(self.device).float().repeat_interleave(self.rows_per_latent, dim=0))
        steady = self.hist_chunks == cfg.window_chunks
        use_graph = cfg.use_cuda_graph and steady and self.device.type == "cuda"
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        if use_graph:
            if self._graphs is None:
                self._pos_ready()
                self._capture()
            x0 = self._denoise_chunk(self._graphs.replay)
        else:
            x0 = self._denoise_chunk(self._chunk_eval)
        # commit: clean forward writes the chunk's keys / values, then the window advances
        self._x_in.copy_(x0.to(self._x_in.dtype))
        self._t_in.fill_(1.0)
        self._t_host = 1.0
        (self._graphs.replay if use_graph else self._chunk_eval)()
        self._slide()
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
            if self.fx is not None:
                # the fused exchange's device-side waits are bounded: one that gave up set the status word and let the
                # consumers run on what had arrived.  The chunk is complete here (the synchronize above), so reading
                # the word costs nothing; a non-zero word means a peer fell behind or left, and the chunk is discarded
                # (the peers' own waits run out the same way, so every rank raises)
                from ..ops.functional import read_status

                code = read_status(self.device, clear=True)
                if code:
                    raise RuntimeError(f"streaming chunk {self.chunk_index}: a device-side exchange wait gave up "
                                       f"(code {code}); a sequence-parallel peer did not deliver its rows in time")
        self.timings.append(ChunkTiming(self.chunk_index, (time.perf_counter() - t0) * 1e3, use_graph))
        self.chunk_index += 1
        h, w = cfg.grid_hw
        return unpatchify_rows(x0.to(self.model.dtype), cfg.latent_channels, cfg.chunk_latents, 2 * h, 2 * w)

    def _pos_ready(self) -> None:
        first = 1 + self.hist_chunks * self.cfg.chunk_latents
        if first not in self._pos_cache:
            pos = self._frame_pos([float(self._tpos[first + i]) for i in range(self.cfg.chunk_latents)])
            self._pos_cache[first] = self._tables(pos, self.chunk_rows)

    def _capture(self) -> None:
        """Capture one chunk evaluation against the full window.  The denoise evaluations and the commit
        evaluation run the same program (they differ only in the loaded inputs), so one graph serves both."""
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._chunk_eval()                       # warm-up on the side stream (allocator, lazy init)
        torch.cuda.current_stream(self.device).wait_stream(s)
        g = torch.cuda.CUDAGraph()
        # with several ranks other threads of the process (the collective library's watchdog) make CUDA calls of
        # their own: only this thread's calls belong to the capture
        with torch.cuda.graph(g, capture_error_mode="thread_local" if self.P > 1 else "global"):
            self._chunk_eval()
        self._graphs = g
