"""Block-causal rendering: the structure-conditioned renderer generated chunk by chunk, for clips of any length.

A clip of ``F`` latent frames is cut into chunks of at most ``chunk`` frames.  The packed document is the renderer's
ordinary one -- ``[text | first frame | structure | target]``, the structure laid over the target frames on their rotary
times -- and a training document appends a clean copy of the target (teacher forcing).  Who sees whom:

  static rows (text, first frame)   see the static rows;
  structure chunk c                 sees the static rows and itself: its rows never depend on another chunk, so they are
                                    the same in training and in a stream that holds only the last ``window`` chunks;
  noisy chunk c                     sees the static rows, the structure of chunks c-window+1 .. c, the clean frames of
                                    chunks c-window+1 .. c-1, and itself;
  clean chunk c                     sees what noisy chunk c sees with its own clean frames in place of the noisy ones --
                                    exactly what a stream computes when it commits chunk c to its key / value cache.

Nothing sees a later chunk.  Attention runs per query segment over exactly its visible keys (dense calls on concatenated
key spans, no token mask): ``training_plan`` lists ``(query span, key spans)`` for the whole document and
``segment_attention`` evaluates it; ``plan_mask`` is the dense oracle.  ``CausalRenderer`` is the stream: per chunk it
evaluates ``[static | structure c | target c]`` while every layer's keys and values of the committed chunks inside the
window come from ``ChunkKVCache``; a chunk is denoised with data-ward Euler steps over the shifted grid and then committed
at the condition level.  ``tests/test_renderer_causal.py`` checks that the stream's evaluation of chunk c equals the
training document's prediction for noisy chunk c.

Reference: solar/renderer/causal.py:1-720 (visibility rule, training plan, generate_causal / stream).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .. import ops
from ..backends.minimax_h3 import flow
from ..backends.minimax_h3.layout import TAG_TEXT, TAG_VIDEO, patchify_latents, spatial_axis, temporal_positions, unpatchify_rows
from ..models.h3 import H3DiT

STATIC_TIME = 1.0
CLEAN_LEVEL = 0.999
Span = Tuple[int, int]


def chunk_spans(frames: int, chunk: int) -> List[Span]:
    if frames < 1 or chunk < 1:
        raise ValueError("frames and chunk are positive")
    return [(a, min(a + chunk, frames)) for a in range(0, frames, chunk)]


def _merge(spans: Sequence[Span]) -> Tuple[Span, ...]:
    out: List[List[int]] = []
    for a, b in sorted(s for s in spans if s[1] > s[0]):
        if out and a <= out[-1][1]:
            out[-1][1] = max(out[-1][1], b)
        else:
            out.append([a, b])
    return tuple((a, b) for a, b in out)


@dataclass(frozen=True)
class DocumentRows:
    """Row spans of a packed causal document ``[static | structure chunks | clean chunks | noisy chunks]``."""
    static: Span
    structure: Tuple[Span, ...]          # empty when the sample carries no structure stream
    clean: Tuple[Span, ...]              # empty without the teacher-forcing copy
    noisy: Tuple[Span, ...]

    @property
    def total(self) -> int:
        return self.noisy[-1][1]


def document_rows(n_static: int, chunk_rows: Sequence[int], *, structure: bool, clean_copy: bool) -> DocumentRows:
    at = n_static

    def lay():
        nonlocal at
        spans = []
        for n in chunk_rows:
            spans.append((at, at + n))
            at += n
        return tuple(spans)

    s = lay() if structure else ()
    c = lay() if clean_copy else ()
    return DocumentRows((0, n_static), s, c, lay())


def training_plan(rows: DocumentRows, window: int) -> List[Tuple[Span, Tuple[Span, ...]]]:
    """``(query span, merged key spans)`` for every segment of the document under the visibility rule."""
    if window < 1:
        raise ValueError("window is at least one chunk")
    plan = [(rows.static, (rows.static,))]
    for j, span in enumerate(rows.structure):
        plan.append((span, _merge([rows.static, span])))
    for kind in ("clean", "noisy"):
        own = getattr(rows, kind)
        for j, span in enumerate(own):
            lo = max(0, j - window + 1)
            keys = [rows.static, span]
            keys += list(rows.structure[lo:j + 1])
            # the history is the CLEAN copy when there is one (teacher forcing), else the noisy chunks themselves
            keys += list((rows.clean if rows.clean else rows.noisy)[lo:j])
            plan.append((span, _merge(keys)))
    return plan


def plan_mask(plan, total: int) -> torch.Tensor:
    m = torch.zeros(total, total, dtype=torch.bool)
    for (qa, qb), keys in plan:
        for ka, kb in keys:
            m[qa:qb, ka:kb] = True
    return m


def segment_attention(q, k, v, plan):
    """q / k / v ``[1, S, H, D]``; every query segment attends the concatenation of its key spans."""
    out = torch.empty_like(q)
    for (qa, qb), keys in plan:
        kk = k[:, keys[0][0]:keys[0][1]] if len(keys) == 1 else torch.cat([k[:, a:b] for a, b in keys], dim=1)
        vv = v[:, keys[0][0]:keys[0][1]] if len(keys) == 1 else torch.cat([v[:, a:b] for a, b in keys], dim=1)
        out[:, qa:qb] = ops.attention(q[:, qa:qb].contiguous(), kk.contiguous(), vv.contiguous())
    return out


# ---------------------------------------------------------------------------------------------------------------------
# documents
# ---------------------------------------------------------------------------------------------------------------------
def _frame_positions(n_text: int, total_frames: int, h: int, w: int):
    rows = h * w
    grid = torch.from_numpy(np.stack(np.meshgrid(spatial_axis(h, w), spatial_axis(w, h), indexing="ij"), -1).reshape(rows, 2))
    tpos = torch.from_numpy(temporal_positions(total_frames + 1, origin=float(n_text)))       # [0] is the first frame's time

    def at(frame_times):
        p = torch.zeros(len(frame_times) * rows, 3, dtype=torch.float64)
        p[:, 0] = torch.as_tensor(frame_times, dtype=torch.float64).repeat_interleave(rows)
        p[:, 1:] = grid.repeat(len(frame_times), 1)
        return p

    text = torch.zeros(n_text, 3, dtype=torch.float64)
    text[:, 0] = torch.arange(n_text)
    return text, at([float(tpos[0])]), lambda a, b: at(tpos[1 + a:1 + b].tolist())


def _forward(model: H3DiT, *, prompt, anchor_rows, video_segments, total_frames: int, grid_hw, cameras, attn_fn):
    """``video_segments``: list of ``(rows [n, 96], row times [n] or a float, (first frame, last frame))`` in document
    order.  Returns the model's output on all video rows."""
    h, w = grid_hw
    n_text, dev = prompt.shape[0], prompt.device
    pos_text, pos_anchor, frames_at = _frame_positions(n_text, total_frames, h, w)
    times = [torch.full((n_text,), STATIC_TIME), torch.full((anchor_rows.shape[0],), CLEAN_LEVEL)]
    pos, view = [pos_text, pos_anchor], None
    if cameras is not None:
        view = [torch.eye(4).repeat(n_text, 1, 1), cameras[:1].float().repeat(anchor_rows.shape[0], 1, 1)]
    for rows, t, (a, b) in video_segments:
        times.append(torch.full((rows.shape[0],), float(t)) if not torch.is_tensor(t) else t.detach().float().cpu())
        pos.append(frames_at(a, b))
        if view is not None:
            view.append(cameras[1 + a:1 + b].float().repeat_interleave(h * w, dim=0))
    values = torch.cat(times)
    uniq, inverse = torch.unique(values, return_inverse=True)
    n_video = sum(r.shape[0] for r, _, _ in video_segments)
    tags = torch.cat([torch.full((n_text,), TAG_TEXT), torch.full((anchor_rows.shape[0] + n_video,), TAG_VIDEO)]).to(torch.int32)
    out, _ = model(video_rows=torch.cat([r for r, _, _ in video_segments]), text_rows=prompt, anchor_rows=anchor_rows, timesteps=uniq,
                   t_index=inverse.to(torch.int32).to(dev), tags=tags.to(dev), position_ids=torch.cat(pos),
                   viewmats=None if view is None else torch.cat(view), attn_fn=attn_fn)
    return out


def teacher_forcing_prediction(model: H3DiT, sample: Mapping[str, torch.Tensor], noisy_rows: torch.Tensor, t_chunks: torch.Tensor, *,
                               chunk: int = 5, window: int = 6):
    """The training document ``[static | structure | clean | noisy]`` under the visibility rule: the prediction on the
    noisy rows ``[F h w, 96]``.  ``t_chunks`` holds one time per chunk."""
    dev, dt = model.proj_in.device, model.dtype
    lat = sample["target_latents"].to(dev)
    C, F, H, W = lat.shape
    h, w = H // 2, W // 2
    spans = chunk_spans(F, chunk)
    per = [(b - a) * h * w for a, b in spans]
    prompt = sample["prompt_embeds"].to(dev, dt)
    anchor_rows = patchify_latents(sample["anchor_latents"].to(dev)).to(dt)
    structure = sample.get("structure_latents")
    rows = document_rows(prompt.shape[0] + anchor_rows.shape[0], per, structure=structure is not None, clean_copy=True)
    plan = training_plan(rows, window)
    clean_rows = patchify_latents(lat).to(dt)
    segs = []
    if structure is not None:
        s_rows = patchify_latents(structure.to(dev)).to(dt)
        segs += [(s_rows[a * h * w:b * h * w], STATIC_TIME, (a, b)) for a, b in spans]
    segs += [(clean_rows[a * h * w:b * h * w], CLEAN_LEVEL, (a, b)) for a, b in spans]
    segs += [(noisy_rows[a * h * w:b * h * w].to(dt), float(t_chunks[i]), (a, b)) for i, (a, b) in enumerate(spans)]
    out = _forward(model, prompt=prompt, anchor_rows=anchor_rows, video_segments=segs, total_frames=F, grid_hw=(h, w),
                   cameras=sample.get("camera_w2c"), attn_fn=lambda q, k, v: segment_attention(q, k, v, plan))
    return out[-F * h * w:]


# ---------------------------------------------------------------------------------------------------------------------
# the stream
# ---------------------------------------------------------------------------------------------------------------------
class ChunkKVCache:
    """Per layer, the keys / values of the structure rows and of the committed clean rows of the last ``window - 1``
    chunks (the current chunk is the window's last)."""

    def __init__(self, window: int):
        self.keep = max(0, int(window) - 1)
        self.layers: List[List[Tuple[torch.Tensor, ...]]] = []      # layers[l] = [(ks, vs, kc, vc) per committed chunk]

    def history(self, layer: int):
        return self.layers[layer] if layer < len(self.layers) else []

    def commit(self, per_layer: Sequence[Tuple[torch.Tensor, ...]]) -> None:
        if not self.layers:
            self.layers = [[] for _ in per_layer]
        for held, fresh in zip(self.layers, per_layer):
            held.append(tuple(t.detach() for t in fresh))
            del held[:max(0, len(held) - self.keep)]

    @property
    def chunks(self) -> int:
        return len(self.layers[0]) if self.layers else 0


class CausalRenderer:
    def __init__(self, model: H3DiT, *, chunk: int = 5, window: int = 6, steps: int = 8, shift: float = flow.VIDEO_SHIFT):
        self.model, self.chunk, self.window, self.steps, self.shift = model, int(chunk), int(window), int(steps), float(shift)

    def _evaluate(self, cache: ChunkKVCache, *, prompt, anchor_rows, structure_rows, target_rows, t: float, frames: Span, total_frames: int,
                  grid_hw, cameras, commit: bool):
        n_static = prompt.shape[0] + anchor_rows.shape[0]
        ns = 0 if structure_rows is None else structure_rows.shape[0]
        a0, a1 = n_static, n_static + ns
        state = {"layer": 0, "fresh": []}

        def attn(q, k, v):
            layer = state["layer"]
            state["layer"] += 1
            hist = cache.history(layer)
            out = torch.empty_like(q)
            ks, vs = k[:, :a0], v[:, :a0]
            out[:, :a0] = ops.attention(q[:, :a0].contiguous(), ks.contiguous(), vs.contiguous())
            if ns:
                out[:, a0:a1] = ops.attention(q[:, a0:a1].contiguous(), k[:, :a1].contiguous(), v[:, :a1].contiguous())
            keys = [ks] + [c[0] for c in hist] + ([k[:, a0:a1]] if ns else []) + [c[2] for c in hist] + [k[:, a1:]]
            vals = [vs] + [c[1] for c in hist] + ([v[:, a0:a1]] if ns else []) + [c[3] for c in hist] + [v[:, a1:]]
            out[:, a1:] = ops.attention(q[:, a1:].contiguous(), torch.cat(keys, 1).contiguous(), torch.cat(vals, 1).contiguous())
            if commit:
                state["fresh"].append((k[:, a0:a1].clone(), v[:, a0:a1].clone(), k[:, a1:].clone(), v[:, a1:].clone()))
            return out

        segs = ([(structure_rows, STATIC_TIME, frames)] if ns else []) + [(target_rows, t, frames)]
        out = _forward(self.model, prompt=prompt, anchor_rows=anchor_rows, video_segments=segs, total_frames=total_frames,
                       grid_hw=grid_hw, cameras=cameras, attn_fn=attn)
        if commit:
            cache.commit(state["fresh"])
        return out[ns:]

    @torch.no_grad()
    def render(self, sample: Mapping[str, torch.Tensor], *, seed: int = 0, record: Optional[list] = None) -> torch.Tensor:
        """``sample`` as ``renderer.core.render`` takes it (``shape`` = (C, F, H, W)); returns latents ``[C, F, H, W]``."""
        model = self.model
        dev, dt = model.proj_in.device, model.dtype
        C, F, H, W = sample["shape"]
        h, w = H // 2, W // 2
        per = h * w
        prompt = sample["prompt_embeds"].to(dev, dt)
        anchor_rows = patchify_latents(sample["anchor_latents"].to(dev)).to(dt)
        structure = sample.get("structure_latents")
        s_rows = None if structure is None else patchify_latents(structure.to(dev)).to(dt)
        cameras = sample.get("camera_w2c")
        g = torch.Generator(device=dev).manual_seed(int(seed))
        times = [float(t) for t in flow.rollout_times(self.steps, self.shift)]
        cache = ChunkKVCache(self.window)
        done = []
        for (a, b) in chunk_spans(F, self.chunk):
            n = (b - a) * per
            x = torch.randn(n, C * 4, generator=g, device=dev)
            kw = dict(prompt=prompt, anchor_rows=anchor_rows, structure_rows=None if s_rows is None else s_rows[a * per:b * per],
                      frames=(a, b), total_frames=F, grid_hw=(h, w), cameras=cameras)
            for i, t in enumerate(times[:self.steps]):
                v = self._evaluate(cache, target_rows=x.to(dt), t=t, commit=False, **kw).float()
                t_next = times[i + 1] if i + 1 < len(times) else 1.0
                x = x + max(t_next - t, 0.0) * v                               # data-ward Euler
            self._evaluate(cache, target_rows=x.to(dt), t=CLEAN_LEVEL, commit=True, **kw)
            if record is not None:
                record.append({"frames": [a, b], "cached_chunks": cache.chunks})
            done.append(x)
        return unpatchify_rows(torch.cat(done).to(dt), C, F, H, W)


class CausalOmniTrainer:
    """Teacher-forcing training of the block-causal renderer: every chunk draws its own shifted time, the noisy chunks are
    predicted in ONE pass over the training document, the loss is the flow-matching error over all target rows.  Shares
    the ``compute_loss`` / ``last_plan`` surface of ``renderer.core.OmniFlowTrainer`` so the training runtime drives either."""

    def __init__(self, model: H3DiT, optimizer, *, chunk: int = 5, window: int = 6, seed: int = 0):
        from types import SimpleNamespace

        self.model, self.opt, self.chunk, self.window = model, optimizer, int(chunk), int(window)
        self.device = model.proj_in.device
        self.rng = np.random.default_rng(seed)
        self.gen = torch.Generator(device=self.device).manual_seed(int(seed) * 100003 + 31)
        self.last_plan = SimpleNamespace(pattern="block_causal", generated_fraction=1.0)

    def compute_loss(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        dev = self.device
        lat = sample["target_latents"].to(dev)
        C, F, H, W = lat.shape
        per = (H // 2) * (W // 2)
        spans = chunk_spans(F, self.chunk)
        t_chunks = torch.tensor([float(1.0 - flow.shifted_sigma(torch.tensor(self.rng.random()), flow.VIDEO_SHIFT)) for _ in spans])
        noise = torch.randn(lat.shape, generator=self.gen, device=dev, dtype=torch.float32)
        x0, n = patchify_latents(lat).float(), patchify_latents(noise)
        t_rows = torch.cat([torch.full(((b - a) * per,), float(t_chunks[i])) for i, (a, b) in enumerate(spans)]).to(dev).view(-1, 1)
        noisy = t_rows * x0 + (1.0 - t_rows) * n
        pred = teacher_forcing_prediction(self.model, sample, noisy, t_chunks, chunk=self.chunk, window=self.window)
        return (pred.float() - (x0 - n)).pow(2).mean()
