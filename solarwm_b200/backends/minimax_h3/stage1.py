"""H3 Stage1: teacher-forcing training under the chunk-window ("W6") visibility rule.

Packed document ``[text | anchor | clean video | noisy video]``; the clean copy sits at t = 1, every
chunk of the noisy copy at its own timestep.  Visibility (rows = queries):

    condition (text + anchor)   sees   condition
    clean chunk i               sees   condition + clean chunks max(0, i - W) .. i
    noisy chunk i               sees   condition + clean chunks max(0, i - W) .. i-1 + its own noisy chunk

executed as one dense attention per (role, chunk) over the union of its visible key spans -- the
27 %-dense mask never materialises (reference: W6 attention, solar/backends/minimax_h3/w6_attention.py:
35-324 and mask.py:44-72; Stage1 core stage1.py:27-243).

Objectives in the data-ward convention (``x_t = t x0 + (1 - t) n``, network output ``x0 - n``):
  * ``tf_fm``    plain flow matching on the noisy half;
  * ``anyflow``  AnyFlow v1.5 forward map: the trainable evaluation plus no-grad evaluations at
                 ``t +/- eps`` for the central difference (solar/backends/minimax_h3/anyflow_loss.py:22-81).
"""
from __future__ import annotations

from typing import Mapping, Optional

import numpy as np
import torch

from ... import ops
from ...engine import anyflow as af
from ...engine.master_adamw import FP32MasterAdamW
from ...models.h3 import H3DiT
from . import flow
from .layout import TAG_AUDIO, TAG_TEXT, TAG_VIDEO, patchify_latents, spatial_axis, temporal_positions


def w6_attention(q, k, v, *, n_cond: int, chunk_rows: int, n_chunks: int, window_chunks: int, n_audio: int = 0):
    """q / k / v [1, S, H, D] with S = n_cond + n_audio + 2 * n_chunks * chunk_rows, rows in the order
    [condition | audio | clean | noisy].  Returns [1, S, H, D].  Condition rows see condition rows, audio rows see
    condition and audio rows, every video row sees both on top of its own window.  On the device one masked
    flash-attention call evaluates the whole rule (prefix rows, clean windows, noisy chunks) with the audio rows counted
    into the prefix, and the condition rows -- the only ones that rule shows too much -- are evaluated again on their
    own; the per-chunk loop below is the CPU form."""
    L = n_chunks * chunk_rows
    cond_rows, n_cond = n_cond, n_cond + n_audio    # from here on ``n_cond`` is the whole common prefix
    if q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and ops.get_backend() == "native":
        from ...models.wan_tf import _cached_mask
        from ...ops.attention_mask import masked_attention

        out = masked_attention(q, k, v, _cached_mask("tf", L, chunk_rows, window_chunks, 0, n_cond))
        if n_audio:
            out = torch.cat([ops.attention(q[:, :cond_rows], k[:, :cond_rows], v[:, :cond_rows]), out[:, cond_rows:]], 1)
        return out
    c0, n0 = n_cond, n_cond + L                     # first clean row, first noisy row
    outs = [ops.attention(q[:, :cond_rows], k[:, :cond_rows], v[:, :cond_rows])]
    if n_audio:
        outs.append(ops.attention(q[:, cond_rows:n_cond], k[:, :n_cond], v[:, :n_cond]))
    clean, noisy = [], []
    for i in range(n_chunks):
        lo = c0 + max(0, i - window_chunks) * chunk_rows
        hi = c0 + (i + 1) * chunk_rows
        kk = torch.cat([k[:, :n_cond], k[:, lo:hi]], 1)
        vv = torch.cat([v[:, :n_cond], v[:, lo:hi]], 1)
        clean.append(ops.attention(q[:, c0 + i * chunk_rows:hi], kk, vv))
        own = slice(n0 + i * chunk_rows, n0 + (i + 1) * chunk_rows)
        kn = torch.cat([k[:, :n_cond], k[:, lo:c0 + i * chunk_rows], k[:, own]], 1)
        vn = torch.cat([v[:, :n_cond], v[:, lo:c0 + i * chunk_rows], v[:, own]], 1)
        noisy.append(ops.attention(q[:, own], kn, vn))
    return torch.cat(outs + clean + noisy, 1)


def w6_mask(n_cond: int, chunk_rows: int, n_chunks: int, window_chunks: int, n_audio: int = 0) -> torch.Tensor:
    """Dense boolean oracle of ``w6_attention`` (True = visible)."""
    L = n_chunks * chunk_rows
    cond_rows, n_cond = n_cond, n_cond + n_audio
    S = n_cond + 2 * L
    m = torch.zeros(S, S, dtype=torch.bool)
    m[:, :n_cond] = True
    m[:n_cond, n_cond:] = False
    m[:cond_rows, cond_rows:] = False
    ch = torch.arange(L) // chunk_rows
    qc, kc = ch.view(-1, 1), ch.view(1, -1)
    m[n_cond:n_cond + L, n_cond:n_cond + L] = (kc <= qc) & (kc >= qc - window_chunks)
    m[n_cond + L:, n_cond:n_cond + L] = (kc < qc) & (kc >= qc - window_chunks)
    m[n_cond + L:, n_cond + L:] = kc == qc
    return m


def teacher_forcing_forward(model: H3DiT, *, prompt, anchor_rows, clean_rows, noisy_rows, t_chunks: torch.Tensor,
                            grid_hw, chunk_latents: int, window_chunks: int, cameras: Optional[torch.Tensor] = None,
                            capture: Optional[list] = None, audio_rows: Optional[torch.Tensor] = None, t_audio: float = 0.5):
    """Rows are already patchified ([n, 96]); ``t_chunks`` [n_chunks] in [0, 1] (1 = clean).  Returns the
    prediction for the noisy rows [L, 96].  ``audio_rows`` [Na, 32] (the silent soundtrack already noised to
    ``t_audio``) sit between the anchor and the video; their prediction is dropped.  With ``capture`` (an empty list)
    every main block appends the detached keys / values of the prefix rows ``[text | anchor | audio | clean]``: under
    W6 those rows never see a noisy row, so they are the same in every evaluation of the step and ``suffix_forward``
    can reuse them."""
    h, w = grid_hw
    rows = h * w
    L = clean_rows.shape[0]
    F = L // rows
    n_chunks = F // chunk_latents
    n_text = prompt.shape[0]
    n_cond = n_text + anchor_rows.shape[0]
    n_audio = 0 if audio_rows is None else audio_rows.shape[0]
    dev = clean_rows.device
    # ---- per-row timestep groups: text / clean -> 1.0 ; anchor -> 0.999 ; audio -> t_audio ; noisy chunk i -> t_chunks[i]
    values = torch.cat([torch.tensor([1.0, 0.999, float(t_audio)]), t_chunks.detach().float().cpu()])
    uniq, inverse = torch.unique(values, return_inverse=True)
    chunk_rows = chunk_latents * rows
    t_index = torch.cat([torch.full((n_text,), int(inverse[0])), torch.full((anchor_rows.shape[0],), int(inverse[1])),
                         torch.full((n_audio,), int(inverse[2])),
                         torch.full((L,), int(inverse[0])), inverse[3:].repeat_interleave(chunk_rows)]).to(torch.int32)
    tags = torch.cat([torch.full((n_text,), TAG_TEXT), torch.full((anchor_rows.shape[0],), TAG_VIDEO),
                      torch.full((n_audio,), TAG_AUDIO), torch.full((2 * L,), TAG_VIDEO)]).to(torch.int32)
    # ---- positions: both video copies share the native grid positions
    pos_text = torch.zeros(n_text, 3, dtype=torch.float64)
    pos_text[:, 0] = torch.arange(n_text)
    ys, xs = spatial_axis(h, w), spatial_axis(w, h)
    grid = torch.from_numpy(np.stack(np.meshgrid(ys, xs, indexing="ij"), -1).reshape(rows, 2))
    tpos = torch.from_numpy(temporal_positions(F + 1, origin=float(n_text)))

    def frames(ts):
        p = torch.zeros(len(ts) * rows, 3, dtype=torch.float64)
        p[:, 0] = torch.as_tensor(ts, dtype=torch.float64).repeat_interleave(rows)
        p[:, 1:] = grid.repeat(len(ts), 1)
        return p

    vid_pos = frames(tpos[1:].tolist())
    pos_audio = torch.zeros(n_audio, 3, dtype=torch.float64)          # (origin + j, 0, first | last column), as in the
    pos_audio[:, 0] = n_text + torch.arange(n_audio)                   # bidirectional document
    pos_audio[:, 2] = torch.from_numpy(np.where(np.arange(n_audio) < n_audio // 2, float(xs[0]), float(xs[-1])))
    pos = torch.cat([pos_text, frames([float(tpos[0])])[:anchor_rows.shape[0]], pos_audio, vid_pos, vid_pos])
    view = None
    if cameras is not None:                 # [1 + F, 4, 4]: anchor then frames
        per = cameras[1:].float().repeat_interleave(rows, dim=0)
        view = torch.cat([torch.eye(4).repeat(n_text, 1, 1), cameras[:1].float().repeat(anchor_rows.shape[0], 1, 1),
                          torch.eye(4).repeat(n_audio, 1, 1), per, per])

    def attn(q, k, v):
        if capture is not None:
            capture.append((k[:, :n_cond + n_audio + L].detach(), v[:, :n_cond + n_audio + L].detach()))
        return w6_attention(q, k, v, n_cond=n_cond, chunk_rows=chunk_rows, n_chunks=n_chunks, window_chunks=window_chunks,
                            n_audio=n_audio)

    vid, _ = model(video_rows=torch.cat([clean_rows, noisy_rows]), text_rows=prompt, anchor_rows=anchor_rows, audio_rows=audio_rows,
                   timesteps=uniq, t_index=t_index.to(dev), tags=tags.to(dev), position_ids=pos, viewmats=view,
                   attn_fn=attn)
    return vid[L:]


@torch.no_grad()
def suffix_forward(model: H3DiT, *, captured, noisy_rows, t_chunks: torch.Tensor, n_text: int, n_anchor: int, grid_hw,
                   chunk_latents: int, window_chunks: int, cameras: Optional[torch.Tensor] = None, n_audio: int = 0):
    """The noisy half alone against captured prefix keys / values (one ``(k, v)`` pair per main block from
    ``teacher_forcing_forward(capture=...)``): the same prediction as a full evaluation for these noisy rows, at
    about half its cost -- the text, anchor and clean rows are not recomputed.  No-grad evaluations only (the
    central-difference probes of the AnyFlow objective); reference: prefix-KV capture / suffix reuse,
    solar/backends/minimax_h3/w6_attention.py:218-324."""
    from ...models.h3 import mm_rope_tables, prope_row_matrices
    from ...ops import functional as F_

    cfg = model.cfg
    h, w = grid_hw
    rows = h * w
    L = noisy_rows.shape[0]
    F = L // rows
    n_chunks = F // chunk_latents
    chunk_rows = chunk_latents * rows
    n_cond = n_text + n_anchor + n_audio            # the common prefix every video row sees
    dev = noisy_rows.device
    if len(captured) != len(model.blocks):
        raise ValueError("one captured (k, v) pair per main block is required")
    uniq, inverse = torch.unique(t_chunks.detach().float().cpu(), return_inverse=True)
    idx = (inverse.repeat_interleave(chunk_rows).to(torch.int32) * 3 + TAG_VIDEO).to(dev).contiguous()
    ys, xs = spatial_axis(h, w), spatial_axis(w, h)
    grid = torch.from_numpy(np.stack(np.meshgrid(ys, xs, indexing="ij"), -1).reshape(rows, 2))
    tpos = torch.from_numpy(temporal_positions(F + 1, origin=float(n_text)))
    pos = torch.zeros(L, 3, dtype=torch.float64)
    pos[:, 0] = tpos[1:].to(torch.float64).repeat_interleave(rows)
    pos[:, 1:] = grid.repeat(F, 1)
    cos, sin = mm_rope_tables(pos.to(dev), cfg.rot_dims, cfg.rope_sections)
    cam_q = cam_kv = cam_o = None
    if cameras is not None:
        cam_q, cam_kv, cam_o = prope_row_matrices(cameras[1:].float().repeat_interleave(rows, dim=0).to(dev), 0.505, 0.898)
    temb = model.time_embed(uniq.to(dev))
    layer = [0]

    def attn(q, k, v):
        pk, pv = captured[layer[0]]
        layer[0] += 1
        outs = []
        for i in range(n_chunks):
            lo = n_cond + max(0, i - window_chunks) * chunk_rows
            hi = n_cond + i * chunk_rows                                   # clean chunks lo .. i-1
            own = slice(i * chunk_rows, (i + 1) * chunk_rows)
            kk = torch.cat([pk[:, :n_cond], pk[:, lo:hi], k[:, own]], 1)
            vv = torch.cat([pv[:, :n_cond], pv[:, lo:hi], v[:, own]], 1)
            outs.append(ops.attention(q[:, own], kk, vv))
        return torch.cat(outs, 1)

    x = F_.linear(noisy_rows.to(model.dtype), model.proj_in)
    for blk in model.blocks:
        x = blk(x, blk.tables(temb), idx, cos, sin, cam_q, cam_kv, cam_o, attn_fn=attn)
    return F_.linear(F_.norm_modulate(x, mode=1, w=model.norm_out, eps=cfg.eps), model.proj_out)


class H3Stage1Trainer:
    def __init__(self, cfg, device, *, objective: str = "tf_fm", chunk_latents: int = 5, window_chunks: int = 5,
                 lr: float = 1e-4, seed: int = 0, diffusion_ratio: float = 0.5, consistency_ratio: float = 0.25,
                 epsilon: float = 0.005, reuse_prefix: bool = True, model=None, optimizer=None, generator=None):
        """``model`` / ``optimizer`` / ``generator``: objects a training runtime already owns (it then drives
        ``compute_loss`` itself and this class builds nothing)."""
        self.reuse_prefix = bool(reuse_prefix)     # AnyFlow probes reuse the trainable evaluation's prefix K / V
        dtype = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
        self.model = model if model is not None else H3DiT(cfg, device=device, dtype=dtype, seed=seed)
        self.opt = optimizer if optimizer is not None else FP32MasterAdamW(self.model.trainable_parameters(), lr=lr)
        self.device = torch.device(device)
        self.gen = generator if generator is not None else \
            torch.Generator(device=self.device).manual_seed(seed * 100003 + 1)
        self.objective, self.chunk_latents, self.window_chunks = objective, chunk_latents, window_chunks
        self.ratios, self.epsilon = (diffusion_ratio, consistency_ratio), float(epsilon)
        self.silence: Optional[torch.Tensor] = None     # packed rows of encoded silence [Na, 32]; None = no audio rows
        self._audio = None                              # this step's (noised rows, audio time), shared by its evaluations

    def _predict(self, sample, lat, noise, t_chunks, capture=None, captured=None):
        dev, dt = self.device, self.model.dtype
        C, F, H, W = lat.shape
        rows = (H // 2) * (W // 2)
        t_rows = t_chunks.repeat_interleave(self.chunk_latents * rows).view(-1, 1)
        clean = patchify_latents(lat).to(dt)
        noisy = (t_rows * clean.float() + (1.0 - t_rows) * patchify_latents(noise).float()).to(dt)
        anchor = sample["anchor_latents"].to(dev)
        audio, t_audio = self._audio if self._audio is not None else (None, 0.5)
        if captured is not None:                   # probe: the noisy half against the captured prefix
            return suffix_forward(self.model, captured=captured, noisy_rows=noisy, t_chunks=t_chunks,
                                  n_text=sample["prompt_embeds"].shape[0], n_anchor=patchify_latents(anchor).shape[0],
                                  grid_hw=(H // 2, W // 2), chunk_latents=self.chunk_latents,
                                  window_chunks=self.window_chunks, cameras=sample.get("camera_w2c"),
                                  n_audio=0 if audio is None else audio.shape[0])
        a_noise = torch.randn(anchor.shape, generator=self.gen, device=dev, dtype=torch.float32).to(anchor.dtype)
        return teacher_forcing_forward(self.model, capture=capture, prompt=sample["prompt_embeds"].to(dev, dt),
                                       anchor_rows=patchify_latents(flow.interpolate(anchor, a_noise, 0.999)).to(dt),
                                       clean_rows=clean, noisy_rows=noisy, t_chunks=t_chunks, grid_hw=(H // 2, W // 2),
                                       chunk_latents=self.chunk_latents, window_chunks=self.window_chunks,
                                       cameras=sample.get("camera_w2c"), audio_rows=None if audio is None else audio.to(dt),
                                       t_audio=t_audio)

    def train_step(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        loss = self.compute_loss(sample)
        loss.backward()
        self.opt.gather_grads()
        self.opt.clip_(1.0)
        self.opt.step()
        self.opt.zero_grad()
        return loss.detach()

    def compute_loss(self, sample: Mapping[str, torch.Tensor]) -> torch.Tensor:
        """The objective of one packed sample (teacher-forcing flow matching or AnyFlow), with its graph."""
        dev = self.device
        lat = sample["target_latents"].to(dev)
        C, F, H, W = lat.shape
        n_chunks = F // self.chunk_latents
        rows = (H // 2) * (W // 2)
        noise = torch.randn(lat.shape, generator=self.gen, device=dev, dtype=torch.float32).to(lat.dtype)
        self._audio = None
        if self.silence is not None:     # one audio time and one audio noise per step: every evaluation of the step sees them
            from .silence import noised_silence

            self._audio = noised_silence(self.silence, self.gen, dev)
        target = patchify_latents((lat.float() - noise.float())).float()                 # x0 - n
        per_chunk = lambda e: e.view(n_chunks, -1).mean(dim=1)   # noqa: E731
        if self.objective == "tf_fm":
            u = torch.rand(n_chunks, generator=self.gen, device=dev)
            t = 1.0 - flow.shifted_sigma(u, flow.VIDEO_SHIFT)
            pred = self._predict(sample, lat, noise, t)
            loss = (pred.float() - target).pow(2).mean()
        else:
            # AnyFlow on the noise level s = 1 - t (its time runs from noise, like the reference grid): the
            # network's data-ward output is negated into the noise-ward velocity
            pairs = af.sample_time_pairs(n_chunks, diffusion_ratio=self.ratios[0], consistency_ratio=self.ratios[1],
                                         generator=self.gen, device=dev)
            s = flow.shifted_sigma(pairs.t, flow.VIDEO_SHIFT)
            r = flow.shifted_sigma(pairs.r, flow.VIDEO_SHIFT)
            need_probes = bool((~pairs.is_diffusion).any())
            prefix = [] if (self.reuse_prefix and need_probes) else None
            u_pred = -self._predict(sample, lat, noise, 1.0 - s, capture=prefix).float()
            s_p, s_m = (s + self.epsilon).clamp(max=1.0), torch.maximum(s - self.epsilon, r)
            du = torch.zeros_like(u_pred)
            if need_probes:
                with torch.no_grad():
                    up = -self._predict(sample, lat, noise, 1.0 - s_p, captured=prefix).float()
                    um = -self._predict(sample, lat, noise, 1.0 - s_m, captured=prefix).float()
                    width = (s_p - s_m).clamp_min(1e-6).repeat_interleave(self.chunk_latents * rows).view(-1, 1)
                    du = (up - um) / width
            span = (s - r).repeat_interleave(self.chunk_latents * rows).view(-1, 1)
            resid = u_pred + span * du - (-target)
            chunk_loss = per_chunk(resid.pow(2).mean(dim=1))
            chunk_loss = af.adaptive_rescale(chunk_loss, pairs.is_diffusion)
            loss = chunk_loss.mean()
        return loss
