"""Temporal and structural video metrics that need no learned weights, plus the registry for the ones that do.

  flow_flicker      warp frame t+1 onto frame t along the forward optical flow and measure what does not match, on the
                    pixels whose forward and backward flows agree (|f + b(x + f)|^2 < 0.01 (|f|^2 + |b|^2) + 0.5).  Read
                    raw (``warp_l1``) and after a Gaussian low-pass of the residual (``warp_l1_lp``: sub-pixel misalignment
                    of fine texture cancels, brightness / colour flicker stays), with the Laplacian-variance sharpness
                    beside them since the raw reading rises with sharpness.  The flow comes from ``flow_fn`` (default:
                    OpenCV's Farneback flow; a learned estimator can be passed in).
  edge_f1           Canny edges of the render against those of the conditioning clip; an edge counts as found when the
                    other side has one within ``tolerance`` pixels.  Precision, recall, F1, every 4th frame.
  motion_compare    point tracks of the conditioning clip against tracks of the render from the same query points: position
                    and velocity error in units of the frame diagonal, on the (point, frame) pairs where the conditioning
                    track is reliable, with the "frozen render" baseline (every track stays at its query) for scale.
                    ``track_grid`` is a pyramidal Lucas-Kanade tracker over a grid re-seeded every 40 frames; a learned
                    tracker with the same output can be passed in.
  Scorers           named model-based scorers (perceptual quality, text-video score, embedding consistency) register a
                    loader; a scorer whose weights cannot be loaded reports ``{"unavailable": why}`` instead of failing the
                    run, so a metrics pass over a benchmark completes with what the machine has.

Reference: eval/solar_renderer/metrics.py:298-508 (flows, warp, m_flicker, track, motion_compare, canny, edge_errors).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

QUERY_FRAMES = (0, 40, 80, 120)
GRID = (20, 12)                     # points along x, y
RELIABLE = 0.6


# ---------------------------------------------------------------------------------------------------------------------
# optical flow and flicker
# ---------------------------------------------------------------------------------------------------------------------
def farneback_flows(frames: np.ndarray) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """RGB8 [T, H, W, 3] -> (frames in [-1, 1] [T, 3, H, W], forward flow [T-1, 2, H, W], backward flow [T-1, 2, H, W])."""
    import cv2

    gray = [cv2.cvtColor(f, cv2.COLOR_RGB2GRAY) for f in frames]
    args = dict(pyr_scale=0.5, levels=4, winsize=21, iterations=3, poly_n=7, poly_sigma=1.5, flags=0)
    fw = [cv2.calcOpticalFlowFarneback(a, b, None, **args) for a, b in zip(gray[:-1], gray[1:])]
    bw = [cv2.calcOpticalFlowFarneback(b, a, None, **args) for a, b in zip(gray[:-1], gray[1:])]
    x = torch.from_numpy(frames.astype(np.float32) / 127.5 - 1.0).permute(0, 3, 1, 2)
    to = lambda v: torch.from_numpy(np.stack(v)).permute(0, 3, 1, 2).float()                   # noqa: E731
    return x, to(fw), to(bw)


def warp(img: torch.Tensor, flow: torch.Tensor):
    """Sample ``img`` [N, C, H, W] at x + flow(x) (pixels).  Returns the warped image and the in-bounds mask."""
    _, _, h, w = img.shape
    yy, xx = torch.meshgrid(torch.arange(h, device=img.device), torch.arange(w, device=img.device), indexing="ij")
    gx, gy = xx[None] + flow[:, 0], yy[None] + flow[:, 1]
    grid = torch.stack([2 * gx / (w - 1) - 1, 2 * gy / (h - 1) - 1], dim=-1)
    out = F.grid_sample(img, grid, mode="bilinear", padding_mode="border", align_corners=True)
    return out, (gx >= 0) & (gx <= w - 1) & (gy >= 0) & (gy <= h - 1)


def _gauss_blur(z: torch.Tensor, sigma: float = 2.0, radius: int = 6) -> torch.Tensor:
    k = torch.exp(-0.5 * (torch.arange(-radius, radius + 1, device=z.device).float() / sigma) ** 2)
    k = k / k.sum()
    c = z.shape[1]
    z = F.conv2d(F.pad(z, (radius, radius, 0, 0), mode="replicate"), k.view(1, 1, 1, -1).repeat(c, 1, 1, 1), groups=c)
    return F.conv2d(F.pad(z, (0, 0, radius, radius), mode="replicate"), k.view(1, 1, -1, 1).repeat(c, 1, 1, 1), groups=c)


@torch.no_grad()
def flow_flicker(frames: np.ndarray, flow_fn: Callable = farneback_flows) -> Dict[str, float]:
    x, fw, bw = flow_fn(frames)
    now, nxt = x[:-1], x[1:]
    warped, inside = warp(nxt, fw)
    back_there = warp(bw, fw)[0]
    disagreement = ((fw + back_there) ** 2).sum(1)
    ok = (inside & (disagreement < 0.01 * ((fw ** 2).sum(1) + (back_there ** 2).sum(1)) + 0.5)).float()
    residual = now - warped
    per_pair = ((residual.abs().mean(1) * 127.5) * ok).sum((1, 2)) / ok.sum((1, 2)).clamp(min=1)
    m = ok[:, None]
    weight = _gauss_blur(m)
    low = (_gauss_blur(residual * m) / weight.clamp(min=1e-3)).abs().mean(1) * 127.5
    valid = ok * (weight[:, 0] > 0.5)
    low_pair = (low * valid).sum((1, 2)) / valid.sum((1, 2)).clamp(min=1)
    g = (0.299 * x[:, 0] + 0.587 * x[:, 1] + 0.114 * x[:, 2]) * 127.5
    lap = -4 * g[:, 1:-1, 1:-1] + g[:, :-2, 1:-1] + g[:, 2:, 1:-1] + g[:, 1:-1, :-2] + g[:, 1:-1, 2:]
    pp, lp = per_pair.numpy(), low_pair.numpy()
    return {"warp_l1": float(pp.mean()), "warp_l1_p90": float(np.percentile(pp, 90)), "warp_l1_max": float(pp.max()),
            "warp_l1_lp": float(lp.mean()), "warp_l1_lp_p90": float(np.percentile(lp, 90)),
            "sharpness_lapvar": float(lap.flatten(1).var(1).mean()), "consistent_frac": float(ok.mean()),
            "flow_mag": float(fw.norm(dim=1).mean()), "pairs": int(len(pp))}


# ---------------------------------------------------------------------------------------------------------------------
# structure: edges
# ---------------------------------------------------------------------------------------------------------------------
def canny_edges(frames: np.ndarray) -> np.ndarray:
    import cv2

    return np.stack([cv2.Canny(cv2.GaussianBlur(cv2.cvtColor(f, cv2.COLOR_RGB2GRAY), (5, 5), 1.2), 50, 150) for f in frames])


def edge_f1(made: np.ndarray, want: np.ndarray, tolerance: int = 2, level: int = 64) -> Dict[str, float]:
    n = min(len(made), len(want))
    found = torch.from_numpy(np.ascontiguousarray(made[:n]) >= level).float()[:, None]
    given = torch.from_numpy(np.ascontiguousarray(want[:n]) >= level).float()[:, None]
    near = lambda e: F.max_pool2d(e, 2 * tolerance + 1, stride=1, padding=tolerance)          # noqa: E731
    precision = float((found * near(given)).sum()) / max(float(found.sum()), 1.0)
    recall = float((given * near(found)).sum()) / max(float(given.sum()), 1.0)
    f1 = 2 * precision * recall / (precision + recall) if precision + recall > 0 else 0.0
    return {"F1": f1, "precision": precision, "recall": recall, "frames": n}


def structure_edges(render: np.ndarray, condition: np.ndarray, every: int = 4) -> Dict[str, float]:
    r, c = render[::every], condition[::every]
    n = min(len(r), len(c))
    want = canny_edges(c[:n])
    out = edge_f1(canny_edges(r[:n]), want)
    out["cond_edge_density"] = float((want > 0).mean())
    return out


# ---------------------------------------------------------------------------------------------------------------------
# motion: point tracks
# ---------------------------------------------------------------------------------------------------------------------
def track_grid(frames: np.ndarray, query_frames: Sequence[int] = QUERY_FRAMES, grid: Tuple[int, int] = GRID):
    """Pyramidal Lucas-Kanade tracks of a grid seeded at every query frame.  Returns tracks [T, N, 2] (pixels), visibility
    and confidence [T, N], the query points [N, 2] and their query frames [N]; a track before its query frame sits at
    the query point with zero confidence."""
    import cv2

    T, H, W, _ = frames.shape
    gray = [cv2.cvtColor(f, cv2.COLOR_RGB2GRAY) for f in frames]
    gx, gy = (np.arange(grid[0]) + 0.5) / grid[0] * W, (np.arange(grid[1]) + 0.5) / grid[1] * H
    seeds = np.array([(x, y) for y in gy for x in gx], np.float32)
    starts = [t for t in query_frames if t < T - 1]
    pts = np.concatenate([seeds] * len(starts))
    qt = np.repeat(np.array(starts), len(seeds))
    tracks = np.tile(pts[None], (T, 1, 1)).astype(np.float32)
    vis, conf = np.zeros((T, len(pts)), np.float32), np.zeros((T, len(pts)), np.float32)
    lk = dict(winSize=(21, 21), maxLevel=3, criteria=(cv2.TERM_CRITERIA_EPS | cv2.TERM_CRITERIA_COUNT, 30, 0.01))
    for s, t0 in enumerate(starts):
        sl = slice(s * len(seeds), (s + 1) * len(seeds))
        cur, alive = seeds.copy().reshape(-1, 1, 2), np.ones(len(seeds), bool)
        vis[t0, sl] = conf[t0, sl] = 1.0
        for t in range(t0 + 1, T):
            nxt, status, err = cv2.calcOpticalFlowPyrLK(gray[t - 1], gray[t], cur, None, **lk)
            back, status_b, _ = cv2.calcOpticalFlowPyrLK(gray[t], gray[t - 1], nxt, None, **lk)
            round_trip = np.linalg.norm((back - cur).reshape(-1, 2), axis=1)
            inside = (nxt[:, 0, 0] >= 0) & (nxt[:, 0, 0] < W) & (nxt[:, 0, 1] >= 0) & (nxt[:, 0, 1] < H)
            alive &= (status.ravel() == 1) & (status_b.ravel() == 1) & inside
            tracks[t, sl] = nxt.reshape(-1, 2)
            vis[t, sl] = alive
            conf[t, sl] = alive * np.exp(-round_trip)                # 1 for a perfect round trip, falling with its error
            cur = nxt
    return tracks, vis, conf, pts, qt


def motion_compare(cond, render, frame_size: Tuple[int, int]) -> Dict[str, object]:
    """``cond`` / ``render``: the 5-tuples of ``track_grid`` (or a learned tracker) from the SAME query points."""
    tc, vc, cc, pts, qt = cond
    tm, vm, cm, _, _ = render
    W, H = frame_size
    diag = math.hypot(W, H)
    n = min(len(tc), len(tm))
    t = np.arange(n)[:, None]
    after = t > qt[None]
    reliable = ((vc[:n] * cc[:n]) > RELIABLE) & after
    if reliable.sum() == 0:
        return {"kept_frac": 0.0, "err_mean": None}
    err = np.linalg.norm(tm[:n] - tc[:n], axis=-1) / diag
    frozen = np.linalg.norm(tc[:n] - pts[None], axis=-1) / diag
    start_ok = (((vc[:n - 1] * cc[:n - 1]) > RELIABLE) & (t[:-1] > qt[None])) | (t[:-1] == qt[None])
    vel_ok = reliable[1:] & start_ok
    vel_err = np.linalg.norm((tm[1:n] - tm[:n - 1]) - (tc[1:n] - tc[:n - 1]), axis=-1) / diag
    return {"err_mean": float(err[reliable].mean()), "err_median": float(np.median(err[reliable])),
            "frac_lt_2pct": float((err[reliable] < 0.02).mean()),
            "vel_err_mean": float(vel_err[vel_ok].mean()) if vel_ok.any() else None,
            "frozen_err_mean": float(frozen[reliable].mean()), "frozen_frac_lt_2pct": float((frozen[reliable] < 0.02).mean()),
            "kept_frac": float(reliable.sum() / max(after.sum(), 1)), "kept_pairs": int(reliable.sum()),
            "kept_frac_by_query": [round(float(reliable[:, qt == q].sum() / max(after[:, qt == q].sum(), 1)), 3) for q in np.unique(qt)],
            "render_reliable_frac": float(((vm[:n] * cm[:n]) > RELIABLE)[reliable].mean()), "frames": int(n)}


# ---------------------------------------------------------------------------------------------------------------------
# model-based scorers
# ---------------------------------------------------------------------------------------------------------------------
class Scorers:
    """``register(name, loader)``: ``loader()`` returns ``score(frames RGB8 [T, H, W, 3], case) -> mapping`` or raises when
    its weights are not on this machine.  Loaded scorers are kept; failures are remembered and reported per call."""

    def __init__(self):
        self._loaders: Dict[str, Callable[[], Callable]] = {}
        self._ready: Dict[str, Callable] = {}
        self._failed: Dict[str, str] = {}

    def register(self, name: str, loader: Callable[[], Callable]) -> None:
        if name in self._loaders:
            raise ValueError(f"scorer {name!r} is already registered")
        self._loaders[name] = loader

    def names(self):
        return sorted(self._loaders)

    def score(self, name: str, frames: np.ndarray, case: Optional[Mapping] = None) -> Mapping[str, object]:
        if name not in self._loaders:
            raise KeyError(name)
        if name not in self._ready and name not in self._failed:
            try:
                self._ready[name] = self._loaders[name]()
            except Exception as exc:  # noqa: BLE001 - missing weights or libraries: the run goes on without this scorer
                self._failed[name] = f"{type(exc).__name__}: {exc}"
        if name in self._failed:
            return {"unavailable": self._failed[name]}
        return dict(self._ready[name](frames, case))
