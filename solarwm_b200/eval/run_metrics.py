"""Run the metric suite over a benchmark's renders, resumably, and summarise methods.

    python -m solarwm_b200.eval.run_metrics compute --root BENCH --renders DIR --method NAME --out SCORES
                                                    [--metrics flicker,edges,motion,gt] [--split all]
    python -m solarwm_b200.eval.run_metrics summary --out SCORES --methods a,b [--split all]

``compute`` writes one JSON per (metric, method, case) under ``<out>/<metric>/<method>/<split>/<id>.json`` through a
temporary name, and skips the ones that are already there, so an interrupted pass continues where it stopped and two
workers can split the cases (``--shard i --shards n``).  A case whose render is missing is listed, not fatal.  ``summary``
reads the readings back, averages each over the cases every listed method has (methods are compared on common cases
only), maps them to 0..100 scales and averages the groups (stability, structure, fidelity) into one score per method.

Reference: eval/solar_renderer/metrics.py:525-664 (compute / result_path / main), summary.py:51-140.
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
from typing import Callable, Dict, List, Mapping, Optional, Sequence

import numpy as np

from .benchmark import Case, load_cases

# reading -> (metric file, how to take it from the JSON, group, map to 0..100)
READINGS = {
    "warp_l1_lp": ("flicker", lambda j: j["warp_l1_lp"], "stability", lambda x: 100 * max(0.0, 1 - x / 10)),
    "motion_err": ("motion", lambda j: j["err_mean"], "structure", lambda x: 100 * max(0.0, 1 - x / 0.5)),
    "edge_f1": ("edges", lambda j: j["F1"], "structure", lambda x: 100 * x),
    "ssim": ("gt", lambda j: j["ssim"], "fidelity", lambda x: 100 * max(0.0, x)),
    "psnr": ("gt", lambda j: j["psnr"], "fidelity", lambda x: 100 * min(1.0, max(0.0, x / 40.0))),
}
GROUPS = ("stability", "structure", "fidelity")


def read_video(path, size=None) -> np.ndarray:
    import cv2

    cap = cv2.VideoCapture(str(path))
    frames = []
    try:
        while True:
            ok, f = cap.read()
            if not ok:
                break
            f = cv2.cvtColor(f, cv2.COLOR_BGR2RGB)
            frames.append(f if size is None else cv2.resize(f, size, interpolation=cv2.INTER_AREA))
    finally:
        cap.release()
    if not frames:
        raise FileNotFoundError(path)
    return np.stack(frames)


def result_path(out, metric: str, method: str, case: Case) -> Path:
    return Path(out) / metric / method / case.split / f"{case.id}.json"


def _metric_fns() -> Dict[str, Callable[[Case, np.ndarray], Optional[Mapping]]]:
    import torch

    from . import metrics as M
    from . import motion

    def flicker(case, render):
        return motion.flow_flicker(render)

    def edges(case, render):
        cond = read_video(case.condition, size=(render.shape[2], render.shape[1]))
        return motion.structure_edges(render, cond)

    def mot(case, render):
        cond = read_video(case.condition, size=(render.shape[2], render.shape[1]))
        n = min(len(cond), len(render))
        return motion.motion_compare(motion.track_grid(cond[:n]), motion.track_grid(render[:n]), (render.shape[2], render.shape[1]))

    def gt(case, render):
        if not case.ground_truth:
            return None
        real = read_video(case.ground_truth, size=(render.shape[2], render.shape[1]))
        n = min(len(real), len(render))
        to = lambda v: torch.from_numpy(v[:n].astype(np.float32) / 255.0).permute(0, 3, 1, 2)      # noqa: E731
        return M.compute(to(render), to(real))

    return {"flicker": flicker, "edges": edges, "motion": mot, "gt": gt}


def compute(root, renders, method: str, out, *, metrics: Sequence[str] = ("flicker", "edges", "motion", "gt"), split: str = "all",
            shard: int = 0, shards: int = 1, scorers=None, max_frames: Optional[int] = None) -> Mapping[str, object]:
    fns = _metric_fns()
    unknown = [m for m in metrics if m not in fns and not (scorers is not None and m in scorers.names())]
    if unknown:
        raise ValueError(f"unknown metrics {unknown}")
    done, skipped, missing = 0, 0, []
    for case in load_cases(root, split)[shard::shards]:
        video = case.render(renders)
        todo = [m for m in metrics if not result_path(out, m, method, case).is_file()]
        skipped += len(metrics) - len(todo)
        if not todo:
            continue
        if not video.is_file():
            missing.append(case.key)
            continue
        render = read_video(video)[:max_frames]
        for m in todo:
            value = fns[m](case, render) if m in fns else scorers.score(m, render, {"prompt": case.prompt, "key": case.key})
            if value is None:
                continue
            target = result_path(out, m, method, case)
            target.parent.mkdir(parents=True, exist_ok=True)
            tmp = target.with_name(f".{target.name}.{os.getpid()}.tmp")
            tmp.write_text(json.dumps({**dict(value), "case": case.key, "tags": case.tags, "kind": case.kind}, sort_keys=True))
            os.replace(tmp, target)
            done += 1
    return {"written": done, "skipped": skipped, "missing_renders": missing}


def load_readings(out, method: str, split: str = "all") -> Dict[str, Dict[str, float]]:
    """case key -> reading -> value, for the readings whose files exist and hold a number."""
    got: Dict[str, Dict[str, float]] = {}
    for name, (metric, take, _, _) in READINGS.items():
        base = Path(out) / metric / method
        for p in (base.rglob("*.json") if base.exists() else []):
            rel = p.relative_to(base).with_suffix("").as_posix()
            if split != "all" and not rel.startswith(split + "/"):
                continue
            try:
                v = take(json.loads(p.read_text()))
            except (KeyError, TypeError, ValueError):
                continue
            if v is not None:
                got.setdefault(rel, {})[name] = float(v)
    return got


def summarise(out, methods: Sequence[str], split: str = "all") -> Mapping[str, object]:
    per = {m: load_readings(out, m, split) for m in methods}
    table = {}
    for name, (_, _, group, scale) in READINGS.items():
        common = set.intersection(*[{k for k, v in per[m].items() if name in v} for m in methods]) if methods else set()
        if not common:
            continue
        for m in methods:
            mean = float(np.mean([per[m][k][name] for k in sorted(common)]))
            table.setdefault(m, {})[name] = {"mean": mean, "scaled": scale(mean), "cases": len(common), "group": group}
    ranking = []
    for m, rows in table.items():
        groups = {g: [r["scaled"] for r in rows.values() if r["group"] == g] for g in GROUPS}
        groups = {g: float(np.mean(v)) for g, v in groups.items() if v}
        ranking.append({"method": m, "score": float(np.mean(list(groups.values()))) if groups else None, **groups})
    ranking.sort(key=lambda r: -(r["score"] or -1))
    return {"readings": table, "ranking": ranking}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="solar-eval-metrics")
    ap.add_argument("command", choices=["compute", "summary"])
    ap.add_argument("--root")
    ap.add_argument("--renders")
    ap.add_argument("--method")
    ap.add_argument("--methods", default="")
    ap.add_argument("--out", required=True)
    ap.add_argument("--metrics", default="flicker,edges,motion,gt")
    ap.add_argument("--split", default="all")
    ap.add_argument("--shard", type=int, default=0)
    ap.add_argument("--shards", type=int, default=1)
    args = ap.parse_args(argv)
    if args.command == "compute":
        if not (args.root and args.renders and args.method):
            ap.error("compute needs --root, --renders and --method")
        print(json.dumps(compute(args.root, args.renders, args.method, args.out, metrics=tuple(args.metrics.split(",")),
                                 split=args.split, shard=args.shard, shards=args.shards), sort_keys=True))
    else:
        print(json.dumps(summarise(args.out, [m for m in args.methods.split(",") if m], args.split), sort_keys=True, indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
