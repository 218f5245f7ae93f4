"""Renderer benchmark: case loader and the pairwise-judge harness.

Cases come from a local copy of the benchmark (two splits, one case format -- a structure video, a first frame, a
prompt; held-out clips also carry the real video):

    <root>/benchmark/hard/cases.jsonl      rows {case_id, files{prompt.txt, condition.mp4, first_frame.png}, tags, condition}
    <root>/benchmark/heldout/cases.jsonl   rows {clip_id, prompt, files{condition.mp4, first_frame.png}, ground_truth, condition}

A method's renders sit at ``<renders>/<split>/<id>.mp4``.

The judge harness asks every pair twice with the two renders in swapped positions and keeps a verdict only when the
two orders agree (one decided + one tie counts as decided; each order picking its own position is position bias and
becomes a tie).  The "judge" itself is a callable -- a VLM client in production, any function in tests; no model is
bundled.  Net preference comes with a bootstrap interval: on the hard split whole structure videos are resampled
(their cases share layout and motion), held-out clips one by one
(reference behaviour: eval/solar_renderer/bench.py:20-78, judge.py:192-300).
"""
from __future__ import annotations

import collections
import json
import random
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple


@dataclass
class Case:
    split: str                      # "hard" | "heldout"
    id: str
    prompt: str
    condition: str                  # structure video
    first_frame: str
    ground_truth: Optional[str]     # held-out clips only
    tags: List[str] = field(default_factory=list)
    kind: Optional[str] = None      # structure type

    @property
    def key(self) -> str:
        return f"{self.split}/{self.id}"

    def render(self, renders) -> Path:
        return Path(renders) / self.split / f"{self.id}.mp4"


def _rows(path: Path) -> List[dict]:
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()]


def load_cases(root, split: str = "all") -> List[Case]:
    if split not in ("hard", "heldout", "all"):
        raise ValueError("split must be hard, heldout or all")
    root = Path(root)
    out: List[Case] = []
    if split in ("hard", "all"):
        for r in _rows(root / "benchmark" / "hard" / "cases.jsonl"):
            f = r["files"]
            out.append(Case("hard", r["case_id"], (root / f["prompt.txt"]).read_text().strip(), str(root / f["condition.mp4"]),
                            str(root / f["first_frame.png"]), None, list(r.get("tags") or []), r.get("condition")))
    if split in ("heldout", "all"):
        for r in _rows(root / "benchmark" / "heldout" / "cases.jsonl"):
            f = r["files"]
            out.append(Case("heldout", r["clip_id"], r["prompt"], str(root / f["condition.mp4"]), str(root / f["first_frame.png"]),
                            str(root / r["ground_truth"]), [], r.get("condition")))
    return out


# ------------------------------------------------------------------------------------------------ judge
Judge = Callable[[Case, str, str, Sequence[str]], Mapping[str, str]]
"""``judge(case, video_in_position_A, video_in_position_B, questions) -> {question: "A" | "B" | "tie"}``"""


def debiased_verdict(first: Mapping[str, str], swapped: Mapping[str, str], question: str, a: str, b: str) -> str:
    """``first`` had method ``a`` in position A; ``swapped`` had ``b`` there.  Returns ``a``, ``b`` or ``"tie"``."""
    v = [{"A": a, "B": b}.get(first.get(question, "tie"), "tie"), {"A": b, "B": a}.get(swapped.get(question, "tie"), "tie")]
    if v[0] == v[1]:
        return v[0]
    if "tie" in v:
        return next(t for t in v if t != "tie")
    return "tie"


def judge_pairs(cases: Iterable[Case], renders_a, renders_b, judge: Judge, questions: Sequence[str],
                a: str = "a", b: str = "b") -> List[dict]:
    """One row per case: ``{"case": key, question: a | b | "tie", ...}``; cases missing either render are skipped."""
    rows = []
    for case in cases:
        va, vb = case.render(renders_a), case.render(renders_b)
        if not (va.exists() and vb.exists()):
            continue
        first = judge(case, str(va), str(vb), questions)
        swapped = judge(case, str(vb), str(va), questions)
        rows.append({"case": case.key, **{q: debiased_verdict(first, swapped, q, a, b) for q in questions}})
    return rows


def bootstrap_ci(xs: Sequence[float], groups: Optional[Sequence[str]] = None, n: int = 2000, seed: int = 0) -> Tuple[float, float, float]:
    """Mean and 95 % bootstrap interval; with ``groups`` whole groups are resampled."""
    if not xs:
        raise ValueError("no observations")
    rng = random.Random(seed)
    mean = sum(xs) / len(xs)
    if groups is None:
        draws = sorted(sum(rng.choice(xs) for _ in xs) / len(xs) for _ in range(n))
    else:
        by = collections.defaultdict(list)
        for x, g in zip(xs, groups):
            by[g].append(x)
        units = list(by.values())
        draws = []
        for _ in range(n):
            d = [x for _ in units for x in rng.choice(units)]
            draws.append(sum(d) / len(d))
        draws.sort()
    return mean, draws[int(0.025 * n)], draws[int(0.975 * n)]


def structure_segment(case_key: str) -> str:
    """``hard/<segment>__<look>`` -> the structure video it came from; a held-out clip is its own unit."""
    return case_key.split("__")[0] if case_key.startswith("hard/") else case_key


def net_preference(rows: Sequence[Mapping[str, str]], question: str, a: str = "a", b: str = "b") -> Dict[str, float]:
    """Net preference of ``a`` over ``b`` (+1 / 0 / -1 per case) with its interval and the win / tie / loss counts."""
    xs = [1 if r[question] == a else (-1 if r[question] == b else 0) for r in rows]
    keys = [r["case"] for r in rows]
    if keys and all(k.startswith("hard/") for k in keys):
        mean, lo, hi = bootstrap_ci(xs, [structure_segment(k) for k in keys], n=2000)
    else:
        mean, lo, hi = bootstrap_ci(xs, n=10000)
    return {"net": mean, "lo": lo, "hi": hi, "wins": xs.count(1), "ties": xs.count(0), "losses": xs.count(-1), "cases": len(xs)}
