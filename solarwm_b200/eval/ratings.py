"""Pairwise-judgement ratings.

``pair_verdict`` folds the two presentation orders of one comparison into a winner or a tie (a
judge that follows the slot rather than the content produces contradicting answers, which count as
a tie).  ``fit_bradley_terry`` estimates strengths by minorisation-maximisation with one virtual tie
per method against a fixed reference of strength 1 (keeps undefeated methods finite) and reports
them on the Elo scale with the mean of the rated methods at 1000
(reference: eval/solar_renderer/elo.py:31-81, judge.py).
"""
from __future__ import annotations

import collections
import math
from typing import Dict, Iterable, Optional, Sequence, Tuple


def pair_verdict(first_order_answer: str, swapped_order_answer: str, a: str, b: str) -> Optional[str]:
    """Answers are "1" / "2" / "tie" for the clip shown first / second.  Returns a, b or None (tie)."""
    def who(ans, first, second):
        return first if ans == "1" else second if ans == "2" else None

    x, y = who(first_order_answer, a, b), who(swapped_order_answer, b, a)
    return x if x == y else None


def fit_bradley_terry(games: Iterable[Tuple[str, str, Optional[str]]], *, iterations: int = 2000,
                      tolerance: float = 1e-7) -> Dict[str, float]:
    """games: (a, b, winner-or-None).  Returns Elo-scale ratings."""
    games = list(games)
    methods = sorted({g[0] for g in games} | {g[1] for g in games})
    wins, n = collections.Counter(), collections.Counter()
    for a, b, w in games:
        n[a, b] += 1
        if w == a:
            wins[a, b] += 1
        elif w == b:
            wins[b, a] += 1
        else:
            wins[a, b] += 0.5
            wins[b, a] += 0.5
    p = {m: 1.0 for m in methods}
    for _ in range(iterations):
        new = {}
        for i in methods:
            w = sum(wins[i, j] for j in methods if j != i) + 0.5
            d = sum((n[i, j] + n[j, i]) / (p[i] + p[j]) for j in methods if j != i) + 1.0 / (p[i] + 1.0)
            new[i] = w / d
        step = max(abs(math.log(new[m] / p[m])) for m in methods)
        p = new
        if step < tolerance:
            break
    g = math.exp(sum(math.log(v) for v in p.values()) / len(p))
    return {m: 1000.0 + 400.0 * math.log10(p[m] / g) for m in methods}


def win_rates(games: Sequence[Tuple[str, str, Optional[str]]]) -> Dict[str, float]:
    score, count = collections.Counter(), collections.Counter()
    for a, b, w in games:
        for m in (a, b):
            count[m] += 1
        if w is None:
            score[a] += 0.5
            score[b] += 0.5
        else:
            score[w] += 1
    return {m: score[m] / count[m] for m in count}
