"""Phase tracing: NVTX ranges for a profiler timeline and CUDA-event phase timers for plain runs.

Both are off unless asked for, and an inactive ``span`` costs one attribute test:

* ``SOLAR_NVTX=1`` (or ``enable_nvtx(True)``): ``span("block.07")`` pushes / pops an NVTX range, so a captured
  timeline shows steps, forward / backward / optimizer phases and transformer blocks by name;
* ``PhaseTimer``: ``with timer.phase("forward"): ...`` brackets the phase with CUDA events on the current stream (host
  clock on CPU); ``summary()`` synchronises once and returns mean / total milliseconds per phase -- the phase split
  the trainers' step events carry when ``SOLAR_PHASE_TIMES=1``.

The reference has no tracing layer (timing is ``perf_counter`` around synchronisations); the counters it does keep
("did the fused path run") live in ``ops._lib.COUNTERS``.
"""
from __future__ import annotations

import contextlib
import os
import time
from typing import Dict, List, Optional, Tuple

import torch

_NVTX = os.environ.get("SOLAR_NVTX", "0") == "1"
_ACTIVE_TIMER: Optional["PhaseTimer"] = None


def enable_nvtx(on: bool) -> bool:
    """Returns the previous setting."""
    global _NVTX
    previous, _NVTX = _NVTX, bool(on)
    return previous


def nvtx_enabled() -> bool:
    return _NVTX and torch.cuda.is_available()


class _Span:
    __slots__ = ("name", "pushed", "phase")

    def __init__(self, name: str):
        self.name, self.pushed, self.phase = name, False, None

    def __enter__(self):
        if _NVTX and torch.cuda.is_available():
            torch.cuda.nvtx.range_push(self.name)
            self.pushed = True
        if _ACTIVE_TIMER is not None:
            self.phase = _ACTIVE_TIMER.phase(self.name)
            self.phase.__enter__()
        return self

    def __exit__(self, *exc):
        if self.phase is not None:
            self.phase.__exit__(*exc)
        if self.pushed:
            torch.cuda.nvtx.range_pop()
        return False


_NULL = contextlib.nullcontext()


def span(name: str):
    """A named range: NVTX when enabled, a timed phase when a ``PhaseTimer`` is installed, else nothing."""
    if not _NVTX and _ACTIVE_TIMER is None:
        return _NULL
    return _Span(name)


class PhaseTimer:
    """Per-phase durations measured on the device (CUDA events on the current stream) without a synchronisation
    per phase; ``summary`` synchronises once."""

    def __init__(self, device=None):
        dev = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.cuda = dev.type == "cuda"
        self._events: Dict[str, List[Tuple[object, object]]] = {}
        self._host: Dict[str, List[float]] = {}

    @contextlib.contextmanager
    def phase(self, name: str):
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._events.setdefault(name, []).append((a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._host.setdefault(name, []).append((time.perf_counter() - t0) * 1e3)

    @contextlib.contextmanager
    def installed(self):
        """Route every ``span`` in the code under this context into the timer."""
        global _ACTIVE_TIMER
        previous, _ACTIVE_TIMER = _ACTIVE_TIMER, self
        try:
            yield self
        finally:
            _ACTIVE_TIMER = previous

    def summary(self) -> Dict[str, Dict[str, float]]:
        if self.cuda:
            torch.cuda.synchronize()
            for name, pairs in self._events.items():
                self._host.setdefault(name, []).extend(a.elapsed_time(b) for a, b in pairs)
            self._events.clear()
        return {name: {"count": len(v), "total_ms": round(sum(v), 4), "mean_ms": round(sum(v) / len(v), 4)}
                for name, v in self._host.items() if v}
