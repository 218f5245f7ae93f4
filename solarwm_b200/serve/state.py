"""Session state machine of the realtime server: idle -> preparing -> ready -> running -> stopped,
a command queue consumed by the worker loop, and the JSON snapshot served at ``/state``
(reference: deploy/solar_wm/shared/state.py, worker command loop worker.py:253-300)."""
from __future__ import annotations

import queue
import threading
import time
from typing import Optional

PHASES = ("idle", "preparing", "ready", "running", "stopped", "failed")
COMMANDS = ("prepare", "start", "chunk", "stop", "shutdown")


class SessionState:
    def __init__(self):
        self.lock = threading.Lock()
        self.phase = "idle"
        self.commands: "queue.Queue[dict]" = queue.Queue()
        self.chunks = []
        self.error: Optional[str] = None
        self.started = time.time()

    def submit(self, op: str, **payload) -> None:
        if op not in COMMANDS:
            raise ValueError(f"unknown command {op!r}")
        self.commands.put({"op": op, **payload})

    def next_command(self, timeout: float = 0.05) -> dict:
        try:
            return self.commands.get(timeout=timeout)
        except queue.Empty:
            return {"op": "chunk"} if self.phase == "running" else {"op": "idle"}

    def set_phase(self, phase: str, error: Optional[str] = None) -> None:
        if phase not in PHASES:
            raise ValueError(phase)
        with self.lock:
            self.phase, self.error = phase, error

    def generated(self, index: int, dit_ms: float, vae_ms: float) -> None:
        with self.lock:
            self.chunks.append({"index": index, "dit_ms": dit_ms, "vae_ms": vae_ms})

    def snapshot(self) -> dict:
        with self.lock:
            last = self.chunks[-8:]
            return {"phase": self.phase, "error": self.error, "chunks": len(self.chunks), "recent": last,
                    "uptime_s": time.time() - self.started}
