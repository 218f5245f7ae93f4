"""Optimizer-step state machine shared by every backend.

One step = zero_grad -> ``grad_accum`` x (train_microbatch, SP-peer identity check) ->
prepare_optimizer_step (gradient sync / clip; must report a finite norm) -> optimizer_step ->
scheduler_step -> set_global_step -> ema_update -> zero_grad -> JSONL event -> optional checkpoint
and validation.  A failing microbatch or a non-finite gradient leaves optimizer, EMA, step counter
and checkpoints untouched.  The cyclic garbage collector is paused inside the loop and run at
checkpoint/validation boundaries (reference: solar/training/engine.py:18-252).
"""
from __future__ import annotations

import gc
import json
import math
import os
from contextlib import contextmanager
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable, Mapping, Protocol, Sequence

from ..errors import BackendContractError

STEP_SCHEMA = "solarwm.training-step.v1"
EVENT_SCHEMA = "solarwm.training-event.v1"


@dataclass(frozen=True)
class BatchIdentity:
    sample_ids: tuple
    start_frames: tuple
    noise_seeds: tuple
    checkpoint_id: str
    plan_fingerprint: str

    def __post_init__(self):
        n = len(self.sample_ids)
        if n < 1:
            raise BackendContractError("microbatch identity has no samples")
        if len(self.start_frames) != n or len(self.noise_seeds) != n:
            raise BackendContractError("microbatch identity fields have different lengths")
        if not self.checkpoint_id or not self.plan_fingerprint:
            raise BackendContractError("microbatch identity lacks checkpoint/plan identity")


@dataclass(frozen=True)
class MicrobatchResult:
    identity: BatchIdentity
    losses: Mapping[str, float]

    def __post_init__(self):
        if not self.losses:
            raise BackendContractError("microbatch produced no loss fields")
        for name, value in self.losses.items():
            if not name or isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value):
                raise BackendContractError(f"non-finite or invalid loss {name!r}: {value!r}")


@dataclass(frozen=True)
class GradientStatus:
    finite: bool
    norm: float

    def __post_init__(self):
        if self.finite and not math.isfinite(self.norm):
            raise BackendContractError("finite gradients reported a non-finite norm")


@dataclass(frozen=True)
class StepPolicy:
    max_steps: int
    grad_accum: int = 1
    save_every: int = 0
    validate_every: int = 0
    validation_steps: tuple = ()
    save_steps: tuple = ()

    def __post_init__(self):
        if self.max_steps < 1 or self.grad_accum < 1:
            raise BackendContractError("max_steps and grad_accum must be positive")
        if self.save_every < 0 or self.validate_every < 0:
            raise BackendContractError("save/validate intervals must be non-negative")
        if any(s < 1 for s in (*self.validation_steps, *self.save_steps)):
            raise BackendContractError("validation_steps must be positive")

    def should_save(self, step: int) -> bool:
        return step in self.save_steps or bool(self.save_every and step % self.save_every == 0)

    def should_validate(self, step: int) -> bool:
        return step in self.validation_steps or bool(self.validate_every and step % self.validate_every == 0)


class TrainingRuntime(Protocol):
    @property
    def global_step(self) -> int: ...
    def zero_grad(self) -> None: ...
    def train_microbatch(self, micro_index: int, grad_accum: int) -> MicrobatchResult: ...
    def assert_sp_peer_identity(self, identity: BatchIdentity) -> None: ...
    def prepare_optimizer_step(self) -> GradientStatus: ...
    def optimizer_step(self) -> None: ...
    def scheduler_step(self) -> None: ...
    def ema_update(self, step: int) -> None: ...
    def set_global_step(self, step: int) -> None: ...
    def save_checkpoint(self, step: int) -> str: ...
    def validate(self, step: int) -> Mapping[str, Any]: ...


@contextmanager
def paused_cycle_collection():
    was_on = gc.isenabled()
    if was_on:
        gc.disable()
    try:
        yield
    finally:
        if was_on:
            gc.enable()


class JsonlEventSink:
    """Appends one canonical JSON line per event with a single O_APPEND write."""

    def __init__(self, path):
        self.path = Path(path)
        self.path.parent.mkdir(parents=True, exist_ok=True)

    def __call__(self, event: Mapping[str, Any]) -> None:
        try:
            line = json.dumps(event, allow_nan=False, ensure_ascii=False, separators=(",", ":"), sort_keys=True) + "\n"
        except (TypeError, ValueError) as exc:
            raise BackendContractError(f"invalid training event: {exc}") from exc
        fd = os.open(self.path, os.O_APPEND | os.O_CREAT | os.O_WRONLY, 0o644)
        try:
            os.write(fd, line.encode())
        finally:
            os.close(fd)


def mean_losses(results: Sequence[MicrobatchResult]) -> dict:
    names = set(results[0].losses)
    if any(set(r.losses) != names for r in results):
        raise BackendContractError("loss fields changed inside one optimizer step")
    return {n: sum(float(r.losses[n]) for r in results) / len(results) for n in sorted(names)}


class TrainingEngine:
    def __init__(self, runtime: TrainingRuntime, policy: StepPolicy, *, event_sink: Callable[[Mapping], None] = None):
        self.runtime, self.policy = runtime, policy
        self.event_sink = event_sink or (lambda event: None)

    def run(self) -> int:
        with paused_cycle_collection():
            while self.runtime.global_step < self.policy.max_steps:
                self.step()
        return self.runtime.global_step

    def step(self) -> None:
        if os.environ.get("SOLAR_PHASE_TIMES", "0") == "1":
            from ..utils.trace import PhaseTimer

            timer = PhaseTimer()
            with timer.installed():
                self._step(timer)
        else:
            self._step(None)

    def _step(self, timer) -> None:
        rt, policy = self.runtime, self.policy
        target = rt.global_step + 1
        rt.zero_grad()
        done = []
        try:
            for micro in range(policy.grad_accum):
                result = rt.train_microbatch(micro, policy.grad_accum)
                rt.assert_sp_peer_identity(result.identity)
                done.append(result)
        except Exception:
            rt.zero_grad()
            raise
        from ..utils.trace import span

        with span("optimizer"):
            status = rt.prepare_optimizer_step()
            if not status.finite or not math.isfinite(status.norm):
                rt.zero_grad()
                raise BackendContractError(f"non-finite gradients before optimizer step {target}: {status.norm}")
            rt.optimizer_step()
        rt.scheduler_step()
        rt.set_global_step(target)
        rt.ema_update(target)
        rt.zero_grad()
        self.event_sink({
            "schema": STEP_SCHEMA, "event": "optimizer_step", "step": target, "grad_accum": policy.grad_accum,
            "gradient_norm": status.norm, "losses": mean_losses(done),
            **({} if timer is None else {"phase_ms": {k: v["total_ms"] for k, v in timer.summary().items()
                                                      if not k.startswith("block.")}}),
            "microbatches": [{"identity": asdict(r.identity), "losses": dict(r.losses)} for r in done]})
        boundary = False
        if policy.should_save(target):
            ident = rt.save_checkpoint(target)
            if not ident:
                raise BackendContractError("checkpoint hook returned an empty identity")
            self.event_sink({"schema": EVENT_SCHEMA, "event": "checkpoint", "step": target, "checkpoint_id": ident})
            boundary = True
        if policy.should_validate(target):
            report = rt.validate(target)
            self.event_sink({"schema": EVENT_SCHEMA, "event": "validation", "step": target, "report": dict(report)})
            boundary = True
        if boundary:
            gc.collect()
