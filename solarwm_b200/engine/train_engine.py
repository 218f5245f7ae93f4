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


@dataclass
class StepRecord:
    """What one optimizer step produced, filled in phase by phase; ``event`` is its JSONL form."""

    step: int
    grad_accum: int
    microbatches: list
    gradient_norm: float = float("nan")
    phase_ms: Mapping[str, float] = None

    def event(self) -> dict:
        out = {"schema": STEP_SCHEMA, "event": "optimizer_step", "step": self.step, "grad_accum": self.grad_accum,
               "gradient_norm": self.gradient_norm, "losses": mean_losses(self.microbatches),
               "microbatches": [{"identity": asdict(r.identity), "losses": dict(r.losses)} for r in self.microbatches]}
        if self.phase_ms is not None:
            out["phase_ms"] = dict(self.phase_ms)
        return out


class TrainingEngine:
    """Drives a ``TrainingRuntime`` through optimizer steps.  A step is four phases run in a fixed order --
    ``_accumulate`` (microbatches + peer identity), ``_update`` (gradient preparation, finite check, optimizer),
    ``_advance`` (schedule, step counter, EMA) and ``_boundaries`` (checkpoint / validation when the policy says so) --
    and one JSONL record.  The ORDER of the runtime hooks inside the phases is the protocol every backend relies on;
    a failure in ``_accumulate`` or a non-finite norm in ``_update`` clears the gradients and leaves optimizer, EMA,
    counter and checkpoints as they were."""

    def __init__(self, runtime: TrainingRuntime, policy: StepPolicy, *, event_sink: Callable[[Mapping], None] = None):
        self.runtime, self.policy = runtime, policy
        self.event_sink = event_sink or (lambda event: None)
        # (policy test, runtime hook, event builder) for everything that can follow a step
        self._boundary_table = (
            (policy.should_save, self._save, lambda step, ident: {"event": "checkpoint", "checkpoint_id": ident}),
            (policy.should_validate, runtime.validate, lambda step, report: {"event": "validation", "report": dict(report)}),
        )

    def run(self) -> int:
        with paused_cycle_collection():
            while self.runtime.global_step < self.policy.max_steps:
                self.step()
        return self.runtime.global_step

    def step(self) -> None:
        timer = None
        if os.environ.get("SOLAR_PHASE_TIMES", "0") == "1":
            from ..utils.trace import PhaseTimer

            timer = PhaseTimer()
        record = StepRecord(self.runtime.global_step + 1, self.policy.grad_accum, [])
        if timer is None:
            self._train(record)
        else:
            with timer.installed():
                self._train(record)
            record.phase_ms = {k: v["total_ms"] for k, v in timer.summary().items() if not k.startswith("block.")}
        self.event_sink(record.event())
        self._boundaries(record.step)

    # -- phases ---------------------------------------------------------------------------------------------------
    def _train(self, record: StepRecord) -> None:
        self.runtime.zero_grad()
        self._accumulate(record)
        self._update(record)
        self._advance(record)

    def _accumulate(self, record: StepRecord) -> None:
        rt = self.runtime
        try:
            for index in range(record.grad_accum):
                outcome = rt.train_microbatch(index, record.grad_accum)
                rt.assert_sp_peer_identity(outcome.identity)
                record.microbatches.append(outcome)
        except BaseException:
            rt.zero_grad()
            raise

    def _update(self, record: StepRecord) -> None:
        from ..utils.trace import span

        rt = self.runtime
        with span("optimizer"):
            status = rt.prepare_optimizer_step()
            record.gradient_norm = status.norm
            if not (status.finite and math.isfinite(status.norm)):
                rt.zero_grad()
                raise BackendContractError(f"non-finite gradients before optimizer step {record.step}: {status.norm}")
            rt.optimizer_step()

    def _advance(self, record: StepRecord) -> None:
        rt = self.runtime
        rt.scheduler_step()
        rt.set_global_step(record.step)
        rt.ema_update(record.step)
        rt.zero_grad()

    def _save(self, step: int) -> str:
        ident = self.runtime.save_checkpoint(step)
        if not ident:
            raise BackendContractError("checkpoint hook returned an empty identity")
        return ident

    def _boundaries(self, step: int) -> None:
        crossed = False
        for due, hook, describe in self._boundary_table:
            if due(step):
                self.event_sink({"schema": EVENT_SCHEMA, "step": step, **describe(step, hook(step))})
                crossed = True
        if crossed:
            gc.collect()             # cycle collection is paused inside the loop; boundaries are where it runs
