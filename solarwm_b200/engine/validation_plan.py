"""Deterministic validation plans.

A plan fixes, before any rank generates anything, which validation rows are rendered, with which
seed, into which slot, and by which data-parallel rank: rows are taken from the validation index in
ordinal order (optionally a stable-hash subset), slot ``i`` gets ``stable_validation_seed(run, id, i)``
and belongs to rank ``i % dp_world``.  The plan is published create-only as ``validation-plan.json``
with a digest so that every rank -- and a later re-run -- can prove it rendered the same plan
(reference: solar/inference/validation_plan.py:21-137).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Mapping, Sequence

from ..errors import SolarWMError
from ..runtime.create_only import write_file_create_only
from ..runtime.randomness import stable_validation_seed


@dataclass(frozen=True)
class PlannedCase:
    slot: int
    sample_id: str
    seed: int
    dp_rank: int
    prompt: str = ""
    start_frame: int = 0


@dataclass(frozen=True)
class ValidationPlan:
    run_id: str
    step: int
    pass_name: str
    cases: tuple

    def as_dict(self) -> dict:
        return {"schema": "solarwm.validation-plan.v1", "run_id": self.run_id, "step": self.step,
                "pass_name": self.pass_name, "cases": [asdict(c) for c in self.cases]}

    @property
    def digest(self) -> str:
        return hashlib.blake2s(json.dumps(self.as_dict(), sort_keys=True, separators=(",", ":")).encode()).hexdigest()

    def for_rank(self, dp_rank: int) -> tuple:
        return tuple(c for c in self.cases if c.dp_rank == dp_rank)


def build_plan(rows: Sequence[Mapping[str, Any]], *, run_id: str, step: int, pass_name: str, count: int,
               dp_world: int = 1, base_seed: int = 0) -> ValidationPlan:
    if count < 1 or dp_world < 1:
        raise SolarWMError("validation plan needs count >= 1 and dp_world >= 1")
    if len(rows) < count:
        raise SolarWMError(f"validation index has {len(rows)} rows, the plan asks for {count}")
    ids = [str(r["sample_id"]) for r in rows]
    if len(set(ids)) != len(ids):
        raise SolarWMError("validation rows must have unique sample ids")
    cases = tuple(PlannedCase(slot=i, sample_id=ids[i], seed=stable_validation_seed(base_seed, ids[i], i),
                              dp_rank=i % dp_world, prompt=str(rows[i].get("caption", "")),
                              start_frame=int(rows[i].get("start_frame", 0))) for i in range(count))
    return ValidationPlan(run_id, int(step), pass_name, cases)


def publish_plan(plan: ValidationPlan, directory) -> Path:
    path = Path(directory) / "validation-plan.json"
    path.parent.mkdir(parents=True, exist_ok=True)
    body = dict(plan.as_dict(), digest=plan.digest)
    write_file_create_only(path, json.dumps(body, sort_keys=True, indent=1).encode())
    return path


def load_plan(path) -> ValidationPlan:
    body = json.loads(Path(path).read_text())
    plan = ValidationPlan(body["run_id"], int(body["step"]), body["pass_name"],
                          tuple(PlannedCase(**c) for c in body["cases"]))
    if body.get("digest") != plan.digest:
        raise SolarWMError("validation plan digest mismatch")
    return plan
