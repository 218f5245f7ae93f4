"""Checkpointable plan streams for a rank's loader workers.

A data loader with ``W`` workers hands out batches in worker order 0, 1, ..., W-1, 0, ...; each worker is one
*reader* of the canonical sampler with its own random stream.  ``PlanMultiplexer`` reproduces that interleaving in the
parent process so that the position of the whole rank is a small explicit state: per worker the epoch, the cursor
into the epoch's plan list and the reader's random state AT THE START of that epoch, plus whose turn it is.  A resumed
run rebuilds every worker's current epoch from its saved random state (one epoch of planning, no shard is read) and
continues with the very next plan, instead of replaying every batch consumed so far.

Reference: WanPlanMultiplexer (solar/backends/wan22/runtime/data.py:182-300).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, List, Mapping, Sequence

from ..errors import DataContractError
from ..runtime.safe_state import decode_python_rng, encode_python_rng
from .sampling import CanonicalSampler, ReaderIdentity, SamplePlan, SamplingConfig

SCHEMA = "solarwm.plan-multiplexer.v1"


@dataclass
class _Worker:
    sampler: CanonicalSampler
    epoch: int = 0
    cursor: int = 0
    plans: List[SamplePlan] = field(default_factory=list)
    epoch_rng: Any = None                      # the reader's random state before ``epoch`` was planned

    def plan_epoch(self) -> None:
        self.epoch_rng = self.sampler.rng_state()
        self.plans = list(self.sampler.iter_epoch(self.epoch))
        if not self.plans:
            raise DataContractError("a loader worker owns no samples in this epoch")
        self.cursor = 0


class PlanMultiplexer:
    def __init__(self, rows: Sequence, sampling: SamplingConfig, topology, *, num_workers: int = 1):
        if num_workers < 1:
            raise DataContractError("num_workers must be positive")
        self.num_workers = int(num_workers)
        self.workers = [_Worker(CanonicalSampler(rows, sampling, ReaderIdentity.from_topology(
            topology, worker_id=w, num_workers=self.num_workers))) for w in range(self.num_workers)]
        for w in self.workers:
            w.plan_epoch()
        self.next_worker = 0

    # -- the stream ---------------------------------------------------------------------------------------------------
    def next_plan(self, worker_id: int) -> SamplePlan:
        w = self.workers[int(worker_id)]
        if w.cursor == len(w.plans):
            w.epoch += 1
            w.plan_epoch()
        plan = w.plans[w.cursor]
        w.cursor += 1
        return plan

    def finish_batch(self, worker_id: int) -> None:
        """A batch of ``worker_id`` was consumed: batches complete in worker order, anything else is a bug upstream."""
        if int(worker_id) != self.next_worker:
            raise DataContractError(f"batch of worker {worker_id} completed out of order (expected {self.next_worker})")
        self.next_worker = (self.next_worker + 1) % self.num_workers

    def next_batch(self, batch_size: int = 1) -> List[SamplePlan]:
        """The next batch in loader order: ``batch_size`` plans of the worker whose turn it is."""
        worker = self.next_worker
        plans = [self.next_plan(worker) for _ in range(int(batch_size))]
        self.finish_batch(worker)
        return plans

    # -- state ----------------------------------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"schema": SCHEMA, "num_workers": self.num_workers, "next_worker": self.next_worker,
                "workers": [{"epoch": w.epoch, "cursor": w.cursor, "epoch_rng": encode_python_rng(w.epoch_rng),
                             "plans_in_epoch": len(w.plans)} for w in self.workers]}

    def load_state_dict(self, state: Mapping[str, Any]) -> None:
        if state.get("schema") != SCHEMA:
            raise DataContractError("unknown plan-multiplexer state schema")
        if int(state.get("num_workers", 0)) != self.num_workers:
            raise DataContractError(f"the run was saved with {state.get('num_workers')} loader workers, "
                                    f"this one has {self.num_workers}")
        saved = state.get("workers")
        if not isinstance(saved, (list, tuple)) or len(saved) != self.num_workers:
            raise DataContractError("plan-multiplexer state lists another number of workers")
        turn = int(state["next_worker"])
        if not 0 <= turn < self.num_workers:
            raise DataContractError("plan-multiplexer state names a worker that does not exist")
        for w, s in zip(self.workers, saved):
            w.epoch = int(s["epoch"])
            w.sampler.set_rng_state(decode_python_rng(s["epoch_rng"]))
            w.plan_epoch()
            if len(w.plans) != int(s["plans_in_epoch"]):
                raise DataContractError("the index or the sampling configuration changed since the state was saved "
                                        f"({len(w.plans)} plans in the epoch, {s['plans_in_epoch']} then)")
            cursor = int(s["cursor"])
            if not 0 <= cursor <= len(w.plans):
                raise DataContractError("plan-multiplexer cursor is outside its epoch")
            w.cursor = cursor
        self.next_worker = turn
