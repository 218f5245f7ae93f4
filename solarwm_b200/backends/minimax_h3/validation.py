"""Fixed, source-balanced validation for the H3 stages, straight from a validation index.

  selection   windows cut from one source video share a source id (``source_sample_id`` of the row, else the sample id up
              to its window suffix).  Slots are dealt to the datasets round-robin (the first path component of the sample
              id), every dataset's source videos are ordered by a seeded hash, and slot ``s`` of a dataset gets candidate
              ``s``, with ``s + quota``, ``s + 2 quota``, ... as its reserves: slots never share a source video, and a
              slot whose first candidate cannot be read (a missing shard, a camera the filter refuses) falls back to a
              reserve of the same dataset.
  freezing    the ids that were finally chosen are written once (``validation-selection.json``, create-only) and read
              back by later passes and by resumed runs, so every validation pass of a run scores the same clips even
              when an earlier reserve has become readable in the meantime.
  scoring     the flow-matching loss at fixed times with noise seeded per (slot, time): a pure function of the weights.
              Slots belong to logical data-parallel ranks round-robin; ranks hold the same number of slots (the count is
              rounded down to whole waves) and the losses are averaged over all of them.

Reference: validation_candidates and H3IndexedValidationStream (solar/backends/minimax_h3/validation_stream.py:24-318).
"""
from __future__ import annotations

import hashlib
import json
from collections import defaultdict
from pathlib import Path
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import torch

from ...errors import DataContractError
from ...runtime.create_only import write_file_create_only
from ...runtime.randomness import stable_validation_seed

SELECTION_SCHEMA = "solarwm.h3-validation-selection.v1"
TIMES = (0.25, 0.5, 0.75)


def source_video_id(sample_id: str, values: Optional[Mapping[str, Any]] = None) -> str:
    given = (values or {}).get("source_sample_id")
    if given:
        return str(given)
    head, sep, _ = sample_id.partition("/h3-158f-occ-")
    return head if sep else sample_id


def balanced_candidates(rows: Sequence, *, sample_count: int, seed: int, balance: bool = True) -> Tuple[Tuple, ...]:
    """``rows`` have ``sample_id`` and ``values``.  Returns one tuple of candidates per slot (first choice, then reserves)."""
    groups: Dict[str, Dict[str, Any]] = defaultdict(dict)
    for row in rows:
        dataset = row.sample_id.split("/")[0] if balance else "all"
        groups[dataset].setdefault(source_video_id(row.sample_id, getattr(row, "values", None)), row)
    datasets = sorted(groups)
    if not datasets or sample_count < len(datasets):
        raise DataContractError("validation needs at least one slot per eligible dataset")
    slots = []
    for slot in range(sample_count):
        pos = slot % len(datasets)
        dataset = datasets[pos]
        quota = sample_count // len(datasets) + (pos < sample_count % len(datasets))
        ordered = sorted(groups[dataset].values(), key=lambda r: hashlib.sha256(f"{seed}:{r.sample_id}".encode()).hexdigest())
        if len(ordered) < quota:
            raise DataContractError(f"validation has too few distinct source videos in {dataset}")
        slots.append(tuple(ordered[slot // len(datasets)::quota]))
    return tuple(slots)


class IndexedValidation:
    """``read(row) -> sample`` loads one clip (it may raise ``DataContractError`` / ``OSError`` for a clip that cannot be
    used); ``dp_rank`` / ``dp_size`` are the logical data-parallel coordinates."""

    def __init__(self, rows: Sequence, read: Callable[[Any], Mapping[str, torch.Tensor]], *, sample_count: int, seed: int,
                 dp_rank: int = 0, dp_size: int = 1, balance: bool = True, freeze_path=None):
        self.read, self.seed, self.dp_rank, self.dp_size = read, int(seed), int(dp_rank), int(dp_size)
        self.count = (int(sample_count) // self.dp_size) * self.dp_size
        if self.count < 1:
            raise DataContractError("validation.sample_count is smaller than the number of data-parallel replicas")
        self.by_id = {r.sample_id: r for r in rows}
        self.candidates = balanced_candidates(rows, sample_count=self.count, seed=self.seed, balance=balance)
        self.freeze_path = None if freeze_path is None else Path(freeze_path)
        self.selected: Dict[int, str] = {}
        self.samples: Dict[int, Mapping[str, torch.Tensor]] = {}

    @property
    def my_slots(self) -> List[int]:
        return [s for s in range(self.count) if s % self.dp_size == self.dp_rank]

    def _frozen(self) -> Optional[Dict[int, str]]:
        if self.freeze_path is None or not self.freeze_path.is_file():
            return None
        doc = json.loads(self.freeze_path.read_text())
        if doc.get("schema") != SELECTION_SCHEMA or doc.get("seed") != self.seed or doc.get("slots") != self.count:
            raise DataContractError("the frozen validation selection was made under another seed or slot count")
        chosen = {int(k): str(v) for k, v in doc["selected"].items()}
        if sorted(chosen) != list(range(self.count)) or any(v not in self.by_id for v in chosen.values()):
            raise DataContractError("the frozen validation selection names clips that are not in the index")
        return chosen

    def prepare(self, dist=None) -> Mapping[int, str]:
        """Choose (or re-read the frozen choice of) one clip per slot, load this rank's, agree on the whole selection."""
        frozen = self._frozen()
        mine: Dict[int, str] = {}
        for slot in self.my_slots:
            options = [self.by_id[frozen[slot]]] if frozen else list(self.candidates[slot])
            problems = []
            for row in options:
                try:
                    self.samples[slot] = self.read(row)
                    mine[slot] = row.sample_id
                    break
                except (DataContractError, OSError) as exc:
                    problems.append(f"{row.sample_id}: {exc}")
            else:
                raise DataContractError(f"validation slot {slot} has no usable clip ({'; '.join(problems)[:400]})")
        everyone = [mine]
        if dist is not None and self.dp_size > 1:
            everyone = [None] * dist.get_world_size()
            dist.all_gather_object(everyone, mine)
        self.selected = {s: i for part in everyone for s, i in part.items()}
        if sorted(self.selected) != list(range(self.count)):
            raise DataContractError("the ranks did not cover every validation slot")
        sources = [source_video_id(i, getattr(self.by_id[i], "values", None)) for i in self.selected.values()]
        if len(set(sources)) != len(sources):
            raise DataContractError("two validation slots ended on the same source video")
        if frozen is None and self.freeze_path is not None and self.dp_rank == 0:
            self.freeze_path.parent.mkdir(parents=True, exist_ok=True)
            write_file_create_only(self.freeze_path, json.dumps(
                {"schema": SELECTION_SCHEMA, "seed": self.seed, "slots": self.count,
                 "selected": {str(s): self.selected[s] for s in sorted(self.selected)}}, sort_keys=True, indent=1).encode())
        return dict(self.selected)

    def items(self):
        """This rank's (slot, sample id, sample) in slot order."""
        for slot in self.my_slots:
            yield slot, self.selected[slot], self.samples[slot]


def score(validation: IndexedValidation, loss_at: Callable[[Mapping[str, torch.Tensor], float, torch.Generator], torch.Tensor], *,
          device, times: Sequence[float] = TIMES, dist=None, group=None) -> Mapping[str, Any]:
    """``loss_at(sample, t, generator)`` is the stage's loss at time ``t`` with all randomness drawn from ``generator``."""
    total = torch.zeros(len(times) + 1, dtype=torch.float64, device=device)
    per_slot = {}
    with torch.no_grad():
        for slot, sample_id, sample in validation.items():
            values = []
            for t in times:
                g = torch.Generator(device=device).manual_seed(stable_validation_seed("h3-validation", sample_id, f"{slot}:{t}") % (2 ** 63))
                values.append(float(loss_at(sample, float(t), g)))
            if not all(v == v and abs(v) != float("inf") for v in values):
                raise FloatingPointError(f"non-finite validation loss on {sample_id}")
            per_slot[slot] = values
            total[:-1] += torch.tensor(values, dtype=torch.float64, device=device)
            total[-1] += 1
    if dist is not None and validation.dp_size > 1:
        dist.all_reduce(total, group=group)
    n = float(total[-1])
    by_time = {f"loss_t{t:g}": float(total[i]) / n for i, t in enumerate(times)}
    return {"loss": sum(by_time.values()) / len(by_time), **by_time, "clips": int(n), "local": {str(k): v for k, v in per_slot.items()},
            "selected": {str(s): validation.selected[s] for s in sorted(validation.selected)}}
