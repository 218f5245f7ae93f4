"""Deterministic sample plans.

Every (row, repeat) pair is a *virtual occurrence*; occurrence ``i`` belongs to reader
``i % total_readers`` where a reader is one DataLoader worker of one LOGICAL data-parallel rank
(sequence-parallel peers map to the same reader and therefore read identical samples).  Owned
occurrences stream through a finite shuffle buffer; start frames are random, fixed from the index
or zero; frame offsets resample the source fps to the output fps.  ``node_shard`` mode assigns whole
shards to nodes with a sha256 draw so a node only downloads its own shards.
``plan_fingerprint`` hashes a plan sequence for cross-run / cross-peer comparison.

Reference: solar/data/sampling.py:26-366.
"""
from __future__ import annotations

import hashlib
import random
from dataclasses import dataclass
from pathlib import PurePosixPath
from typing import Iterable, Iterator, Optional, Sequence

import numpy as np

from ..errors import DataContractError
from .index import IndexRow


@dataclass(frozen=True)
class SamplingConfig:
    seed: int
    pixel_frames: int
    random_start: bool = True
    fixed_start_from_index: bool = False
    clip_seconds: Optional[float] = None
    output_fps: Optional[float] = None
    shuffle_buffer: int = 4096
    partition_mode: str = "global_occurrence"      # or "node_shard"
    shard_partition_scope: str = "complete"        # or "collection_relative"

    def __post_init__(self):
        if self.pixel_frames < 1:
            raise DataContractError("pixel_frames must be positive")
        if self.shuffle_buffer < 1:
            raise DataContractError("shuffle_buffer must be positive")
        if self.partition_mode not in ("global_occurrence", "node_shard"):
            raise DataContractError("unknown partition_mode")
        if self.shard_partition_scope not in ("complete", "collection_relative"):
            raise DataContractError("unknown shard_partition_scope")
        if self.random_start and self.fixed_start_from_index:
            raise DataContractError("random_start and fixed_start_from_index are mutually exclusive")
        if (self.clip_seconds is None) != (self.output_fps is None):
            raise DataContractError("clip_seconds and output_fps must be set together")
        if self.clip_seconds is not None:
            implied = round(self.clip_seconds * float(self.output_fps)) + 1
            if implied != self.pixel_frames:
                raise DataContractError(f"clip_seconds/output_fps imply {implied} frames, expected {self.pixel_frames}")


@dataclass(frozen=True)
class ReaderIdentity:
    rank: int
    world_size: int
    worker_id: int = 0
    num_workers: int = 1
    node_id: int = 0
    node_count: int = 1
    local_rank: int = 0
    local_world_size: int = 1

    def __post_init__(self):
        if not 0 <= self.rank < self.world_size:
            raise DataContractError("reader rank is outside world_size")
        if not 0 <= self.worker_id < self.num_workers:
            raise DataContractError("worker_id is outside num_workers")
        if not 0 <= self.node_id < self.node_count:
            raise DataContractError("node_id is outside node_count")
        if not 0 <= self.local_rank < self.local_world_size:
            raise DataContractError("local_rank is outside local_world_size")

    @classmethod
    def from_topology(cls, topology, *, worker_id: int = 0, num_workers: int = 1) -> "ReaderIdentity":
        """Logical-DP reader of a ``runtime.topology.Topology`` (all SP peers get the same identity)."""
        try:
            sp, local_world = int(topology.sp_size), int(topology.local_world_size)
            local_dp_world = max(local_world // sp, 1)
            return cls(rank=int(topology.dp_rank), world_size=int(topology.dp_size), worker_id=worker_id,
                       num_workers=num_workers, node_id=int(topology.node_rank), node_count=int(topology.num_nodes),
                       local_rank=(int(topology.local_rank) // sp) % local_dp_world, local_world_size=local_dp_world)
        except (AttributeError, TypeError, ValueError) as exc:
            raise DataContractError("invalid distributed topology") from exc

    @property
    def global_reader(self) -> int:
        return self.rank * self.num_workers + self.worker_id

    @property
    def total_readers(self) -> int:
        return self.world_size * self.num_workers

    @property
    def local_reader(self) -> int:
        return self.local_rank * self.num_workers + self.worker_id

    @property
    def local_readers(self) -> int:
        return self.local_world_size * self.num_workers


@dataclass(frozen=True)
class SamplePlan:
    sample_id: str
    key: str
    shard: str
    row_ordinal: int
    repeat_ordinal: int
    epoch: int
    start_frame: int
    source_frame_indices: tuple
    reader_rank: int
    worker_id: int


def frame_offsets(config: SamplingConfig, source_fps: float) -> np.ndarray:
    if config.clip_seconds is None:
        return np.arange(config.pixel_frames, dtype=np.int64)
    fps = source_fps if source_fps > 0 else float(config.output_fps)
    off = np.rint(np.arange(config.pixel_frames, dtype=np.float64) * (fps / float(config.output_fps))).astype(np.int64)
    return np.maximum.accumulate(off)


class CanonicalSampler:
    def __init__(self, rows: Sequence[IndexRow], config: SamplingConfig, identity: ReaderIdentity):
        if not rows:
            raise DataContractError("sampler needs at least one index row")
        self.rows, self.config, self.identity = tuple(rows), config, identity
        self._rng = random.Random(config.seed + identity.global_reader * 100003)

    # public ---------------------------------------------------------------------------
    def iter_epoch(self, epoch: int) -> Iterator[SamplePlan]:
        if epoch < 0:
            raise DataContractError("epoch must be non-negative")
        if self.config.partition_mode == "node_shard":
            yield from self._by_node_shard(epoch)
        else:
            yield from self._by_occurrence(epoch)

    def rng_state(self):
        return self._rng.getstate()

    def set_rng_state(self, state) -> None:
        self._rng.setstate(state)

    # internals ------------------------------------------------------------------------
    def _plan(self, row: IndexRow, repeat: int, epoch: int) -> SamplePlan:
        v = row.values
        try:
            n = int(v.get("num_frames") or v["manifest"]["video"]["num_frames"])
        except (KeyError, TypeError, ValueError) as exc:
            raise DataContractError(f"sample {row.sample_id} lacks num_frames") from exc
        try:
            fps = float(v.get("fps") or v.get("manifest", {}).get("video", {}).get("fps") or 0.0)
        except (TypeError, ValueError) as exc:
            raise DataContractError(f"sample {row.sample_id} has invalid fps") from exc
        off = frame_offsets(self.config, fps)
        span = int(off[-1])
        if n <= span:
            raise DataContractError(f"sample {row.sample_id} has {n} frames, needs an offset through {span}")
        if self.config.random_start:
            start = self._rng.randint(0, n - span - 1)
        elif self.config.fixed_start_from_index:
            try:
                start = int(v["start_frame"])
            except (KeyError, TypeError, ValueError) as exc:
                raise DataContractError(f"sample {row.sample_id} lacks a valid fixed start_frame") from exc
        else:
            start = 0
        if start < 0 or start + span >= n:
            raise DataContractError(f"sample {row.sample_id} fixed start {start} is outside {n} source frames")
        return SamplePlan(row.sample_id, row.key, row.shard, row.ordinal, repeat, epoch, start,
                          tuple(int(i) for i in start + off), self.identity.rank, self.identity.worker_id)

    def _by_occurrence(self, epoch: int) -> Iterator[SamplePlan]:
        me, total = self.identity.global_reader, self.identity.total_readers
        owned, virtual = [], 0
        for row in self.rows:
            for rep in range(row.epoch_repeats):
                if virtual % total == me:
                    owned.append((row, rep))
                virtual += 1
        if not owned:
            raise DataContractError("this reader owns no virtual occurrences")
        pool = []
        for item in owned:
            if self.config.shuffle_buffer == 1:
                yield self._plan(*item, epoch)     # no RNG draw for a one-slot buffer
                continue
            pool.append(item)
            if len(pool) >= self.config.shuffle_buffer:
                yield self._plan(*pool.pop(self._rng.randrange(len(pool))), epoch)
        while pool:
            yield self._plan(*pool.pop(self._rng.randrange(len(pool))), epoch)

    def node_shard_groups(self, epoch: int) -> tuple:
        if self.config.partition_mode != "node_shard":
            raise DataContractError("node shard groups require partition_mode=node_shard")
        if epoch < 0:
            raise DataContractError("epoch must be non-negative")
        groups, current, name = [], [], ""
        for row in self.rows:
            if current and row.shard != name:
                groups.append((name, current))
                current = []
            name = row.shard
            current.append(row)
        if current:
            groups.append((name, current))
        rng = random.Random(self.config.seed + self.identity.node_id * 1000003 + epoch * 1000000007)
        chosen, pool = [], []
        for shard, rows in groups:
            key = _partition_key(shard, self.config.shard_partition_scope)
            draw = hashlib.sha256(f"{self.config.seed}|{epoch}|{key}".encode()).digest()[:8]
            if int.from_bytes(draw, "big") % self.identity.node_count != self.identity.node_id:
                continue
            pool.append((shard, rows))
            if len(pool) >= self.config.shuffle_buffer:
                s, r = pool.pop(rng.randrange(len(pool)))
                chosen.append((s, tuple(r)))
        while pool:
            s, r = pool.pop(rng.randrange(len(pool)))
            chosen.append((s, tuple(r)))
        return tuple(chosen)

    def _by_node_shard(self, epoch: int) -> Iterator[SamplePlan]:
        cursor = emitted = 0
        for _, rows in self.node_shard_groups(epoch):
            mine = []
            for row in rows:
                for rep in range(row.epoch_repeats):
                    if cursor % self.identity.local_readers == self.identity.local_reader:
                        mine.append((row, rep))
                    cursor += 1
            self._rng.shuffle(mine)
            for item in mine:
                emitted += 1
                yield self._plan(*item, epoch)
        if not emitted:
            raise DataContractError("this node-shard reader emitted no occurrences")


def _partition_key(shard: str, scope: str) -> str:
    if scope == "complete":
        return shard
    parts = PurePosixPath(shard).parts
    at = max((i for i, p in enumerate(parts) if p == "shards"), default=-1)
    return "/".join(parts[at - 1:]) if at > 0 else shard


def plan_fingerprint(plans: Iterable[SamplePlan]) -> str:
    h = hashlib.blake2s()
    h.update(b"solarwm.sample-plan.v1\n")
    for p in plans:
        h.update((f"{p.sample_id}\t{p.key}\t{p.shard}\t{p.row_ordinal}\t{p.repeat_ordinal}\t{p.epoch}\t"
                  f"{p.start_frame}\t{','.join(map(str, p.source_frame_indices))}\t{p.reader_rank}\t{p.worker_id}\n").encode())
    return h.hexdigest()
