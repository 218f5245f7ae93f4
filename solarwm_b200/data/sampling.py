"""Deterministic sample plans: who reads which clip, in what order, from which frame.

The plan sequence is a CONTRACT between runs, between sequence-parallel peers and with corpora prepared elsewhere:
for the same index, configuration and reader identity this module must emit exactly the sequence (and therefore the
same ``plan_fingerprint``) as the reference sampler does; ``tests/test_reference_contracts.py`` holds it to that
against the reference package (contract: solar/data/sampling.py:26-366).  What the contract fixes:

  * every (index row, repeat) pair is a *virtual occurrence*, numbered in index order;
  * ``global_occurrence`` mode: occurrence ``v`` belongs to reader ``v mod readers`` where a reader is one loader
    worker of one LOGICAL data-parallel rank (sequence-parallel peers are the same reader); a reader's occurrences
    pass through a bounded shuffle reservoir driven by the reader's own ``random.Random(seed + reader * 100003)``,
    which also draws the random start frames and lives across epochs;
  * ``node_shard`` mode: whole shards are dealt to nodes by ``sha256(seed|epoch|shard key) mod nodes``, shuffled
    through the same kind of reservoir with a per-node, per-epoch generator, and the occurrences inside a shard are
    split round-robin over the node's local readers and shuffled with the reader's generator;
  * frame offsets resample the clip's frame rate to the output rate (rounded, never decreasing).

The code is organised as small parts that can be tested alone: ``Reservoir`` (the bounded shuffle), a start-frame
policy chosen once per sampler, ``FrameGrid`` (cached offsets per source rate), ``deal_shards`` (node assignment).
"""
from __future__ import annotations

import hashlib
import random
from dataclasses import dataclass
from pathlib import PurePosixPath
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import numpy as np

from ..errors import DataContractError
from .index import IndexRow

_PARTITION_MODES = ("global_occurrence", "node_shard")
_SHARD_SCOPES = ("complete", "collection_relative")


def _require(ok: bool, message: str) -> None:
    if not ok:
        raise DataContractError(message)


@dataclass(frozen=True)
class SamplingConfig:
    seed: int
    pixel_frames: int
    random_start: bool = True
    fixed_start_from_index: bool = False
    clip_seconds: Optional[float] = None
    output_fps: Optional[float] = None
    shuffle_buffer: int = 4096
    partition_mode: str = "global_occurrence"
    shard_partition_scope: str = "complete"

    def __post_init__(self):
        _require(self.pixel_frames >= 1, "pixel_frames must be positive")
        _require(self.shuffle_buffer >= 1, "shuffle_buffer must be positive")
        _require(self.partition_mode in _PARTITION_MODES, "unknown partition_mode")
        _require(self.shard_partition_scope in _SHARD_SCOPES, "unknown shard_partition_scope")
        _require(not (self.random_start and self.fixed_start_from_index),
                 "random_start and fixed_start_from_index are mutually exclusive")
        _require((self.clip_seconds is None) == (self.output_fps is None),
                 "clip_seconds and output_fps must be set together")
        if self.clip_seconds is not None:
            implied = round(self.clip_seconds * float(self.output_fps)) + 1
            _require(implied == self.pixel_frames,
                     f"clip_seconds/output_fps imply {implied} frames, expected {self.pixel_frames}")


@dataclass(frozen=True)
class ReaderIdentity:
    """One loader worker of one logical data-parallel rank (never a raw sequence-parallel process)."""

    rank: int
    world_size: int
    worker_id: int = 0
    num_workers: int = 1
    node_id: int = 0
    node_count: int = 1
    local_rank: int = 0
    local_world_size: int = 1

    def __post_init__(self):
        for value, bound, what in ((self.rank, self.world_size, "reader rank is outside world_size"),
                                   (self.worker_id, self.num_workers, "worker_id is outside num_workers"),
                                   (self.node_id, self.node_count, "node_id is outside node_count"),
                                   (self.local_rank, self.local_world_size, "local_rank is outside local_world_size")):
            _require(0 <= value < bound, what)

    @classmethod
    def from_topology(cls, topology, *, worker_id: int = 0, num_workers: int = 1) -> "ReaderIdentity":
        """The reader of a ``runtime.topology.Topology``: every SP peer of a DP rank maps to the same identity."""
        try:
            sp = int(topology.sp_size)
            local_dp = max(int(topology.local_world_size) // sp, 1)
            return cls(rank=int(topology.dp_rank), world_size=int(topology.dp_size), worker_id=worker_id,
                       num_workers=num_workers, node_id=int(topology.node_rank), node_count=int(topology.num_nodes),
                       local_rank=(int(topology.local_rank) // sp) % local_dp, local_world_size=local_dp)
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


# ---------------------------------------------------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------------------------------------------------
class Reservoir:
    """Bounded shuffle: items enter in order; once ``capacity`` are held, each arrival releases one held item chosen
    by ``rng.randrange``; ``drain`` releases the rest the same way.  Capacity 1 passes items through untouched and
    draws nothing."""

    def __init__(self, capacity: int, rng: random.Random):
        self.capacity, self.rng, self._held = int(capacity), rng, []

    def feed(self, item) -> Iterator:
        if self.capacity == 1:
            yield item
            return
        self._held.append(item)
        if len(self._held) >= self.capacity:
            yield self._held.pop(self.rng.randrange(len(self._held)))

    def drain(self) -> Iterator:
        while self._held:
            yield self._held.pop(self.rng.randrange(len(self._held)))

    def through(self, items: Iterable) -> Iterator:
        for item in items:
            yield from self.feed(item)
        yield from self.drain()


class FrameGrid:
    """Frame offsets of one clip window relative to its start, per source frame rate (cached)."""

    def __init__(self, config: SamplingConfig):
        self.config = config
        self._by_rate: Dict[float, np.ndarray] = {}

    def offsets(self, source_fps: float) -> np.ndarray:
        cfg = self.config
        if cfg.clip_seconds is None:
            source_fps = 0.0                                   # one grid for every clip
        hit = self._by_rate.get(source_fps)
        if hit is None:
            hit = self._by_rate[source_fps] = frame_offsets(cfg, source_fps)
        return hit


def frame_offsets(config: SamplingConfig, source_fps: float) -> np.ndarray:
    steps = np.arange(config.pixel_frames, dtype=np.int64)
    if config.clip_seconds is None:
        return steps
    rate = float(source_fps) if source_fps > 0 else float(config.output_fps)
    resampled = np.rint(steps.astype(np.float64) * (rate / float(config.output_fps))).astype(np.int64)
    return np.maximum.accumulate(resampled)


def _clip_geometry(row: IndexRow) -> Tuple[int, float]:
    v = row.values
    video = v.get("manifest", {}).get("video", {}) if isinstance(v.get("manifest"), dict) else {}
    try:
        frames = int(v.get("num_frames") or video["num_frames"])
    except (KeyError, TypeError, ValueError) as exc:
        raise DataContractError(f"sample {row.sample_id} lacks num_frames") from exc
    try:
        fps = float(v.get("fps") or video.get("fps") or 0.0)
    except (TypeError, ValueError) as exc:
        raise DataContractError(f"sample {row.sample_id} has invalid fps") from exc
    return frames, fps


def _start_policy(config: SamplingConfig, rng: random.Random) -> Callable[[IndexRow, int, int], int]:
    """``(row, frames, span) -> start``; only the random policy touches the generator."""
    if config.random_start:
        return lambda row, frames, span: rng.randint(0, frames - span - 1)
    if config.fixed_start_from_index:
        def from_index(row, frames, span):
            try:
                return int(row.values["start_frame"])
            except (KeyError, TypeError, ValueError) as exc:
                raise DataContractError(f"sample {row.sample_id} lacks a valid fixed start_frame") from exc
        return from_index
    return lambda row, frames, span: 0


def partition_key(shard: str, scope: str) -> str:
    """What identifies a shard for the node draw: its whole path, or the path from the collection directory (the
    parent of the last ``shards`` component) down, so that a corpus keeps its assignment when its root moves."""
    if scope == "complete":
        return shard
    parts = PurePosixPath(shard).parts
    marks = [i for i, p in enumerate(parts) if p == "shards"]
    return "/".join(parts[marks[-1] - 1:]) if marks and marks[-1] > 0 else shard


def shard_runs(rows: Sequence[IndexRow]) -> List[Tuple[str, List[IndexRow]]]:
    """Consecutive rows of the same shard, in index order."""
    runs: List[Tuple[str, List[IndexRow]]] = []
    for row in rows:
        if runs and runs[-1][0] == row.shard:
            runs[-1][1].append(row)
        else:
            runs.append((row.shard, [row]))
    return runs


def deal_shards(rows: Sequence[IndexRow], config: SamplingConfig, node_id: int, node_count: int, epoch: int) -> tuple:
    """The shards of ``node_id`` for ``epoch`` in reading order."""
    rng = random.Random(config.seed + node_id * 1000003 + epoch * 1000000007)

    def mine():
        for shard, members in shard_runs(rows):
            ticket = hashlib.sha256(f"{config.seed}|{epoch}|{partition_key(shard, config.shard_partition_scope)}".encode())
            if int.from_bytes(ticket.digest()[:8], "big") % node_count == node_id:
                yield shard, tuple(members)

    return tuple(Reservoir(config.shuffle_buffer, rng).through(mine())) if config.shuffle_buffer > 1 else tuple(mine())


# ---------------------------------------------------------------------------------------------------------------------
# the sampler
# ---------------------------------------------------------------------------------------------------------------------
class CanonicalSampler:
    def __init__(self, rows: Sequence[IndexRow], config: SamplingConfig, identity: ReaderIdentity):
        _require(len(rows) > 0, "sampler needs at least one index row")
        self.rows, self.config, self.identity = tuple(rows), config, identity
        self._rng = random.Random(config.seed + identity.global_reader * 100003)
        self._grid = FrameGrid(config)
        self._start = _start_policy(config, self._rng)

    def rng_state(self):
        return self._rng.getstate()

    def set_rng_state(self, state) -> None:
        self._rng.setstate(state)

    def iter_epoch(self, epoch: int) -> Iterator[SamplePlan]:
        _require(epoch >= 0, "epoch must be non-negative")
        stream = self._node_shard_stream(epoch) if self.config.partition_mode == "node_shard" \
            else self._occurrence_stream()
        for row, repeat in stream:
            yield self._plan(row, repeat, epoch)

    def node_shard_groups(self, epoch: int) -> tuple:
        _require(self.config.partition_mode == "node_shard", "node shard groups require partition_mode=node_shard")
        _require(epoch >= 0, "epoch must be non-negative")
        return deal_shards(self.rows, self.config, self.identity.node_id, self.identity.node_count, epoch)

    # -- streams of (row, repeat) ---------------------------------------------------------------------------------
    def _occurrence_stream(self) -> Iterator[Tuple[IndexRow, int]]:
        me, readers = self.identity.global_reader, self.identity.total_readers
        owned, number = [], 0
        for row in self.rows:
            for repeat in range(row.epoch_repeats):
                if number % readers == me:
                    owned.append((row, repeat))
                number += 1
        _require(bool(owned), "this reader owns no virtual occurrences")
        # plans are built as items leave the reservoir, so start-frame draws interleave with the shuffle draws
        yield from Reservoir(self.config.shuffle_buffer, self._rng).through(owned)

    def _node_shard_stream(self, epoch: int) -> Iterator[Tuple[IndexRow, int]]:
        me, readers = self.identity.local_reader, self.identity.local_readers
        number = emitted = 0
        for _, members in self.node_shard_groups(epoch):
            mine = []
            for row in members:
                for repeat in range(row.epoch_repeats):
                    if number % readers == me:
                        mine.append((row, repeat))
                    number += 1
            self._rng.shuffle(mine)
            emitted += len(mine)
            yield from mine
        _require(emitted > 0, "this node-shard reader emitted no occurrences")

    # -- one plan ---------------------------------------------------------------------------------------------------
    def _plan(self, row: IndexRow, repeat: int, epoch: int) -> SamplePlan:
        frames, fps = _clip_geometry(row)
        offsets = self._grid.offsets(fps)
        span = int(offsets[-1])
        _require(frames > span, f"sample {row.sample_id} has {frames} frames, needs an offset through {span}")
        start = self._start(row, frames, span)
        _require(0 <= start and start + span < frames,
                 f"sample {row.sample_id} fixed start {start} is outside {frames} source frames")
        return SamplePlan(row.sample_id, row.key, row.shard, row.ordinal, repeat, epoch, start,
                          tuple(int(i) for i in start + offsets), self.identity.rank, self.identity.worker_id)


def plan_fingerprint(plans: Iterable[SamplePlan]) -> str:
    """blake2s over one tab-separated line per plan under a version header: equal sequences, equal fingerprints."""
    h = hashlib.blake2s(b"solarwm.sample-plan.v1\n")
    for p in plans:
        fields = (p.sample_id, p.key, p.shard, p.row_ordinal, p.repeat_ordinal, p.epoch, p.start_frame,
                  ",".join(str(i) for i in p.source_frame_indices), p.reader_rank, p.worker_id)
        h.update(("\t".join(str(f) for f in fields) + "\n").encode())
    return h.hexdigest()
