"""Shard prefetching and cache warm-up.

``warm_cache`` materialises an explicit working set (the distinct shards of some index rows) before a run starts: it
refuses a set that does not fit the cache BEFORE any transfer (evicting the beginning while warming the end would
prepare nothing), keeps ``max_workers`` transfers in flight, waits out transient time-outs until one overall deadline,
and reports shards / bytes / seconds.  It creates no reader cursors and advances no random streams.

``ShardPrefetcher`` keeps the shards of upcoming sample plans in flight on a small thread pool so that the training
loop never waits on transport: ``schedule(plan)`` starts a transfer (once per shard), ``wait(plan)`` blocks until the
plan's shard is local and returns its path, ``iterate(plans)`` does both with a look-ahead window.  On a node with
several reader processes ``node_order`` staggers which shard each process asks for first, so that the processes do
not all queue behind the same per-shard lock (reference: solar/data/prefetch.py:30-346).
"""
from __future__ import annotations

import threading
import time
from collections import OrderedDict
from concurrent.futures import FIRST_COMPLETED, Future, ThreadPoolExecutor, wait
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Iterable, Iterator, Optional, Sequence

from ..errors import DataContractError
from .transport import DownloadTimeout


@dataclass(frozen=True)
class WarmupResult:
    shards: int
    bytes: int
    seconds: float


def _shard_sizes(rows) -> "OrderedDict[str, Optional[int]]":
    sizes: "OrderedDict[str, Optional[int]]" = OrderedDict()
    for r in rows:
        size = r.values.get("shard_size")
        size = None if size is None else int(size)
        if r.shard in sizes and sizes[r.shard] != size:
            raise DataContractError(f"rows disagree on the size of shard {r.shard}")
        sizes[r.shard] = size
    return sizes


def warm_cache(resolver, rows, max_workers: int = 8, *, max_bytes: Optional[int] = None, timeout_s: float = 7200.0,
               progress: Optional[Callable[[int, int], None]] = None) -> WarmupResult:
    """Resolve every distinct shard of ``rows`` once.  ``max_bytes``: the cache capacity the working set must fit."""
    if max_workers < 1 or timeout_s <= 0 or (max_bytes is not None and max_bytes < 1):
        raise DataContractError("cache warm-up needs positive workers, capacity and time budget")
    sizes = _shard_sizes(rows)
    total = sum(v or 0 for v in sizes.values())
    capacity = int(getattr(resolver, "max_cache_bytes", 0) or 0)
    if max_bytes is not None and capacity and max_bytes > capacity:
        raise DataContractError("the warm-up capacity exceeds the resolver's cache capacity")
    limit = max_bytes if max_bytes is not None else (capacity or None)
    if limit is not None and total > limit:
        raise DataContractError(f"the working set needs {total} bytes, the cache holds {limit}: warm a smaller index "
                                "or enlarge the cache")
    start = time.monotonic()
    deadline, stop = start + timeout_s, threading.Event()

    def fetch(item) -> Path:
        shard, size = item
        while True:
            if stop.is_set() or time.monotonic() >= deadline:
                raise DownloadTimeout(f"cache warm-up ran out of time at {shard}")
            try:
                return resolver.resolve(shard, size)
            except DownloadTimeout:
                stop.wait(min(1.0, max(0.0, deadline - time.monotonic())))

    items, done_count = iter(sizes.items()), 0
    pool = ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="cache-warmup")
    pending = set()
    try:
        for item in items:
            pending.add(pool.submit(fetch, item))
            if len(pending) >= max_workers:
                break
        while pending:
            finished, pending = wait(pending, timeout=max(0.0, deadline - time.monotonic()), return_when=FIRST_COMPLETED)
            if not finished:
                raise DownloadTimeout("cache warm-up ran out of time")
            for f in finished:
                f.result()
                done_count += 1
                if progress is not None:
                    progress(done_count, len(sizes))
                nxt = next(items, None)
                if nxt is not None:
                    pending.add(pool.submit(fetch, nxt))
    finally:
        stop.set()
        for f in pending:
            f.cancel()
        pool.shutdown(wait=True, cancel_futures=True)
    return WarmupResult(done_count, total, time.monotonic() - start)


def node_order(shards: Sequence[str], local_rank: int, local_world: int) -> list:
    """The distinct shards of a look-ahead window in the order THIS process should request them: rotated by its
    position on the node, so that ``local_world`` processes start on different shards."""
    distinct = list(OrderedDict.fromkeys(shards))
    if local_world <= 1 or not distinct:
        return distinct
    k = (local_rank * max(1, len(distinct) // local_world)) % len(distinct)
    return distinct[k:] + distinct[:k]


class ShardPrefetcher:
    def __init__(self, resolver, lookahead: int = 4, max_workers: int = 4, local_rank: int = 0, local_world: int = 1):
        if lookahead < 1 or max_workers < 1:
            raise DataContractError("prefetch depth and workers must be positive")
        self.resolver, self.lookahead = resolver, int(lookahead)
        self.local_rank, self.local_world = int(local_rank), int(local_world)
        self.pool = ThreadPoolExecutor(max_workers=max_workers, thread_name_prefix="shard-prefetch")
        self.pending: "OrderedDict[str, Future]" = OrderedDict()
        self.waited_s = 0.0                      # time the consumer actually blocked (0 when prefetch keeps up)

    def _submit(self, shard: str, size=None) -> None:
        if shard not in self.pending:
            self.pending[shard] = self.pool.submit(self.resolver.resolve, shard, size)

    def schedule(self, plan) -> None:
        self._submit(plan.shard, getattr(plan, "shard_size", None))

    def schedule_plans(self, plans: Sequence) -> None:
        for shard in node_order([p.shard for p in plans], self.local_rank, self.local_world):
            self._submit(shard)

    def wait(self, plan) -> Path:
        self.schedule(plan)
        t0 = time.monotonic()
        try:
            return self.pending[plan.shard].result()
        except BaseException:
            self.pending.pop(plan.shard, None)        # a failed transfer is retried by the next schedule
            raise
        finally:
            self.waited_s += time.monotonic() - t0

    def prepare(self, plan) -> Path:
        return self.wait(plan)

    def iterate(self, plans: Iterable) -> Iterator:
        """Yield ``(plan, local_shard_path)`` while keeping ``lookahead`` distinct shards in flight."""
        window, it = [], iter(plans)
        for plan in it:
            window.append(plan)
            self.schedule(plan)
            if len({p.shard for p in window}) > self.lookahead:
                head = window.pop(0)
                yield head, self.wait(head)
                self._trim(window)
        for head in window:
            yield head, self.wait(head)

    def _trim(self, window) -> None:
        live = {p.shard for p in window}
        for shard in [s for s, f in self.pending.items() if s not in live and f.done()]:
            del self.pending[shard]

    def close(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)
