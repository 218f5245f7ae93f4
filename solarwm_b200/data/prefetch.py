"""Shard prefetching: resolve the shards of upcoming sample plans on a small thread pool so the
training loop never waits on transport (reference: solar/data/prefetch.py:30-346)."""
from __future__ import annotations

from collections import OrderedDict
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Iterable, Iterator


def warm_cache(resolver, rows, max_workers: int = 8) -> int:
    """Resolve every distinct shard of ``rows`` once; returns the number of shards touched."""
    shards = OrderedDict((r.shard, r.values.get("shard_size")) for r in rows)
    with ThreadPoolExecutor(max_workers=max_workers) as pool:
        list(pool.map(lambda kv: resolver.resolve(kv[0], kv[1]), shards.items()))
    return len(shards)


class ShardPrefetcher:
    def __init__(self, resolver, lookahead: int = 4, max_workers: int = 4):
        self.resolver, self.lookahead = resolver, max(int(lookahead), 1)
        self.pool = ThreadPoolExecutor(max_workers=max_workers)
        self.pending: "OrderedDict[str, Future]" = OrderedDict()

    def _submit(self, shard: str) -> None:
        if shard not in self.pending:
            self.pending[shard] = self.pool.submit(self.resolver.resolve, shard)

    def iterate(self, plans: Iterable) -> Iterator:
        """Yield ``(plan, local_shard_path)`` while keeping ``lookahead`` distinct shards in flight."""
        window, it = [], iter(plans)
        for plan in it:
            window.append(plan)
            self._submit(plan.shard)
            if len({p.shard for p in window}) > self.lookahead:
                head = window.pop(0)
                yield head, self.pending[head.shard].result()
                self._trim(window)
        for head in window:
            yield head, self.pending[head.shard].result()

    def _trim(self, window) -> None:
        live = {p.shard for p in window}
        for shard in [s for s, f in self.pending.items() if s not in live and f.done()]:
            del self.pending[shard]

    def close(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)
