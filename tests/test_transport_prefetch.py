"""Bucket downloader (against a fake opener: no network), token provider, cache warm-up and the prefetcher."""
import io
import json
import threading
import time
import urllib.error
from types import SimpleNamespace

import pytest

from solarwm_b200.data.prefetch import ShardPrefetcher, node_order, warm_cache
from solarwm_b200.data.transport import (CachedRemoteResolver, DownloadTimeout, GCSRestDownloader, TokenProvider, is_transient,
                                         parse_gs_uri)
from solarwm_b200.errors import DataContractError


class _Response(io.BytesIO):
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _http(code):
    return urllib.error.HTTPError("u", code, "x", {}, None)


def test_token_sources_in_order(tmp_path):
    f = tmp_path / "tok"
    f.write_text(" from-file \n")
    assert TokenProvider(f, environ={"GOOGLE_OAUTH_ACCESS_TOKEN": "env"})() == "from-file"
    assert TokenProvider(tmp_path / "none", environ={"GOOGLE_OAUTH_ACCESS_TOKEN": "env"})() == "env"
    seen = []

    def meta(request, timeout):
        seen.append((request.full_url, dict(request.header_items())))
        return _Response(json.dumps({"access_token": "meta"}).encode())

    assert TokenProvider(opener=meta, environ={})() == "meta" and seen[0][1]["Metadata-flavor"] == "Google"
    with pytest.raises(DataContractError):
        TokenProvider(opener=lambda r, timeout: _Response(b"{}"), environ={})()
    with pytest.raises(DataContractError):
        TokenProvider(opener=lambda r, timeout: (_ for _ in ()).throw(OSError("no route")), environ={})()


def test_downloader_retries_the_right_failures(tmp_path):
    assert parse_gs_uri("gs://b/a/b c.tar") == ("b", "a/b c.tar")
    assert GCSRestDownloader.media_url("gs://b/a/b c.tar").endswith("/b/b/o/a%2Fb%20c.tar?alt=media")
    with pytest.raises(DataContractError):
        parse_gs_uri("gs://bucket-only")
    assert is_transient(_http(503)) and is_transient(_http(429)) and is_transient(TimeoutError()) and not is_transient(_http(404))
    sleeps, calls = [], []

    def flaky(request, timeout):
        calls.append(request.get_header("Authorization"))
        if len(calls) == 1:
            raise _http(503)
        if len(calls) == 2:
            raise _http(401)                                     # a rotated token: retried with a fresh one
        return _Response(b"shard-bytes")

    tokens = iter(["t1", "t2", "t3"])
    dl = GCSRestDownloader(lambda: next(tokens), opener=flaky, sleep=sleeps.append)
    assert dl("gs://b/x.tar", tmp_path / "x") == 11 and (tmp_path / "x").read_bytes() == b"shard-bytes"
    assert calls == ["Bearer t1", "Bearer t2", "Bearer t3"] and sleeps == [0.5, 1.0]
    gone = GCSRestDownloader(lambda: "t", opener=lambda r, timeout: (_ for _ in ()).throw(_http(404)), sleep=sleeps.append)
    with pytest.raises(DataContractError) as err:
        gone("gs://b/missing.tar", tmp_path / "m")
    assert not isinstance(err.value, DownloadTimeout) and len(sleeps) == 2           # a 404 is not retried
    always = GCSRestDownloader(lambda: "t", attempts=3, opener=lambda r, timeout: (_ for _ in ()).throw(_http(500)), sleep=lambda s: None)
    with pytest.raises(DownloadTimeout):
        always("gs://b/x.tar", tmp_path / "y")
    clock = iter([0.0, 0.0, 400.0, 400.0, 400.0])
    late = GCSRestDownloader(lambda: "t", opener=lambda r, timeout: _Response(b"z"), clock=lambda: next(clock), time_budget_s=300)
    with pytest.raises(DownloadTimeout):
        late("gs://b/x.tar", tmp_path / "z")


def test_warm_up_checks_capacity_before_any_transfer_and_waits_out_timeouts(tmp_path):
    served = {}

    def downloader(uri, path):
        served[uri] = served.get(uri, 0) + 1
        if uri.endswith("s1.tar") and served[uri] == 1:
            raise DownloadTimeout("try again")
        with open(path, "wb") as fh:
            fh.write(b"x" * 10)

    res = CachedRemoteResolver("gs://bucket/data", tmp_path / "cache", downloader, max_cache_bytes=25)
    rows = [SimpleNamespace(shard=f"s{i % 3}.tar", values={"shard_size": 10}) for i in range(6)]
    with pytest.raises(DataContractError):                                        # 30 bytes into a 25-byte cache
        warm_cache(res, rows)
    assert served == {}
    ticks = []
    done = warm_cache(res, rows[:2] * 2, max_workers=2, progress=lambda a, b: ticks.append((a, b)))
    assert (done.shards, done.bytes) == (2, 20) and served["gs://bucket/data/s1.tar"] == 2 and ticks[-1] == (2, 2)
    with pytest.raises(DataContractError):
        warm_cache(res, [SimpleNamespace(shard="a", values={"shard_size": 1}), SimpleNamespace(shard="a", values={"shard_size": 2})])
    with pytest.raises(DownloadTimeout):                                          # the overall deadline ends the waiting
        warm_cache(SimpleNamespace(resolve=lambda s, n: (_ for _ in ()).throw(DownloadTimeout("slow"))), rows[:1], timeout_s=0.3)


def test_prefetcher_schedule_wait_and_node_order():
    assert node_order(["a", "b", "a", "c", "d"], 0, 2) == ["a", "b", "c", "d"]
    assert node_order(["a", "b", "a", "c", "d"], 1, 2) == ["c", "d", "a", "b"]
    order, gate = [], threading.Event()

    class Resolver:
        def resolve(self, shard, size=None):
            order.append(shard)
            if shard == "bad":
                raise DataContractError("corrupt")
            gate.wait(1.0)
            return f"/l/{shard}"

    pf = ShardPrefetcher(Resolver(), lookahead=2, max_workers=1, local_rank=1, local_world=2)
    plans = [SimpleNamespace(shard=s) for s in ("a", "b", "c", "d")]
    pf.schedule_plans(plans)
    gate.set()
    assert pf.wait(plans[0]) == "/l/a" and order[0] == "c"                        # this process started elsewhere
    assert pf.prepare(plans[3]) == "/l/d" and len(order) == 4                     # nothing is fetched twice
    with pytest.raises(DataContractError):
        pf.wait(SimpleNamespace(shard="bad"))
    with pytest.raises(DataContractError):                                        # a failed transfer is tried again
        pf.wait(SimpleNamespace(shard="bad"))
    assert order.count("bad") == 2 and pf.waited_s >= 0.0
    pf.close()
