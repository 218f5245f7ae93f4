"""Fragmented-MP4 preview delivery on synthetic box streams (no encoder binary is needed)."""
import struct

import pytest

from solarwm_b200.serve.fragments import (FragmentedPreviewWriter, FragmentSplitter, MediaStore, TraceIndex,
                                          fragment_sample_count, iter_boxes)


def box(kind: bytes, body: bytes = b"") -> bytes:
    return struct.pack(">I4s", 8 + len(body), kind) + body


def moof(samples: int) -> bytes:
    trun = box(b"trun", struct.pack(">II", 0, samples) + b"\0" * 4)
    return box(b"moof", box(b"mfhd", b"\0" * 8) + box(b"traf", box(b"tfhd", b"\0" * 8) + trun))


def stream(fragments):
    data = box(b"ftyp", b"isom") + box(b"moov", b"m" * 40)
    for i, n in enumerate(fragments):
        data += moof(n) + box(b"mdat", bytes([i]) * (50 + i))
    return data


def test_boxes_and_sample_counts():
    assert [k for k, _ in iter_boxes(box(b"ftyp", b"x") + box(b"free"))] == [b"ftyp", b"free"]
    assert fragment_sample_count(moof(4)) == 4
    with pytest.raises(ValueError):
        list(iter_boxes(box(b"ftyp", b"x")[:-1]))
    with pytest.raises(ValueError):
        fragment_sample_count(moof(0))


@pytest.mark.parametrize("chunk", [1, 7, 64, 10 ** 6])
def test_splitter_is_independent_of_chunking(chunk):
    data, sp, out = stream([4, 4, 1]), FragmentSplitter(), []
    for i in range(0, len(data), chunk):
        out += sp.feed(data[i:i + chunk])
    sp.finish()
    assert [(k, n) for k, _, n in out] == [("init", 0), ("fragment", 4), ("fragment", 4), ("fragment", 1)]
    assert b"".join(d for _, d, _ in out) == data
    cut = FragmentSplitter()
    cut.feed(data[:-10])
    with pytest.raises(ValueError):
        cut.finish()                                               # the stream ended inside a fragment
    with pytest.raises(ValueError):
        FragmentSplitter().feed(box(b"mdat", b"x"))               # media before the initialisation segment


def test_store_serves_fragments_by_cursor_while_live_and_after(tmp_path):
    store = MediaStore(tmp_path)
    w = FragmentedPreviewWriter(store, "harbour_01", 3)
    data = stream([4, 4, 4, 2])
    assert w.write(data[:200]) >= 1
    live = store.fragments("harbour_01", 3, 0, limit=8)
    assert live["init"] == data[:len(box(b"ftyp", b"isom") + box(b"moov", b"m" * 40))] and not live["done"]
    n_live = len(live["rows"])
    assert n_live >= 1 and live["rows"][0]["first"] == 0 and live["data"][0][4:8] == b"moof"
    w.write(data[200:])
    w.finish()
    rest = store.fragments("harbour_01", 3, live["next_cursor"], limit=8)          # resume where the client stopped
    assert rest["done"] and rest["produced"] == 4 and n_live + len(rest["rows"]) == 4
    assert [r["first"] for r in live["rows"] + rest["rows"]] == [0, 4, 8, 12]
    assert b"".join(live["data"] + rest["data"]) == data[len(live["init"]):]
    assert (tmp_path / "harbour_01-session-3-live.mp4").read_bytes() == data        # renamed when finished
    one = store.fragments("harbour_01", 3, 2, limit=1)
    assert [r["serial"] for r in one["rows"]] == [2] and one["init"] is None and one["next_cursor"] == 3
    for bad in (("../x", 3, 0), ("harbour_01", 0, 0), ("harbour_01", 3, -1)):
        with pytest.raises(ValueError):
            store.fragments(*bad)
    with pytest.raises(ValueError):
        store.fragments("harbour_01", 3, 9)                                        # beyond what was produced
    with pytest.raises(FileExistsError):
        FragmentedPreviewWriter(store, "harbour_01", 3)                            # an owned, fresh output only


def test_trace_index_window_gaps_and_unclean_ends(tmp_path):
    store = MediaStore(tmp_path)
    w = FragmentedPreviewWriter(store, "a", 1)
    w.write(stream([1] * 12))
    idx = TraceIndex(store.paths("a", 1)[2], capacity=4)
    rows, produced, done = idx.batch(0, 3)                          # older than the 4-row window: read from the file
    assert [r["serial"] for r in rows] == [0, 1, 2] and produced == 12 and not done
    assert [r["serial"] for r in idx.batch(9, 8)[0]] == [9, 10, 11]
    w.finish(rc=1, error="encoder died")
    with pytest.raises(ValueError):
        idx.batch(0, 1)
    bad = tmp_path / "gap.jsonl"
    bad.write_text('{"event": "fragment", "serial": 1, "offset": 0, "first": 0, "count": 1, "length": 10}\n')
    with pytest.raises(ValueError):
        TraceIndex(bad).batch(0, 1)


def test_media_endpoint_over_http(tmp_path):
    import base64
    import json
    import urllib.error
    import urllib.request

    from solarwm_b200.serve.web import make_server, serve_in_thread

    store = MediaStore(tmp_path)
    w = FragmentedPreviewWriter(store, "scene", 1)
    data = stream([2, 2])
    w.write(data)
    w.finish()

    class State:
        def snapshot(self):
            return {}

    server = make_server(State(), None, media=store, port=0)
    serve_in_thread(server)
    base = f"http://127.0.0.1:{server.server_address[1]}"
    try:
        got = json.loads(urllib.request.urlopen(f"{base}/media?scene=scene&sequence=1&cursor=0&limit=4").read())
        assert got["done"] and got["next_cursor"] == 2 and base64.b64decode(got["init"]) + b"".join(
            base64.b64decode(b) for b in got["data"]) == data
        for query, code in (("scene=../etc&sequence=1", 400), ("scene=missing&sequence=1", 404)):
            with pytest.raises(urllib.error.HTTPError) as err:
                urllib.request.urlopen(f"{base}/media?{query}")
            assert err.value.code == code
    finally:
        server.shutdown()
