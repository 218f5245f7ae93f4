"""The bucket store against a fake server (no network): identity, no-overwrite, resumable sessions, pagination."""
import base64
import hashlib
import json
import re
from urllib.parse import parse_qs, unquote, urlsplit

import pytest

from solarwm_b200.runtime.object_store import DirectoryStore, GCSStore, ObjectInfo, StoreError, relative_key, store_for


class FakeBucket:
    """Plays the JSON API: objects, resumable sessions, scripted failures."""

    def __init__(self):
        self.objects, self.sessions, self.log = {}, {}, []
        self.fail_next_put = 0           # transport failures to inject into chunk uploads
        self.lose_bytes = 0              # ... after which the session holds only this many bytes of the chunk
        self.page_size = 1000

    def __call__(self, method, path, body, headers):
        assert headers["Authorization"] == "Bearer tok"
        self.log.append((method, path.split("?")[0]))
        url = urlsplit(path)
        q = parse_qs(url.query)
        if url.path.startswith("/upload/") and "upload_id" not in q:          # open a session
            meta = json.loads(body)
            if meta["name"] in self.objects:
                return 412, {}, b""
            sid = f"s{len(self.sessions)}"
            self.sessions[sid] = {"name": meta["name"], "md5": meta["md5Hash"], "size": int(headers["X-Upload-Content-Length"]), "data": b""}
            return 200, {"location": f"https://storage.googleapis.com/upload/storage/v1/b/b/o?uploadType=resumable&upload_id={sid}"}, b""
        if url.path.startswith("/upload/"):
            s = self.sessions[q["upload_id"][0]]
            rng = headers["Content-Range"]
            if not rng.startswith("bytes */"):
                if self.fail_next_put:
                    self.fail_next_put -= 1
                    s["data"] += body[:self.lose_bytes]
                    raise OSError("connection reset")
                start = int(re.match(r"bytes (\d+)-", rng)[1])
                assert start == len(s["data"]), "the client must continue where the session is"
                s["data"] += body
            if len(s["data"]) == s["size"]:
                assert base64.b64encode(hashlib.md5(s["data"]).digest()).decode() == s["md5"]
                self.objects[s["name"]] = s["data"]
                return 200, {}, b"{}"
            return 308, ({"range": f"bytes=0-{len(s['data']) - 1}"} if s["data"] else {}), b""
        if url.path.endswith("/o"):                                            # list
            names = sorted(n for n in self.objects if n.startswith(q["prefix"][0]))
            start = int(q.get("pageToken", ["0"])[0])
            items = [{"name": n, "size": str(len(self.objects[n])), "md5Hash": ObjectInfo.of_bytes(self.objects[n]).md5}
                     for n in names[start:start + self.page_size]]
            out = {"items": items}
            if start + self.page_size < len(names):
                out["nextPageToken"] = str(start + self.page_size)
            return 200, {}, json.dumps(out).encode()
        name = unquote(url.path.split("/o/", 1)[1])
        if name not in self.objects:
            return 404, {}, b""
        if q.get("alt") == ["media"]:
            return 200, {}, self.objects[name]
        return 200, {}, json.dumps({"size": str(len(self.objects[name])), "md5Hash": ObjectInfo.of_bytes(self.objects[name]).md5}).encode()


def _store(bucket, **kw):
    return GCSStore("gs://b/runs/r1", token=lambda: "tok", transport=bucket, sleep=lambda s: None, **kw)


def test_put_is_idempotent_never_overwrites_and_streams_in_chunks(tmp_path):
    bucket = FakeBucket()
    st = _store(bucket, chunk=1000)
    f = tmp_path / "video.mp4"
    f.write_bytes(bytes(range(256)) * 13)                                     # 3,328 bytes -> 4 chunks
    assert st.put_file("val/step_1/video.mp4", f) is True
    assert bucket.objects["runs/r1/val/step_1/video.mp4"] == f.read_bytes()
    assert sum(1 for m, p in bucket.log if m == "PUT") == 4
    assert st.put_file("val/step_1/video.mp4", f) is False                    # same identity: nothing is sent
    with pytest.raises(StoreError) as err:
        st.put_bytes("val/step_1/video.mp4", b"other content")
    assert err.value.code == "object_content_conflict"
    assert st.metadata("val/step_1/video.mp4") == ObjectInfo.of_file(f) and st.metadata("missing") is None
    assert st.read("val/step_1/video.mp4") == f.read_bytes()
    with pytest.raises(StoreError):
        st.put_bytes("empty", b"")
    for bad in ("", "/abs", "a/../b", "a//b"):
        with pytest.raises(StoreError):
            relative_key(bad)
    with pytest.raises(StoreError):
        GCSStore("https://b/x", token=lambda: "t")


def test_an_interrupted_chunk_resumes_from_what_the_session_holds():
    bucket = FakeBucket()
    bucket.fail_next_put, bucket.lose_bytes = 1, 300                          # the first chunk dies after 300 bytes
    st = _store(bucket, chunk=1000)
    data = bytes(range(251)) * 10
    assert st.put_bytes("blob.bin", data) is True and bucket.objects["runs/r1/blob.bin"] == data
    probes = [h for h in bucket.log if h[0] == "PUT"]
    assert len(probes) >= 4                                                   # failed chunk, probe, then the rest
    stalled = FakeBucket()
    stalled.fail_next_put, stalled.lose_bytes = 99, 0                         # never acknowledges anything
    with pytest.raises(StoreError) as err:
        _store(stalled, chunk=1000).put_bytes("blob.bin", data)
    assert err.value.code == "upload_stalled"


def test_listing_is_paginated_and_retries_follow_the_status_class():
    bucket = FakeBucket()
    st = _store(bucket)
    for i in range(5):
        st.put_bytes(f"receipts/node-{i}.json", b"{%d}" % i)
    st.put_bytes("other/x", b"1")
    bucket.page_size = 2
    got = st.list("receipts")
    assert sorted(got) == [f"receipts/node-{i}.json" for i in range(5)] and got["receipts/node-3.json"].size == 3
    calls = {"n": 0}

    def flaky(method, path, body, headers):
        calls["n"] += 1
        if calls["n"] < 3:
            return 503, {}, b""
        return bucket(method, path, body, headers)

    assert GCSStore("gs://b/runs/r1", token=lambda: "tok", transport=flaky, sleep=lambda s: None).read("other/x") == b"1"
    with pytest.raises(StoreError) as err:
        GCSStore("gs://b/runs/r1", token=lambda: "tok", transport=lambda *a: (403, {}, b""), sleep=lambda s: None).read("other/x")
    assert err.value.code == "storage_http_403" and not err.value.retryable
    with pytest.raises(StoreError) as err:
        GCSStore("gs://b/runs/r1", token=lambda: "", transport=bucket).read("other/x")
    assert err.value.code == "storage_authentication_failed"


def test_directory_store_speaks_the_same_protocol(tmp_path):
    st = store_for(f"file://{tmp_path / 'out'}")
    assert isinstance(st, DirectoryStore) and st.put_bytes("a/b.json", b"{}") is True and st.put_bytes("a/b.json", b"{}") is False
    with pytest.raises(StoreError):
        st.put_bytes("a/b.json", b"[]")
    assert st.read("a/b.json") == b"{}" and list(st.list("a")) == ["a/b.json"] and st.metadata("nope") is None


def _node_view(root, step, name, slots, failed=(), total=4):
    import json as js

    d = root / "validation" / f"step_{step:06d}_{name}"
    for g in ("compare", "manifests", "errors"):
        (d / g).mkdir(parents=True, exist_ok=True)
    for s in slots:
        (d / "compare" / f"rank{s:03d}_round00_dp{s:03d}_clip_start000000.mp4").write_bytes(b"mp4-%d" % s)
        (d / "manifests" / f"rank_{s:03d}.json").write_text(js.dumps({"slot": s, "step": step, "pass": name}))
    for s in failed:
        (d / "errors" / f"rank_{s:03d}.json").write_text(js.dumps({"slot": s, "step": step, "pass": name, "error": "decode failed"}))
    (d / "compare" / "notes.txt").write_text("never uploaded")
    (d / "COMPLETE.json").write_text(js.dumps({"step": step, "pass": name, "slots": total}))
    return d


def test_two_nodes_publish_and_node_zero_finalizes_only_when_every_receipt_is_in(tmp_path):
    import json as js

    from solarwm_b200.runtime.validation_publish import ValidationPublisher, finalize, read_partition

    store = DirectoryStore(tmp_path / "bucket")
    n0, n1 = tmp_path / "n0", tmp_path / "n1"
    _node_view(n0, 100, "val", [0, 2])
    _node_view(n1, 100, "val", [1], failed=[3])
    p0 = ValidationPublisher(n0, store, node=0, nodes=2)
    first = p0.scan()
    assert first["passes"][0]["status"] == "published" and first["pending"] == 1 and first["passes"][0]["objects_sent"] == 4
    assert store.metadata("validation/step_000100_val/COMPLETE.json") is None
    assert store.metadata("validation/step_000100_val/compare/notes.txt") is None
    p1 = ValidationPublisher(n1, store, node=1, nodes=2)
    assert p1.scan()["passes"][0]["status"] == "published"
    done = p0.scan()
    assert done["passes"][0]["status"] == "partial" and done["partial"] == 1 and done["errors"] == 0
    marker = js.loads(store.read("validation/step_000100_val/COMPLETE.json"))
    assert marker["failed_slots"] == [3] and marker["ok_slots"] == 3 and marker["nodes"] == 2
    assert p0.scan()["passes"][0]["status"] == "partial"                      # cached; and a fresh publisher is idempotent
    again = ValidationPublisher(n0, store, node=0, nodes=2).scan()
    assert again["passes"][0] == {"pass": "step_000100_val", "status": "partial", "objects_sent": 0}
    # a stray object under the pass, or a slot claimed twice, blocks the marker
    like = read_partition(n0.resolve(), n0.resolve() / "validation" / "step_000100_val", node=0, nodes=2).receipt
    store.put_bytes("validation/step_000100_val/compare/rank009_x.mp4", b"stray")
    with pytest.raises(StoreError) as err:
        finalize(store, "validation/step_000100_val", like)
    assert err.value.code == "global_object_inventory_mismatch"


def test_local_partition_checks(tmp_path):
    import json as js

    from solarwm_b200.runtime.validation_publish import read_partition

    root = (tmp_path / "n").resolve()
    d = _node_view(root, 7, "val", [0, 1])
    part = read_partition(root, d, node=0, nodes=1)
    assert part.receipt["ok_slots"] == [0, 1] and len(part.uploads) == 4 and part.prefix == "validation/step_000007_val"
    (d / "manifests" / "rank_001.json").write_text(js.dumps({"slot": 1, "step": 7, "pass": "val", "access_token": "abc"}))
    with pytest.raises(StoreError) as err:
        read_partition(root, d, node=0, nodes=1)
    assert err.value.code == "credential_in_publication_json"
    (d / "manifests" / "rank_001.json").write_text(js.dumps({"slot": 0, "step": 7, "pass": "val"}))
    with pytest.raises(StoreError) as err:
        read_partition(root, d, node=0, nodes=1)
    assert err.value.code == "sample_identity_mismatch"
    (d / "manifests" / "rank_001.json").unlink()
    with pytest.raises(StoreError) as err:
        read_partition(root, d, node=0, nodes=1)
    assert err.value.code == "local_slot_inventory_mismatch"


def test_cli_publishes_a_run_directory(tmp_path, capsys):
    import json as js

    from solarwm_b200.cli import main

    _node_view(tmp_path / "run", 5, "val", [0, 1], total=2)
    assert main(["publish-validation", "--run-dir", str(tmp_path / "run"), "--destination", str(tmp_path / "dest")]) == 0
    report = js.loads(capsys.readouterr().out)
    assert report["passes"][0]["status"] == "complete"
    assert (tmp_path / "dest" / "validation" / "step_000005_val" / "COMPLETE.json").is_file()
