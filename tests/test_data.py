import io
import tarfile

import numpy as np
import pytest

from solarwm_b200.data import camera as cam
from solarwm_b200.data.archive import TarShardReader
from solarwm_b200.data.index import IndexRow, assert_disjoint, inventory, read_index, write_index
from solarwm_b200.data.sampling import (CanonicalSampler, ReaderIdentity, SamplingConfig, frame_offsets,
                                        plan_fingerprint)
from solarwm_b200.data.transport import LocalResolver, resolver_from_config
from solarwm_b200.errors import DataContractError


def _rows(n=24, shards=4):
    return [IndexRow.from_mapping(i, {"sample_id": f"s{i}", "key": f"k{i}", "shard": f"set/shards/{i % shards:03d}.tar",
                                      "epoch_repeats": 1 + (i % 3 == 0), "num_frames": 200, "fps": 24.0})
            for i in range(n)]


def test_index_round_trip_inventory_and_disjointness(tmp_path):
    rows = [r.values for r in _rows(5)]
    for name in ("i.jsonl", "i.jsonl.gz"):
        assert write_index(tmp_path / name, rows) == 5
        got = read_index(tmp_path / name)
        assert [r.sample_id for r in got] == [f"s{i}" for i in range(5)]
    a, b = inventory(tmp_path / "i.jsonl"), inventory(tmp_path / "i.jsonl.gz")
    assert a.rows == 5 and a.virtual_occurrences == 7 and a.ordered_row_digest == b.ordered_row_digest
    with pytest.raises(DataContractError):
        IndexRow.from_mapping(0, {"sample_id": "a", "key": "k", "shard": "../x.tar"})
    with pytest.raises(DataContractError):
        IndexRow.from_mapping(0, {"sample_id": "a", "key": "k", "shard": "x.tar", "epoch_repeats": 0})
    with pytest.raises(DataContractError):
        assert_disjoint(_rows(3), _rows(2))


def test_sampler_is_deterministic_and_partitions_occurrences():
    rows = _rows()
    cfg = SamplingConfig(seed=11, pixel_frames=81, shuffle_buffer=5)
    total = sum(r.epoch_repeats for r in rows)
    seen = []
    for rank in range(2):
        for worker in range(2):
            ident = ReaderIdentity(rank, 2, worker, 2)
            a = list(CanonicalSampler(rows, cfg, ident).iter_epoch(0))
            b = list(CanonicalSampler(rows, cfg, ident).iter_epoch(0))
            assert plan_fingerprint(a) == plan_fingerprint(b)
            seen += [(p.sample_id, p.repeat_ordinal) for p in a]
            assert all(0 <= p.start_frame and p.source_frame_indices[-1] < 200 for p in a)
    assert len(seen) == total and len(set(seen)) == total
    other = list(CanonicalSampler(rows, SamplingConfig(seed=12, pixel_frames=81, shuffle_buffer=5),
                                  ReaderIdentity(0, 2, 0, 2)).iter_epoch(0))
    mine = list(CanonicalSampler(rows, cfg, ReaderIdentity(0, 2, 0, 2)).iter_epoch(0))
    assert plan_fingerprint(other) != plan_fingerprint(mine)


def test_frame_resampling_fixed_start_and_node_shards():
    cfg = SamplingConfig(seed=0, pixel_frames=5, random_start=False, clip_seconds=0.25, output_fps=16.0)
    assert frame_offsets(cfg, 32.0).tolist() == [0, 2, 4, 6, 8]
    with pytest.raises(DataContractError):
        SamplingConfig(seed=0, pixel_frames=5, clip_seconds=1.0, output_fps=16.0)
    rows = [IndexRow.from_mapping(0, {"sample_id": "a", "key": "k", "shard": "x.tar", "num_frames": 50, "start_frame": 7})]
    p = next(CanonicalSampler(rows, SamplingConfig(seed=0, pixel_frames=4, random_start=False, fixed_start_from_index=True,
                                                   shuffle_buffer=1), ReaderIdentity(0, 1)).iter_epoch(0))
    assert p.source_frame_indices == (7, 8, 9, 10)
    rows = _rows(32, shards=8)
    rows.sort(key=lambda r: r.shard)
    cfg = SamplingConfig(seed=3, pixel_frames=81, partition_mode="node_shard")
    per_node = []
    for node in range(2):
        s = CanonicalSampler(rows, cfg, ReaderIdentity(node, 2, node_id=node, node_count=2))
        per_node.append({g[0] for g in s.node_shard_groups(0)})
    assert per_node[0].isdisjoint(per_node[1]) and len(per_node[0] | per_node[1]) == 8


def test_camera_conventions():
    rng = np.random.default_rng(0)
    from solarwm_b200.data.synthetic import random_camera_path

    c2w = random_camera_path(9, seed=1)
    inv = cam.invert_se3(c2w)
    assert np.allclose(inv @ c2w, np.eye(4), atol=1e-5)
    rel = cam.relative_w2c(c2w, "absolute_c2w")
    assert np.allclose(rel[0], np.eye(4), atol=1e-5)
    assert np.allclose(cam.relative_w2c(inv, "absolute_w2c"), rel, atol=1e-5)
    comp = cam.transform_translation(rel, "logd4")
    t, tc = np.linalg.norm(rel[1:, :3, 3], axis=-1), np.linalg.norm(comp[1:, :3, 3], axis=-1)
    assert np.allclose(tc, np.log1p(t) / 4.0, atol=1e-6) and np.allclose(comp[:, :3, :3], rel[:, :3, :3])
    far = rel.copy()
    far[3, :3, 3] = [30, 0, 0]
    with pytest.raises(cam.CameraGuardError):
        cam.CameraGuards().apply(far)
    cam.CameraGuards().apply(far, audit_rows=2)
    assert cam.causal_pixel_indices(81, 4).tolist() == [0] + list(range(1, 81, 4))
    tok = cam.camera_tokens(random_camera_path(81, 2), pixel_frames=81, temporal_stride=4, tokens_per_frame=3)
    assert tok["viewmats"].shape == (21 * 3, 4, 4) and tok["K"].shape == (63, 3, 3)
    P, Pinv = cam.prope_matrices(tok["viewmats"], tok["K"])
    assert np.allclose(P @ Pinv, np.eye(4), atol=1e-8)
    buf = io.BytesIO()
    np.savez(buf, c2w=c2w)
    m, storage = cam.load_camera_npz(buf.getvalue(), "c2w")
    assert storage == "absolute_c2w" and m.shape == (9, 4, 4)
    with pytest.raises(DataContractError):
        cam.load_camera_npz(buf.getvalue(), "w2c")


def test_tar_reader_and_local_transport(tmp_path):
    shard = tmp_path / "root" / "a" / "0.tar"
    shard.parent.mkdir(parents=True)
    with tarfile.open(shard, "w") as tf:
        for name, data in (("s0.video.bin", b"VID"), ("s0.camera.npz", b"CAM")):
            info = tarfile.TarInfo(name)
            info.size = len(data)
            tf.addfile(info, io.BytesIO(data))
    res = resolver_from_config({"transport": {"kind": "local", "root": str(tmp_path / "root")}})
    assert isinstance(res, LocalResolver)
    path = res.resolve("a/0.tar", expected_size=shard.stat().st_size)
    reader = TarShardReader(max_open=1)
    s = reader.read_sample(path, "s0", {"video": "s0.video.bin", "camera": "s0.camera.npz"})
    assert s.members == {"video": b"VID", "camera": b"CAM"}
    with pytest.raises(DataContractError):
        reader.read_members(path, ["nope"])
    with pytest.raises(DataContractError):
        res.resolve("a/1.tar")
    with pytest.raises(DataContractError):
        resolver_from_config({"transport": {"root": "gs://bucket/x"}})
    reader.close()


def test_window_index_build_query_and_slices(tmp_path):
    import pytest

    from solarwm_b200.data.windows import WindowIndex, build_index, enumerate_windows
    from solarwm_b200.errors import DataContractError

    assert list(enumerate_windows(10, 4, 3)) == [0, 3, 6]
    clips = [{"sample_id": "a", "shard": "s0.tar", "num_frames": 10}, {"sample_id": "b", "shard": "s1.tar", "num_frames": 3},
             {"sample_id": "c", "shard": "s1.tar", "num_frames": 7}]
    path = tmp_path / "windows.sqlite"
    assert build_index(path, clips, window=4, stride=3) == 5
    idx = WindowIndex(path)
    assert len(idx) == 5 and idx[3] == (3, "c", "s1.tar", 0, 4)
    assert [w.ordinal for w in idx.slice(1, 2)] == [1, 3]
    idx.close()
    with pytest.raises(DataContractError):
        build_index(path, clips, window=4, stride=3)
    with pytest.raises(DataContractError):
        build_index(tmp_path / "none.sqlite", clips, window=64, stride=1)
    assert not (tmp_path / "none.sqlite").exists()


def test_raw_video_decode_matches_written_frames(tmp_path):
    import numpy as np
    import pytest

    cv2 = pytest.importorskip("cv2")
    from solarwm_b200.data import raw_video
    from solarwm_b200.errors import DataContractError

    path = str(tmp_path / "clip.mp4")
    w = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 24.0, (64, 48))
    assert w.isOpened()
    for i in range(80):
        w.write(np.full((48, 64, 3), (i * 3, 255 - i * 3, 40), np.uint8))     # BGR
    w.release()
    blob = open(path, "rb").read()
    info = raw_video.probe(blob)
    assert info["frames"] == 80 and abs(info["fps"] - 24.0) < 1e-3 and (info["height"], info["width"]) == (48, 64)
    idx = [0, 2, 2, 5, 70]                                   # a repeat and a jump beyond the seek threshold
    got = raw_video.decode_frames(blob, idx)
    assert got.shape == (5, 48, 64, 3) and got.dtype == np.uint8
    for j, i in enumerate(idx):                              # RGB order, lossy codec: a few grey levels of slack
        assert abs(float(got[j, ..., 2].mean()) - i * 3) < 6 and abs(float(got[j, ..., 0].mean()) - 40) < 6
    assert raw_video.decode_frames(blob, [1, 3], size=(24, 32)).shape == (2, 24, 32, 3)
    clip = raw_video.load_clip("a.mp4", blob, 4, offsets=[0, 3, 6, 9])
    assert clip.shape == (4, 48, 64, 3)
    buf = __import__("io").BytesIO()
    np.save(buf, np.zeros((5, 4, 4, 3), np.uint8))
    assert raw_video.load_clip("a.npy", buf.getvalue(), 3).shape == (3, 4, 4, 3)
    with pytest.raises(DataContractError):
        raw_video.decode_frames(blob, [3, 1])
    with pytest.raises(DataContractError):
        raw_video.decode_frames(blob, [200])
    with pytest.raises(DataContractError):
        raw_video.decode_frames(b"not a video", [0])


def test_plan_multiplexer_interleaves_workers_and_resumes_anywhere():
    """Two loader workers of one rank: batches alternate between them, each worker follows its own canonical plan
    stream across epochs, and a state saved at ANY point continues with exactly the plans an uninterrupted run sees."""
    from solarwm_b200.data.plan_mux import PlanMultiplexer
    from solarwm_b200.runtime.topology import Topology

    rows, cfg, topo = _rows(10, 2), SamplingConfig(seed=3, pixel_frames=81, shuffle_buffer=4), Topology(2, 1, 2, 1, 1)
    full = PlanMultiplexer(rows, cfg, topo, num_workers=2)
    stream = [full.next_batch(2) for _ in range(12)]                      # three epochs' worth for this rank
    workers = [p.worker_id for batch in stream for p in batch]
    assert workers[:8] == [0, 0, 1, 1, 0, 0, 1, 1] and {p.reader_rank for b in stream for p in b} == {1}
    # each worker's sub-stream is the canonical sampler's, epoch after epoch
    for w in range(2):
        ref = CanonicalSampler(rows, cfg, ReaderIdentity.from_topology(topo, worker_id=w, num_workers=2))
        want = [p for e in range(4) for p in ref.iter_epoch(e)]
        got = [p for batch in stream for p in batch if p.worker_id == w]
        assert got == want[:len(got)] and max(p.epoch for p in got) >= 1
    for cut in (0, 1, 5, 8):                                              # including a cut at an epoch boundary
        a = PlanMultiplexer(rows, cfg, topo, num_workers=2)
        for _ in range(cut):
            a.next_batch(2)
        state = a.state_dict()
        assert state["schema"] == "solarwm.plan-multiplexer.v1"
        import json
        b = PlanMultiplexer(rows, cfg, topo, num_workers=2)
        b.load_state_dict(json.loads(json.dumps(state)))                  # the state is plain JSON
        assert [b.next_batch(2) for _ in range(12 - cut)] == stream[cut:]
    m = PlanMultiplexer(rows, cfg, topo, num_workers=2)
    with pytest.raises(DataContractError):
        m.finish_batch(1)                                                 # worker 0's batch comes first
    with pytest.raises(DataContractError):
        PlanMultiplexer(rows, cfg, topo, num_workers=3).load_state_dict(m.state_dict())
    with pytest.raises(DataContractError):
        PlanMultiplexer(_rows(14, 2), cfg, topo, num_workers=2).load_state_dict(m.state_dict())   # another index
    with pytest.raises(DataContractError):
        m.load_state_dict({"schema": "other"})
