import os
import random
import threading

import numpy as np
import pytest

from solarwm_b200.errors import BackendContractError, CheckpointError, ConfigurationError
from solarwm_b200.runtime import create_only, distributed as rdist, output_layout, provenance, randomness, safe_state
from solarwm_b200.runtime.topology import Topology


def test_topology_rank_algebra():
    t = Topology(16, 11, 8, 3, 4)
    assert (t.dp_rank, t.sp_rank, t.dp_size, t.node_rank, t.num_nodes) == (2, 3, 4, 1, 2)
    assert t.sp_group_ranks() == (8, 9, 10, 11) and t.dp_group_ranks() == (3, 7, 11, 15)
    env = {"WORLD_SIZE": "8", "RANK": "5", "LOCAL_WORLD_SIZE": "8", "LOCAL_RANK": "5"}
    assert Topology.from_environ(2, env).dp_rank == 2
    with pytest.raises(ConfigurationError):
        Topology(8, 0, 8, 0, 3)
    with pytest.raises(ConfigurationError):
        Topology.from_environ(1, {})


class FakeDist:
    """Stands in for torch.distributed: every rank's record is supplied up front."""

    def __init__(self, rank, world, records=None, broadcast_value=None):
        self.rank, self.world, self.records, self.broadcast_value = rank, world, records, broadcast_value
        self.ran_broadcast = False

    def is_initialized(self):
        return True

    def get_rank(self):
        return self.rank

    def get_world_size(self):
        return self.world

    def all_gather_object(self, out, local):
        for i in range(self.world):
            out[i] = local if i == self.rank else self.records[i]

    def broadcast_object_list(self, box, src=0):
        self.ran_broadcast = True
        if self.rank != src:
            box[0] = self.broadcast_value


def test_collective_error_is_rank_sorted_text_on_every_rank():
    records = {0: (0, ""), 1: (1, "ValueError: bad shard"), 2: (2, ""), 3: (3, "OSError: disk")}
    messages = []
    for rank in range(4):
        d = FakeDist(rank, 4, records)
        with pytest.raises(BackendContractError) as e:
            rdist.propagate_collective_error(records[rank][1], dist=d, label="phase")
        messages.append(str(e.value))
    assert len(set(messages)) == 1
    assert messages[0] == "phase failed collectively: rank 1: ValueError: bad shard | rank 3: OSError: disk"


def test_collective_call_chains_local_exception_and_rank_zero_call():
    d = FakeDist(1, 2, {0: (0, "")})
    with pytest.raises(BackendContractError) as e:
        rdist.collective_call(lambda: (_ for _ in ()).throw(KeyError("k")), dist=d, label="load")
    assert isinstance(e.value.__cause__, KeyError) and "rank 1: KeyError" in str(e.value)
    ran = []
    d1 = FakeDist(1, 2, {0: (0, "")}, broadcast_value="from-zero")
    assert rdist.collective_rank_zero_call(lambda: ran.append(1) or "mine", dist=d1, label="x") == "from-zero"
    assert ran == [] and d1.ran_broadcast
    d0 = FakeDist(0, 2, {1: (1, "")})
    assert rdist.collective_rank_zero_call(lambda: "zero", dist=d0, label="x") == "zero"
    assert rdist.collective_call(lambda: 5, dist=None, label="single") == 5


def test_malformed_exchange_and_fingerprints():
    with pytest.raises(BackendContractError, match="malformed"):
        rdist.propagate_collective_error("", dist=FakeDist(0, 2, {1: "oops"}), label="p")
    with pytest.raises(BackendContractError, match="every raw rank"):
        rdist.propagate_collective_error("", dist=FakeDist(0, 2, {1: (0, "")}), label="p")
    a = rdist.identity_fingerprint({"s": ["a"], "n": [1]})
    assert rdist.assert_peer_fingerprints([a, a]) == a
    with pytest.raises(BackendContractError):
        rdist.assert_peer_fingerprints([a, rdist.identity_fingerprint({"s": ["b"], "n": [1]})])
    assert rdist.gather_and_assert_sp_identity({"x": 1}, sp_size=1) == rdist.identity_fingerprint({"x": 1})


def test_create_only_publish_race_winner_is_never_replaced(tmp_path):
    results = []

    def publisher(i):
        staging = tmp_path / f".stage{i}"
        staging.mkdir()
        (staging / "who").write_text(str(i))
        try:
            create_only.publish_directory_no_replace(staging, tmp_path / "public")
            results.append(("won", i))
        except FileExistsError:
            results.append(("lost", i))

    threads = [threading.Thread(target=publisher, args=(i,)) for i in range(6)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    winners = [i for s, i in results if s == "won"]
    assert len(winners) == 1 and (tmp_path / "public" / "who").read_text() == str(winners[0])
    create_only.write_file_create_only(tmp_path / "f.bin", b"one")
    with pytest.raises(FileExistsError):
        create_only.write_file_create_only(tmp_path / "f.bin", b"two")
    assert (tmp_path / "f.bin").read_bytes() == b"one"
    create_only.link_file_create_only(tmp_path / "f.bin", tmp_path / "g.bin")
    with pytest.raises(FileExistsError):
        create_only.link_file_create_only(tmp_path / "f.bin", tmp_path / "g.bin")
    src = tmp_path / "a"
    src.write_text("a")
    (tmp_path / "b").write_text("b")
    with pytest.raises(FileExistsError):
        create_only.rename_noreplace(src, tmp_path / "b")


def test_rng_state_round_trip_is_plain_data():
    random.seed(7)
    np.random.seed(7)
    enc_p, enc_n = safe_state.encode_python_rng(), safe_state.encode_numpy_rng()

    def plain(v):
        if isinstance(v, dict):
            return all(isinstance(k, str) and plain(x) for k, x in v.items())
        if isinstance(v, list):
            return all(plain(x) for x in v)
        return v is None or isinstance(v, (int, float, str))

    assert plain(enc_p) and plain(enc_n)
    want = (random.random(), np.random.rand())
    random.random(), np.random.rand()
    safe_state.restore_python_rng(enc_p)
    safe_state.restore_numpy_rng(enc_n)
    assert (random.random(), np.random.rand()) == want
    with pytest.raises(CheckpointError):
        safe_state.decode_python_rng({"schema": "other"})


def test_seed_domains_layout_and_secrets():
    assert randomness.objective_seed(3, 0) == 300009 and randomness.objective_seed(3, 2) == 300009 + 2048
    assert randomness.model_init_seed("minimax_h3", 1) != randomness.model_init_seed("ltx25_video", 1)
    assert randomness.stable_validation_seed("a", 1) == randomness.stable_validation_seed("a", 1)
    assert output_layout.checkpoint_model_dir("/o", 12).name == "checkpoint_model_000012"
    assert output_layout.public_validation_dir("/o", 5, "ema").as_posix() == "/o/validation/step_000005_ema"
    assert output_layout.events_path("/o", 3).name == "rank-00003.jsonl"
    assert output_layout.inference_layout({"inference": {"length_policy": "camera"}}) == "dataset_triplet_v1"
    with pytest.raises(ConfigurationError):
        output_layout.public_validation_dir("/o", 1, "../x")
    provenance.reject_inline_secrets({"data": {"token_file": "/secrets/t"}})
    with pytest.raises(ConfigurationError):
        provenance.reject_inline_secrets({"data": {"api_key": "abc123"}})
    with pytest.raises(ConfigurationError):
        provenance.reject_inline_secrets({"x": ["ghp_" + "a" * 36]})


def test_validation_publish_partition_and_receipts(tmp_path):
    import json

    import pytest

    from solarwm_b200.errors import SolarWMError
    from solarwm_b200.runtime.validation_publish import owner_node, publish_validation

    src = tmp_path / "validation" / "step_000010_main"
    (src / "slot-000000").mkdir(parents=True)
    (src / "slot-000000" / "video.mp4").write_bytes(b"abc")
    (src / "slot-000000" / "manifest.json").write_text("{}")
    (src / "COMPLETE.json").write_text("{}")
    dest = tmp_path / "published"
    total = 0
    for node in range(2):
        out = publish_validation(src, f"file://{dest}", node=node, nodes=2)
        total += out["objects_sent"]
    assert total == 3
    assert (dest / "step_000010_main" / "slot-000000" / "video.mp4").read_bytes() == b"abc"
    receipt = json.loads((src / ".published" / "node-0000.json").read_text())
    assert all(owner_node(o["key"].split("/", 1)[1], 2) == 0 for o in receipt["objects"])
    again = publish_validation(src, f"file://{dest}", node=0, nodes=2)       # re-runnable
    assert again["skipped_passes"] == 1 and again["objects_sent"] == 0
    with pytest.raises(SolarWMError):
        publish_validation(tmp_path / "validation", f"file://{dest}", node=2, nodes=2)


def test_gcs_uploader_create_only_and_retry():
    import io
    import json
    import urllib.error

    import pytest

    from solarwm_b200.runtime.gcs_upload import GCSUploader, UploadError

    calls = []

    class _Resp(io.BytesIO):
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    def opener(req):
        calls.append(req)
        if len(calls) == 1:
            raise urllib.error.HTTPError(req.full_url, 503, "busy", {}, None)
        if "exists" in req.full_url:
            raise urllib.error.HTTPError(req.full_url, 412, "precondition", {}, None)
        return _Resp(json.dumps({"generation": "42"}).encode())

    import tempfile

    with tempfile.NamedTemporaryFile() as fh:
        fh.write(b"payload")
        fh.flush()
        up = GCSUploader("bucket", lambda: "tok", prefix="runs/x", opener=opener, sleep=lambda s: None)
        r = up.upload(fh.name, "a/b.bin")
        assert r["generation"] == "42" and r["key"] == "runs/x/a/b.bin" and len(calls) == 2
        assert "ifGenerationMatch=0" in calls[-1].full_url and calls[-1].headers["Authorization"] == "Bearer tok"
        with pytest.raises(UploadError):
            up.upload(fh.name, "exists.bin")


def test_balanced_descending_sequence_partition():
    import pytest

    from solarwm_b200.parallel.ulysses import balanced_bounds, balanced_lengths

    assert balanced_lengths(5040, 8) == [630] * 8
    lens = balanced_lengths(2108, 8)                       # 1100 prompt tokens + 1008 anchor rows
    assert sum(lens) == 2108 and lens == sorted(lens, reverse=True) and lens[0] - lens[-1] <= 1
    spans = [balanced_bounds(2108, 8, r) for r in range(8)]
    assert spans[0][0] == 0 and spans[-1][1] == 2108 and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    with pytest.raises(ValueError):
        balanced_lengths(3, 8)


def test_train_section_maps_to_activation_and_sharding_options():
    import pytest

    from solarwm_b200.backends.wan22.runtime import activation_and_sharding_options as opts
    from solarwm_b200.errors import ConfigurationError

    assert opts({}, 1) == dict(checkpointing="none", keep_blocks=0, lean_kept=False, zero=False, zero_transport="collective",
                               shard_params=False, cuda_graph=False)
    assert opts({"fsdp": {"activation_checkpointing": True}}, 8)["checkpointing"] == "full"
    assert opts({"fsdp": {"activation_checkpointing": True, "saved_attention_blocks": 30}}, 8)["checkpointing"] == "selective"
    assert opts({"fsdp": {"activation_checkpointing": "selective"}, "activation_memory": {"keep_blocks": 19, "lean": True}}, 1) == \
        dict(checkpointing="selective", keep_blocks=19, lean_kept=True, zero=False, zero_transport="collective",
             shard_params=False, cuda_graph=False)
    sharded = opts({"zero": {"enabled": True, "transport": "fused"}, "fsdp": {"shard_parameters": True}, "cuda_graph": True}, 8)
    assert sharded["shard_params"] is True and sharded["cuda_graph"] is True
    assert opts({"zero": {"enabled": True, "transport": "fused"}, "fsdp": {"shard_parameters": True}}, 1)["shard_params"] is False
    with pytest.raises(ConfigurationError):                                  # parameter sharding rides the fused transport
        opts({"zero": {"enabled": True}, "fsdp": {"shard_parameters": True}}, 8)
    assert opts({"zero": {"enabled": True, "transport": "fused"}}, 8)["zero"] is True
    assert opts({"zero": {"enabled": True}}, 1)["zero"] is False             # one rank: nothing to shard over
    assert opts({"fsdp": {"enabled": True}}, 2)["zero"] is True
    with pytest.raises(ConfigurationError):
        opts({"fsdp": {"activation_checkpointing": "sometimes"}}, 1)
    with pytest.raises(ConfigurationError):
        opts({"zero": {"transport": "smoke-signals"}}, 2)


def test_device_wait_failure_is_raised_by_every_rank_with_one_message():
    """A faked status word: rank 1's bounded wait gave up (code 5); both ranks must raise the same text, and a clean
    exchange raises nothing."""
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.runtime.distributed import raise_if_device_wait_failed

    class FakeDist:
        def __init__(self, rank, records):
            self.rank, self.records = rank, records

        def is_initialized(self):
            return True

        def get_rank(self):
            return self.rank

        def get_world_size(self):
            return 2

        def all_gather_object(self, out, mine):
            self.records[self.rank] = mine
            out[:] = [self.records[0], self.records[1]]

    codes = {0: 0, 1: 5}
    messages = []
    for rank in (0, 1):
        records = {r: (r, "" if codes[r] == 0 else f"a device-side bounded wait gave up (status code {codes[r]})")
                   for r in (0, 1)}
        with pytest.raises(BackendContractError) as err:
            raise_if_device_wait_failed(codes[rank], dist=FakeDist(rank, records))
        messages.append(str(err.value))
    assert messages[0] == messages[1] and "rank 1" in messages[0] and "status code 5" in messages[0]
    clean = {0: (0, ""), 1: (1, "")}
    raise_if_device_wait_failed(0, dist=FakeDist(0, clean))
    raise_if_device_wait_failed(0, dist=None)
