"""Wan fixed-window rules and the 153-frame window index join (``solar data materialize-wan153f``)."""
import gzip
import hashlib
import json

import pytest

from solarwm_b200.backends.wan22 import windows as W
from solarwm_b200.cli import main
from solarwm_b200.errors import DataContractError


def test_start_frame_rules():
    assert [W.window_count_81f(n) for n in (81, 120, 121, 160, 200, 201)] == [1, 1, 2, 2, 2, 3]
    assert W.window_start_81f({"window_index": 0, "window_count": 1}, 101) == 10            # centred
    starts = [W.window_start_81f({"window_index": i, "window_count": 3}, 241) for i in range(3)]
    assert starts == [0, 80, 160]                                                         # both ends included
    with pytest.raises(DataContractError):
        W.window_start_81f({"window_index": 0, "window_count": 2}, 100)
    long_form = {"source_sample_id": "miradata/x", "source_dataset": "miradata", "window_count": 6}
    got = [W.window_start_153f(dict(long_form, window_index=i), 1153) for i in range(6)]
    assert got == [0, 200, 400, 600, 800, 1000]
    one = {"source_sample_id": "re10k/abc", "source_dataset": "re10k", "window_index": 0, "window_count": 1}
    want = int.from_bytes(hashlib.blake2b(b"solarwm-latent-153f-v1\0re10k/abc", digest_size=8).digest(), "little") % (200 - 153 + 1)
    assert W.window_start_153f(one, 200) == want
    with pytest.raises(DataContractError):
        W.window_start_153f(dict(one, window_count=6), 200)


def _write(path, rows):
    with open(path, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")


def _raw(sample_id, dataset, frames, split):
    return {"sample_id": sample_id, "key": sample_id.replace("/", "_"), "shard": f"{dataset}/s0.tar", "epoch_repeats": 1,
            "dataset": dataset, "num_frames": frames, "split": split}


def _authority(raw, ordinal, start):
    return {"sample_id": f"{raw['sample_id']}/latent-153f-w{ordinal:02d}", "key": f"{raw['key']}__latent153f_w{ordinal:02d}",
            "shard": raw["shard"], "epoch_repeats": 1, "start_frame": start,
            "source_frame_indices": list(range(start, start + 153))}


def test_window_index_join_is_strict_deterministic_and_create_only(tmp_path, capsys):
    a = _raw("re10k/clip-a", "re10k", 200, "train")
    b = _raw("miradata/clip-b", "miradata", 653, "train")
    c = _raw("re10k/clip-c", "re10k", 160, "test")
    _write(tmp_path / "train.jsonl", [a, b])
    _write(tmp_path / "test.jsonl", [c])
    b_starts = [W.window_start_153f({"source_sample_id": b["sample_id"], "source_dataset": "miradata", "window_index": i,
                                     "window_count": 6}, 653) for i in range(6)]
    _write(tmp_path / "train_w.jsonl", [_authority(a, 0, 17)] + [_authority(b, i, s) for i, s in enumerate(b_starts)])
    _write(tmp_path / "test_w.jsonl", [_authority(c, 0, 3)])
    args = ["data", "materialize-wan153f", "--train-index", str(tmp_path / "train.jsonl"), "--test-index",
            str(tmp_path / "test.jsonl"), "--train-window-index", str(tmp_path / "train_w.jsonl"), "--test-window-index",
            str(tmp_path / "test_w.jsonl")]
    assert main(args + ["--output", str(tmp_path / "out.jsonl.gz")]) == 0
    summary = json.loads(capsys.readouterr().out)
    assert summary["schema"] == "solarwm.wan22-153f-window-index.v1"
    assert (summary["train_sources"], summary["test_sources"], summary["train_windows"], summary["test_windows"]) == (2, 1, 7, 1)
    rows = [json.loads(l) for l in gzip.open(tmp_path / "out.jsonl.gz")]
    assert len(rows) == 8 and rows[0]["start_frame"] == 17 and rows[0]["window_count"] == 1 and rows[0]["split"] == "train"
    assert rows[3]["source_dataset"] == "miradata" and rows[3]["window_index"] == 2 and rows[3]["num_frames"] == 653
    assert rows[-1]["split"] == "test" and rows[-1]["source_sample_id"] == "re10k/clip-c"
    assert hashlib.sha256(gzip.open(tmp_path / "out.jsonl.gz").read()).hexdigest() == summary["decompressed_sha256"]
    # create-only; and the same inputs give the same bytes
    assert main(args + ["--output", str(tmp_path / "out.jsonl.gz")]) == 2
    assert main(args + ["--output", str(tmp_path / "again.jsonl.gz")]) == 0
    assert (tmp_path / "again.jsonl.gz").read_bytes() == (tmp_path / "out.jsonl.gz").read_bytes()
    capsys.readouterr()
    # a clip without its full set of windows, a wrong long-form start and a role mismatch are refused
    _write(tmp_path / "short_w.jsonl", [_authority(a, 0, 17)] + [_authority(b, i, s) for i, s in enumerate(b_starts[:5])])
    with pytest.raises(DataContractError, match="complete window authority"):
        W.write_window_index(tmp_path / "train.jsonl", tmp_path / "test.jsonl", tmp_path / "short_w.jsonl",
                             tmp_path / "test_w.jsonl", tmp_path / "x.gz")
    bad = [_authority(a, 0, 17)] + [_authority(b, i, s + (1 if i == 2 else 0)) for i, s in enumerate(b_starts)]
    _write(tmp_path / "bad_w.jsonl", bad)
    with pytest.raises(DataContractError, match="long-form authority start"):
        W.write_window_index(tmp_path / "train.jsonl", tmp_path / "test.jsonl", tmp_path / "bad_w.jsonl",
                             tmp_path / "test_w.jsonl", tmp_path / "y.gz")
    with pytest.raises(DataContractError, match="role"):
        W.write_window_index(tmp_path / "train.jsonl", tmp_path / "test.jsonl", tmp_path / "test_w.jsonl",
                             tmp_path / "train_w.jsonl", tmp_path / "z.gz")
    assert not list(tmp_path.glob(".*partial"))
