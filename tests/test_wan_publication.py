import io
import json

import numpy as np
import pytest

from solarwm_b200.backends.wan22.publication import plan_triplets, preflight, publish_triplets
from solarwm_b200.engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from solarwm_b200.errors import BackendContractError


def _case(i, **meta):
    base = {"physical_dataset": "re10k", "publish_stem": f"clip_{i:03d}", "publication_pixel_frames": 5,
            "camera_publication_convention": "authoritative_absolute_c2w"}
    return InferenceCase(slot=i, sample_id=f"s{i}", prompt="p", start_frame=0, noise_seed=i, camera_fingerprint="c", metadata={**base, **meta})


class _Adapter:
    family = "wan22_ti2v_5b"

    def __init__(self, frames=5, dtype=np.float64):
        self.frames, self.dtype = frames, dtype

    def generate(self, case, *, weights_id):
        buf = io.BytesIO()
        np.save(buf, np.tile(np.eye(4), (self.frames, 1, 1)).astype(self.dtype))
        return GeneratedSample({"video.mp4": b"v%d" % case.slot, "compare.mp4": b"c%d" % case.slot, "camera.npy": buf.getvalue()},
                               (1,), "uint8")


def test_triplets_are_linked_receipted_and_sealed_last(tmp_path):
    cases = [_case(0), _case(1)]
    plan = plan_triplets(tmp_path / "out", "run-a", cases)
    preflight(plan)                                                       # before generation: all names are free
    gen = tmp_path / "out" / "runs" / "run-a" / "generation"
    InferenceEngine(_Adapter()).run(cases, weights_id="w", output_dir=gen)
    done = publish_triplets(gen, plan, family="wan22_ti2v_5b", weights_id="w")
    out = tmp_path / "out"
    assert (out / "generate" / "re10k" / "clip_001.mp4").read_bytes() == b"v1"
    assert (out / "compare" / "re10k" / "clip_000.mp4").read_bytes() == b"c0"
    assert np.load(out / "camera" / "re10k" / "clip_000.npy").shape == (5, 4, 4)
    assert (out / "generate" / "re10k" / "clip_000.mp4").stat().st_ino == (gen / "slot-000000" / "video.mp4").stat().st_ino
    prov = out / "runs" / "run-a" / "publication"
    seal = json.loads((prov / "COMPLETE.json").read_text())
    assert seal == done and seal["cases"] == 2 and seal["layout"] == "dataset_triplet_v1"
    receipt = json.loads((prov / "samples" / "slot-000001.json").read_text())
    assert receipt["artifacts"]["camera.npy"]["path"] == "camera/re10k/clip_001.npy" and receipt["published_pixel_frames"] == 5
    assert len((prov / "ordered-manifest.jsonl").read_text().splitlines()) == 2
    with pytest.raises(BackendContractError):                             # a second publication of the same run
        publish_triplets(gen, plan, family="wan22_ti2v_5b", weights_id="w")


def test_plans_and_sources_are_checked_before_anything_becomes_public(tmp_path):
    for bad in ({"physical_dataset": "../x"}, {"publish_stem": ""}, {"publication_pixel_frames": 0}, {"camera_publication_convention": "relative"}):
        with pytest.raises(BackendContractError):
            plan_triplets(tmp_path, "r", [_case(0, **bad)])
    with pytest.raises(BackendContractError):
        plan_triplets(tmp_path, "r", [_case(0), _case(1, publish_stem="clip_000")])           # same destination
    with pytest.raises(BackendContractError):
        plan_triplets(tmp_path, "r", [])
    cases = [_case(0)]

    def attempt(name, adapter, tamper=None, **kw):
        root = tmp_path / name
        plan = plan_triplets(root, "r", cases)
        gen = root / "runs" / "r" / "generation"
        InferenceEngine(adapter).run(cases, weights_id="w", output_dir=gen)
        if tamper:
            tamper(gen)
        with pytest.raises(BackendContractError):
            publish_triplets(gen, plan, **{"family": "wan22_ti2v_5b", "weights_id": "w", **kw})
        assert not (root / "generate").exists() and not (root / "runs" / "r" / "publication").exists()   # nothing leaked

    attempt("frames", _Adapter(frames=4))                                  # camera file of the wrong length
    attempt("dtype", _Adapter(dtype=np.float32))
    attempt("weights", _Adapter(), weights_id="other")
    attempt("drift", _Adapter(), tamper=lambda g: (g / "slot-000000" / "video.mp4").write_bytes(b"changed"))
    attempt("unsealed", _Adapter(), tamper=lambda g: (g / "COMPLETE.json").unlink())
    taken = tmp_path / "taken"
    plan = plan_triplets(taken, "r", cases)
    (taken / "camera" / "re10k").mkdir(parents=True)
    (taken / "camera" / "re10k" / "clip_000.npy").write_bytes(b"x")
    with pytest.raises(BackendContractError):
        preflight(plan)
