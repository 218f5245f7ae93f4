import json

import pytest

from solarwm_b200.engine.comparison import publish_comparison_view, seal_comparison_view
from solarwm_b200.engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from solarwm_b200.errors import BackendContractError


class _Adapter:
    family = "toy"

    def __init__(self, with_video=True):
        self.with_video = with_video

    def generate(self, case, *, weights_id):
        art = {"latents.pt": b"x"}
        if self.with_video:
            art["compare.mp4"] = b"video-%d" % case.slot
        return GeneratedSample(art, (1,), "uint8", metrics={"psnr": 20.0 + case.slot}, provenance={"steps": 50})


def _case(i):
    return InferenceCase(slot=i, sample_id=f"clip/{i:02d} a", prompt="p", start_frame=4 * i, noise_seed=7 + i, camera_fingerprint="none")


def test_partitions_merge_into_one_browsable_view(tmp_path):
    run = tmp_path / "run"
    parts = []
    for d in range(2):                                            # two replicas, round-robin slots
        part = run / "validation" / ".staging" / f"replica-{d}"
        InferenceEngine(_Adapter()).run([_case(i) for i in range(4) if i % 2 == d], weights_id="w", output_dir=part)
        parts.append(part)
    view = run / "validation" / "step_000010_live"
    kw = dict(step=10, pass_name="live", cases=4, dp_world_size=2, sp_size=1, run_root=run, cases_per_round=2)
    first = publish_comparison_view(parts[0], view, **kw)
    with pytest.raises(BackendContractError):                     # half of the slots: not sealable yet
        seal_comparison_view(view, step=10, pass_name="live", cases=4)
    publish_comparison_view(parts[1], view, **kw)
    seal = seal_comparison_view(view, step=10, pass_name="live", cases=4)
    names = sorted(p.name for p in (view / "compare").iterdir())
    assert names == ["rank000_round00_dp000_clip-00-a_start000000.mp4", "rank001_round00_dp001_clip-01-a_start000004.mp4",
                     "rank002_round01_dp000_clip-02-a_start000008.mp4", "rank003_round01_dp001_clip-03-a_start000012.mp4"]
    assert seal["videos"] == names and json.loads((view / "COMPLETE.json").read_text())["slots"] == 4
    assert (view / "compare" / names[2]).read_bytes() == b"video-2"
    assert (view / "compare" / names[2]).stat().st_ino == (parts[0] / "slot-000002" / "compare.mp4").stat().st_ino   # a link
    summary = json.loads((view / "manifests" / "rank_003.json").read_text())
    assert summary["dp_rank"] == 1 and summary["round"] == 1 and summary["metrics"]["psnr"] == 23.0
    assert summary["compare_mp4"] == f"validation/step_000010_live/compare/{names[3]}" and first[0].slot == 0
    with pytest.raises(BackendContractError):                     # merging a partition twice
        publish_comparison_view(parts[0], view, **kw)
    with pytest.raises(BackendContractError):                     # incomplete rounds
        publish_comparison_view(parts[0], tmp_path / "v2", **dict(kw, cases=3))
    bare = run / "validation" / ".staging" / "bare"
    InferenceEngine(_Adapter(with_video=False)).run([_case(0)], weights_id="w", output_dir=bare)
    with pytest.raises(BackendContractError):                     # a slot without its comparison video
        publish_comparison_view(bare, tmp_path / "v3", **dict(kw, cases=2))
