import json

import pytest

from solarwm_b200.engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from solarwm_b200.engine.train_engine import (BatchIdentity, GradientStatus, JsonlEventSink, MicrobatchResult,
                                              StepPolicy, TrainingEngine)
from solarwm_b200.errors import BackendContractError


class FakeRuntime:
    def __init__(self, bad_grad_at=None, fail_micro_at=None):
        self.calls, self._step, self.bad, self.fail = [], 0, bad_grad_at, fail_micro_at

    @property
    def global_step(self):
        return self._step

    def _log(self, name, *a):
        self.calls.append((name, *a))

    def zero_grad(self):
        self._log("zero_grad")

    def train_microbatch(self, i, n):
        self._log("micro", i, n)
        if self.fail == self._step + 1:
            raise RuntimeError("reader died")
        ident = BatchIdentity(("s",), (0,), (1,), "ck", "plan")
        return MicrobatchResult(ident, {"fm": 1.0 + i})

    def assert_sp_peer_identity(self, ident):
        self._log("identity")

    def prepare_optimizer_step(self):
        self._log("prepare")
        if self.bad == self._step + 1:
            return GradientStatus(False, float("nan"))
        return GradientStatus(True, 0.5)

    def optimizer_step(self):
        self._log("opt")

    def scheduler_step(self):
        self._log("sched")

    def ema_update(self, step):
        self._log("ema", step)

    def set_global_step(self, step):
        self._log("set", step)
        self._step = step

    def save_checkpoint(self, step):
        self._log("save", step)
        return f"id{step}"

    def validate(self, step):
        self._log("validate", step)
        return {"ok": True}


def test_step_order_events_and_boundaries(tmp_path):
    rt = FakeRuntime()
    sink = JsonlEventSink(tmp_path / "events" / "rank-00000.jsonl")
    assert TrainingEngine(rt, StepPolicy(2, grad_accum=2, save_every=2, validate_every=2), event_sink=sink).run() == 2
    first = [c[0] for c in rt.calls[:11]]
    assert first == ["zero_grad", "micro", "identity", "micro", "identity", "prepare", "opt", "sched", "set", "ema", "zero_grad"]
    assert [c for c in rt.calls if c[0] in ("save", "validate")] == [("save", 2), ("validate", 2)]
    events = [json.loads(l) for l in (tmp_path / "events" / "rank-00000.jsonl").read_text().splitlines()]
    assert [e["event"] for e in events] == ["optimizer_step", "optimizer_step", "checkpoint", "validation"]
    assert events[0]["schema"] == "solarwm.training-step.v1" and events[0]["losses"] == {"fm": 1.5}
    assert events[2]["checkpoint_id"] == "id2"


def test_non_finite_gradient_stops_before_any_mutation():
    rt = FakeRuntime(bad_grad_at=2)
    with pytest.raises(BackendContractError, match="non-finite"):
        TrainingEngine(rt, StepPolicy(3)).run()
    assert rt.global_step == 1
    tail = [c[0] for c in rt.calls[-3:]]
    assert tail == ["identity", "prepare", "zero_grad"]
    assert sum(1 for c in rt.calls if c[0] == "opt") == 1


def test_failing_microbatch_zeroes_grads_and_reraises():
    rt = FakeRuntime(fail_micro_at=1)
    with pytest.raises(RuntimeError, match="reader died"):
        TrainingEngine(rt, StepPolicy(1)).run()
    assert [c[0] for c in rt.calls] == ["zero_grad", "micro", "zero_grad"]


def test_contract_dataclasses_validate():
    with pytest.raises(BackendContractError):
        MicrobatchResult(BatchIdentity(("s",), (0,), (1,), "c", "p"), {"x": float("nan")})
    with pytest.raises(BackendContractError):
        BatchIdentity((), (), (), "c", "p")
    with pytest.raises(BackendContractError):
        StepPolicy(0)
    with pytest.raises(BackendContractError):
        JsonlEventSink("/tmp/_nan_events.jsonl")({"x": float("nan")})


class FakeAdapter:
    family = "fake"

    def __init__(self, fail_slot=None):
        self.fail_slot = fail_slot

    def generate(self, case, *, weights_id):
        if case.slot == self.fail_slot:
            raise ValueError("decode failed")
        return GeneratedSample({"video.mp4": b"v" * (case.slot + 1), "meta/info.json": b"{}"}, (1, 2), "uint8")


def _cases(n):
    return [InferenceCase(i, f"s{i}", "p", 0, i, "cam") for i in range(n)]


def test_inference_publication_layout_and_digest(tmp_path):
    s = InferenceEngine(FakeAdapter()).run(_cases(2), weights_id="w", output_dir=tmp_path / "out")
    out = tmp_path / "out"
    assert (out / "slot-000001" / "video.mp4").read_bytes() == b"vv"
    m = json.loads((out / "slot-000000" / "manifest.json").read_text())
    assert m["schema"] == "solarwm.inference-sample.v1" and m["artifacts"][1]["bytes"] == 1
    complete = json.loads((out / "COMPLETE.json").read_text())
    assert complete["cases"] == 2 and complete["ordered_manifest_digest"] == s.ordered_manifest_digest
    assert len((out / "ordered-manifest.jsonl").read_text().splitlines()) == 2
    assert not [p for p in tmp_path.iterdir() if p.name.endswith(".partial")]
    with pytest.raises(BackendContractError, match="already exists"):
        InferenceEngine(FakeAdapter()).run(_cases(1), weights_id="w", output_dir=out)
    assert (out / "slot-000001").exists()          # the published winner is untouched


def test_inference_failure_never_publishes_and_waves_are_collective(tmp_path):
    phases = []
    with pytest.raises(BackendContractError, match="case wave 1"):
        InferenceEngine(FakeAdapter(fail_slot=1)).run(_cases(3), weights_id="w", output_dir=tmp_path / "o",
                                                      collective_error=lambda e, p: phases.append((p, e)))
    assert not (tmp_path / "o").exists()
    assert phases[0] == ("output setup", None) and phases[2][0] == "case wave 1" and "decode failed" in phases[2][1]
    phases.clear()
    InferenceEngine(FakeAdapter()).run(_cases(1), weights_id="w", output_dir=tmp_path / "p",
                                       collective_error=lambda e, p: phases.append(p), collective_case_waves=3)
    assert phases == ["output setup", "case wave 0", "case wave 1", "case wave 2", "partition commit"]
    with pytest.raises(BackendContractError):
        GeneratedSample({"a": b"1", "a/b": b"2"}, (1,), "u8")
    with pytest.raises(BackendContractError):
        InferenceEngine(FakeAdapter()).run([_cases(1)[0], _cases(1)[0]], weights_id="w", output_dir=tmp_path / "q")


def test_comparison_view_and_validation_plan(tmp_path):
    import json

    import pytest
    import torch

    from solarwm_b200.engine.comparison import side_by_side, write_comparison
    from solarwm_b200.engine.validation_plan import build_plan, load_plan, publish_plan
    from solarwm_b200.errors import SolarWMError

    g, s = torch.zeros(5, 3, 16, 24), torch.ones(4, 3, 8, 16) * 0.5
    view = side_by_side(g, s, separator=4)
    assert view.shape == (4, 3, 16, 24 + 4 + 16)
    assert float(view[0, 0, 0, 30]) == -1.0 and float(view[0, 0, 8, 30]) == 0.5      # letter-boxed source
    info = write_comparison(tmp_path / "cmp", g, s, use_ffmpeg=False, meta={"sample_id": "a"})
    assert info["frames"] == 4 and json.loads((tmp_path / "cmp" / "comparison.json").read_text())["sample_id"] == "a"

    rows = [{"sample_id": f"v{i}", "caption": f"c{i}"} for i in range(5)]
    plan = build_plan(rows, run_id="r", step=10, pass_name="main", count=4, dp_world=2, base_seed=7)
    again = build_plan(rows, run_id="r", step=10, pass_name="main", count=4, dp_world=2, base_seed=7)
    assert plan.digest == again.digest
    assert [c.slot for c in plan.for_rank(1)] == [1, 3]
    path = publish_plan(plan, tmp_path / "val")
    assert load_plan(path).digest == plan.digest
    with pytest.raises(FileExistsError):
        publish_plan(plan, tmp_path / "val")                   # create-only
    with pytest.raises(SolarWMError):
        build_plan(rows, run_id="r", step=10, pass_name="main", count=9)
