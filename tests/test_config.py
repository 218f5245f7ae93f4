import json

import pytest

from solarwm_b200.config import load_config, supported_routes, validate_route
from solarwm_b200.config.loader import canonical_json
from solarwm_b200.errors import ConfigurationError

BASE = """
schema: solarwm.run.v1
action: train
name: t
model: {family: wan2.2-ti2v-5b, camera_translation_transform: linear}
data: {pixel_frames: 81, root: "${DATA_ROOT}"}
train: {stage: stage0p5, causal_mode: bidirectional, objective: flow_matching}
runtime: {output_dir: /tmp/x}
"""


def _write(tmp_path, text, name="c.yaml"):
    p = tmp_path / name
    p.write_text(text)
    return p


def test_load_expand_override_and_digests(tmp_path, monkeypatch):
    monkeypatch.setenv("DATA_ROOT", "/data")
    p = _write(tmp_path, BASE)
    a = load_config(p)
    assert a.values["data"]["root"] == "/data"
    b = load_config(p, ["train.max_steps=7", "data.extra.nested=[1, 2]"])
    assert b.values["train"]["max_steps"] == 7 and b.values["data"]["extra"]["nested"] == [1, 2]
    assert a.source_digest == b.source_digest and a.resolved_digest != b.resolved_digest
    out = tmp_path / "resolved.json"
    b.write_json(out)
    again = load_config(out)                      # a resolved config is accepted back as JSON
    assert again.resolved_digest == b.resolved_digest
    assert canonical_json({"b": 1, "a": 2}) == b'{"a":2,"b":1}\n'


@pytest.mark.parametrize("mutation,needle", [
    ("schema: solarwm.run.v1", "schema: other.v9"),
    ("action: train", "action: destroy"),
    ("name: t", "name: ''"),
    ("runtime: {output_dir: /tmp/x}", "runtime: 3"),
    ("name: t", "name: t\nbogus_section: {}"),
    ("name: t", "name: t\nname: again"),
    ("data: {pixel_frames: 81", "data: {1: 2, pixel_frames: 81"),
    ("objective: flow_matching", "objective: flow_matching, lr: .nan"),
])
def test_strict_rejections(tmp_path, monkeypatch, mutation, needle):
    monkeypatch.setenv("DATA_ROOT", "/data")
    with pytest.raises(ConfigurationError):
        load_config(_write(tmp_path, BASE.replace(mutation, needle)))


def test_unset_env_and_bad_override(tmp_path, monkeypatch):
    monkeypatch.delenv("DATA_ROOT", raising=False)
    with pytest.raises(ConfigurationError, match="DATA_ROOT"):
        load_config(_write(tmp_path, BASE))
    monkeypatch.setenv("DATA_ROOT", "/d")
    with pytest.raises(ConfigurationError):
        load_config(_write(tmp_path, BASE), ["novalue"])
    with pytest.raises(ConfigurationError):
        load_config(_write(tmp_path, BASE), ["name.sub=1"])


def _cfg(**kw):
    base = {"action": "train", "model": {"family": "wan22_ti2v_5b"}, "data": {"pixel_frames": 81},
            "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching"}}
    for k, v in kw.items():
        base[k] = {**base.get(k, {}), **v} if isinstance(v, dict) else v
    return base


def test_routes_table_and_gates():
    assert len(supported_routes()) == 9
    assert validate_route(_cfg()).key == "wan22_ti2v_5b:stage0p5:bidirectional:flow_matching"
    r = validate_route(_cfg(train={"stage": "stage1", "causal_mode": "teacher_forcing", "objective": "anyflow_forward_map"}))
    assert r.variant == "v1_5"
    assert validate_route(_cfg(model={"family": "ltx-2.5"}, data={"pixel_frames": 153})).objective == "native_rectified_flow"
    with pytest.raises(ConfigurationError):
        validate_route(_cfg(data={"pixel_frames": 80}))
    with pytest.raises(ConfigurationError):
        validate_route(_cfg(model={"family": "minimax_h3"}, data={"pixel_frames": 158}))   # needs logd4
    assert validate_route(_cfg(model={"family": "minimax_h3", "camera_translation_transform": "logd4"},
                               data={"pixel_frames": 158})).family == "minimax_h3"
    with pytest.raises(ConfigurationError):
        validate_route(_cfg(model={"family": "wan22_i2v_a14b"}, train={"stage": "stage2"}))
    assert validate_route({"action": "preencode", "model": {"family": "minimax-h3"}}).stage == "preencode"
    with pytest.raises(ConfigurationError):
        validate_route(_cfg(model={"family": "unknown"}))
