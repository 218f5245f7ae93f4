import json
import struct

import pytest

from solarwm_b200.backends.wan22.readiness import AssetLayout, probe_runtime
from solarwm_b200.errors import BackendContractError


def _config(tmp_path=None, **over):
    cfg = {"schema": "solarwm.run.v1", "action": "train",
           "model": {"family": "wan22_ti2v_5b", "architecture": "tiny"},
           "data": {"source": "synthetic", "pixel_frames": 81},
           "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 1},
           "runtime": {"output_dir": "/tmp/x"}}
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v} if isinstance(v, dict) else v
    return cfg


def _safetensors(path, tensors):
    header, blob = {}, b""
    for name, shape in tensors.items():
        n = 1
        for d in shape:
            n *= d
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [len(blob), len(blob) + 2 * n]}
        blob += b"\0" * (2 * n)
    raw = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(raw)) + raw + blob)


def test_synthetic_runs_need_nothing_and_say_so():
    r = probe_runtime(_config(), family="wan22_ti2v_5b")
    assert r.ready and r.as_dict()["schema"] == "solarwm.wan22-readiness.v1"
    assert [i.code for i in r.issues if i.severity == "info"] == ["assets"] and r.assets["base"] is None
    r.require_ready()


def test_a_released_package_is_checked_file_by_file_in_one_pass(tmp_path):
    base = tmp_path / "Wan2.2-TI2V-5B"
    base.mkdir()
    cfg = _config(model={"base_path": str(base), "assets": {"vae": "codecs/vae.pth"}}, data={"source": "index", "index": str(tmp_path / "i.jsonl"), "encoding": "online"},
                  inference={"steps": 0, "solver": "heun", "compare_source": "seeded"})
    r = probe_runtime(cfg, family="wan22_ti2v_5b")
    codes = sorted({i.code for i in r.issues if i.severity == "error"})
    # everything that is wrong is listed at once
    assert codes == ["index", "inference", "text_encoder", "tokenizer", "transformer_config", "transformer_weights", "vae"]
    assert r.assets["vae"] == str(base / "codecs" / "vae.pth") and not r.ready
    with pytest.raises(BackendContractError) as err:
        r.require_ready()
    assert "transformer_weights" in str(err.value) and "tokenizer" in str(err.value)
    # repair it
    (base / "codecs").mkdir()
    for f in ("codecs/vae.pth", "models_t5_umt5-xxl-enc-bf16.pth"):
        (base / f).write_bytes(b"x")
    (base / "google" / "umt5-xxl").mkdir(parents=True)
    (base / "config.json").write_text(json.dumps({"dim": 128, "num_layers": 2, "num_heads": 4}))
    _safetensors(base / "model-00001.safetensors", {"blocks.0.ffn.0.weight": (512, 128), "head.head.bias": (64,)})
    from solarwm_b200.data.index import write_index

    write_index(tmp_path / "i.jsonl", [{"sample_id": "a", "key": "k", "shard": "s/0.tar", "num_frames": 200, "fps": 24.0}])
    good = probe_runtime({**cfg, "inference": {"steps": 4}}, family="wan22_ti2v_5b")
    assert good.ready, good.issues
    assert good.weight_inventory == {"tensors": 2, "shards": 1, "parameters": 512 * 128 + 64, "dtypes": ["BF16"]}
    assert good.index_inventories["index"]["rows"] == 1
    (base / "config.json").write_text(json.dumps({"dim": 3072}))
    bad = probe_runtime({**cfg, "inference": {}}, family="wan22_ti2v_5b")
    assert [i.code for i in bad.issues if i.severity == "error"] == ["transformer_config"]


def test_placeholders_resume_sources_and_layout_rules(tmp_path):
    r = probe_runtime(_config(model={"base_path": "/path/to/Wan2.2"}), family="wan22_ti2v_5b")
    assert any("placeholder" in i.message for i in r.issues) and not r.ready
    with pytest.raises(BackendContractError):
        AssetLayout.from_config({"model": {"base_path": "relative/dir"}})
    with pytest.raises(BackendContractError):
        AssetLayout.from_config({"model": {"assets": {"vae": "x"}}})
    resumed = probe_runtime(_config(model={"base_path": str(tmp_path), "assets": {"transformer_config": "builtin"}},
                                    checkpoint={"mode": "full_resume", "resume_from": str(tmp_path / "missing")}), family="wan22_ti2v_5b")
    assert [i.code for i in resumed.issues if i.severity == "error"] == ["checkpoint"] and resumed.weight_inventory == {"source": "checkpoint"}
    needs_gpu = probe_runtime(_config(), family="wan22_ti2v_5b", require_cuda=True)
    import torch

    assert needs_gpu.ready == torch.cuda.is_available() or any(i.code == "device" for i in needs_gpu.issues)


def test_cli_readiness_exit_codes(tmp_path, monkeypatch, capsys):
    from pathlib import Path

    from solarwm_b200.cli import main

    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    config = str(Path(__file__).resolve().parent.parent / "configs" / "wan22_ti2v_5b" / "tiny_stage0p5_cpu.yaml")
    assert main(["environment", "readiness", "--config", config]) == 0
    assert json.loads(capsys.readouterr().out)["ready"] is True
    assert main(["environment", "readiness", "--config", config, "--set", "model.base_path=/path/to/weights"]) == 3
    assert json.loads(capsys.readouterr().out)["ready"] is False
