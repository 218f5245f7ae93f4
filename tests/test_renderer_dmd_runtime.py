"""Renderer distillation runtime: roles from the control adapters, exact resume, parent identity, CLI dispatch."""
import json

import pytest
import torch

from solarwm_b200.errors import BackendContractError, ConfigurationError
from tests.test_renderer_runtime import _config, _corpus


def _control(tmp_path):
    """A control run whose exported adapters the distillation starts from."""
    from solarwm_b200.renderer.runtime import export_adapter, run_control_training

    _corpus(tmp_path / "corpus", n=4)
    out = run_control_training(_config(tmp_path / "corpus", tmp_path / "control", train={"max_steps": 1, "gradient_accumulation_steps": 1}))
    return export_adapter(out["checkpoint"], tmp_path / "control.pt")["path"]


def _dmd_config(tmp_path, out, control, **over):
    cfg = _config(tmp_path / "corpus", out, train={"objective": "dmd", "max_steps": 4, "optimizer": {"lr": 1e-3}, "critic_optimizer": {"lr": 1e-3},
                                                  "dmd": {"control": control, "student_steps": 2, "critic_updates_per_student": 2, "guidance": 2.0}})
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v}
    return cfg


def test_distillation_starts_from_control_resumes_exactly_and_names_its_parents(tmp_path, capsys):
    from solarwm_b200.checkpoint.store import verify_checkpoint
    from solarwm_b200.renderer.dmd_runtime import COMPONENTS, RendererDMDRuntime, run_dmd_training
    from solarwm_b200.renderer.runtime import read_adapter

    control = _control(tmp_path)
    rt = RendererDMDRuntime(_dmd_config(tmp_path, tmp_path / "probe", control))
    want = read_adapter(control)
    for model in (rt.trainer.student, rt.trainer.critic, rt.trainer.teacher):
        got = {n: p for n, p in model.named_parameters() if "lora_" in n}
        assert all(torch.equal(got[n], want[n].to(got[n])) for n in want)
    assert not any(p.requires_grad for p in rt.trainer.teacher.parameters()) and rt.parents["student_init"] == rt.parents["control"]
    rt.close()
    straight = run_dmd_training(_dmd_config(tmp_path, tmp_path / "a", control, checkpoint={"save_steps": [2]}))
    assert straight["final_step"] == 4 and straight["student_step"] == 1
    end = verify_checkpoint(straight["checkpoint"])
    assert end.contract.stage == "fewstep" and end.contract.objective == "dmd" and all((end.path / c).is_file() for c in COMPONENTS)
    resumed = run_dmd_training(_dmd_config(tmp_path, tmp_path / "b", control, checkpoint={"resume_from": str(tmp_path / "a" / "checkpoint_model_000002")}))
    for name in ("optimizer.pt", "critic-optimizer.pt"):
        a, b = (torch.load(p / name, weights_only=True) for p in (end.path, verify_checkpoint(resumed["checkpoint"]).path))
        assert torch.equal(a["master"], b["master"]) and a["step"] == b["step"]
    events = [json.loads(l) for f in (tmp_path / "a").rglob("*.jsonl") for l in f.read_text().splitlines()]
    assert [e["student_updated"] for e in events if e.get("event") == "train_step"] == [0.0, 0.0, 1.0, 0.0]
    # another control parent, or other distillation settings, refuse the checkpoint
    torch.save({**torch.load(control, weights_only=True), "note": "another file"}, tmp_path / "control2.pt")
    with pytest.raises(BackendContractError):
        RendererDMDRuntime(_dmd_config(tmp_path, tmp_path / "c", str(tmp_path / "control2.pt"), checkpoint={"resume_from": straight["checkpoint"]}))
    other = _dmd_config(tmp_path, tmp_path / "d", control, checkpoint={"resume_from": straight["checkpoint"]})
    other["train"]["dmd"] = {**other["train"]["dmd"], "guidance": 3.0}
    with pytest.raises(BackendContractError):
        RendererDMDRuntime(other)
    with pytest.raises(ConfigurationError):
        bad = _dmd_config(tmp_path, tmp_path / "e", control)
        bad["train"]["dmd"] = {"student_steps": 2}
        RendererDMDRuntime(bad)
    # the command line dispatches on the objective
    import yaml

    from solarwm_b200.renderer.cli import main

    (tmp_path / "dmd.yaml").write_text(yaml.safe_dump(_dmd_config(tmp_path, tmp_path / "cli", control, train={"max_steps": 1})))
    assert main(["train", "--config", str(tmp_path / "dmd.yaml")]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["final_step"] == 1
