"""Wan Stage2 run loop: roles started from earlier checkpoints, exact resume, schedule check, events."""
import json
from pathlib import Path

import pytest
import torch
import yaml

from solarwm_b200.errors import BackendContractError

ROOT = Path(__file__).resolve().parent.parent


def _config(out, **over):
    cfg = yaml.safe_load((ROOT / "configs" / "wan22_ti2v_5b" / "tiny_stage2_sgf_cpu.yaml").read_text())
    cfg["runtime"].update(output_dir=str(out), device="cpu")
    cfg["train"]["max_steps"] = 4
    cfg["train"]["ema"] = {"enabled": True, "decay": 0.5, "start_step": 0}
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v}
    return cfg


def _role(path):
    return torch.load(Path(path) / "role.pt", map_location="cpu", weights_only=True)


def test_resume_is_exact_and_counters_follow_the_schedule(tmp_path):
    from solarwm_b200.backends.wan22.stage2 import expected_student_updates, run_stage2_training

    assert [expected_student_updates(n, 2) for n in range(6)] == [0, 0, 0, 1, 1, 2]
    straight = run_stage2_training(_config(tmp_path / "a", checkpoint={"save_steps": [2, 4]}))
    assert straight["final_step"] == 4 and straight["checkpoint_dir"].endswith("checkpoint_model_000004")
    mid = tmp_path / "a" / "checkpoint_model_000002"
    resumed = run_stage2_training(_config(tmp_path / "b", checkpoint={"resume_from": str(mid), "save_steps": [4]}))
    assert resumed["final_step"] == 4
    a, b = _role(tmp_path / "a" / "checkpoint_model_000004"), _role(tmp_path / "b" / "checkpoint_model_000004")
    # the roles continue where they stopped; threaded CPU reductions may differ in the last bits between two runs of one
    # process (seen at 1e-14 on the critic's time-embedding biases), so the comparison allows that much and no more
    for role in ("student", "critic", "ema_student"):
        assert all(torch.allclose(a[role][k].float(), b[role][k].float(), rtol=1e-5, atol=1e-9) for k in a[role]), role
    run = torch.load(tmp_path / "a" / "checkpoint_model_000004" / "runtime.pt", weights_only=True)
    assert run["student_updates"] == 1 and run["global_step"] == 4
    events = [json.loads(l) for f in (tmp_path / "a").rglob("*.jsonl") for l in f.read_text().splitlines()]
    steps = [e for e in events if e.get("event") == "train_step"]
    assert [e["step"] for e in steps] == [1, 2, 3, 4] and "student" in steps[2] and "student" not in steps[0]
    # a checkpoint whose counters were tampered with is refused
    bad = tmp_path / "tampered"
    import shutil

    shutil.copytree(mid, bad)
    with pytest.raises(Exception):
        torch.save({"global_step": 2, "student_updates": 5, "initialization": {}}, bad / "runtime.pt")
        run_stage2_training(_config(tmp_path / "c", checkpoint={"resume_from": str(bad)}))


def test_roles_start_from_earlier_checkpoints(tmp_path):
    from solarwm_b200.backends.wan22.stage2 import Stage2Options, WanStage2Trainer, load_role_weights, run_stage2_training
    from solarwm_b200.backends.wan22.contracts import architecture

    first = run_stage2_training(_config(tmp_path / "parent", checkpoint={"save_steps": [3]}, train={"max_steps": 3}))
    parent = first["checkpoint_dir"]
    cfg = _config(tmp_path / "child", checkpoint={"save_steps": [1], "initialization": {"student": {"path": parent, "weight_source": "ema"},
                                                                                        "teacher": parent}}, train={"max_steps": 1})
    out = run_stage2_training(cfg)
    rec = out["initialization"]
    assert rec["student"]["taken"] == "role.pt:ema_student" and rec["teacher"]["taken"] == "role.pt:student"
    assert rec["critic"]["taken"].endswith("(teacher's)") and rec["student"]["stage"] == "stage2" and rec["student"]["step"] == 3
    saved = torch.load(Path(out["checkpoint_dir"]) / "runtime.pt", weights_only=True)
    assert saved["initialization"]["teacher"]["checkpoint"] == rec["teacher"]["checkpoint"]
    # the loader itself: strict names, the right entry, verified source
    arch = architecture(cfg)
    tr = WanStage2Trainer(arch, "cpu", Stage2Options(chunk_frames=2, window_chunks=2, denoising_steps=(1000.0, 500.0)), dtype=torch.float32)
    before = tr.critic.get_parameter("blocks.0.ffn.0.weight").detach().clone()
    got = load_role_weights(tr.critic, parent, role="critic")
    assert got["taken"] == "role.pt:critic" and not torch.equal(before, tr.critic.get_parameter("blocks.0.ffn.0.weight"))
    want = _role(parent)["critic"]["blocks.0.ffn.0.weight"]
    assert torch.equal(tr.critic.get_parameter("blocks.0.ffn.0.weight"), want.to(torch.float32))
    with pytest.raises(BackendContractError):
        load_role_weights(tr.critic, parent, role="critic", weight_source="other")
    with pytest.raises(Exception):
        load_role_weights(tr.critic, tmp_path / "nowhere", role="critic")
    # resuming a child under another parent is refused
    other = _config(tmp_path / "child2", checkpoint={"resume_from": out["checkpoint_dir"]}, train={"max_steps": 2})
    with pytest.raises(BackendContractError):
        run_stage2_training(other)


WORKER = """
import json, os, sys, torch
sys.path.insert(0, os.environ["REPO"])
from tests.test_wan_stage2_runtime import _config, _role
from solarwm_b200.backends.wan22.stage2 import run_stage2_training
cfg = _config(os.environ["OUT"], checkpoint={"save_steps": [3]}, distributed={"world_size": 2, "sequence_parallel_size": 1})
cfg["train"]["max_steps"] = 3
out = run_stage2_training(cfg)
rank = int(os.environ["RANK"])
print("RESULT " + json.dumps({"rank": rank, "losses": out["losses"], "final": out["final_step"]}), flush=True)
"""


def test_two_data_parallel_ranks_average_their_gradients(tmp_path):
    import os
    import socket
    import subprocess
    import sys

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, REPO=repo, OUT=str(tmp_path / "run"), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    rows = [json.loads(l.split("RESULT ", 1)[1]) for o in outs for l in o.splitlines() if l.startswith("RESULT ")]
    assert len(rows) == 2 and all(r["final"] == 3 for r in rows)
    assert rows[0]["losses"]["critic"] != rows[1]["losses"]["critic"]           # the replicas rolled out different prompts and noise
    saved = _role(tmp_path / "run" / "checkpoint_model_000003")
    ranks = torch.load(tmp_path / "run" / "checkpoint_model_000003" / "rank-state.pt", weights_only=True)
    assert ranks["world_size"] == 2 and len(ranks["ranks"]) == 2 and "student" in saved
