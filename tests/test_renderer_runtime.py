"""Renderer corpus reader (validation, rank ownership, length buckets, resume) and the config-driven training runtime
(engine hooks, checkpoints, exact resume, parent identity, adapter export, CLI)."""
import json

import numpy as np
import pytest
import torch

from solarwm_b200.errors import BackendContractError, DataContractError
from solarwm_b200.renderer.data import MemberContract, OmniStream, read_member, views_from_c2w, write_member

CONTRACT = MemberContract(latent_channels=24, text_dim=64, grids=((8, 8),), frames_period=1, frames_offset=2)


def _member(path, seed, frames=4, camera=True, extra=None, observations=()):
    g = torch.Generator().manual_seed(seed)
    t = {"target_latents": torch.randn(24, frames, 8, 8, generator=g), "prompt_embeds": torch.randn(6, 64, generator=g),
         "text_token_tags": torch.zeros(6, dtype=torch.int64), "anchor_latents": torch.randn(24, 1, 8, 8, generator=g),
         "structure_latents": torch.randn(24, frames, 8, 8, generator=g)}
    if camera:
        c2w = torch.eye(4).repeat(frames, 1, 1)
        c2w[:, 2, 3] = torch.arange(frames) * 0.1 + 5.0
        t["camera_c2w"], t["camera_K"] = c2w, torch.tensor([[0.5, 0, 0.5], [0, 0.9, 0.5], [0, 0, 1.0]])
    t.update(extra or {})
    write_member(path, t, observations=observations, source="unit")


def _corpus(root, n=6, frames=lambda i: 4):
    rows = []
    for i in range(n):
        _member(root / "members" / f"m{i:02d}.safetensors", i, frames=frames(i))
        rows.append({"id": f"clip-{i:02d}", "member": f"members/m{i:02d}.safetensors", "latent_frames": frames(i), "observations": 0})
    (root / "index.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    return rows


def test_member_validation_and_camera_normalisation(tmp_path):
    _member(tmp_path / "ok.safetensors", 0, extra={"known_degrees": torch.linspace(0, 1, 4 * 16), "observation_0_latents": torch.randn(24, 2, 4, 4)},
            observations=[{"frames": [0, 3], "degree": 0.9}])
    s = read_member(tmp_path / "ok.safetensors", {"id": "a"}, CONTRACT)
    assert s.camera_w2c.shape == (5, 4, 4) and torch.equal(s.camera_w2c[0], torch.eye(4)) and torch.equal(s.camera_w2c[1], torch.eye(4))
    assert torch.allclose(s.camera_w2c[-1, 2, 3], torch.tensor(-0.3), atol=1e-6) and s.camera_K.shape == (4, 3, 3)
    assert s.observations[0].frames == (0, 3) and s.observations[0].degree == 0.9 and s.known_degree.shape == (64,) and s.source == "unit"
    assert read_member(tmp_path / "ok.safetensors", {"id": "a", "free_observations": True}, CONTRACT).observations[0].frames is None
    train = s.as_training_sample()
    assert set(train) >= {"target_latents", "anchor_latents", "prompt_embeds", "structure_latents", "camera_w2c", "known_degree", "shape"}
    c2w = torch.eye(4).repeat(3, 1, 1)
    c2w[:, 0, 3] = torch.tensor([2.0, 3.0, 5.0])
    assert torch.allclose(views_from_c2w(c2w)[:, 0, 3], torch.tensor([0.0, -1.0, -3.0]))
    bad = {"nan": {"target_latents": torch.full((24, 4, 8, 8), float("nan"))}, "grid": {"target_latents": torch.randn(24, 4, 6, 8)},
           "tags": {"text_token_tags": torch.full((6,), 3, dtype=torch.int64)}, "known": {"known_degrees": torch.full((64,), 1.5)},
           "far": {"camera_c2w": torch.eye(4).repeat(4, 1, 1) + torch.tensor([0, 0, 0, 1.0]).view(1, 1, 4) * torch.tensor([0, 0, 99.0, 0]).view(1, 4, 1) * torch.arange(4).view(4, 1, 1)},
           "halfcam": {"camera_K": None}}
    for name, extra in bad.items():
        if name == "halfcam":
            _member(tmp_path / f"{name}.safetensors", 1, camera=False, extra={"camera_c2w": torch.eye(4).repeat(4, 1, 1)})
        else:
            _member(tmp_path / f"{name}.safetensors", 1, extra=extra)
        with pytest.raises(DataContractError):
            read_member(tmp_path / f"{name}.safetensors", {"id": name}, CONTRACT)
    _member(tmp_path / "obs.safetensors", 2, extra={"observation_0_latents": torch.randn(24, 2, 4, 4)}, observations=[{"frames": [0, 9]}])
    with pytest.raises(DataContractError):
        read_member(tmp_path / "obs.safetensors", {"id": "o"}, CONTRACT)


def test_stream_partitions_ranks_buckets_lengths_and_resumes(tmp_path):
    _corpus(tmp_path, n=10, frames=lambda i: 4 if i % 2 else 7)
    kw = dict(root=tmp_path, index=tmp_path / "index.jsonl", seed=3, contract=CONTRACT)
    a, b = OmniStream(dp_rank=0, dp_size=2, length_buckets=True, **kw), OmniStream(dp_rank=1, dp_size=2, length_buckets=True, **kw)
    assert a.plan_fingerprint == b.plan_fingerprint != OmniStream(dp_rank=0, dp_size=2, **kw).plan_fingerprint
    seen = []
    for _ in range(4):                                             # 2 runs per length per epoch (5 rows -> 4 usable)
        x, y = a.next(), b.next()
        assert x.target_latents.shape[1] == y.target_latents.shape[1] and x.sample_id != y.sample_id
        seen += [x.sample_id, y.sample_id]
    assert len(set(seen)) == 8 and a.epoch == 0 and a.cursor == 4
    state = a.state_dict()
    nxt = a.next()
    assert a.epoch == 1 and a.cursor == 1                          # rolled into the next epoch
    fresh = OmniStream(dp_rank=0, dp_size=2, length_buckets=True, **kw)
    fresh.load_state_dict(state)
    assert fresh.next().sample_id == nxt.sample_id
    with pytest.raises(DataContractError):
        OmniStream(dp_rank=0, dp_size=2, **kw).load_state_dict(state)          # another plan
    with pytest.raises(DataContractError):
        fresh.load_state_dict(dict(state, cursor=99))
    # without buckets every epoch is one seeded permutation cut to the world size
    plain = OmniStream(dp_rank=0, dp_size=3, **kw)
    order = plain.global_order(0)
    assert len(order) == 9 and sorted(order.tolist()) != order.tolist() and np.array_equal(order, plain.global_order(0))
    # a failed read leaves the cursor in place
    (tmp_path / "members" / "m00.safetensors").write_bytes(b"broken")
    r = OmniStream(dp_rank=0, dp_size=1, shuffle=False, **kw)
    with pytest.raises(DataContractError):
        r.next()
    assert (r.epoch, r.cursor) == (0, 0)
    (tmp_path / "dup.jsonl").write_text('{"id": "x", "member": "a"}\n{"id": "x", "member": "b"}\n')
    with pytest.raises(DataContractError):
        OmniStream(root=tmp_path, index=tmp_path / "dup.jsonl", dp_rank=0, dp_size=1, seed=0)


def _config(tmp_path, out, **over):
    cfg = {"schema": "solarwm.run.v1", "action": "train", "name": "renderer-unit",
           "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}},
           "data": {"omni_root": str(tmp_path), "omni_index": str(tmp_path / "index.jsonl"), "seed": 5, "omni_length_buckets": False,
                    "member_contract": {"text_dim": 64, "grids": [[8, 8]], "frames_period": 1, "frames_offset": 2}},
           "train": {"objective": "flow_matching", "max_steps": 4, "gradient_accumulation_steps": 2,
                     "optimizer": {"lr": 1e-3, "warmup_steps": 1},
                     "observations": {"patterns": {"shared": 1.0, "known_frames": 1.0}}},
           "checkpoint": {"save_steps": [2], "ema": {"decay": 0.5}},
           "runtime": {"device": "cpu", "output_dir": str(out)}}
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v}
    return cfg


def test_runtime_trains_resumes_exactly_and_exports(tmp_path, capsys):
    from solarwm_b200.checkpoint.store import verify_checkpoint
    from solarwm_b200.models.h3 import h3_preset
    from solarwm_b200.renderer.cli import main
    from solarwm_b200.renderer.runtime import (COMPONENTS, RendererTrainingRuntime, export_adapter, read_adapter,
                                               run_control_training, validate_config)

    assert h3_preset("tiny").text_dim == 64
    _corpus(tmp_path / "corpus", n=6)
    cfg = _config(tmp_path / "corpus", tmp_path / "a")
    out = run_control_training(cfg)
    assert out["final_step"] == 4 and out["last_loss"] == out["last_loss"]
    mid, end = tmp_path / "a" / "checkpoint_model_000002", tmp_path / "a" / "checkpoint_model_000004"
    found = verify_checkpoint(str(end))
    assert found.contract.family == "minimax_h3_renderer" and all((found.path / c).is_file() for c in COMPONENTS)
    assert torch.load(end / "rank-state.pt", weights_only=True)["ranks"][0]["reader"]["cursor"] == 2          # 8 samples over 6 rows
    # resume from step 2 reproduces step 4 bit for bit (optimizer, average, reader position, random streams)
    cfg_b = _config(tmp_path / "corpus", tmp_path / "b", checkpoint={"resume_from": str(mid)})
    run_control_training(cfg_b)
    a, b = (torch.load(p / "optimizer.pt", weights_only=True) for p in (end, tmp_path / "b" / "checkpoint_model_000004"))
    assert torch.equal(a["master"], b["master"]) and torch.equal(a["exp_avg_sq"], b["exp_avg_sq"])
    ea, eb = (torch.load(p / "ema.pt", weights_only=True)["state"] for p in (end, tmp_path / "b" / "checkpoint_model_000004"))
    assert all(torch.equal(ea[k], eb[k]) for k in ea)
    # another observation profile or corpus refuses the checkpoint
    other = _config(tmp_path / "corpus", tmp_path / "c", checkpoint={"resume_from": str(mid)},
                    train={"observations": {"patterns": {"shared": 1.0}}})
    with pytest.raises(BackendContractError):
        RendererTrainingRuntime(other)
    # export: live and averaged weights; the export initialises a child run whose contract names its parent
    live = export_adapter(end, tmp_path / "export" / "live.pt")
    ema = export_adapter(end, tmp_path / "export" / "ema.pt", weight_source="ema")
    assert live["tensors"] == ema["tensors"] > 0 and live["identity"] != ema["identity"]
    assert set(read_adapter(tmp_path / "export" / "ema.pt")) == set(read_adapter(end))
    child_cfg = _config(tmp_path / "corpus", tmp_path / "d", checkpoint={"initialization": {"student": {"path": str(tmp_path / "export" / "ema.pt")}}},
                        train={"max_steps": 1, "gradient_accumulation_steps": 1})
    child = RendererTrainingRuntime(child_cfg)
    assert child.parents["control_initialization"] == ema["identity"] and child.checkpoint_id.startswith("init:sha256:")
    got = {n: p for n, p in child.model.named_parameters() if p.requires_grad}
    want = read_adapter(tmp_path / "export" / "ema.pt")
    assert all(torch.equal(got[n], want[n].to(got[n])) for n in want)
    child.close()
    for broken in ({"train": {"max_steps": 0}}, {"distributed": {"sequence_parallel_size": 2}}, {"train": {"objective": "other"}}):
        from solarwm_b200.errors import ConfigurationError

        with pytest.raises(ConfigurationError):
            validate_config(_config(tmp_path / "corpus", tmp_path / "x", **broken))
    # the command line: resolve, train, export
    import yaml

    (tmp_path / "cfg.yaml").write_text(yaml.safe_dump(_config(tmp_path / "corpus", tmp_path / "e", train={"max_steps": 1, "gradient_accumulation_steps": 1})))
    assert main(["train", "--config", str(tmp_path / "cfg.yaml"), "--resolve"]) == 0
    assert json.loads(capsys.readouterr().out)["train"]["max_steps"] == 1
    assert main(["train", "--config", str(tmp_path / "cfg.yaml"), "--set", "train.max_steps=2"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["final_step"] == 2
    assert main(["export", "--checkpoint", str(tmp_path / "e" / "checkpoint_model_000002"), "--out", str(tmp_path / "e.pt")]) == 0
    assert (tmp_path / "e.pt").is_file()


WORKER = """
import json, os, sys, torch
sys.path.insert(0, os.environ["REPO"])
from pathlib import Path
from tests.test_renderer_runtime import _config
from solarwm_b200.renderer.runtime import RendererTrainingRuntime
from solarwm_b200.engine.train_engine import StepPolicy, TrainingEngine
root = Path(os.environ["CORPUS"])
cfg = _config(root, os.environ["OUT"], train={"max_steps": 2, "gradient_accumulation_steps": 1}, data={"omni_length_buckets": True})
rt = RendererTrainingRuntime(cfg)
ids = []
TrainingEngine(rt, StepPolicy(max_steps=2, grad_accum=1, save_steps=(2,)),
               event_sink=lambda e: ids.extend(e.get("sample_ids", [])) if e.get("event") == "optimizer_step" else None).run()
print("RESULT " + json.dumps({"rank": rt.topology.raw_rank, "master": float(rt.optimizer.master.double().sum()), "cursor": rt.reader.cursor}), flush=True)
rt.close()
"""


def test_two_data_parallel_ranks_share_one_set_of_adapters(tmp_path):
    import os
    import socket
    import subprocess
    import sys

    _corpus(tmp_path / "corpus", n=6)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(2):
        env = dict(os.environ, REPO=repo, CORPUS=str(tmp_path / "corpus"), OUT=str(tmp_path / "run"), RANK=str(rank), LOCAL_RANK=str(rank),
                   WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    rows = [json.loads(l.split("RESULT ", 1)[1]) for o in outs for l in o.splitlines() if l.startswith("RESULT ")]
    assert len(rows) == 2 and rows[0]["master"] == rows[1]["master"] and rows[0]["cursor"] == rows[1]["cursor"] == 2
    saved = torch.load(tmp_path / "run" / "checkpoint_model_000002" / "rank-state.pt", weights_only=True)
    assert saved["world_size"] == 2 and [r["reader"]["cursor"] for r in saved["ranks"]] == [2, 2]


def test_example_config_trains_on_a_corpus(tmp_path, monkeypatch, capsys):
    from pathlib import Path

    from solarwm_b200.renderer.cli import main

    _corpus(tmp_path / "corpus", n=4)
    monkeypatch.setenv("SOLAR_OMNI_ROOT", str(tmp_path / "corpus"))
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "out"))
    config = str(Path(__file__).resolve().parent.parent / "configs" / "renderer" / "control_tiny_cpu.yaml")
    assert main(["train", "--config", config, "--set", "train.max_steps=2"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["final_step"] == 2
