"""LTX adapter training runtime: exact resume, the resume identity, gradient accumulation, SP = 2 and DP = 2 on gloo."""
import json
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

from solarwm_b200.errors import BackendContractError


def _config(out, **over):
    cfg = {"schema": "solarwm.run.v1", "action": "train", "name": "ltx-lora",
           "model": {"family": "ltx25_video", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "linear"},
           "data": {"source": "synthetic", "seed": 2, "pixel_frames": 153, "latent_frames": 2, "latent_height": 4, "latent_width": 4},
           "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 4, "grad_accum": 2,
                     "optimizer": {"lr": 1e-3, "warmup_steps": 1}, "ema": {"decay": 0.5}},
           "runtime": {"output_dir": str(out), "device": "cpu", "save_every": 2}}
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v}
    return cfg


def test_resume_is_exact_and_needs_the_same_runtime_semantics(tmp_path):
    from solarwm_b200.backends.ltx25.runtime import COMPONENTS, LTXTrainingRuntime, run_training
    from solarwm_b200.checkpoint.store import verify_checkpoint

    a = run_training(_config(tmp_path / "a"))
    assert a["final_step"] == 4 and a["last_loss"] == a["last_loss"]
    end = verify_checkpoint(a["checkpoint"])
    assert all((end.path / c).is_file() for c in COMPONENTS)
    run = torch.load(end.path / "runtime.pt", weights_only=True)
    assert run["fingerprint"]["schema"] == "solarwm.ltx25.checkpoint.v1" and run["fingerprint"]["lora"]["rank"] == 4
    assert len(run["adapter_targets"]) == 2 * 10 and run["fingerprint"]["lora"]["target_count"] == 20
    mid = tmp_path / "a" / "checkpoint_model_000002"
    b = run_training(_config(tmp_path / "b", checkpoint={"mode": "full_resume", "resume_from": str(mid)}))
    ea, eb = (torch.load(p / "optimizer.pt", weights_only=True) for p in (end.path, verify_checkpoint(b["checkpoint"]).path))
    assert torch.equal(ea["master"], eb["master"]) and torch.equal(ea["exp_avg_sq"], eb["exp_avg_sq"])
    xa, xb = (torch.load(p / "ema.pt", weights_only=True) for p in (end.path, verify_checkpoint(b["checkpoint"]).path))
    assert torch.equal(xa["flat"], xb["flat"]) and xa["num_updates"] == xb["num_updates"] == 4
    # another camera transform, another averaging recipe or another rank is not the same run
    for over in ({"model": {"camera_translation_transform": "logd4"}}, {"train": {"ema": {"decay": 0.9}}}):
        with pytest.raises(BackendContractError) as err:
            LTXTrainingRuntime(_config(tmp_path / "c", checkpoint={"mode": "full_resume", "resume_from": str(mid)}, **over))
        assert "differing" in str(err.value)
    with pytest.raises(BackendContractError):
        LTXTrainingRuntime(_config(tmp_path / "c", checkpoint={"mode": "full_resume", "resume_from": str(mid)}, model={"adapter": {"rank": 8}}))
    with pytest.raises(BackendContractError):
        LTXTrainingRuntime(_config(tmp_path / "c", model={"adapter": {"rank": 0}}))


WORKER = textwrap.dedent("""
    import json, os, sys, torch
    sys.path.insert(0, os.environ["REPO"])
    from tests.test_ltx_runtime import _config
    from solarwm_b200.backends.ltx25.runtime import LTXTrainingRuntime
    from solarwm_b200.engine.train_engine import StepPolicy, TrainingEngine
    sp = int(os.environ["SP"])
    cfg = _config(os.environ["OUT"], distributed={"sequence_parallel_size": sp}, train={"grad_accum": 1, "max_steps": 2})
    rt = LTXTrainingRuntime(cfg)
    losses = []
    TrainingEngine(rt, StepPolicy(max_steps=2, grad_accum=1), event_sink=lambda e: losses.append(e["losses"]["loss"]) if e.get("event") == "optimizer_step" else None).run()
    print("RESULT " + json.dumps({"rank": rt.topology.raw_rank, "master": float(rt.optimizer.master.double().sum()),
                                   "abs": float(rt.optimizer.master.double().abs().sum()), "losses": losses}), flush=True)
    rt.close()
""")


def _spawn(tmp_path, world, sp):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / f"worker_{world}_{sp}.py"
    script.write_text(WORKER)
    procs = []
    for rank in range(world):
        env = dict(os.environ, REPO=repo, OUT=str(tmp_path / f"run_{world}_{sp}"), SP=str(sp), RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    return [json.loads(l.split("RESULT ", 1)[1]) for o in outs for l in o.splitlines() if l.startswith("RESULT ")]


def test_sequence_parallel_equals_one_process_and_data_parallel_keeps_replicas_identical(tmp_path):
    one = _spawn(tmp_path, 1, 1)[0]
    sp2 = _spawn(tmp_path, 2, 2)
    assert sp2[0]["master"] == sp2[1]["master"]
    # two ranks splitting one sample's tokens take the same steps as one process
    assert sp2[0]["losses"] == pytest.approx(one["losses"], rel=2e-4) and sp2[0]["abs"] == pytest.approx(one["abs"], rel=1e-4)
    dp2 = _spawn(tmp_path, 2, 1)
    assert dp2[0]["master"] == dp2[1]["master"] and dp2[0]["losses"] != dp2[1]["losses"]     # different samples, one set of adapters


def test_inference_samples_with_trained_adapters_live_or_averaged(tmp_path):
    from solarwm_b200.backends.ltx25.runtime import adapter_weights, run_training
    from solarwm_b200.registry import load_backend

    out = run_training(_config(tmp_path / "train"))
    meta, live, _ = adapter_weights(out["checkpoint"], "live")
    _, ema, _ = adapter_weights(out["checkpoint"], "ema")
    assert set(live) == set(ema) == set(meta["state_keys"]) and all(live[k].shape == ema[k].shape for k in live)
    moved = [k for k in live if "lora_B" in k and float((live[k] - ema[k]).abs().max()) > 0]
    assert moved                                                    # the average trails the live weights
    be = load_backend("ltx25_video")
    base = {"schema": "solarwm.run.v1", "action": "infer", "model": {"family": "ltx25_video", "architecture": "tiny"},
            "data": {"seed": 2}, "inference": {"cases": 1, "latent_frames": 2, "latent_height": 4, "latent_width": 4, "steps": 2}}
    got = {}
    for name, ck in (("random", {}), ("live", {"resume_from": out["checkpoint"], "weight_source": "live"}),
                     ("ema", {"resume_from": out["checkpoint"], "weight_source": "ema"})):
        r = be.infer({**base, "checkpoint": ck, "runtime": {"output_dir": str(tmp_path / name), "device": "cpu"}})
        got[name] = torch.load(next((tmp_path / name / "generate").rglob("latents.pt")), weights_only=True)
        assert (r["weights_id"] == "init:random") == (name == "random")
    assert not torch.equal(got["live"], got["ema"]) and got["live"].shape == got["ema"].shape
    with pytest.raises(BackendContractError):
        adapter_weights(out["checkpoint"], "other")


def test_cameras_condition_the_adapter_training_step(tmp_path):
    from solarwm_b200.backends.ltx25.runtime import LTXTrainingRuntime

    losses = {}
    for name, data in (("plain", {}), ("cameras", {"cameras": True})):
        rt = LTXTrainingRuntime(_config(tmp_path / name, data=data))
        try:
            losses[name] = rt.train_microbatch(0, 1).losses["loss"]
            cond = rt._camera_condition()
            assert (cond is None) == (name == "plain")
            if cond is not None:
                assert cond["viewmats"].shape == (1, 2, 4, 4) and torch.equal(cond["viewmats"][0, 0], torch.eye(4)) and cond["Ks"].shape == (1, 2, 3, 3)
        finally:
            rt.close()
    assert losses["plain"] != losses["cameras"]                       # same sample and noise, another attention geometry


def test_validation_loss_on_frozen_clips(tmp_path):
    from solarwm_b200.backends.ltx25.runtime import LTXTrainingRuntime
    from solarwm_b200.registry import load_backend

    be = load_backend("ltx25_video")
    pre = {"schema": "solarwm.run.v1", "action": "preencode", "model": {"family": "ltx25_video", "architecture": "tiny"},
           "data": {"pixel_frames": 9, "pixel_height": 64, "pixel_width": 64, "seed": 1}, "runtime": {"device": "cpu", "output_dir": str(tmp_path / "pre")},
           "preencode": {"source": "synthetic", "num_samples": 3, "output_root": str(tmp_path / "enc"),
                         "codecs": {"z_dim": 16, "vae_base": 4, "t5": {"vocab": 512, "dim": 64, "dim_attn": 32, "dim_ffn": 64, "num_heads": 2,
                                                                      "num_layers": 1, "text_len": 16}}}}
    assert be.preencode(pre)["samples"] == 3
    cfg = _config(tmp_path / "run", validation={"index": str(tmp_path / "enc" / "index.jsonl"), "sample_count": 2, "balance_sources": False})
    rt = LTXTrainingRuntime(cfg)
    try:
        first = rt.validate(0)["validation"]
        assert first["clips"] == 2 and first["loss"] > 0 and rt.validate(0)["validation"] == first
        with torch.no_grad():
            rt.optimizer.master.add_(0.05)
            rt.optimizer.live.copy_(rt.optimizer.master.to(rt.optimizer.live.dtype))
        assert rt.validate(1)["validation"]["loss"] != first["loss"]
    finally:
        rt.close()
