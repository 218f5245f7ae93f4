"""H3 Stage2 runtime: phases on separate samples, exact resume of both roles, the EMA's creation boundary, role
initialisation from adapter files, refusal of non-finite updates, and two data-parallel ranks on gloo."""
import copy
import os
import subprocess
import sys
import textwrap

import pytest
import torch


def _config(tmp, **over):
    cfg = {"schema": "solarwm.run.v1", "action": "train",
           "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4},
                     "camera_translation_transform": "logd4", "causal": {"chunk_latents": 2, "window_chunks": 1}},
           "data": {"seed": 3, "latent_frames": 4, "latent_height": 4, "latent_width": 4, "prompt_len": 6, "pixel_frames": 158},
           "runtime": {"device": "cpu", "output_dir": str(tmp)},
           "train": {"stage": "stage2", "causal_mode": "self_gradient_forcing", "objective": "flow_matching", "objective_variant": "",
                     "max_steps": 6, "optimizer": {"lr": 1e-3}, "critic_optimizer": {"lr": 5e-4}, "denoise_steps": 1,
                     "critic_updates_per_student": 2},
           "checkpoint": {"ema": {"start_step": 2, "decay": 0.5}, "save_steps": [4]}}
    for k, v in over.items():
        cfg[k] = {**cfg.get(k, {}), **v}
    return cfg


def _model_config():
    from solarwm_b200.backends.minimax_h3.backend import MiniMaxH3Backend

    return lambda cfg: MiniMaxH3Backend("minimax_h3")._cfg(cfg)


def _kick(runtime):
    """LoRA up-projections start at zero; give them values so the student's gradients are not trivially zero."""
    for opt in (runtime.trainer.opt_s, runtime.trainer.opt_c):
        g = torch.Generator().manual_seed(5)
        opt.master.copy_(torch.randn(opt.master.shape, generator=g) * 0.02)
        opt.live.copy_(opt.master.to(opt.live.dtype))


def test_resume_continues_both_roles_exactly_and_the_ema_starts_at_its_boundary(tmp_path):
    from solarwm_b200.backends.minimax_h3.stage2_runtime import COMPONENTS, H3SGFRuntime
    from solarwm_b200.checkpoint.store import verify_checkpoint
    from solarwm_b200.errors import BackendContractError

    mc = _model_config()
    cfg = _config(tmp_path / "a")
    straight = H3SGFRuntime(cfg, model_config=mc(cfg))
    _kick(straight)
    seen = []
    for _ in range(6):
        stats = straight.train_outer_step()
        seen.append((stats["student_updated"], straight.student_step, straight.ema is not None))
        if straight.global_step == 4:
            straight.save_checkpoint(4)
    # two critic-only steps come first; student updates on outer steps 3 and 5; the average exists from the 2nd one on
    assert seen == [(0.0, 0, False), (0.0, 0, False), (1.0, 1, False), (0.0, 1, False), (1.0, 2, True), (0.0, 2, True)]
    assert all(stats[k] == stats[k] for k in ("loss_critic", "critic_grad_norm", "loss"))
    ck = tmp_path / "a" / "checkpoint_model_000004"
    found = verify_checkpoint(str(ck))
    assert found.step == 4 and all((found.path / c).is_file() for c in COMPONENTS)
    assert torch.load(found.path / "ema.pt", weights_only=True)["state"] is None
    cfg_b = _config(tmp_path / "b", checkpoint={"resume_from": str(ck)})
    resumed = H3SGFRuntime(cfg_b, model_config=mc(cfg_b))
    assert resumed.global_step == 4 and resumed.student_step == 1 and resumed.ema is None
    while resumed.global_step < 6:
        resumed.train_outer_step()
    for a, b in ((straight.trainer.opt_s, resumed.trainer.opt_s), (straight.trainer.opt_c, resumed.trainer.opt_c)):
        assert torch.equal(a.master, b.master) and torch.equal(a.exp_avg_sq, b.exp_avg_sq) and a.step_count == b.step_count
    assert torch.equal(straight.ema.shadow, resumed.ema.shadow)
    # a checkpoint with an average, resumed under a later boundary, is refused
    resumed.save_checkpoint(6)
    late = _config(tmp_path / "c", checkpoint={"resume_from": str(tmp_path / "b" / "checkpoint_model_000006"),
                                                "ema": {"start_step": 9, "decay": 0.5}})
    with pytest.raises(BackendContractError):
        H3SGFRuntime(late, model_config=mc(late))
    for r in (straight, resumed):
        r.close()


def test_roles_start_from_adapter_files_and_the_teacher_is_a_frozen_third_role(tmp_path):
    from solarwm_b200.backends.minimax_h3.runtime import ADAPTER_SCHEMA
    from solarwm_b200.backends.minimax_h3.stage2_runtime import H3SGFRuntime, run_sgf_training
    from solarwm_b200.errors import BackendContractError

    mc = _model_config()
    cfg = _config(tmp_path / "a")
    first = H3SGFRuntime(cfg, model_config=mc(cfg))
    _kick(first)
    state = {n: p.detach().clone() for n, p in first.trainer.student.named_parameters() if p.requires_grad}
    first.close()
    torch.save({"schema": ADAPTER_SCHEMA, "state": state, "rank": 4}, tmp_path / "stage1-adapter.pt")
    torch.save({"schema": "other", "state": state}, tmp_path / "bad.pt")
    init = {"student": str(tmp_path / "stage1-adapter.pt"), "teacher": str(tmp_path / "stage1-adapter.pt")}
    cfg2 = _config(tmp_path / "b", checkpoint={"initialization": init})
    rt = H3SGFRuntime(cfg2, model_config=mc(cfg2))
    tr = rt.trainer
    assert tr.teacher is not None and not any(p.requires_grad for p in tr.teacher.parameters())
    got = {n: p for n, p in tr.student.named_parameters() if p.requires_grad}
    assert all(torch.equal(got[n], state[n]) for n in state) and torch.equal(tr.opt_s.master[:8], tr.opt_s.live[:8].float())
    # the three roles alias one base
    base_s = {n: p.data_ptr() for n, p in tr.student.named_parameters() if not p.requires_grad}
    base_t = {n: p.data_ptr() for n, p in tr.teacher.named_parameters() if "lora_" not in n}
    shared = [n for n in base_s if n in base_t and base_s[n] == base_t[n]]
    assert len(shared) > 10
    teacher_before = {n: p.detach().clone() for n, p in tr.teacher.named_parameters() if "lora_" in n}
    for _ in range(3):
        rt.train_outer_step()
    assert rt.student_step == 1
    assert all(torch.equal(p, teacher_before[n]) for n, p in tr.teacher.named_parameters() if "lora_" in n)
    assert rt.initialization["teacher"].endswith("stage1-adapter.pt")
    rt.close()
    bad = _config(tmp_path / "c", checkpoint={"initialization": {"critic": str(tmp_path / "bad.pt")}})
    with pytest.raises(BackendContractError):
        H3SGFRuntime(bad, model_config=mc(bad))
    # the whole loop through the backend entry: events, final checkpoint
    cfg3 = _config(tmp_path / "d", train={"max_steps": 3})
    out = run_sgf_training(cfg3, model_config=mc(cfg3))
    assert out["final_step"] == 3 and out["student_step"] == 1 and out["checkpoint"].endswith("checkpoint_model_000003")
    events = (tmp_path / "d" / "events").glob("*.jsonl") if (tmp_path / "d" / "events").is_dir() else (tmp_path / "d").rglob("*.jsonl")
    lines = [l for f in events for l in f.read_text().splitlines()]
    assert sum('"train_step"' in l for l in lines) == 3


def test_a_non_finite_update_is_refused_before_the_weights_change(tmp_path):
    from solarwm_b200.backends.minimax_h3.stage2_runtime import H3SGFRuntime

    mc = _model_config()
    cfg = _config(tmp_path)
    rt = H3SGFRuntime(cfg, model_config=mc(cfg))
    _kick(rt)
    before = rt.trainer.opt_c.master.clone()
    rt.trainer.sync = lambda params, flat: flat.fill_(float("nan"))          # a poisoned reduction
    with pytest.raises(FloatingPointError):
        rt.trainer.critic_phase(rt._next_sample(), 2)
    assert torch.equal(rt.trainer.opt_c.master, before) and rt.trainer.opt_c.step_count == 0
    assert all(p.grad is None for p in rt.trainer.opt_c.params)
    rt.close()


WORKER = textwrap.dedent("""
    import json, os, sys, torch
    sys.path.insert(0, os.environ["REPO"])
    from tests.test_h3_sgf_runtime import _config, _kick, _model_config
    from solarwm_b200.backends.minimax_h3.stage2_runtime import H3SGFRuntime
    cfg = _config(os.environ["OUT"], distributed={"world_size": 2})
    rt = H3SGFRuntime(cfg, model_config=_model_config()(cfg))
    _kick(rt)
    for _ in range(3):
        rt.train_outer_step()
    rt.save_checkpoint(3)
    tr = rt.trainer
    print("RESULT " + json.dumps({"rank": rt.topology.raw_rank, "s": float(tr.opt_s.master.double().sum()),
                                   "c": float(tr.opt_c.master.double().sum()), "consumed": rt.batches_consumed}), flush=True)
    rt.close()
""")


def test_two_data_parallel_ranks_keep_their_adapters_identical(tmp_path):
    import json
    import socket

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
    assert len(rows) == 2 and rows[0]["s"] == rows[1]["s"] and rows[0]["c"] == rows[1]["c"]
    assert all(r["consumed"] == 4 for r in rows)                   # one critic sample per step, one more for the student on step 3
    saved = torch.load(tmp_path / "run" / "checkpoint_model_000003" / "rank-state.pt", weights_only=True)
    assert saved["world_size"] == 2 and len(saved["ranks"]) == 2


def test_the_silent_soundtrack_enters_the_replay_and_every_score(tmp_path):
    """With ``data.silence_latents_path`` the teacher-forced replay and the critic / real score evaluations carry the
    audio rows (the score evaluations of one student phase share one draw); a run with them repeats itself exactly."""
    from safetensors.torch import save_file

    from solarwm_b200.backends.minimax_h3.silence import LENGTHS
    from solarwm_b200.backends.minimax_h3.stage2_runtime import H3SGFRuntime

    path = tmp_path / "s.safetensors"
    save_file({"silence_158f": (torch.randn(2, 32, LENGTHS[158], generator=torch.Generator().manual_seed(0)) * 0.1).to(torch.bfloat16)}, str(path))
    mc = _model_config()

    def run(name, silent):
        cfg = _config(tmp_path / name, data={"silence_latents_path": str(path)} if silent else {})
        rt = H3SGFRuntime(cfg, model_config=mc(cfg))
        _kick(rt)
        seen = []
        for role, model in (("student", rt.trainer.student), ("critic", rt.trainer.critic)):
            held = model.forward
            model.forward = (lambda held, role: lambda **k: (seen.append(
                (role, None if k.get("audio_rows") is None else (tuple(k["audio_rows"].shape), float(k["audio_rows"].float().sum())))), held(**k))[1])(held, role)
        stats = [rt.train_outer_step() for _ in range(3)]
        return seen, stats, [p.detach().clone() for p in rt.trainer.student.trainable_parameters()]

    plain_seen, plain_stats, _ = run("plain", False)
    assert plain_seen and all(a is None for _, a in plain_seen)
    seen, stats, weights = run("silent", True)
    # the streaming rollout itself carries no audio rows; every teacher-forced and bidirectional evaluation does
    with_audio = [(r, a) for r, a in seen if a is not None]
    assert with_audio and all(a[0] == (2 * LENGTHS[158], 32) for _, a in with_audio)
    assert {r for r, _ in with_audio} == {"student", "critic"}
    third = stats[2]
    assert third["student_updated"] == 1.0 and third["loss"] == third["loss"]
    assert stats[0]["loss_critic"] != plain_stats[0]["loss_critic"]
    again_seen, again_stats, again_weights = run("silent-again", True)
    assert again_seen == seen and all(torch.equal(a, b) for a, b in zip(weights, again_weights))
