"""Real two-process gloo runs on CPU: fail-together error propagation, the data-readiness side
channel with a failing and a slow reader, and the tiny Wan-style DiT (2 blocks, dim 128, SP=2 on gloo) trained
with Ulysses SP=2 matches the single-process oracle in loss and in every parameter gradient."""
import json
import os
import time
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _init(rank, world, path):
    dist.init_process_group("gloo", init_method=f"file://{path}", rank=rank, world_size=world,
                            timeout=timedelta(seconds=60))


def _failure_worker(rank, world, path, out):
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.runtime import distributed as rdist

    _init(rank, world, path)
    result = {}
    try:
        rdist.collective_call(lambda: (_ for _ in ()).throw(ValueError("shard 7 missing")) if rank == 1 else 1,
                              dist=dist, label="preflight")
    except BackendContractError as exc:
        result["collective"] = str(exc)
    state = torch.get_rng_state().clone()
    ready = rdist.DataReadiness(enabled=True, timeout=timedelta(seconds=30))

    def slow_then_fail():
        if rank == 0:
            time.sleep(1.0)            # a slow reader only delays its peers
            return "batch"
        raise OSError("bucket read failed")

    try:
        ready.read(slow_then_fail)
    except BackendContractError as exc:
        result["readiness"] = str(exc)
    result["rng_unchanged"] = bool(torch.equal(state, torch.get_rng_state()))
    result["ok_read"] = ready.read(lambda: rank)
    torch.save(result, f"{out}.{rank}")
    dist.destroy_process_group()


def test_errors_and_data_readiness_fail_together(tmp_path):
    out = str(tmp_path / "res")
    mp.spawn(_failure_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    r0, r1 = (torch.load(f"{out}.{r}", weights_only=True) for r in range(2))
    assert r0["collective"] == r1["collective"] == "preflight failed collectively: rank 1: ValueError: shard 7 missing"
    assert r0["readiness"] == r1["readiness"] and "rank 1: OSError: bucket read failed" in r0["readiness"]
    assert r0["rng_unchanged"] and r1["rng_unchanged"] and (r0["ok_read"], r1["ok_read"]) == (0, 1)


def _make_trainer(sp=None):
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer
    from solarwm_b200.models.wan import wan_preset

    tr = WanStage0p5Trainer(wan_preset("tiny"), "cpu", Stage0p5Options(lr=1e-3, seed=0, sigma_sampling="uniform_index"),
                            sp=sp, dtype=torch.float32)
    with torch.no_grad():
        tr.model.get_parameter("head.head.weight").normal_(0, 0.02, generator=torch.Generator().manual_seed(5))
    return tr


def _batch():
    g = torch.Generator().manual_seed(0)
    return torch.randn(1, 5, 16, 16, 16, generator=g), torch.randn(1, 32, 256, generator=g)


def _sp_worker(rank, world, path, out):
    from solarwm_b200.parallel.ulysses import UlyssesCollective

    _init(rank, world, path)
    tr = _make_trainer(UlyssesCollective(None))
    lat, txt = _batch()
    loss = tr.microbatch(lat, txt)
    tr.model.finalize_grads()
    tr.sp.sum_gradients_([g for u in tr.model.units() for g in (u.grad, u.grad_v)])
    grads = {n: p.main_grad.clone() for n, p in tr.model.named_parameters()}
    torch.save({"loss": loss, "grads": grads}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_tiny_wan_sp2_matches_single_process_oracle(tmp_path):
    tr = _make_trainer()
    lat, txt = _batch()
    loss = tr.microbatch(lat, txt)
    tr.model.finalize_grads()
    want = {n: p.main_grad.clone() for n, p in tr.model.named_parameters()}
    out = str(tmp_path / "sp")
    mp.spawn(_sp_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    got = [torch.load(f"{out}.{r}", weights_only=True) for r in range(2)]
    for r in got:
        assert abs(float(r["loss"]) - float(loss)) < 1e-5 * max(1.0, abs(float(loss)))
    worst = 0.0
    for name, ref in want.items():
        for r in got:
            err = (r["grads"][name] - ref).norm().item() / max(ref.norm().item(), 1e-8)
            worst = max(worst, err)
            assert err < 2e-4, (name, err)
    assert torch.equal(got[0]["grads"]["blocks.0.ffn.0.weight"], got[1]["grads"]["blocks.0.ffn.0.weight"])


def _zero_worker(rank, world, path, out):
    from solarwm_b200.engine.optim import FlatAdamW
    from solarwm_b200.parallel.flat import FlatUnit
    from solarwm_b200.parallel.zero import ZeroAdamW

    _init(rank, world, path)
    specs = [("a.weight", (24, 16), False), ("a.bias", (24,), False), ("n.weight", (16,), True)]

    def make():
        torch.manual_seed(0)
        u = FlatUnit(specs, "cpu", dtype=torch.float32, pad_to=world)
        for n, _, _ in specs:
            u.parameter(n)
        u.flat.normal_()
        u.flat_v.normal_()
        u.ensure_grads()
        return u

    u_ref, u_z = make(), make()
    ref = FlatAdamW([u_ref], lr=1e-2, weight_decay=0.1)
    zero = ZeroAdamW([u_z], None, lr=1e-2, weight_decay=0.1)
    for step in range(3):
        grads = []
        for r in range(world):                       # the gradient every rank would hold
            g = torch.Generator().manual_seed(100 * step + r)
            grads.append((torch.randn(u_ref.numel_m, generator=g), torch.randn(u_ref.numel_v, generator=g)))
        u_ref.grad.copy_(sum(g[0] for g in grads))
        u_ref.grad_v.copy_(sum(g[1] for g in grads))
        n_ref = ref.local_grad_sumsq().sqrt().clone()
        ref.set_clip(n_ref, 1.0)
        ref.step()
        u_z.grad.copy_(grads[rank][0])
        u_z.grad_v.copy_(grads[rank][1])
        n_z = zero.sharded_step(1.0)
        assert torch.allclose(n_z, n_ref, rtol=1e-5), (n_z, n_ref)
    torch.save({"flat": u_z.flat.clone(), "flat_v": u_z.flat_v.clone(), "ref": u_ref.flat.clone(),
                "ref_v": u_ref.flat_v.clone(), "state_numel": zero.state[0]["m"]["exp_avg"].numel(),
                "full": u_z.numel_m}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_zero_sharded_adamw_matches_unsharded(tmp_path):
    out = str(tmp_path / "zero")
    mp.spawn(_zero_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(f"{out}.{r}", weights_only=True)
        assert got["state_numel"] * 2 == got["full"]            # each rank holds half of the moments
        assert torch.allclose(got["flat"], got["ref"], atol=1e-6)
        assert torch.allclose(got["flat_v"], got["ref_v"], atol=1e-6)


def _tp_worker(rank, world, path, out):
    from solarwm_b200.models.vit_decoder import TensorParallelViT, ViTDecoderConfig, ViTVideoDecoder, rope_tables

    _init(rank, world, path)
    cfg = ViTDecoderConfig(latent_channels=4, dim=64, depth=2, heads=4, dim_head=16, ffn_dim=96, registers=2, patch=2)
    m = ViTVideoDecoder(cfg, device="cpu", dtype=torch.float32, seed=0)
    tp = TensorParallelViT(m)
    x = torch.randn(2, 12, 64, generator=torch.Generator().manual_seed(3))
    cos, sin = rope_tables(1, cfg.window, 3, 4, cfg.dim_head)
    want = x
    for blk in m.blocks:
        q, k, v = m.block_qkv(blk, want, cos, sin)
        want = m.block_finish(blk, want, m.attend(q, k, v))
    got = x
    for li in range(cfg.depth):
        got = tp.block(li, got, cos, sin)
    torch.save({"err": float((got - want).abs().max()), "shard_rows": tp.shards[0]["qkv"].shape[0]}, f"{out}.{rank}")
    dist.destroy_process_group()


def test_tensor_parallel_vit_block_matches_unsharded(tmp_path):
    out = str(tmp_path / "tp")
    mp.spawn(_tp_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(f"{out}.{r}", weights_only=True)
        assert got["err"] < 1e-4 and got["shard_rows"] == 3 * 2 * 16


def _h3_stream_worker(rank, world, path, out):
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.parallel.ulysses import UlyssesCollective
    from solarwm_b200.serve.h3_stream import H3StreamConfig, H3StreamingGenerator

    _init(rank, world, path)
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    scfg = H3StreamConfig(grid_hw=(2, 4), chunk_latents=2, window_chunks=2, denoise_steps=2, use_cuda_graph=False, seed=5)
    g = torch.Generator().manual_seed(1)
    text, anchor = torch.randn(9, cfg.text_dim, generator=g), torch.randn(24, 1, 4, 8, generator=g)
    outs = {}
    for name, sp in (("single", None), ("sp", UlyssesCollective(None))):
        gen = H3StreamingGenerator(model, scfg, sp=sp)
        gen.start(text, anchor, torch.eye(4))
        outs[name] = torch.stack([gen.next_chunk(None) for _ in range(4)])
    torch.save({"err": float((outs["single"] - outs["sp"]).abs().max()), "scale": float(outs["single"].abs().max())},
               f"{out}.{rank}")
    dist.destroy_process_group()


def test_h3_streaming_with_ulysses_matches_single_rank(tmp_path):
    out = str(tmp_path / "h3sp")
    mp.spawn(_h3_stream_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    for r in range(2):
        got = torch.load(f"{out}.{r}", weights_only=True)
        assert got["err"] < 1e-4 * max(got["scale"], 1.0), got


def _scene_worker(rank, world, path, out):
    from solarwm_b200.serve import scene_guard as sg

    _init(rank, world, path)
    good = {"text": torch.randn(6, 16), "anchor_latent": torch.randn(4, 1, 4, 6)}
    bad = dict(good, anchor_latent=torch.full((4, 1, 4, 6), float("nan")))
    kw = dict(text_dim=16, latent_channels=4, grid_hw=(2, 3))
    result = {"parked": 0}
    sg.admit_scene(sg.check_scene(good, **kw), dist=dist)                   # every rank agrees: proceeds
    try:                                                                     # only rank 1 holds a bad copy
        sg.admit_scene(sg.check_scene(bad if rank == 1 else good, **kw), dist=dist)
        result["raised"] = False
    except sg.SceneRejected as exc:
        result.update(raised=True, message=str(exc), agreed=exc.pre_call_collective_agreement)
        result["stage"] = sg.recover(exc, lambda: result.__setitem__("parked", result["parked"] + 1))
    try:
        sg.recover(sg.SceneRejected("local only", stage="x", pre_call_collective_agreement=False), lambda: None)
        result["local_recoverable"] = True
    except RuntimeError:
        result["local_recoverable"] = False
    sg.admit_scene(sg.check_scene(good, **kw), dist=dist)                   # the group is still usable afterwards
    torch.save(result, f"{out}.{rank}")
    dist.destroy_process_group()


def test_scene_rejection_is_agreed_before_any_device_work_and_parks(tmp_path):
    from solarwm_b200.serve.scene_guard import check_scene

    out = str(tmp_path / "scene")
    mp.spawn(_scene_worker, args=(2, str(tmp_path / "rdv"), out), nprocs=2, join=True)
    got = [torch.load(f"{out}.{r}", weights_only=True) for r in range(2)]
    assert all(g["raised"] and g["agreed"] and g["parked"] == 1 and g["stage"] == "scene_start" for g in got)
    assert got[0]["message"] == got[1]["message"] and "rank 1" in got[0]["message"] and "non-finite" in got[0]["message"]
    assert not got[0]["local_recoverable"]
    kw = dict(text_dim=16, latent_channels=4, grid_hw=(2, 3))
    assert "tokens" in check_scene({"text": torch.randn(0, 16), "anchor_latent": torch.randn(4, 1, 4, 6)}, **kw)
    assert "anchor" in check_scene({"text": torch.randn(3, 16), "anchor_latent": torch.randn(4, 1, 4, 5)}, **kw)
    assert "embedding" in check_scene({"text": torch.randn(3, 8), "anchor_latent": torch.randn(4, 1, 4, 6)}, **kw)


def _corpus_dp_worker(rank, world, path, out, index):
    import json
    import os

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    _init(rank, world, path)
    from solarwm_b200.backends.wan22.runtime import run_training

    root = f"{out}-run"
    config = {"schema": "solarwm.run.v1", "action": "train", "name": "dp-corpus",
              "model": {"family": "wan22_ti2v_5b", "architecture": "tiny", "timestep_shift": 5.0, "nonzero_head_init": True,
                        "camera_translation_transform": "linear"},
              "data": {"source": "index", "index": index, "seed": 0, "pixel_frames": 81, "latent_height": 4, "latent_width": 4},
              "distributed": {"world_size": 2, "sequence_parallel_size": 1},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "micro_batch_size": 1,
                        "grad_accum": 1, "global_batch_size": 2, "max_steps": 2, "warmup_steps": 0,
                        "optimizer": {"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.01, "grad_clip": 1.0}},
              "checkpoint": {"mode": "none"}, "runtime": {"output_dir": root, "device": "cpu", "save_every": 0, "validate_every": 0}}
    result = run_training(config)
    events = [json.loads(l) for l in open(os.path.join(root, "events", f"rank-{rank:05d}.jsonl"))]
    ids = [m["identity"]["sample_ids"][0] for e in events if e["event"] == "optimizer_step" for m in e["microbatches"]]
    norms = [e["gradient_norm"] for e in events if e["event"] == "optimizer_step"]
    torch.save({"ids": ids, "norms": norms, "final": result["final_step"]}, f"{out}.{rank}")
    if dist.is_initialized():
        dist.destroy_process_group()


def test_data_parallel_ranks_read_disjoint_corpus_samples(tmp_path):
    from solarwm_b200.backends.wan22.preencode import run_preencode

    pre = {"data": {"pixel_frames": 81, "pixel_height": 32, "pixel_width": 32, "seed": 3}, "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 4, "output_root": str(tmp_path / "enc"), "samples_per_shard": 2,
                         "codecs": {"z_dim": 16, "vae_base": 8, "t5": {"vocab": 512, "dim": 256, "dim_attn": 32, "dim_ffn": 64,
                                                                      "num_heads": 2, "num_layers": 1, "text_len": 32}}}}
    assert run_preencode(pre, "wan22_ti2v_5b")["samples"] == 4
    out = str(tmp_path / "dp")
    mp.spawn(_corpus_dp_worker, args=(2, str(tmp_path / "rdv"), out, str(tmp_path / "enc" / "index.jsonl")), nprocs=2, join=True)
    got = [torch.load(f"{out}.{r}", weights_only=True) for r in range(2)]
    assert got[0]["final"] == got[1]["final"] == 2
    assert len(got[0]["ids"]) == 2 and not set(got[0]["ids"]) & set(got[1]["ids"])          # disjoint ownership
    assert got[0]["norms"] == got[1]["norms"]                                               # one all-reduced gradient


def _sharded_ckpt_worker(rank, world, path, out, root, resume_from):
    """SP = 2 with the optimizer (and its EMA shadow) sharded over both ranks: train, save, or resume and continue."""
    import json
    import os

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    _init(rank, world, path)
    from solarwm_b200.backends.wan22.runtime import run_training

    config = {"schema": "solarwm.run.v1", "action": "train", "name": "sharded-ckpt",
              "model": {"family": "wan22_ti2v_5b", "architecture": "tiny", "timestep_shift": 5.0, "nonzero_head_init": True,
                        "camera_translation_transform": "linear"},
              "data": {"source": "synthetic", "seed": 0, "pixel_frames": 81, "latent_height": 4, "latent_width": 4},
              "distributed": {"world_size": 2, "sequence_parallel_size": 2},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "micro_batch_size": 1,
                        "grad_accum": 1, "global_batch_size": 1, "max_steps": 4, "warmup_steps": 1,
                        "optimizer": {"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8, "weight_decay": 0.01, "grad_clip": 1.0},
                        "ema": {"enabled": True, "decay": 0.9}, "zero": {"enabled": True, "transport": "collective"}},
              "checkpoint": ({"mode": "full_resume", "resume_from": resume_from} if resume_from else {"mode": "none"}),
              "runtime": {"output_dir": root, "device": "cpu", "save_every": 0 if resume_from else 2, "validate_every": 0}}
    result = run_training(config)
    events = [json.loads(l) for l in open(os.path.join(root, "events", f"rank-{rank:05d}.jsonl"))]
    steps = {e["step"]: (e["losses"], e["gradient_norm"]) for e in events if e["event"] == "optimizer_step"}
    torch.save({"steps": steps, "final": result["final_step"]}, f"{out}.{rank}")
    if dist.is_initialized():
        dist.destroy_process_group()


def test_sharded_optimizer_and_ema_checkpoint_resumes_exactly(tmp_path):
    """Two ranks, optimizer state and EMA sharded over them: the checkpoint holds EVERY rank's share (un-sharded
    layout), and a run resumed from step 2 reproduces steps 3 and 4 of the uninterrupted run."""
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    mp.spawn(_sharded_ckpt_worker, args=(2, str(tmp_path / "rdv-a"), str(tmp_path / "ra"), a, None), nprocs=2, join=True)
    ckpt_dir = tmp_path / "a" / "checkpoint_model_000002"
    payload = torch.load(ckpt_dir / "model.pt", map_location="cpu", weights_only=True)
    opt = payload["optimizer"]
    assert opt["layout"] == "full"
    for unit in opt["units"]:
        for key in ("m", "v"):
            n = unit[key]["numel"]
            assert unit[key]["exp_avg"].numel() == n and unit[key]["exp_avg_sq"].numel() == n and unit[key]["ema"].numel() == n
    # second halves (rank 1's shards) are real state, not zeros
    first = opt["units"][1]["m"]
    half = first["numel"] // 2
    assert first["exp_avg_sq"][half:].abs().sum() > 0 and first["exp_avg_sq"][:half].abs().sum() > 0
    assert first["master"] is None or first["master"][half:].abs().sum() > 0      # fp32 runs have no separate master
    assert set(payload["generator_ema"]) == set(payload["generator"])
    name = "blocks.0.ffn.0.weight"
    assert not torch.equal(payload["generator_ema"][name].float(), payload["generator"][name].float())
    mp.spawn(_sharded_ckpt_worker, args=(2, str(tmp_path / "rdv-b"), str(tmp_path / "rb"), b, str(ckpt_dir)), nprocs=2, join=True)
    ra = [torch.load(f"{tmp_path / 'ra'}.{r}", weights_only=True) for r in range(2)]
    rb = [torch.load(f"{tmp_path / 'rb'}.{r}", weights_only=True) for r in range(2)]
    assert sorted(rb[0]["steps"]) == [3, 4] and rb[0]["final"] == rb[1]["final"] == 4
    for s in (3, 4):
        for r in range(2):
            assert rb[r]["steps"][s] == ra[r]["steps"][s], (s, r, rb[r]["steps"][s], ra[r]["steps"][s])


def _h3_config(root, world, sp, resume_from=None, max_steps=4, save_every=2, stage="stage0p5"):
    route = {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching"} if stage == "stage0p5" else \
        {"stage": "stage1", "causal_mode": "teacher_forcing", "objective": "anyflow_forward_map", "objective_variant": "v1_5"}
    frames = {"latent_frames": 3, "latent_height": 8, "latent_width": 8} if stage == "stage0p5" else \
        {"latent_frames": 4, "latent_height": 4, "latent_width": 4}
    return {"schema": "solarwm.run.v1", "action": "train", "name": "h3-multi",
            "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4},
                      "camera_translation_transform": "logd4", "causal": {"chunk_latents": 2, "window_chunks": 1}},
            "data": {"source": "synthetic", "seed": 0, "pixel_frames": 158, "prompt_len": 7, **frames},
            "distributed": {"world_size": world, "sequence_parallel_size": sp},
            "train": {**route, "max_steps": max_steps,
                      "grad_accum": 1, "optimizer": {"lr": 1e-3, "warmup_steps": 1}, "ema": {"enabled": True, "decay": 0.9}},
            "checkpoint": ({"mode": "full_resume", "resume_from": resume_from} if resume_from else {"mode": "none"}),
            "runtime": {"output_dir": root, "device": "cpu", "save_every": 0 if resume_from else save_every,
                        "save_final": not resume_from}}


def _h3_train_worker(rank, world, path, out, root, sp, resume_from, stage="stage0p5"):
    import json
    import os

    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world))
    _init(rank, world, path)
    from solarwm_b200.registry import load_backend

    load_backend("minimax_h3").train(_h3_config(root, world, sp, resume_from, stage=stage))
    events = [json.loads(l) for l in open(os.path.join(root, "events", f"rank-{rank:05d}.jsonl"))]
    steps = {e["step"]: (e["losses"], e["gradient_norm"]) for e in events if e["event"] == "optimizer_step"}
    torch.save({"steps": steps}, f"{out}.{rank}")
    if dist.is_initialized():
        dist.destroy_process_group()


def test_h3_adapter_training_on_two_ranks(tmp_path):
    """SP = 2 (both ranks hold half the packed rows of one sample) reproduces the single-process losses and gradient
    norms; a checkpoint written by both ranks holds ``ema.pt`` and every rank's random streams, and a resumed run
    repeats steps 3 and 4."""
    from solarwm_b200.registry import load_backend

    one = load_backend("minimax_h3").train(_h3_config(str(tmp_path / "one"), 1, 1))
    single = {e["step"]: (e["losses"]["loss"], e["gradient_norm"])
              for e in map(json.loads, open(tmp_path / "one" / "events" / "rank-00000.jsonl")) if e["event"] == "optimizer_step"}
    assert one["final_step"] == 4 and sorted(single) == [1, 2, 3, 4]
    a, b = str(tmp_path / "a"), str(tmp_path / "b")
    mp.spawn(_h3_train_worker, args=(2, str(tmp_path / "rdv-a"), a, str(tmp_path / "ra"), 2, None), nprocs=2, join=True)
    got = [torch.load(f"{a}.{r}", weights_only=False)["steps"] for r in range(2)]
    assert got[0] == got[1]
    for s in range(1, 5):
        assert abs(got[0][s][0]["loss"] - single[s][0]) < 1e-4 * max(1.0, single[s][0]), (s, got[0][s], single[s])
        assert abs(got[0][s][1] - single[s][1]) < 1e-3 * max(1.0, single[s][1]), (s, got[0][s], single[s])
    ckpt = tmp_path / "ra" / "checkpoint_model_000002"
    assert {"adapter.pt", "optimizer.pt", "scheduler.pt", "ema.pt", "rank-state.pt", "runtime.pt"} <= {p.name for p in ckpt.iterdir()}
    ranks = torch.load(ckpt / "rank-state.pt", weights_only=True)
    assert ranks["world_size"] == 2 and len(ranks["ranks"]) == 2
    ema = torch.load(ckpt / "ema.pt", weights_only=True)
    adapter = torch.load(ckpt / "adapter.pt", weights_only=True)["state"]
    assert ema["num_updates"] == 2 and set(ema["state"]) == set(adapter)
    assert any(not torch.allclose(ema["state"][k], adapter[k].float()) for k in adapter)      # an average, not a copy
    mp.spawn(_h3_train_worker, args=(2, str(tmp_path / "rdv-b"), b, str(tmp_path / "rb"), 2, str(ckpt)), nprocs=2, join=True)
    again = torch.load(f"{b}.0", weights_only=False)["steps"]
    assert sorted(again) == [3, 4] and all(again[s] == got[0][s] for s in (3, 4))


def test_h3_data_parallel_ranks_average_their_gradients(tmp_path):
    """DP = 2: the replicas read different samples, report different losses and apply ONE averaged gradient."""
    out = str(tmp_path / "dp")
    mp.spawn(_h3_train_worker, args=(2, str(tmp_path / "rdv"), out, str(tmp_path / "r"), 1, None), nprocs=2, join=True)
    got = [torch.load(f"{out}.{r}", weights_only=False)["steps"] for r in range(2)]
    assert all(got[0][s][0] != got[1][s][0] for s in got[0]) and all(got[0][s][1] == got[1][s][1] for s in got[0])


def test_h3_stage1_anyflow_runs_data_parallel_and_refuses_sequence_parallel(tmp_path):
    """Stage1 (teacher forcing, AnyFlow objective) behind the same runtime: two replicas on different samples apply one
    averaged adapter gradient; SP > 1 is refused up front (one packed video per rank)."""
    out = str(tmp_path / "s1")
    mp.spawn(_h3_train_worker, args=(2, str(tmp_path / "rdv"), out, str(tmp_path / "r"), 1, None, "stage1"), nprocs=2, join=True)
    got = [torch.load(f"{out}.{r}", weights_only=False)["steps"] for r in range(2)]
    assert sorted(got[0]) == [1, 2, 3, 4]
    assert all(got[0][s][0] != got[1][s][0] for s in got[0]) and all(got[0][s][1] == got[1][s][1] for s in got[0])
    assert (tmp_path / "r" / "checkpoint_model_000004" / "ema.pt").is_file()
