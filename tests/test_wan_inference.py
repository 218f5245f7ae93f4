"""Wan generation: UniPC / Euler samplers with first-frame anchoring, data-parallel case partitions and their merge."""
import json
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from solarwm_b200.backends.wan22.inference import merge_partitions, partition_cases, sample_bidirectional
from solarwm_b200.engine.inference_engine import GeneratedSample, InferenceCase, InferenceEngine
from solarwm_b200.errors import BackendContractError
from solarwm_b200.models.wan import WanDiT, wan_preset


def _tiny():
    cfg = wan_preset("tiny")
    model = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=3)
    with torch.no_grad():
        model.get_parameter("head.head.weight").normal_(0, 0.3)       # the released init predicts zero velocity
    return model, cfg


def _case(i):
    return InferenceCase(slot=i, sample_id=f"case-{i:04d}", prompt=f"p{i}", start_frame=0, noise_seed=100 + i,
                         camera_fingerprint="none")


def test_unipc_and_euler_agree_as_steps_grow_and_anchor_holds():
    model, cfg = _tiny()
    torch.manual_seed(0)
    text = torch.randn(1, cfg.text_len, cfg.text_dim)
    kw = dict(frames=3, height=4, width=4, shift=3.0, seed=5)
    fine, _ = sample_bidirectional(model, text, steps=64, solver="euler", **kw)
    uni, sig = sample_bidirectional(model, text, steps=8, solver="unipc", **kw)
    eul, _ = sample_bidirectional(model, text, steps=8, solver="euler", **kw)
    assert len(sig) == 9 and sig[-1] == 0.0 and sig[0] > sig[1]
    # the second-order multistep solver is closer to the fine-grid solution than first-order steps on the same grid
    assert (uni - fine).norm() < (eul - fine).norm()
    anchor = torch.randn(cfg.out_dim, 4, 4)
    for solver in ("unipc", "euler"):
        x, _ = sample_bidirectional(model, text, steps=3, solver=solver, first_frame=anchor, **kw)
        assert torch.equal(x[0, 0], anchor) and torch.isfinite(x).all()
        free, _ = sample_bidirectional(model, text, steps=3, solver=solver, **kw)
        assert not torch.allclose(x[0, 1], free[0, 1])                  # the anchor conditions the other frames
    with pytest.raises(BackendContractError):
        sample_bidirectional(model, text, steps=2, solver="heun", **kw)


def test_partition_is_round_robin_and_rejects_bad_identities():
    cases = [_case(i) for i in range(5)]
    assert [c.slot for c in partition_cases(cases, 0, 2)] == [0, 2, 4]
    assert [c.slot for c in partition_cases(cases, 1, 2)] == [1, 3]
    assert partition_cases(cases, 2, 3) == (cases[2],)
    with pytest.raises(BackendContractError):
        partition_cases(cases, 2, 2)
    with pytest.raises(BackendContractError):
        partition_cases(cases + [_case(0)], 0, 2)


class _Adapter:
    family = "toy"

    def generate(self, case, *, weights_id):
        return GeneratedSample({"x.bin": bytes([case.slot])}, (1,), "uint8", metrics={}, provenance={})


def test_merge_joins_partitions_in_slot_order_and_checks_them(tmp_path):
    cases = [_case(i) for i in range(5)]
    parts = []
    for d in range(2):
        part = tmp_path / f"part{d}"
        InferenceEngine(_Adapter()).run(partition_cases(cases, d, 2), weights_id="w", output_dir=part)
        parts.append(part)
    whole = tmp_path / "whole"
    InferenceEngine(_Adapter()).run(cases, weights_id="w", output_dir=whole)
    digest = merge_partitions(parts, tmp_path / "merged", family="toy", weights_id="w", expected_cases=5)
    seal = json.loads((tmp_path / "merged" / "COMPLETE.json").read_text())
    # a partitioned run publishes byte for byte what one process would have
    assert seal == json.loads((whole / "COMPLETE.json").read_text()) and seal["ordered_manifest_digest"] == digest
    assert (tmp_path / "merged" / "ordered-manifest.jsonl").read_bytes() == (whole / "ordered-manifest.jsonl").read_bytes()
    assert (tmp_path / "merged" / "slot-000003" / "x.bin").read_bytes() == b"\x03"
    with pytest.raises(BackendContractError):                                   # create-only
        merge_partitions(parts, tmp_path / "merged", family="toy", weights_id="w", expected_cases=5)
    again = []
    for d in range(2):
        part = tmp_path / f"again{d}"
        InferenceEngine(_Adapter()).run(partition_cases(cases, d, 2), weights_id="w", output_dir=part)
        again.append(part)
    with pytest.raises(BackendContractError):                                   # a slot is missing
        merge_partitions(again[:1], tmp_path / "m2", family="toy", weights_id="w", expected_cases=5)
    with pytest.raises(BackendContractError):                                   # other weights
        merge_partitions(again, tmp_path / "m3", family="toy", weights_id="other", expected_cases=5)
    with pytest.raises(BackendContractError):                                   # the same replica twice
        merge_partitions([again[1], again[1]], tmp_path / "m4", family="toy", weights_id="w", expected_cases=4)


def _infer_worker(rank, world, rdv, root, sp):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1")
    dist.init_process_group("gloo", init_method=f"file://{rdv}", rank=rank, world_size=world)
    from solarwm_b200.backends.wan22.inference import run_inference

    config = {"schema": "solarwm.run.v1", "action": "infer", "name": "dp-infer",
              "model": {"family": "wan22_ti2v_5b", "architecture": "tiny", "timestep_shift": 5.0, "nonzero_head_init": True},
              "data": {"source": "synthetic", "seed": 0},
              "inference": {"cases": 3, "steps": 2, "latent_frames": 2, "latent_height": 4, "latent_width": 4,
                            "first_frame": "seeded", "sequence_parallel_size": sp},
              "runtime": {"output_dir": root, "device": "cpu"}}
    out = run_inference(config, "wan22_ti2v_5b")
    assert out["cases"] == 3
    dist.destroy_process_group()


@pytest.mark.parametrize("sp", [1, 2])
def test_two_ranks_publish_what_one_rank_does(tmp_path, sp):
    """DP = 2 (each replica generates its share) and SP = 2 (both ranks evaluate every case, one writes): the public
    directory is the single-process one."""
    from solarwm_b200.backends.wan22.inference import run_inference

    mp.spawn(_infer_worker, args=(2, str(tmp_path / "rdv"), str(tmp_path / "two"), sp), nprocs=2, join=True)
    config = {"schema": "solarwm.run.v1", "action": "infer", "name": "dp-infer",
              "model": {"family": "wan22_ti2v_5b", "architecture": "tiny", "timestep_shift": 5.0, "nonzero_head_init": True},
              "data": {"source": "synthetic", "seed": 0},
              "inference": {"cases": 3, "steps": 2, "latent_frames": 2, "latent_height": 4, "latent_width": 4,
                            "first_frame": "seeded"},
              "runtime": {"output_dir": str(tmp_path / "one"), "device": "cpu"}}
    run_inference(config, "wan22_ti2v_5b")
    one, two = tmp_path / "one" / "generate", tmp_path / "two" / "generate"
    assert not (tmp_path / "two" / ".generate.parts").exists()
    a = [json.loads(l) for l in (one / "ordered-manifest.jsonl").read_text().splitlines()]
    b = [json.loads(l) for l in (two / "ordered-manifest.jsonl").read_text().splitlines()]
    assert [m["case"] for m in a] == [m["case"] for m in b] and len(b) == 3
    for slot in range(3):
        x = torch.load(one / f"slot-{slot:06d}" / "latents.pt")
        y = torch.load(two / f"slot-{slot:06d}" / "latents.pt")
        torch.testing.assert_close(x, y, rtol=1e-4, atol=1e-5)


def test_causal_routes_are_sampled_by_chunked_rollout_with_optional_cameras(tmp_path):
    from solarwm_b200.backends.wan22.inference import WanLatentAdapter

    model, cfg = _tiny()
    base = {"model": {"family": "wan22_ti2v_5b", "timestep_shift": 3.0, "causal": {"chunk_frames": 2, "window_chunks": 2}},
            "train": {"stage": "stage2", "causal_mode": "self_gradient_forcing", "denoising_steps": [1000.0, 500.0]},
            "inference": {"latent_frames": 5, "latent_height": 4, "latent_width": 4, "first_frame": "seeded"}}
    ad = WanLatentAdapter("wan22_ti2v_5b", model, base)
    assert ad.autoregressive
    out = ad.generate(_case(0), weights_id="w")
    assert out.shape == (1, 5, cfg.out_dim, 4, 4) and out.provenance["sampler"] == "few-step-rollout"
    assert out.provenance["mode"] == "autoregressive" and out.provenance["chunks"] == 2 and out.provenance["steps"] == 2
    again = ad.generate(_case(0), weights_id="w")
    assert out.artifacts["latents.pt"] == again.artifacts["latents.pt"]                  # seeded by the case
    assert ad.generate(_case(1), weights_id="w").artifacts["latents.pt"] != out.artifacts["latents.pt"]
    # the bidirectional route of the same weights is another sampler; inference.mode overrides the route
    bi = WanLatentAdapter("wan22_ti2v_5b", model, {**base, "inference": {**base["inference"], "mode": "bidirectional", "steps": 2}})
    assert not bi.autoregressive and bi.generate(_case(0), weights_id="w").provenance["sampler"] == "unipc-flow"
    with pytest.raises(BackendContractError):
        WanLatentAdapter("wan22_ti2v_5b", model, {**base, "inference": {"mode": "other"}}).autoregressive
    with pytest.raises(BackendContractError):                                            # 4 + anchor does not split into chunks of 2... 3 does not
        WanLatentAdapter("wan22_ti2v_5b", model, {**base, "inference": {**base["inference"], "latent_frames": 4}}).generate(_case(0), weights_id="w")
    # camera-length rollout: as many frames as the path has
    views = torch.eye(4).repeat(7, 1, 1)
    views[:, 2, 3] = -torch.arange(7) * 0.1
    torch.save({"viewmats": views}, tmp_path / "cams.pt")
    cam = WanLatentAdapter("wan22_ti2v_5b", model, {**base, "inference": {**base["inference"], "cameras": str(tmp_path / "cams.pt")}})
    got = cam.generate(_case(0), weights_id="w")
    assert got.shape[1] == 7 and got.provenance["camera_frames"] == 7


def test_bidirectional_sampling_follows_a_camera_path(tmp_path):
    from solarwm_b200.backends.wan22.inference import WanLatentAdapter

    model, cfg = _tiny()
    base = {"model": {"family": "wan22_ti2v_5b", "timestep_shift": 3.0}, "train": {"stage": "stage0p5", "causal_mode": "bidirectional"},
            "inference": {"latent_frames": 3, "latent_height": 4, "latent_width": 4, "steps": 2}}
    plain = WanLatentAdapter("wan22_ti2v_5b", model, base).generate(_case(0), weights_id="w")
    views = torch.eye(4).repeat(3, 1, 1)
    views[:, 0, 3] = -torch.arange(3) * 0.3
    torch.save({"viewmats": views}, tmp_path / "cams.pt")
    cam_cfg = {**base, "inference": {**base["inference"], "cameras": str(tmp_path / "cams.pt")}}
    moved = WanLatentAdapter("wan22_ti2v_5b", model, cam_cfg).generate(_case(0), weights_id="w")
    assert moved.provenance["camera_frames"] == 3 and moved.artifacts["latents.pt"] != plain.artifacts["latents.pt"]
    torch.save({"viewmats": views[:2]}, tmp_path / "short.pt")
    with pytest.raises(BackendContractError):
        WanLatentAdapter("wan22_ti2v_5b", model, {**base, "inference": {**base["inference"], "cameras": str(tmp_path / "short.pt")}}).generate(_case(0), weights_id="w")
