"""H3 generation through the shared inference engine: stage-dependent samplers, camera identity, packaging."""
import pytest
import torch

from solarwm_b200.backends.minimax_h3.inference import H3InferenceAdapter, build_cases, camera_fingerprint, decoded_pixel_frames
from solarwm_b200.engine.inference_engine import InferenceEngine
from solarwm_b200.errors import BackendContractError
from solarwm_b200.models.h3 import H3DiT, h3_preset
from solarwm_b200.serve.h3_stream import H3StreamConfig


def _conditions(cfg, n=2, frames=4):
    out = []
    for i in range(n):
        g = torch.Generator().manual_seed(i)
        views = torch.eye(4).repeat(frames + 1, 1, 1)
        views[:, 0, 3] = -torch.arange(frames + 1) * 0.05 * (i + 1)
        out.append({"sample_id": f"clip-{i}", "prompt": f"p{i}", "prompt_embeds": torch.randn(6, cfg.text_dim, generator=g),
                    "anchor_latents": torch.randn(24, 1, 4, 4, generator=g), "camera_w2c": views})
    return out


def test_fingerprints_and_frame_rule():
    v = torch.eye(4).repeat(3, 1, 1)
    assert camera_fingerprint(v) == camera_fingerprint(v.clone()) != camera_fingerprint(v + 1e-3)
    assert camera_fingerprint(v, torch.eye(3).repeat(3, 1, 1)) != camera_fingerprint(v)
    assert [decoded_pixel_frames(n) for n in (2, 7, 47)] == [5, 22, 158]
    for bad in (1, 6, 8):
        with pytest.raises(BackendContractError):
            decoded_pixel_frames(bad)


def test_stage_decides_the_sampler_and_the_engine_publishes_the_cases(tmp_path):
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    conds = _conditions(cfg)
    cases = build_cases(conds, noise_seed=7)
    assert [c.slot for c in cases] == [0, 1] and cases[0].camera_fingerprint != cases[1].camera_fingerprint
    assert build_cases(conds, noise_seed=7)[0].noise_seed == cases[0].noise_seed != build_cases(conds, noise_seed=8)[0].noise_seed
    bi = H3InferenceAdapter(model, conds, stage="stage0p5", steps=2)
    a = bi.generate(cases[0], weights_id="w")
    assert a.shape == (24, 4, 4, 4) and a.provenance["sampler"] == "bidirectional-euler" and a.metrics["latent_abs_max"] > 0
    assert a.artifacts["latents.pt"] == bi.generate(cases[0], weights_id="w").artifacts["latents.pt"]
    scfg = H3StreamConfig(grid_hw=(2, 2), chunk_latents=2, window_chunks=2, denoise_steps=1, use_cuda_graph=False)
    causal = H3InferenceAdapter(model, conds, stage="stage2", stream_cfg=scfg)
    b = causal.generate(cases[0], weights_id="w")
    assert b.shape == (24, 4, 4, 4) and b.provenance["sampler"] == "few-step-rollout" and b.artifacts["latents.pt"] != a.artifacts["latents.pt"]
    summary = InferenceEngine(causal).run(cases, weights_id="w", output_dir=tmp_path / "out")
    assert summary.cases == 2 and sorted(p.name for p in (tmp_path / "out").glob("slot-*")) == ["slot-000000", "slot-000001"]
    # a case made for other cameras is refused; block-causal weights need a stream configuration; odd lengths are refused
    moved = [dict(conds[0], camera_w2c=conds[0]["camera_w2c"] + 0.01), conds[1]]
    with pytest.raises(BackendContractError):
        H3InferenceAdapter(model, moved, stage="stage0p5", steps=2).generate(cases[0], weights_id="w")
    with pytest.raises(BackendContractError):
        H3InferenceAdapter(model, conds, stage="stage1")
    with pytest.raises(BackendContractError):
        H3InferenceAdapter(model, conds, stage="stage3", stream_cfg=scfg)
    odd = _conditions(cfg, n=1, frames=3)
    with pytest.raises(BackendContractError):
        H3InferenceAdapter(model, odd, stage="stage1", stream_cfg=scfg).generate(build_cases(odd)[0], weights_id="w")


def test_decoded_frames_travel_with_the_sample():
    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    conds = _conditions(cfg, n=1)
    vit = ViTVideoDecoder(ViTDecoderConfig(latent_channels=24, dim=64, depth=1, heads=2, dim_head=32, ffn_dim=128, registers=2, patch=2),
                          device="cpu", dtype=torch.float32)
    ad = H3InferenceAdapter(model, conds, stage="stage0p5", steps=2, decoder_factory=lambda: StreamingViTDecoder(vit, (4, 4)))
    out = ad.generate(build_cases(conds)[0], weights_id="w")
    assert "frames.pt" in out.artifacts and out.metrics["decoded_frames"] > 0


def test_backend_publishes_cases_for_either_stage(tmp_path):
    from solarwm_b200.registry import load_backend

    be = load_backend("minimax_h3")
    base = {"schema": "solarwm.run.v1", "action": "infer", "model": {"family": "minimax_h3", "architecture": "tiny", "camera_translation_transform": "logd4"},
            "inference": {"cases": 2, "grid_hw": [2, 2], "chunk_latents": 2, "latent_frames": 4, "window_chunks": 2, "denoise_steps": 1, "steps": 2}}
    a = be.infer({**base, "train": {"stage": "stage0p5"}, "runtime": {"device": "cpu", "output_dir": str(tmp_path / "bi")}})
    b = be.infer({**base, "train": {"stage": "stage2"}, "runtime": {"device": "cpu", "output_dir": str(tmp_path / "causal")}})
    assert a["cases"] == b["cases"] == 2 and a["ordered_manifest_digest"] != b["ordered_manifest_digest"]
    assert len(list((tmp_path / "bi" / "generate").glob("slot-*"))) == 2
