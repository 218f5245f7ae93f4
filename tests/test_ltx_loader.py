"""LTX released-layout loader: name rules, verify-before-copy, dropped families, unplaced / missing handling."""
import pytest
import torch

from solarwm_b200.backends.ltx25.checkpoint import PREFIX
from solarwm_b200.backends.ltx25.loader import destination, export_released, load_video_core, plan
from solarwm_b200.errors import BackendContractError
from solarwm_b200.models.ltx import LTXDiT, ltx_preset


def _model(seed):
    cfg = ltx_preset("tiny")
    cfg.gated_attention = True
    return LTXDiT(cfg, device="cpu", dtype=torch.float32, seed=seed)


def _write(path, tensors):
    from safetensors.torch import save_file

    save_file({k: v.contiguous() for k, v in tensors.items()}, str(path))


def test_name_rules():
    assert destination("transformer_blocks.3.attn1.to_out.0.weight") == "blocks.3.self_attn.o.weight"
    assert destination("transformer_blocks.0.attn2.k_norm.weight") == "blocks.0.cross_attn.norm_k.weight"
    assert destination("transformer_blocks.12.ff.net.0.proj.bias") == "blocks.12.ffn.0.bias"
    assert destination("transformer_blocks.1.scale_shift_table") == "blocks.1.modulation"
    assert destination("scale_shift_table") == "head.modulation" and destination("proj_out.weight") == "head.head.weight"
    assert destination("adaln_single.linear.bias") == "time_projection.1.bias"
    assert destination("transformer_blocks.1.prompt_scale_shift_table") is None
    assert destination("transformer_blocks.1.attn1.to_q.lora_A.weight") is None


def test_round_trip_through_the_released_layout(tmp_path):
    src, dst = _model(1), _model(2)
    with torch.no_grad():
        for p in src.parameters():
            p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(p.numel())) * 0.05)
    tensors = dict(export_released(src))
    assert tensors[PREFIX + "patchify_proj.weight"].dim() == 2 and tensors[PREFIX + "scale_shift_table"].dim() == 2
    # families of the audio-video release that the video-only runtime never reads
    tensors[PREFIX + "audio_patchify_proj.weight"] = torch.zeros(4, 4)
    tensors[PREFIX + "transformer_blocks.0.audio_attn1.to_q.weight"] = torch.zeros(4, 4)
    tensors[PREFIX + "transformer_blocks.0.video_to_audio_attn.to_q.weight"] = torch.zeros(4, 4)
    tensors[PREFIX + "video_embeddings_connector.learnable_registers"] = torch.zeros(4, 4)
    _write(tmp_path / "m.safetensors", tensors)
    report = load_video_core(dst, tmp_path / "m.safetensors")
    assert report.placed == len(dict(src.named_parameters())) and report.published_model
    assert report.parameters == sum(p.numel() for p in src.parameters())
    assert report.dropped == {"audio": 2, "av_cross": 1, "video_connector": 1}
    for (n, a), (_, b) in zip(src.named_parameters(), dst.named_parameters()):
        assert torch.equal(a, b), n
    x = torch.randn(1, 16, 2, 4, 4, generator=torch.Generator().manual_seed(0))
    ctx = torch.randn(1, 8, 64, generator=torch.Generator().manual_seed(1))
    t = torch.full((1, 2), 0.5)
    with torch.no_grad():
        assert torch.equal(src(x, t, ctx), dst(x, t, ctx))


def test_nothing_is_copied_when_anything_is_wrong(tmp_path):
    src = _model(1)
    good = dict(export_released(src))
    cases = {
        "shape": {**good, PREFIX + "transformer_blocks.1.ff.net.2.weight": torch.zeros(3, 3)},
        "dtype": {**good, PREFIX + "proj_out.bias": torch.zeros(16, dtype=torch.int32)},
        "unknown": {**good, PREFIX + "mystery.weight": torch.zeros(2)},
        "extra-block": {**good, PREFIX + "transformer_blocks.2.attn1.to_q.weight": torch.zeros(128, 128)},
        "unplaced": {**good, PREFIX + "transformer_blocks.0.prompt_scale_shift_table": torch.zeros(2, 128)},
        "missing": {k: v for k, v in good.items() if "caption_projection" not in k},
    }
    for name, tensors in cases.items():
        dst = _model(2)
        before = [p.detach().clone() for p in dst.parameters()]
        _write(tmp_path / f"{name}.safetensors", tensors)
        with pytest.raises(BackendContractError):
            load_video_core(dst, tmp_path / f"{name}.safetensors")
        assert all(torch.equal(a, b) for a, b in zip(before, dst.parameters())), name
    bad = dict(good)
    bad[PREFIX + "transformer_blocks.0.scale_shift_table"] = torch.full((6, 128), float("nan"))
    _write(tmp_path / "nan.safetensors", bad)
    with pytest.raises(BackendContractError, match="non-finite"):
        load_video_core(_model(2), tmp_path / "nan.safetensors")

    # a release with prompt tables and no caption projection loads only when both gaps are named, and says what it is
    dst = _model(2)
    kept = [p.detach().clone() for n, p in dst.named_parameters() if n.startswith("text_embedding.")]
    mapping, report = plan(dst, tmp_path / "unplaced.safetensors", allow_unplaced=["transformer_blocks.*.prompt_scale_shift_table"])
    assert report.unplaced == ["transformer_blocks.0.prompt_scale_shift_table"] and not report.published_model
    merged = {k: v for k, v in cases["unplaced"].items() if "caption_projection" not in k}
    _write(tmp_path / "both.safetensors", merged)
    report = load_video_core(dst, tmp_path / "both.safetensors", allow_unplaced=["*prompt_scale_shift_table"], allow_missing=["text_embedding.*"])
    assert len(report.missing) == 4 and not report.published_model
    assert all(torch.equal(a, p) for a, (n, p) in zip(kept, [(n, p) for n, p in dst.named_parameters() if n.startswith("text_embedding.")]))
    assert torch.equal(dict(dst.named_parameters())["blocks.1.ffn.2.weight"], dict(src.named_parameters())["blocks.1.ffn.2.weight"])


def test_adapter_training_and_inference_start_from_a_released_base(tmp_path):
    """``model.base_weights``: the released-layout file replaces the seeded base before the adapters are attached; the
    adapter run trains on it and a plain inference run names the file as its weights."""
    from solarwm_b200.backends.ltx25.backend import _arch
    from solarwm_b200.registry import load_backend
    from solarwm_b200.backends.ltx25.runtime import LTXTrainingRuntime

    base = {"schema": "solarwm.run.v1", "action": "train", "name": "ltx-base",
            "model": {"family": "ltx25_video", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "linear"},
            "data": {"source": "synthetic", "seed": 2, "pixel_frames": 153, "latent_frames": 2, "latent_height": 4, "latent_width": 4},
            "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 1,
                      "optimizer": {"lr": 1e-3}}, "runtime": {"output_dir": str(tmp_path / "run"), "device": "cpu"}}
    src = LTXDiT(_arch(base), device="cpu", dtype=torch.float32, seed=9)
    with torch.no_grad():
        for p in src.parameters():
            p.copy_(torch.randn(p.shape, generator=torch.Generator().manual_seed(p.numel() + 1)) * 0.05)
    _write(tmp_path / "base.safetensors", dict(export_released(src)))
    cfg = {**base, "model": {**base["model"], "base_weights": {"path": str(tmp_path / "base.safetensors")}}}
    rt = LTXTrainingRuntime(cfg)
    try:
        assert rt.core.base_report.published_model and rt.core.base_report.placed == len(dict(src.named_parameters()))
        want = dict(src.named_parameters())["blocks.1.self_attn.q.weight"]
        got = [p for n, p in rt.core.model.named_parameters() if n.startswith("blocks.1.self_attn.q.") and p.shape == want.shape]
        assert any(torch.equal(p, want) for p in got)
        loss = rt.train_microbatch(0, 1).losses["loss"]
        assert loss == loss
    finally:
        rt.close()
    plain = LTXTrainingRuntime(base)
    try:
        assert plain.core.base_report is None
    finally:
        plain.close()
    with pytest.raises(BackendContractError):
        LTXTrainingRuntime({**cfg, "model": {**cfg["model"], "base_weights": str(tmp_path / "absent.safetensors")}})
    infer = {**cfg, "action": "infer", "inference": {"cases": 1, "steps": 2}, "runtime": {"output_dir": str(tmp_path / "gen"), "device": "cpu"}}
    infer["model"] = {k: v for k, v in infer["model"].items() if k != "adapter"}
    out = load_backend("ltx25_video").infer(infer)
    assert out["weights_id"].startswith("released:") and out["cases"] == 1
