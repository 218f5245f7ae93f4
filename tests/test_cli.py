import json
import os
from pathlib import Path

import pytest

from solarwm_b200.cli import main

CONFIG = str(Path(__file__).resolve().parent.parent / "configs" / "wan22_ti2v_5b" / "tiny_stage0p5_cpu.yaml")


def _events(root):
    return [json.loads(l) for l in (Path(root) / "events" / "rank-00000.jsonl").read_text().splitlines()]


def test_train_resume_is_exact_and_infer_publishes(tmp_path, monkeypatch):
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "a"))
    assert main(["train", "--config", CONFIG, "--set", "runtime.device=cpu"]) == 0
    a = tmp_path / "a"
    for name in ("resolved-config.json", "launch-manifest.json", "run-result.json"):
        assert (a / name).is_file()
    assert json.loads((a / "run-result.json").read_text())["schema"] == "solarwm.run-result.v1"
    assert json.loads((a / "launch-manifest.json").read_text())["schema"] == "solarwm.launch.v2"
    assert (a / "checkpoint_model_000002" / "model.pt").is_file() and (a / "checkpoint_model_000004" / "COMPLETE.json").is_file()
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "b"))
    assert main(["train", "--config", CONFIG, "--set", "runtime.device=cpu", "--set", "checkpoint.mode=full_resume",
                 "--set", f"checkpoint.resume_from={a / 'checkpoint_model_000002'}", "--set", "runtime.save_every=0"]) == 0
    first = {e["step"]: (e["losses"], e["gradient_norm"]) for e in _events(a) if e["event"] == "optimizer_step"}
    second = {e["step"]: (e["losses"], e["gradient_norm"]) for e in _events(tmp_path / "b") if e["event"] == "optimizer_step"}
    assert sorted(second) == [3, 4] and all(second[s] == first[s] for s in second)
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "c"))
    assert main(["infer", "--config", CONFIG, "--set", "action=infer", "--set", "runtime.device=cpu",
                 "--set", f"checkpoint.resume_from={a / 'checkpoint_model_000004'}", "--set", "inference.cases=2",
                 "--set", "inference.steps=2"]) == 0
    out = tmp_path / "c" / "generate"
    assert (out / "COMPLETE.json").is_file() and (out / "slot-000001" / "latents.pt").is_file()


def test_cli_errors_exit_2_and_helpers(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    assert main(["infer", "--config", CONFIG]) == 2                       # action mismatch
    assert main(["train", "--config", CONFIG, "--set", "train.stage=stage9"]) == 2
    assert main(["train", "--config", CONFIG, "--set", "distributed.sequence_parallel_size=3"]) == 2
    assert main(["train", "--config", str(tmp_path / "missing.yaml")]) == 2
    assert main(["config", "routes"]) == 0
    assert "minimax_h3:stage2:self_gradient_forcing:flow_matching" in capsys.readouterr().out
    assert main(["config", "resolve", "--config", CONFIG, "--output", str(tmp_path / "r.json")]) == 0
    assert json.loads((tmp_path / "r.json").read_text())["schema"] == "solarwm.run.v1"
    assert main(["environment", "probe"]) == 0
    assert "native_library" in capsys.readouterr().out


@pytest.mark.parametrize("rel,action", [
    ("wan22_ti2v_5b/tiny_stage1_anyflow_cpu.yaml", "train"),
    ("wan22_ti2v_5b/tiny_stage2_sgf_cpu.yaml", "train"),
    ("wan22_ti2v_5b/tiny_preencode_cpu.yaml", "preencode"),
    ("wan22_ti2v_5b/tiny_stage0p5_online_cpu.yaml", "train"),
    ("ltx25_video/tiny_stage0p5_cpu.yaml", "train"),
    ("ltx25_video/tiny_lora_cameras_cpu.yaml", "train"),
    ("minimax_h3/tiny_stage2_sgf_cpu.yaml", "train"),
    ("minimax_h3/tiny_infer_cases_cpu.yaml", "infer"),
    ("minimax_h3/tiny_stage0p5_cpu.yaml", "train"),
    ("minimax_h3/tiny_infer_cpu.yaml", "infer"),
])
def test_example_configs_run_on_cpu(rel, action, tmp_path, monkeypatch):
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "out"))
    config = str(Path(__file__).resolve().parent.parent / "configs" / rel)
    assert main([action, "--config", config, "--set", "runtime.device=cpu"]) == 0
    result = json.loads((tmp_path / "out" / "run-result.json").read_text())
    assert result["schema"] == "solarwm.run-result.v1"


def test_benchmark_shape_config_resolves_and_validates(tmp_path, monkeypatch, capsys):
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    config = str(Path(__file__).resolve().parent.parent / "configs" / "wan22_ti2v_5b" / "stage0p5_sp8.yaml")
    assert main(["config", "resolve", "--config", config]) == 0
    assert '"sequence_parallel_size":8' in capsys.readouterr().out


def test_train_from_a_preencoded_corpus_and_resume_exactly(tmp_path, monkeypatch):
    """preencode (synthetic clips, codecs sized to the tiny DiT) -> train from the corpus index -> resume mid-run:
    the resumed steps read the same samples and reproduce the same losses."""
    cfg_dir = Path(__file__).resolve().parent.parent / "configs" / "wan22_ti2v_5b"
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "pre"))
    assert main(["preencode", "--config", str(cfg_dir / "tiny_preencode_cpu.yaml"), "--set", "preencode.num_samples=5",
                 "--set", "data.pixel_frames=81", "--set", "preencode.codecs={z_dim: 16, vae_base: 8, t5: {vocab: 512, dim: 256, dim_attn: 32, dim_ffn: 64, "
                          "num_heads: 2, num_layers: 1, text_len: 32}}"]) == 0
    index = tmp_path / "pre" / "encoded" / "index.jsonl"
    assert index.is_file()
    monkeypatch.setenv("SOLAR_CORPUS_INDEX", str(index))
    common = ["--config", str(cfg_dir / "tiny_train_from_corpus_cpu.yaml"), "--set", "runtime.device=cpu"]
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "a"))
    assert main(["train", *common]) == 0
    ev_a = {e["step"]: e for e in _events(tmp_path / "a") if e["event"] == "optimizer_step"}
    ids = [tuple(m["identity"]["sample_ids"]) for s in sorted(ev_a) for m in ev_a[s]["microbatches"]]
    assert len(ids) == 4 and all(i[0].startswith("synthetic-") for i in ids) and len(set(ids)) >= 3     # real corpus samples
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "b"))
    assert main(["train", *common, "--set", "checkpoint.mode=full_resume", "--set",
                 f"checkpoint.resume_from={tmp_path / 'a' / 'checkpoint_model_000002'}", "--set", "runtime.save_every=0"]) == 0
    ev_b = {e["step"]: e for e in _events(tmp_path / "b") if e["event"] == "optimizer_step"}
    assert sorted(ev_b) == [3, 4]
    for s in (3, 4):
        assert ev_b[s]["losses"] == ev_a[s]["losses"]
        assert ev_b[s]["microbatches"][0]["identity"]["sample_ids"] == ev_a[s]["microbatches"][0]["identity"]["sample_ids"]


def test_infer_with_prompts_and_a_text_encoder(tmp_path, monkeypatch):
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    enc = "{vocab: 512, dim: 256, dim_attn: 32, dim_ffn: 64, num_heads: 2, num_layers: 1, text_len: 32}"
    assert main(["infer", "--config", CONFIG, "--set", "action=infer", "--set", "runtime.device=cpu", "--set", "inference.steps=2",
                 "--set", "inference.prompts=[a harbour at dusk, a street in the rain]", "--set", f"inference.text_encoder={enc}"]) == 0
    out = tmp_path / "generate"
    assert (out / "slot-000000" / "latents.pt").is_file() and (out / "slot-000001" / "latents.pt").is_file()
    manifest = json.loads((out / "slot-000001" / "manifest.json").read_text())
    assert "rain" in json.dumps(manifest)
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path / "bad"))
    wrong = "{vocab: 512, dim: 64, dim_attn: 32, dim_ffn: 64, num_heads: 2, num_layers: 1, text_len: 32}"
    assert main(["infer", "--config", CONFIG, "--set", "action=infer", "--set", "runtime.device=cpu", "--set", "inference.steps=1",
                 "--set", "inference.prompts=[x]", "--set", f"inference.text_encoder={wrong}"]) == 2


def test_infer_decodes_to_a_video_when_a_vae_is_configured(tmp_path, monkeypatch):
    pytest.importorskip("cv2")
    from solarwm_b200.data import raw_video

    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    assert main(["infer", "--config", CONFIG, "--set", "action=infer", "--set", "runtime.device=cpu", "--set", "inference.steps=1",
                 "--set", "inference.latent_frames=3", "--set", "inference.latent_height=4", "--set", "inference.latent_width=6",
                 "--set", "inference.vae={z_dim: 16, base: 8, temporal_ups: [true, false], fps: 8}"]) == 0
    blob = (tmp_path / "generate" / "slot-000000" / "video.mp4").read_bytes()
    info = raw_video.probe(blob)
    assert info["frames"] == 5 and (info["height"], info["width"]) == (16, 24)        # 1 + 2 * 2 frames, 4 x spatial


def test_validation_publishes_a_comparison_view(tmp_path, monkeypatch):
    """Training with inline validation, a decoder and a comparison source: every validation pass publishes its slots
    (latents, video, the generated clip beside its source) and the flat comparison view that links into them."""
    pytest.importorskip("cv2")
    from solarwm_b200.data import raw_video

    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    assert main(["train", "--config", CONFIG, "--set", "runtime.device=cpu", "--set", "train.max_steps=2", "--set", "runtime.save_every=0",
                 "--set", "runtime.validate_every=2", "--set", "validation={sample_count: 2, pass_name: live}",
                 "--set", "inference={steps: 1, latent_frames: 3, latent_height: 4, latent_width: 6, compare_source: seeded, "
                          "vae: {z_dim: 16, base: 8, temporal_ups: [true, false], fps: 8}}"]) == 0
    views = sorted(p for p in (tmp_path / "validation").rglob("COMPLETE.json") if p.parent.name.endswith("_compare"))
    assert len(views) == 1
    view = views[0].parent
    videos = sorted((view / "compare").iterdir())
    assert len(videos) == 2 and videos[0].name.startswith("rank000_round00_dp000_case-0000_start000000")
    info = raw_video.probe(videos[1].read_bytes())
    assert info["frames"] == 5 and info["width"] == 2 * 24 + 8                      # generated | band | source
    assert json.loads((view / "manifests" / "rank_001.json").read_text())["step"] == 2
