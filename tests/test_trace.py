"""Phase tracing: spans are free when off, feed an installed timer, and the trainer reports its phases."""
import torch

from solarwm_b200.utils import trace


def test_span_is_a_shared_null_context_when_nothing_listens():
    assert trace.span("a") is trace.span("b")
    with trace.span("a"):
        pass


def test_phase_timer_collects_spans_and_nested_phases():
    timer = trace.PhaseTimer("cpu")
    with timer.installed():
        for _ in range(3):
            with trace.span("outer"):
                with trace.span("inner"):
                    torch.randn(64, 64) @ torch.randn(64, 64)
    assert trace.span("x") is trace.span("y")                  # uninstalled again
    s = timer.summary()
    assert s["outer"]["count"] == 3 and s["inner"]["count"] == 3
    assert s["outer"]["total_ms"] >= s["inner"]["total_ms"] > 0


def test_trainer_step_reports_forward_backward_optimizer_and_blocks():
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer
    from solarwm_b200.models.wan import WanConfig

    cfg = WanConfig(model_type="ti2v", in_dim=4, out_dim=4, dim=64, ffn_dim=128, num_heads=2, num_layers=2, text_dim=32,
                    text_len=8, freq_dim=32)
    tr = WanStage0p5Trainer(cfg, "cpu", Stage0p5Options(seed=1), dtype=torch.float32)
    batch = {"latents": torch.randn(1, 3, 4, 4, 4), "text": torch.randn(1, 8, 32)}
    timer = trace.PhaseTimer("cpu")
    with timer.installed():
        tr.train_step(batch)
        tr.train_step(batch)
    s = timer.summary()
    assert {"forward", "backward", "optimizer", "block.00", "block.01"} <= set(s)
    assert s["forward"]["count"] == 2 and s["block.01"]["count"] == 2
    previous = trace.enable_nvtx(True)                         # no CUDA here: still a no-op, never an error
    try:
        with trace.span("nvtx-on-cpu"):
            pass
    finally:
        trace.enable_nvtx(previous)


def test_step_events_carry_the_phase_split_when_asked(tmp_path, monkeypatch):
    import json
    from pathlib import Path

    from solarwm_b200.cli import main

    config = str(Path(__file__).resolve().parent.parent / "configs" / "wan22_ti2v_5b" / "tiny_stage0p5_cpu.yaml")
    monkeypatch.setenv("SOLAR_OUTPUT_DIR", str(tmp_path))
    monkeypatch.setenv("SOLAR_PHASE_TIMES", "1")
    assert main(["train", "--config", config, "--set", "runtime.device=cpu", "--set", "train.max_steps=2",
                 "--set", "runtime.save_every=0"]) == 0
    events = [json.loads(l) for l in (tmp_path / "events" / "rank-00000.jsonl").read_text().splitlines()]
    steps = [e for e in events if e["event"] == "optimizer_step"]
    assert len(steps) == 2 and {"forward", "backward", "optimizer"} <= set(steps[0]["phase_ms"])
