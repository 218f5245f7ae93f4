"""Host-side pieces of the benchmark script: argument defaults and the resident-block plan."""
import importlib.util
import sys
from pathlib import Path
from types import SimpleNamespace


def _bench():
    path = Path(__file__).resolve().parents[1] / "bench.py"
    spec = importlib.util.spec_from_file_location("solar_bench_script", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_defaults_run_one_gpu_for_a_few_steps(monkeypatch):
    bench = _bench()
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse_args()
    assert args.gpus == 1 and args.steps >= 1 and args.warmup >= 3 and args.impl == "ours" and args.mode == "train"
    monkeypatch.setattr(sys, "argv", ["bench.py", "--gpus", "8", "--steps", "5", "--warmup", "3", "--impl", "reference"])
    args = bench.parse_args()
    assert (args.gpus, args.steps, args.warmup, args.impl) == (8, 5, 3, "reference")


def test_resident_block_plan_on_the_5b_shape():
    bench = _bench()
    cfg = SimpleNamespace(dim=3072, ffn_dim=14336, num_layers=30)
    total = 183359 * 2 ** 20
    plan = lambda world, **kw: bench.resident_block_plan(cfg, 27280, world, total, zero_on=world > 1,  # noqa: E731
                                                         checkpointing="selective", **kw)
    assert plan(1) == (30, True)                       # one GPU: every block resident only in lean form
    assert plan(1, lean_mode="off") == (19, False)     # plain blocks: 19 fit, 11 are recomputed
    assert plan(2) == (30, False)                      # sharded optimizer: everything fits as it is
    assert plan(1, keep_blocks=7) == (7, False) and plan(1, keep_blocks=7, lean_mode="on") == (7, True)
    assert bench.resident_block_plan(cfg, 27280, 4, total, zero_on=True, checkpointing="none") == (0, False)
    small = bench.resident_block_plan(cfg, 27280, 1, 80 * 2 ** 30, zero_on=False, checkpointing="selective")
    assert small[0] == 0 and small[1] is True          # no room beyond weights and optimizer state: recompute all


def test_model_flops_and_utilization_of_the_5b_shape(tmp_path):
    from solarwm_b200.utils.roofline import block_forward_flops, measured_peaks, step_utilization, training_step_flops

    cfg = SimpleNamespace(dim=3072, ffn_dim=14336, num_layers=30, text_len=512)
    per_block = block_forward_flops(27280, 512, 3072, 14336)
    assert abs(per_block / 1e12 - 17.2) < 0.4                       # 2.06 + 9.14 + ~1.2 + 4.81 TFLOP
    total = training_step_flops(cfg, 27280)
    assert abs(total / 1e15 - 1.55) < 0.05
    (tmp_path / "MEASURED_PEAKS.json").write_text('{"hbm_gbs": 6540.5, "bf16_tflops": 1641.7, "bf16_tflops_sustained": 1390.9}')
    u = step_utilization(cfg, 27280, 1894.0, 1, root=tmp_path)
    assert u["peak_source"] == "measured" and 0.55 < u["fraction_of_sustained_peak"] < 0.62
    assert abs(step_utilization(cfg, 27280, 319.0, 8, root=tmp_path)["fraction_of_sustained_peak"] - u["fraction_of_sustained_peak"] * 1894 / 319 / 8) < 2e-3
    assert measured_peaks(tmp_path / "nowhere")["source"] == "fallback"


def test_reference_arm_prints_an_unavailable_line_without_a_gpu():
    import json
    import subprocess

    import torch

    if torch.cuda.is_available():
        import pytest

        pytest.skip("the reference arm would really run here")
    root = Path(__file__).resolve().parents[1]
    out = subprocess.run([sys.executable, str(root / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3"],
                         capture_output=True, text=True, timeout=300, cwd=str(root))
    assert out.returncode == 0
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line
