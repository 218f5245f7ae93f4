"""The config-driven training runtimes on one GPU: adapters move, losses are finite, the native kernels are the ones
that ran, checkpoints verify."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _moved(optimizer, before):
    return float((optimizer.master - before).abs().max()) > 0


def test_ltx_adapter_runtime_on_the_device(tmp_path):
    from solarwm_b200 import ops
    from solarwm_b200.backends.ltx25.runtime import run_training
    from solarwm_b200.checkpoint.store import verify_checkpoint
    from tests.test_ltx_runtime import _config

    before = ops.total_launches()
    out = run_training(_config(tmp_path / "ltx", runtime={"device": "cuda"}, train={"max_steps": 2, "grad_accum": 1}))
    assert out["final_step"] == 2 and out["last_loss"] == out["last_loss"] and ops.total_launches() > before
    assert verify_checkpoint(out["checkpoint"]).step == 2
    ops.check_status()


def test_h3_sgf_runtime_on_the_device(tmp_path):
    from solarwm_b200 import ops
    from solarwm_b200.backends.minimax_h3.stage2_runtime import H3SGFRuntime
    from tests.test_h3_sgf_runtime import _config, _kick, _model_config

    cfg = _config(tmp_path / "sgf", runtime={"device": "cuda"})
    rt = H3SGFRuntime(cfg, model_config=_model_config()(cfg))
    try:
        _kick(rt)
        s0, c0 = rt.trainer.opt_s.master.clone(), rt.trainer.opt_c.master.clone()
        before = ops.total_launches()
        stats = [rt.train_outer_step() for _ in range(3)]
        assert all(st["loss_critic"] == st["loss_critic"] for st in stats) and stats[2]["student_updated"] == 1.0
        assert _moved(rt.trainer.opt_s, s0) and _moved(rt.trainer.opt_c, c0) and ops.total_launches() > before
        rt.save_checkpoint(3)
        ops.check_status()
    finally:
        rt.close()


def test_renderer_runtimes_on_the_device(tmp_path):
    from solarwm_b200 import ops
    from solarwm_b200.renderer.runtime import run_control_training
    from tests.test_renderer_runtime import _config, _corpus

    _corpus(tmp_path / "corpus", n=4)
    before = ops.total_launches()
    a = run_control_training(_config(tmp_path / "corpus", tmp_path / "control", runtime={"device": "cuda"},
                                     train={"max_steps": 2, "gradient_accumulation_steps": 1}))
    b = run_control_training(_config(tmp_path / "corpus", tmp_path / "causal", runtime={"device": "cuda"},
                                     train={"max_steps": 1, "gradient_accumulation_steps": 1, "causal_omni": {"chunk": 2, "window": 2}}))
    assert a["final_step"] == 2 and b["final_step"] == 1 and a["last_loss"] == a["last_loss"] and b["last_loss"] == b["last_loss"]
    assert ops.total_launches() > before
    ops.check_status()


def test_online_encoding_on_the_device():
    from solarwm_b200.backends.wan22.runtime import online_batches
    from solarwm_b200.models.wan import wan_preset

    config = {"model": {"family": "wan22_ti2v_5b"}, "train": {"micro_batch_size": 1},
              "data": {"source": "synthetic", "encoding": "online", "num_samples": 2, "seed": 1, "pixel_frames": 9, "pixel_height": 32,
                       "pixel_width": 32,
                       "online_codecs": {"t5": {"vocab": 512, "dim": 256, "dim_attn": 64, "dim_ffn": 128, "num_heads": 2, "num_layers": 1, "text_len": 32},
                                         "vae": {"z_dim": 16, "base": 8, "temporal_ups": [True, True, False]}}}}
    batch = next(online_batches(config, wan_preset("tiny"), torch.device("cuda")))
    assert batch["latents"].shape == (1, 3, 16, 4, 4) and batch["latents"].dtype == torch.bfloat16 and bool(torch.isfinite(batch["latents"].float()).all())


def test_adapter_ranks_that_are_not_multiples_of_eight_match_the_fp32_reference():
    from solarwm_b200.ops import functional as F_

    g = torch.Generator().manual_seed(0)
    x = torch.randn(96, 128, generator=g)
    w, b = torch.randn(256, 128, generator=g) / 11, torch.randn(256, generator=g) / 7
    a, bb = torch.randn(4, 128, generator=g) / 11, torch.randn(256, 4, generator=g) / 3
    dy = torch.randn(96, 256, generator=g)
    ref_in = [t.clone().requires_grad_(True) for t in (x, a, bb)]
    ref = ref_in[0] @ w.t() + b + 0.5 * ((ref_in[0] @ ref_in[1].t()) @ ref_in[2].t())
    ref.backward(dy)
    dev = [t.cuda().bfloat16().requires_grad_(True) for t in (x, a, bb)]
    out = F_.lora_linear(dev[0], w.cuda().bfloat16(), b.cuda().bfloat16(), dev[1], dev[2], 0.5)
    out.backward(dy.cuda().bfloat16())
    assert dev[1].grad.shape == (4, 128) and dev[2].grad.shape == (256, 4)
    for got, want in ((out, ref), (dev[0].grad, ref_in[0].grad), (dev[1].grad, ref_in[1].grad), (dev[2].grad, ref_in[2].grad)):
        assert float((got.detach().float().cpu() - want.detach()).abs().max()) < 3e-2 * float(want.detach().abs().max())
