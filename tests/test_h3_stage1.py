"""H3 Stage1: W6 segment attention equals the dense-mask oracle; trainers step (CPU)."""
import torch

from solarwm_b200.backends.minimax_h3.stage1 import H3Stage1Trainer, w6_attention, w6_mask
from solarwm_b200.data.synthetic import h3_sample
from solarwm_b200.models.h3 import h3_preset
from solarwm_b200.ops import reference as R


def test_w6_attention_matches_dense_mask():
    torch.manual_seed(0)
    n_cond, chunk_rows, n_chunks, W = 5, 4, 4, 1
    S = n_cond + 2 * n_chunks * chunk_rows
    q, k, v = (torch.randn(1, S, 2, 16) for _ in range(3))
    got = w6_attention(q, k, v, n_cond=n_cond, chunk_rows=chunk_rows, n_chunks=n_chunks, window_chunks=W)
    mask = w6_mask(n_cond, chunk_rows, n_chunks, W)
    want = R.attention(q, k, v, mask=mask.view(1, 1, S, S))
    assert torch.allclose(got, want, atol=1e-5)
    dense = mask.float().mean()
    assert 0.2 < dense < 0.6


def test_h3_stage1_trainers_step():
    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    for objective in ("tf_fm", "anyflow"):
        tr = H3Stage1Trainer(cfg, "cpu", objective=objective, chunk_latents=2, window_chunks=1, lr=1e-3,
                             diffusion_ratio=0.34, consistency_ratio=0.33)
        s = h3_sample(latent_frames=4, height=4, width=4, prompt_len=6, text_dim=cfg.text_dim, seed=0)
        s["camera_w2c"] = torch.eye(4).repeat(5, 1, 1)
        before = [p.detach().clone() for p in tr.model.trainable_parameters()]
        loss = tr.train_step(s)
        assert torch.isfinite(loss)
        assert any(not torch.equal(a, b) for a, b in zip(before, tr.model.trainable_parameters()))


def test_h3_stage2_outer_steps_share_one_base():
    from solarwm_b200.backends.minimax_h3.stage2 import H3Stage2Trainer
    from solarwm_b200.models.h3 import LoRALinear

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    tr = H3Stage2Trainer(cfg, "cpu", chunk_latents=2, window_chunks=1, denoise_steps=2, grid_hw=(2, 2),
                         critic_updates_per_student=2, lr_student=1e-3, lr_critic=1e-3)
    s_mods = [m for m in tr.student.modules() if isinstance(m, LoRALinear)]
    c_mods = [m for m in tr.critic.modules() if isinstance(m, LoRALinear)]
    assert all(a.weight is b.weight for a, b in zip(s_mods, c_mods))            # one frozen base
    assert all(a.lora_A is not b.lora_A for a, b in zip(s_mods, c_mods))        # private adapters
    s = h3_sample(latent_frames=4, height=4, width=4, prompt_len=6, text_dim=cfg.text_dim, seed=0)
    s["camera_w2c"] = torch.eye(4).repeat(5, 1, 1)
    r0 = tr.train_outer_step(s, n_chunks=2)
    assert "critic" in r0 and "student" not in r0
    tr.train_outer_step(s, n_chunks=2)
    before = s_mods[0].lora_B.detach().clone()
    r2 = tr.train_outer_step(s, n_chunks=2)
    assert "student" in r2 and r2["student"] == r2["student"]
    assert not torch.equal(before, s_mods[0].lora_B)


def test_h3_backend_routes_stage1_and_stage2(tmp_path):
    from solarwm_b200.backends.minimax_h3.backend import MiniMaxH3Backend
    from solarwm_b200.checkpoint.store import verify_checkpoint

    base = {"schema": "solarwm.run.v1", "action": "train",
            "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4},
                      "camera_translation_transform": "logd4", "causal": {"chunk_latents": 2, "window_chunks": 1}},
            "data": {"seed": 0, "latent_frames": 4, "latent_height": 4, "latent_width": 4, "prompt_len": 6, "pixel_frames": 158},
            "runtime": {"device": "cpu"}}
    be = MiniMaxH3Backend("minimax_h3")
    for stage, mode, objective, variant in (("stage1", "teacher_forcing", "anyflow_forward_map", "v1_5"),
                                            ("stage2", "self_gradient_forcing", "flow_matching", "")):
        cfg = dict(base, runtime={"device": "cpu", "output_dir": str(tmp_path / stage)},
                   train={"stage": stage, "causal_mode": mode, "objective": objective, "objective_variant": variant,
                          "max_steps": 1, "optimizer": {"lr": 1e-3}, "denoise_steps": 1, "critic_updates_per_student": 1})
        out = be.train(cfg)
        assert out["final_step"] == 1
        ok = verify_checkpoint(out["checkpoint"])
        assert ok.contract.stage == stage and ok.step == 1


def test_h3_activation_checkpointing_modes_keep_the_gradients():
    import torch

    from solarwm_b200.backends.minimax_h3.stage1 import teacher_forcing_forward  # noqa: F401  (module import check)
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.renderer.cli import _sample
    from solarwm_b200.renderer.core import packed_forward
    from solarwm_b200.backends.minimax_h3.layout import patchify_latents

    cfg = h3_preset("tiny")
    cfg.lora_rank = 4
    s = _sample(cfg, 0)
    grads = {}
    for mode in ("none", "full", "selective"):
        m = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
        for p in m.trainable_parameters():
            torch.nn.init.normal_(p, std=0.02, generator=torch.Generator().manual_seed(p.numel()))
        m.checkpointing = mode
        rows = patchify_latents(s["target_latents"]).float()
        out = packed_forward(m, prompt=s["prompt_embeds"].float(), anchor_rows=patchify_latents(s["anchor_latents"]).float(),
                             structure_rows=None, target_rows=rows, row_times=torch.full((rows.shape[0],), 0.4), grid_hw=(4, 4))
        out.pow(2).mean().backward()
        grads[mode] = [p.grad.clone() for p in m.trainable_parameters()]
        assert len(grads[mode]) > 0 and any(g.abs().max() > 0 for g in grads[mode])
    for mode in ("full", "selective"):
        for a, b in zip(grads["none"], grads[mode]):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-8)


def test_h3_backend_infer_runs_camera_length_generation(tmp_path):
    import json

    from solarwm_b200.registry import load_backend

    config = {"model": {"family": "minimax_h3", "architecture": "tiny", "camera_translation_transform": "logd4"},
              "runtime": {"output_dir": str(tmp_path / "run"), "device": "cpu"},
              "inference": {"source": "synthetic", "grid_hw": [2, 3], "chunk_latents": 2, "chunks": 3, "denoise_steps": 2,
                            "memory": True, "top_k": 2, "seed": 4}}
    out = load_backend("minimax_h3").infer(config)
    manifest = json.loads((tmp_path / "run" / "generate" / "manifest.json").read_text())
    assert out["chunks"] == 3 and manifest["latents"] == 6 and manifest["memory"]["enabled"] is True
    assert len(manifest["chunk_seconds"]) == 3


def test_h3_backend_infer_loads_released_weights(tmp_path):
    import torch
    from safetensors.torch import save_file

    from solarwm_b200.backends.minimax_h3.loader import export_released_layout
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.registry import load_backend

    cfg = h3_preset("tiny")
    weights = tmp_path / "weights"
    weights.mkdir()
    save_file(export_released_layout(H3DiT(cfg, device="cpu", dtype=torch.float32, seed=9)), str(weights / "model.safetensors"))
    config = {"model": {"family": "minimax_h3", "architecture": "tiny", "camera_translation_transform": "logd4",
                        "weights_dir": str(weights)},
              "runtime": {"output_dir": str(tmp_path / "run"), "device": "cpu"},
              "inference": {"source": "synthetic", "grid_hw": [2, 3], "chunk_latents": 2, "chunks": 1, "denoise_steps": 1}}
    assert load_backend("minimax_h3").infer(config)["chunks"] == 1
    config["model"]["weight_rules"] = [["^nothing$", "proj_in"]]
    import pytest

    with pytest.raises(BackendContractError, match="match no rule"):
        load_backend("minimax_h3").infer(config)


def test_suffix_forward_on_captured_prefix_matches_the_full_evaluation():
    """AnyFlow probes: the noisy half evaluated against the captured prefix K / V equals the noisy half of a full
    teacher-forcing evaluation, at other noise levels than the capturing evaluation used; and a trainer with the
    reuse on takes the same step as one with it off."""
    from solarwm_b200.backends.minimax_h3.layout import patchify_latents
    from solarwm_b200.backends.minimax_h3.stage1 import suffix_forward, teacher_forcing_forward
    from solarwm_b200.models.h3 import H3DiT

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    s = h3_sample(latent_frames=4, height=4, width=4, prompt_len=6, text_dim=cfg.text_dim, seed=1)
    cams = torch.eye(4).repeat(5, 1, 1)
    cams[1:, 0, 3] = torch.arange(4) * 0.1
    g = torch.Generator().manual_seed(0)
    clean = patchify_latents(s["target_latents"]).float()
    anchor = patchify_latents(s["anchor_latents"]).float()
    kw = dict(grid_hw=(2, 2), chunk_latents=2, window_chunks=1, cameras=cams)

    def noisy_at(t):
        return clean * 0.5 + torch.randn(clean.shape, generator=torch.Generator().manual_seed(int(t[0] * 1000)))

    t0, t1 = torch.tensor([0.3, 0.7]), torch.tensor([0.35, 0.65])
    with torch.no_grad():
        prefix = []
        teacher_forcing_forward(model, prompt=s["prompt_embeds"].float(), anchor_rows=anchor, clean_rows=clean,
                                noisy_rows=noisy_at(t0), t_chunks=t0, capture=prefix, **kw)
        assert len(prefix) == len(model.blocks) and prefix[0][0].shape[1] == 6 + anchor.shape[0] + clean.shape[0]
        want = teacher_forcing_forward(model, prompt=s["prompt_embeds"].float(), anchor_rows=anchor, clean_rows=clean,
                                       noisy_rows=noisy_at(t1), t_chunks=t1, **kw)
        got = suffix_forward(model, captured=prefix, noisy_rows=noisy_at(t1), t_chunks=t1, n_text=6, n_anchor=anchor.shape[0], **kw)
    assert got.shape == want.shape and torch.allclose(got, want, atol=2e-5, rtol=1e-4)
    cfg.lora_rank = 4
    losses = []
    for reuse in (False, True):
        tr = H3Stage1Trainer(cfg, "cpu", objective="anyflow", chunk_latents=2, window_chunks=1, lr=1e-3,
                             diffusion_ratio=0.0, consistency_ratio=0.5, seed=3, reuse_prefix=reuse)
        for p in tr.model.trainable_parameters():
            torch.nn.init.normal_(p, std=0.02, generator=torch.Generator().manual_seed(p.numel()))
        batch = dict(s, camera_w2c=cams)
        losses.append(float(tr.train_step(batch)))
    # without reuse every probe re-noises the anchor frame on its own, so the two steps agree closely, not bitwise
    assert abs(losses[0] - losses[1]) < 1e-3 * max(1.0, abs(losses[0]))
    del g


def test_h3_backend_train_honours_activation_checkpointing_setting(tmp_path, monkeypatch):
    from solarwm_b200.models import h3 as h3_model
    from solarwm_b200.registry import load_backend

    seen = []
    original = h3_model.H3DiT.forward

    def spy(self, **kw):
        seen.append(self.checkpointing)
        return original(self, **kw)

    monkeypatch.setattr(h3_model.H3DiT, "forward", spy)
    config = {"schema": "solarwm.run.v1", "action": "train",
              "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
              "data": {"seed": 0, "latent_frames": 3, "latent_height": 4, "latent_width": 4, "prompt_len": 6, "pixel_frames": 158},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 1,
                        "optimizer": {"lr": 1e-3}, "fsdp": {"activation_checkpointing": True, "saved_attention_blocks": 2}},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path)}}
    out = load_backend("minimax_h3").train(config)
    assert out["final_step"] == 1 and seen and set(seen) == {"selective"}


def test_h3_backend_trains_from_its_own_preencoded_corpus(tmp_path):
    from solarwm_b200.registry import load_backend

    be = load_backend("minimax_h3")
    pre = {"data": {"pixel_frames": 9, "pixel_height": 64, "pixel_width": 64, "seed": 1}, "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 2, "output_root": str(tmp_path / "enc"),
                         "codecs": {"vae_base": 4, "t5": {"vocab": 512, "dim": 64, "dim_attn": 32, "dim_ffn": 64, "num_heads": 2,
                                                         "num_layers": 1, "text_len": 8}}}}
    assert be.preencode(pre)["samples"] == 2
    config = {"schema": "solarwm.run.v1", "action": "train",
              "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
              "data": {"source": "index", "index": str(tmp_path / "enc" / "index.jsonl"), "seed": 0, "pixel_frames": 158},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 2,
                        "optimizer": {"lr": 1e-3}},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")}}
    out = be.train(config)
    assert out["final_step"] == 2 and out["last_loss"] == out["last_loss"]
    # the same corpus conditions a camera-length generation: prompt + anchor frame of sample 1
    infer = dict(config, action="infer", runtime={"device": "cpu", "output_dir": str(tmp_path / "gen")},
                 inference={"source": "index", "sample": 1, "grid_hw": [2, 2], "chunk_latents": 2, "chunks": 2, "denoise_steps": 1})
    got = be.infer(infer)
    assert got["chunks"] == 2 and (tmp_path / "gen" / "generate" / "manifest.json").is_file()


def test_h3_backend_infer_decodes_frames_when_a_decoder_is_configured(tmp_path):
    from solarwm_b200.registry import load_backend

    config = {"model": {"family": "minimax_h3", "architecture": "tiny", "camera_translation_transform": "logd4"},
              "runtime": {"output_dir": str(tmp_path / "run"), "device": "cpu"},
              "inference": {"source": "synthetic", "grid_hw": [2, 3], "chunk_latents": 2, "chunks": 2, "denoise_steps": 1,
                            "decoder": {"dim": 64, "depth": 1, "heads": 2, "dim_head": 32, "ffn_dim": 128, "registers": 2, "patch": 2}}}
    out = load_backend("minimax_h3").infer(config)
    assert out["frames"] > 0 and out["video"]["frames"] == out["frames"]
    assert (tmp_path / "run" / "generate" / "frames" / "video.rgb").stat().st_size == out["frames"] * (4 * 2) * (6 * 2) * 3


def test_w6_with_audio_rows_matches_its_dense_mask():
    """Condition rows see the condition, audio rows the condition and the audio, video rows both plus their window."""
    torch.manual_seed(1)
    n_cond, n_audio, chunk_rows, n_chunks, W = 5, 3, 4, 3, 1
    S = n_cond + n_audio + 2 * n_chunks * chunk_rows
    q, k, v = (torch.randn(1, S, 2, 16) for _ in range(3))
    mask = w6_mask(n_cond, chunk_rows, n_chunks, W, n_audio=n_audio)
    assert not mask[:n_cond, n_cond:].any() and mask[n_cond:n_cond + n_audio, :n_cond + n_audio].all()
    assert not mask[n_cond:n_cond + n_audio, n_cond + n_audio:].any() and mask[n_cond + n_audio:, :n_cond + n_audio].all()
    got = w6_attention(q, k, v, n_cond=n_cond, chunk_rows=chunk_rows, n_chunks=n_chunks, window_chunks=W, n_audio=n_audio)
    assert torch.allclose(got, R.attention(q, k, v, mask=mask.view(1, 1, S, S)), atol=1e-5)


def test_silent_soundtrack_in_teacher_forcing():
    """Audio rows enter the document (the video prediction depends on them), the prefix capture holds them, the suffix
    evaluation on that prefix equals the full one, and a trainer with silence installed steps on both objectives."""
    from solarwm_b200.backends.minimax_h3.layout import patchify_latents
    from solarwm_b200.backends.minimax_h3.stage1 import suffix_forward, teacher_forcing_forward
    from solarwm_b200.models.h3 import H3DiT

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    s = h3_sample(latent_frames=4, height=4, width=4, prompt_len=6, text_dim=cfg.text_dim, seed=1)
    clean = patchify_latents(s["target_latents"]).float()
    anchor = patchify_latents(s["anchor_latents"]).float()
    audio = torch.randn(6, cfg.audio_row_dim, generator=torch.Generator().manual_seed(5))
    noisy = clean * 0.5 + torch.randn(clean.shape, generator=torch.Generator().manual_seed(2))
    kw = dict(grid_hw=(2, 2), chunk_latents=2, window_chunks=1, cameras=torch.eye(4).repeat(5, 1, 1))
    t0, t1 = torch.tensor([0.3, 0.7]), torch.tensor([0.4, 0.6])
    common = dict(prompt=s["prompt_embeds"].float(), anchor_rows=anchor, clean_rows=clean, noisy_rows=noisy)
    with torch.no_grad():
        prefix = []
        with_audio = teacher_forcing_forward(model, t_chunks=t0, audio_rows=audio, t_audio=0.4, capture=prefix, **common, **kw)
        without = teacher_forcing_forward(model, t_chunks=t0, **common, **kw)
        other_time = teacher_forcing_forward(model, t_chunks=t0, audio_rows=audio, t_audio=0.8, **common, **kw)
        assert with_audio.shape == without.shape == clean.shape
        assert not torch.allclose(with_audio, without, atol=1e-4) and not torch.allclose(with_audio, other_time, atol=1e-5)
        assert prefix[0][0].shape[1] == 6 + anchor.shape[0] + 6 + clean.shape[0]
        want = teacher_forcing_forward(model, t_chunks=t1, audio_rows=audio, t_audio=0.4, **common, **kw)
        got = suffix_forward(model, captured=prefix, noisy_rows=noisy, t_chunks=t1, n_text=6, n_anchor=anchor.shape[0], n_audio=6, **kw)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-4)

    cfg.lora_rank = 4
    for objective in ("tf_fm", "anyflow"):
        losses = {}
        for silent in (False, True):
            tr = H3Stage1Trainer(cfg, "cpu", objective=objective, chunk_latents=2, window_chunks=1, lr=1e-3, seed=3,
                                 diffusion_ratio=0.0, consistency_ratio=0.5)
            for p in tr.model.trainable_parameters():
                torch.nn.init.normal_(p, std=0.02, generator=torch.Generator().manual_seed(p.numel()))
            if silent:
                tr.silence = audio
            before = [p.detach().clone() for p in tr.model.trainable_parameters()]
            losses[silent] = float(tr.train_step(dict(s, camera_w2c=kw["cameras"])))
            assert losses[silent] == losses[silent]
            assert any(not torch.equal(a, b) for a, b in zip(before, tr.model.trainable_parameters()))
        assert losses[False] != losses[True]
