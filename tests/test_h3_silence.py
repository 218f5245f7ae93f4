"""The silent soundtrack of the video-only H3 stages: artifact checks, packed rows, the training step with audio rows."""
import pytest
import torch

from solarwm_b200.backends.minimax_h3.silence import LENGTHS, load_silence_latents, noised_silence, silence_rows
from solarwm_b200.errors import DataContractError


def _artifact(path, frames=158, dtype=torch.bfloat16, length=None):
    from safetensors.torch import save_file

    g = torch.Generator().manual_seed(0)
    save_file({f"silence_{frames}f": (torch.randn(2, 32, length or LENGTHS[frames], generator=g) * 0.1).to(dtype)}, str(path))


def test_artifact_checks_and_row_packing(tmp_path):
    _artifact(tmp_path / "s.safetensors")
    v = load_silence_latents(tmp_path / "s.safetensors", pixel_frames=158)
    assert v.shape == (2, 32, 263)
    rows = silence_rows(v)
    assert rows.shape == (526, 32) and torch.equal(rows[0], v[0, :, 0]) and torch.equal(rows[263], v[1, :, 0]) and torch.equal(rows[1], v[0, :, 1])
    g = torch.Generator().manual_seed(1)
    noised, t = noised_silence(rows, g, torch.device("cpu"))
    assert noised.shape == rows.shape and 0.0 < t < 1.0 and not torch.allclose(noised, rows.float())
    for bad in ({"frames": 153}, {"dtype": torch.float32}, {"length": 100}):
        _artifact(tmp_path / "bad.safetensors", **bad)
        with pytest.raises(DataContractError):
            load_silence_latents(tmp_path / "bad.safetensors", pixel_frames=158)
    with pytest.raises(DataContractError):
        load_silence_latents(tmp_path / "none.safetensors")
    with pytest.raises(DataContractError):
        load_silence_latents(tmp_path / "s.safetensors", pixel_frames=100)
    (tmp_path / "junk.safetensors").write_bytes(b"junk")
    with pytest.raises(DataContractError):
        load_silence_latents(tmp_path / "junk.safetensors")


def test_training_step_packs_the_silent_soundtrack(tmp_path):
    from solarwm_b200.backends.minimax_h3.runtime import H3TrainingRuntime
    from solarwm_b200.registry import load_backend

    _artifact(tmp_path / "s.safetensors")
    be = load_backend("minimax_h3")
    base = {"schema": "solarwm.run.v1", "action": "train",
            "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
            "data": {"source": "synthetic", "seed": 3, "pixel_frames": 158, "latent_frames": 2, "latent_height": 4, "latent_width": 4},
            "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 1, "optimizer": {"lr": 1e-3}},
            "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")}}
    losses, seen = {}, {}
    for name, extra in (("plain", {}), ("silent", {"silence_latents_path": str(tmp_path / "s.safetensors")})):
        cfg = {**base, "data": {**base["data"], **extra}}
        rt = H3TrainingRuntime(cfg, model_config=be._cfg(cfg))
        try:
            held = rt.model.forward
            rt.model.forward = lambda **k: (seen.__setitem__(name, None if k.get("audio_rows") is None else tuple(k["audio_rows"].shape)), held(**k))[1]
            losses[name] = rt.train_microbatch(0, 1).losses["loss"]
        finally:
            rt.close()
    assert seen == {"plain": None, "silent": (526, 32)} and losses["plain"] != losses["silent"]
