"""H3 frame / latent / canvas rules and raw-camera decoding (against the reference functions when they are installed)."""
import io
import sys
from pathlib import Path

import numpy as np
import pytest

from solarwm_b200.backends.minimax_h3.geometry import (FIXED_FOCAL, ResizeCrop, align_pixel_frames, audio_latents_for_video, decode_camera,
                                                       fixed_intrinsics, latent_pixel_indices, latent_to_pixel_frames, normalise_intrinsics,
                                                       pixel_to_latent_frames, validate_canvas)
from solarwm_b200.errors import DataContractError

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


def test_frame_latent_and_canvas_rules():
    assert [align_pixel_frames(n) for n in (1, 5, 6, 22, 23, 158)] == [5, 5, 22, 22, 39, 158]
    assert pixel_to_latent_frames(158) == 47 and latent_to_pixel_frames(47) == 158 and pixel_to_latent_frames(5) == 2
    for n in (5, 22, 39, 158, 362):
        idx = latent_pixel_indices(n)
        assert len(idx) == pixel_to_latent_frames(n) and idx[0] == 0 and idx[-1] < n and (np.diff(idx) > 0).all()
        assert latent_to_pixel_frames(len(idx)) == n
    assert latent_pixel_indices(22).tolist() == [0, 1, 5, 9, 13, 17, 18]
    for bad in (4, 23):
        with pytest.raises(ValueError):
            pixel_to_latent_frames(bad)
    with pytest.raises(ValueError):
        latent_to_pixel_frames(6)
    assert audio_latents_for_video(158) == 165 and audio_latents_for_video(24) == 25
    assert validate_canvas(768, 1344) == (768, 1344)
    for bad in ((0, 32), (100, 64), (64, 70)):
        with pytest.raises(ValueError):
            validate_canvas(*bad)
    if (REF / "solar").exists():
        sys.path.insert(0, str(REF))
        try:
            from solar.backends.minimax_h3 import geometry as theirs
        except Exception:  # noqa: BLE001
            return
        for n in (5, 22, 158, 362):
            assert latent_pixel_indices(n).tolist() == theirs.latent_aligned_pixel_indices(n).tolist()
            assert pixel_to_latent_frames(n) == theirs.pixel_frames_to_latent_frames(n)
        assert [align_pixel_frames(n) for n in range(1, 60)] == [theirs.align_pixel_frames(n) for n in range(1, 60)]


def test_intrinsics_follow_the_resize_and_crop():
    how = ResizeCrop.cover(1920, 1080, 1344, 768)                    # 16:9 -> 1.75: resized to 1365 x 768, 10 px cut left
    assert (how.resized_w, how.resized_h, how.crop_left, how.crop_top) == (1365, 768, 10, 0)
    px = np.array([[1000.0, 0, 960], [0, 1000.0, 540], [0, 0, 1]])
    K = normalise_intrinsics(px, [0, 3], how)
    assert K.shape == (2, 3, 3) and K.dtype == np.float32
    assert K[0, 0, 0] == pytest.approx(1000 * 1365 / 1920 / 1344) and K[0, 1, 1] == pytest.approx(1000 * 768 / 1080 / 768)
    assert K[0, 0, 2] == pytest.approx((960 * 1365 / 1920 - 10) / 1344) and K[0, 1, 2] == pytest.approx(0.5)
    # the same camera given normalised, as (fx, fy, cx, cy) vectors per frame, lands on the same matrices
    vec = np.tile([1000 / 1920, 1000 / 1080, 0.5, 0.5], (5, 1))
    assert np.allclose(normalise_intrinsics(vec, [0, 3], how), K, atol=1e-6)
    assert np.allclose(normalise_intrinsics(px[None], [0, 3], how), K, atol=1e-6)
    assert np.allclose(normalise_intrinsics(None, [0, 3], how), fixed_intrinsics(2)) and fixed_intrinsics(1)[0, 0, 0] == pytest.approx(FIXED_FOCAL[0])
    with pytest.raises(DataContractError):
        normalise_intrinsics(np.tile(px, (2, 1, 1)), [0, 3], how)    # two matrices for frames 0 and 3
    huge = px.copy()
    huge[0, 0] = 9000.0
    with pytest.raises(DataContractError):
        normalise_intrinsics(huge, [0], how)
    assert normalise_intrinsics(huge, [0], how, focal_guard=False)[0, 0, 0] > 4
    with pytest.raises(DataContractError):
        normalise_intrinsics(np.zeros((2, 2)), [0], how)


def _archive(**arrays) -> bytes:
    buf = io.BytesIO()
    np.savez(buf, **arrays)
    return buf.getvalue()


def test_camera_archives_in_their_several_forms():
    how = ResizeCrop.cover(640, 480, 64, 64)
    c2w = np.tile(np.eye(4, dtype=np.float32), (6, 1, 1))
    c2w[:, 0, 3] = np.arange(6)
    got, K = decode_camera(_archive(vipe_c2w=c2w, vipe_status=np.array(["ok"]), fx=np.float64(0.8), fy=np.float64(1.1)), [0, 2, 5], how)
    assert got[:, 0, 3].tolist() == [0.0, 2.0, 5.0] and K.shape == (3, 3, 3) and K[0, 1, 1] == pytest.approx(1.1 * 480 * (64 / 480) / 64)
    w2c = np.linalg.inv(c2w)
    assert np.allclose(decode_camera(_archive(w2c=w2c), [1, 4], how)[0], c2w[[1, 4]], atol=1e-6)
    extra = io.BytesIO()
    np.save(extra, np.array([[500.0, 0, 320], [0, 500.0, 240], [0, 0, 1]]))
    _, K2 = decode_camera(_archive(camera_c2w=c2w), [0], how, intrinsics_bytes=extra.getvalue())
    assert K2[0, 0, 2] == pytest.approx(0.5, abs=0.01)
    assert np.allclose(decode_camera(_archive(c2w=c2w), [0], how)[1], fixed_intrinsics(1))     # no intrinsics anywhere
    for bad in (_archive(vipe_c2w=c2w, vipe_status=np.array(["failed"])), _archive(points=c2w), _archive(c2w=c2w[:2]),
                _archive(c2w=np.full_like(c2w, np.nan)), _archive(c2w=c2w[:, :3])):
        with pytest.raises(DataContractError):
            decode_camera(bad, [0, 3], how)


def test_cameras_travel_from_the_preencoder_to_the_training_sample(tmp_path):
    import torch

    from solarwm_b200.backends.minimax_h3.runtime import H3TrainingRuntime
    from solarwm_b200.registry import load_backend

    be = load_backend("minimax_h3")
    pre = {"data": {"pixel_frames": 9, "pixel_height": 64, "pixel_width": 64, "seed": 1}, "runtime": {"device": "cpu"},
           "preencode": {"source": "synthetic", "num_samples": 2, "cameras": True, "output_root": str(tmp_path / "enc"),
                         "codecs": {"vae_base": 4, "t5": {"vocab": 512, "dim": 64, "dim_attn": 32, "dim_ffn": 64, "num_heads": 2,
                                                         "num_layers": 1, "text_len": 8}}}}
    assert be.preencode(pre)["samples"] == 2
    import json

    contract = json.loads((tmp_path / "enc" / "encoder-contract.json").read_text())
    assert {t["name"] for t in contract["tensors"]} == {"latents", "text", "camera_c2w", "camera_K"}
    config = {"schema": "solarwm.run.v1", "action": "train",
              "model": {"family": "minimax_h3", "architecture": "tiny", "adapter": {"rank": 4}, "camera_translation_transform": "logd4"},
              "data": {"source": "index", "index": str(tmp_path / "enc" / "index.jsonl"), "seed": 0, "pixel_frames": 158},
              "train": {"stage": "stage0p5", "causal_mode": "bidirectional", "objective": "flow_matching", "max_steps": 1, "optimizer": {"lr": 1e-3}},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")}}
    rt = H3TrainingRuntime(config, model_config=be._cfg(config))
    try:
        _, _, sample = rt._next_sample()
        views = sample["camera_w2c"]
        assert views.shape == (3, 4, 4) and torch.equal(views[0], torch.eye(4))
        assert float(views[1:, 2, 3].abs().min()) > 0                  # the dolly of the corpus, relative to the anchor's camera
        rt.train_microbatch(0, 1)
    finally:
        rt.close()
