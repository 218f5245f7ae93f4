"""Source-length H3 evaluation: geometry (against the reference function when it is installed), plan checks,
idempotent preparation, resumable generation with trimming to the source length."""
import json
import sys
from pathlib import Path

import pytest
import torch

from solarwm_b200.errors import BackendContractError
from solarwm_b200.serve.h3_source_length import (exported_fps, full_length_geometry, load_plan, prepare_case, relative_views,
                                                 run_plan, storyboard_indices)

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"


def test_geometry_matches_the_reference_function_and_its_own_rules():
    g = full_length_geometry(81)
    assert (g.decoded_frames, g.decode_latents, g.rollout_latents, g.tail_camera_rows) == (90, 27, 30, 6)
    assert g.camera_indices[:7] == (0, 1, 5, 9, 13, 17, 18) and g.camera_indices[-1] == 77 and len(g.camera_indices) == 30
    for frames in (22, 39, 40, 200, 961):
        g = full_length_geometry(frames)
        assert g.decoded_frames >= frames and g.rollout_latents % 5 == 0 and 0 <= g.rollout_latents - g.decode_latents < 5
        assert max(g.camera_indices) < frames and list(g.camera_indices) == sorted(g.camera_indices)
    for bad in (21, True, 30.0):
        with pytest.raises(ValueError):
            full_length_geometry(bad)
    assert exported_fps(30.0, "source") == 30.0 and exported_fps(30.0, "h3") == 24.0
    for args in ((0.0, "source"), (float("nan"), "h3"), (24.0, "other")):
        with pytest.raises(ValueError):
            exported_fps(*args)
    assert storyboard_indices(101) == [0, 10, 25, 50, 75, 90, 100]
    if (REF / "solar").exists():
        sys.path.insert(0, str(REF))
        try:
            from solar.backends.minimax_h3.full_length import full_length_geometry as theirs
        except Exception:  # noqa: BLE001
            return
        for frames in range(22, 400, 7):
            a, b = full_length_geometry(frames), theirs(frames)
            assert (a.decoded_frames, a.decode_latents, a.rollout_latents, a.camera_indices, a.tail_camera_rows) == \
                   (b.decoded_frames, b.decode_latents, b.rollout_latents, b.camera_indices, b.tail_camera_rows)


def test_plan_rows_are_checked(tmp_path):
    good = [{"key": "a", "dataset": "d", "num_frames": 30, "fps": 24.0, "caption": "x"},
            {"key": "b", "dataset": "d", "num_frames": 1000, "fps": 30.0, "caption": "y"}]
    p = tmp_path / "plan.json"
    p.write_text(json.dumps(good))
    with pytest.raises(BackendContractError):
        load_plan(p)                                               # 1000 frames need streaming decode
    assert len(load_plan(p, stream_decode=True)) == 2
    for broken in ([], [dict(good[0]), dict(good[0])], [dict(good[0], key="a/b")], [dict(good[0], dataset="..")],
                   [dict(good[0], num_frames="30")]):
        p.write_text(json.dumps(broken))
        with pytest.raises(BackendContractError):
            load_plan(p, stream_decode=True)
    p.write_text(json.dumps([dict(good[0], num_frames=10)]))
    with pytest.raises(ValueError):
        load_plan(p)


def test_relative_views_start_at_the_identity_and_refuse_broken_matrices():
    c2w = torch.eye(4).repeat(5, 1, 1)
    c2w[:, 0, 3] = torch.arange(5.0) + 3
    v = relative_views(c2w)
    assert torch.equal(v[0], torch.eye(4)) and torch.allclose(v[2, :3, 3], torch.tensor([-2.0, 0, 0]))
    bad = c2w.clone()
    bad[1, 3, 0] = 0.5
    with pytest.raises(BackendContractError):
        relative_views(bad)


class _FakeDecoder:
    """1 frame for the first latent, 4 for every later one (the codec's cadence)."""

    def __init__(self):
        self.n = 0

    def push(self, latent):
        self.n += 1
        return torch.full((3, 1 if self.n == 1 else 4, 8, 12), float(self.n))


class _Writer:
    made = []

    def __init__(self, path, fps):
        self.path, self.fps, self.frames = Path(path), fps, 0
        _Writer.made.append(self)

    def push(self, frames):
        self.frames += frames.shape[1]

    def close(self):
        self.path.write_bytes(b"mp4:%d" % self.frames)


def test_prepare_is_idempotent_and_generation_resumes_and_trims(tmp_path):
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.serve.h3_stream import H3StreamConfig

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    rows = [{"key": "clip-a", "dataset": "val", "num_frames": 22, "fps": 30.0, "caption": "a room"},
            {"key": "clip-b", "dataset": "val", "num_frames": 22, "fps": 25.0, "caption": "a hall", "validation_noise_seed": 9}]
    calls = {"prompt": 0}

    def encode_prompt(text):
        calls["prompt"] += 1
        return torch.randn(6, cfg.text_dim, generator=torch.Generator().manual_seed(len(text)))

    identity = {"codec": "test", "image": "first-frame"}
    for row in rows:
        F = row["num_frames"]
        c2w = torch.eye(4).repeat(F, 1, 1)
        c2w[:, 2, 3] = torch.linspace(0, 2, F)
        K = torch.tensor([[0.5, 0, 0.5], [0, 0.9, 0.5], [0, 0, 1.0]]).repeat(F, 1, 1)
        r1 = prepare_case(tmp_path / "work", row, c2w=c2w, intrinsics=K, encode_prompt=encode_prompt,
                          encode_anchor=lambda: torch.randn(24, 1, 4, 6, generator=torch.Generator().manual_seed(1)), identity=identity)
        r2 = prepare_case(tmp_path / "work", row, c2w=c2w, intrinsics=K, encode_prompt=encode_prompt,
                          encode_anchor=lambda: torch.zeros(24, 1, 4, 6), identity=identity)
        assert r1 == r2 and r1["geometry"]["rollout_latents"] == 10 and r1["geometry"]["decode_latents"] == 7
    assert calls["prompt"] == 2                                    # the second call of each case reused the receipt
    with pytest.raises(BackendContractError):
        prepare_case(tmp_path / "work", rows[0], c2w=c2w, intrinsics=K, encode_prompt=encode_prompt,
                     encode_anchor=lambda: torch.zeros(24, 1, 4, 6), identity={"codec": "other"})
    scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=5, window_chunks=2, denoise_steps=1, use_cuda_graph=False)
    kw = dict(work_dir=tmp_path / "work", out_dir=tmp_path / "out", stream_cfg=scfg, identity={"checkpoint": "c1"},
              decoder_factory=_FakeDecoder, writer_factory=_Writer, save_latents=True)
    first = run_plan(model, rows[:1], **kw)
    assert first["generated"] == ["clip-a"] and not first["skipped"]
    man = json.loads((tmp_path / "out" / "val" / "clip-a.json").read_text())
    # 7 of the 10 generated latents are decoded (1 + 6 * 4 = 25 frames) and the clip's 22 frames are exported
    assert man["generation"]["frames"] == 22 and man["generation"]["latents"] == 10 and man["fps"] == 30.0
    assert (tmp_path / "out" / "val" / "clip-a.mp4").read_bytes() == b"mp4:22" and man["noise_seed"] == 0
    assert torch.load(tmp_path / "out" / "val" / "clip-a.latents.pt", weights_only=True).shape == (24, 10, 4, 6)
    both = run_plan(model, rows, **kw)
    assert both["generated"] == ["clip-b"] and both["skipped"] == ["clip-a"]
    assert json.loads((tmp_path / "out" / "val" / "clip-b.json").read_text())["noise_seed"] == 9
    with pytest.raises(BackendContractError):                      # the same outputs under another checkpoint identity
        run_plan(model, rows, **{**kw, "identity": {"checkpoint": "c2"}})
    # ranks split the plan
    assert run_plan(model, rows, rank=1, world=2, **kw)["skipped"] == ["clip-b"]
    with pytest.raises(BackendContractError):
        run_plan(model, [dict(rows[0], key="never-prepared")], **kw)


def test_backend_runs_a_source_length_plan_with_the_streaming_decoder(tmp_path):
    from solarwm_b200.backends.minimax_h3.backend import MiniMaxH3Backend
    from solarwm_b200.models.h3 import h3_preset

    cfg = h3_preset("tiny")
    F = 22
    (tmp_path / "sources").mkdir()
    c2w = torch.eye(4).repeat(F, 1, 1)
    c2w[:, 2, 3] = torch.linspace(0, 1, F)
    torch.save({"text": torch.randn(6, cfg.text_dim), "anchor_latent": torch.randn(24, 1, 4, 6), "c2w": c2w,
                "intrinsics": torch.tensor([[0.5, 0, 0.5], [0, 0.9, 0.5], [0, 0, 1.0]]).repeat(F, 1, 1)}, tmp_path / "sources" / "clip.pt")
    (tmp_path / "plan.json").write_text(json.dumps([{"key": "clip", "dataset": "val", "num_frames": F, "fps": 24.0, "caption": "c"}]))
    config = {"schema": "solarwm.run.v1", "action": "infer",
              "model": {"family": "minimax_h3", "architecture": "tiny", "camera_translation_transform": "logd4"},
              "runtime": {"device": "cpu", "output_dir": str(tmp_path / "run")},
              "inference": {"length_policy": "source", "plan": str(tmp_path / "plan.json"), "sources": str(tmp_path / "sources"),
                            "grid_hw": [2, 3], "window_chunks": 2, "denoise_steps": 1, "use_ffmpeg": False,
                            "decoder": {"dim": 64, "depth": 1, "heads": 2, "dim_head": 32, "ffn_dim": 128, "registers": 2, "patch": 2}}}
    be = MiniMaxH3Backend("minimax_h3")
    out = be.infer(config)
    assert out["generated"] == ["clip"]
    man = json.loads((tmp_path / "run" / "generate" / "val" / "clip.json").read_text())
    assert man["generation"]["latents"] == 10 and 0 < man["generation"]["frames"] <= F and man["geometry"]["decode_latents"] == 7
    assert (tmp_path / "run" / "generate" / "val" / "clip.mp4").is_file()
    assert be.infer(config)["skipped"] == ["clip"]
