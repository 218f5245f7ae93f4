"""Model-free temporal / structural metrics, the scorer registry, and the resumable benchmark pass + summary."""
import json

import numpy as np
import pytest


def _scene(T=12, H=64, W=96, shift=2, flicker=0.0, seed=0):
    """A textured pattern translating right by ``shift`` pixels per frame; ``flicker`` adds a per-frame brightness jump."""
    rng = np.random.default_rng(seed)
    import cv2

    base = cv2.GaussianBlur(rng.integers(0, 255, (H, W + T * shift + 8, 3), dtype=np.uint8), (0, 0), 2.0)
    base[20:40, 30:70] = (255, 255, 255)
    frames = []
    for t in range(T):
        f = base[:, t * shift:t * shift + W].astype(np.float32)
        f += flicker * (1 if t % 2 else -1)
        frames.append(np.clip(f, 0, 255).astype(np.uint8))
    return np.stack(frames)


def test_flicker_reads_brightness_jumps_not_motion():
    from solarwm_b200.eval.motion import flow_flicker, warp
    import torch

    steady, flashing = flow_flicker(_scene()), flow_flicker(_scene(flicker=12.0))
    assert steady["pairs"] == 11 and steady["consistent_frac"] > 0.5 and 1.0 < steady["flow_mag"] < 3.0
    assert flashing["warp_l1_lp"] > 5 * max(steady["warp_l1_lp"], 0.5) and flashing["warp_l1_lp"] > 10.0
    assert abs(flashing["sharpness_lapvar"] - steady["sharpness_lapvar"]) < 0.2 * steady["sharpness_lapvar"]
    img = torch.arange(16.0).view(1, 1, 4, 4)
    out, inside = warp(img, torch.ones(1, 2, 4, 4))                      # sample one pixel right and down
    assert out[0, 0, 0, 0] == img[0, 0, 1, 1] and not bool(inside[0, 3, 3]) and bool(inside[0, 0, 0])


def test_edges_and_tracks_follow_structure_and_motion():
    from solarwm_b200.eval.motion import canny_edges, edge_f1, motion_compare, structure_edges, track_grid

    a = _scene()
    same = structure_edges(a, a)
    assert same["F1"] == pytest.approx(1.0) and same["frames"] == 3 and same["cond_edge_density"] > 0
    other = structure_edges(_scene(seed=5)[:, ::-1].copy(), a)
    assert other["F1"] < 0.9
    e = canny_edges(a[:1])
    shifted = np.roll(e, 2, axis=2)
    assert edge_f1(shifted, e, tolerance=2)["F1"] > 0.95 and edge_f1(np.roll(e, 9, axis=2), e, tolerance=2)["F1"] < 0.8
    cond = track_grid(a, query_frames=(0,), grid=(6, 4))
    tracks, vis, conf, pts, qt = cond
    assert tracks.shape == (12, 24, 2) and (qt == 0).all()
    moved = tracks[-1, :, 0] - pts[:, 0]
    ok = (vis[-1] * conf[-1]) > 0.6
    assert ok.sum() >= 8 and np.median(moved[ok]) == pytest.approx(-22.0, abs=2.0)        # the pattern moves left in the frame
    same_motion = motion_compare(cond, track_grid(a, query_frames=(0,), grid=(6, 4)), (96, 64))
    frozen = motion_compare(cond, track_grid(np.repeat(a[:1], 12, axis=0), query_frames=(0,), grid=(6, 4)), (96, 64))
    assert same_motion["err_mean"] < 0.005 and same_motion["kept_frac"] > 0.3
    assert frozen["err_mean"] > 5 * max(same_motion["err_mean"], 1e-3) and frozen["err_mean"] == pytest.approx(frozen["frozen_err_mean"], rel=0.3)


def test_scorers_report_missing_weights_instead_of_failing():
    from solarwm_b200.eval.motion import Scorers

    s = Scorers()
    s.register("mean_level", lambda: (lambda frames, case: {"value": float(frames.mean())}))
    calls = {"n": 0}

    def absent():
        calls["n"] += 1
        raise FileNotFoundError("weights/quality.pt")

    s.register("quality_model", absent)
    assert s.names() == ["mean_level", "quality_model"] and s.score("mean_level", np.full((2, 4, 4, 3), 10, np.uint8))["value"] == 10.0
    assert "FileNotFoundError" in s.score("quality_model", np.zeros((1, 2, 2, 3), np.uint8))["unavailable"]
    s.score("quality_model", np.zeros((1, 2, 2, 3), np.uint8))
    assert calls["n"] == 1                                          # the failed load is remembered, not retried per case
    with pytest.raises(ValueError):
        s.register("mean_level", absent)
    with pytest.raises(KeyError):
        s.score("other", np.zeros((1, 2, 2, 3), np.uint8))


def _write(path, frames):
    import cv2

    path.parent.mkdir(parents=True, exist_ok=True)
    wr = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), 24.0, (frames.shape[2], frames.shape[1]))
    for f in frames:
        wr.write(cv2.cvtColor(f, cv2.COLOR_RGB2BGR))
    wr.release()


def test_benchmark_pass_is_resumable_and_summary_ranks_methods(tmp_path, capsys):
    import cv2

    from solarwm_b200.eval.run_metrics import compute, main, result_path, summarise
    from solarwm_b200.eval.benchmark import load_cases

    root = tmp_path / "bench"
    rows = []
    for i in range(2):
        clip = _scene(seed=i)
        _write(root / "media" / f"c{i}.mp4", clip)
        cv2.imwrite(str(root / "media" / f"f{i}.png"), clip[0])
        rows.append({"clip_id": f"clip{i}", "prompt": "p", "files": {"condition.mp4": f"media/c{i}.mp4", "first_frame.png": f"media/f{i}.png"},
                     "ground_truth": f"media/c{i}.mp4", "condition": "edges"})
        _write(tmp_path / "renders" / "good" / "heldout" / f"clip{i}.mp4", clip)
        _write(tmp_path / "renders" / "bad" / "heldout" / f"clip{i}.mp4", _scene(seed=i + 7, flicker=15.0))
    (root / "benchmark" / "heldout").mkdir(parents=True)
    (root / "benchmark" / "heldout" / "cases.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (tmp_path / "renders" / "bad" / "heldout" / "clip1.mp4").unlink()
    out = tmp_path / "scores"
    first = compute(root, tmp_path / "renders" / "good", "good", out, split="heldout")
    assert first == {"written": 8, "skipped": 0, "missing_renders": []}
    again = compute(root, tmp_path / "renders" / "good", "good", out, split="heldout")
    assert again["written"] == 0 and again["skipped"] == 8
    bad = compute(root, tmp_path / "renders" / "bad", "bad", out, split="heldout")
    assert bad["written"] == 4 and bad["missing_renders"] == ["heldout/clip1"]
    case0 = load_cases(root, "heldout")[0]
    assert json.loads(result_path(out, "gt", "good", case0).read_text())["ssim"] > 0.9
    s = summarise(out, ["good", "bad"], "heldout")
    assert [r["method"] for r in s["ranking"]] == ["good", "bad"] and s["readings"]["good"]["edge_f1"]["cases"] == 1     # common cases only
    assert s["readings"]["good"]["warp_l1_lp"]["mean"] < s["readings"]["bad"]["warp_l1_lp"]["mean"]
    assert main(["summary", "--out", str(out), "--methods", "good,bad", "--split", "heldout"]) == 0
    assert json.loads(capsys.readouterr().out)["ranking"][0]["method"] == "good"
    with pytest.raises(ValueError):
        compute(root, tmp_path / "renders" / "good", "good", out, metrics=("nonsense",))


def test_render_pass_is_resumable_and_survives_a_failing_case(tmp_path):
    import cv2

    from solarwm_b200.eval.render_benchmark import render_cases, write_video
    from solarwm_b200.eval.run_metrics import read_video

    root = tmp_path / "bench"
    rows = []
    for i in range(3):
        clip = _scene(seed=i)
        _write(root / "media" / f"c{i}.mp4", clip)
        cv2.imwrite(str(root / "media" / f"f{i}.png"), clip[0])
        rows.append({"clip_id": f"clip{i}", "prompt": "p", "files": {"condition.mp4": f"media/c{i}.mp4", "first_frame.png": f"media/f{i}.png"},
                     "ground_truth": f"media/c{i}.mp4", "condition": "edges"})
    (root / "benchmark" / "heldout").mkdir(parents=True)
    (root / "benchmark" / "heldout" / "cases.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    calls = []

    def method(case):
        calls.append(case.id)
        if case.id == "clip1":
            raise RuntimeError("out of memory")
        return read_video(case.condition)[:, ::-1].copy()           # a "render": the structure video upside down

    first = render_cases(root, tmp_path / "renders", method, split="heldout")
    assert first["rendered"] == ["heldout/clip0", "heldout/clip2"] and first["failed"][0]["case"] == "heldout/clip1"
    again = render_cases(root, tmp_path / "renders", method, split="heldout")
    assert again["skipped"] == ["heldout/clip0", "heldout/clip2"] and calls.count("clip0") == 1 and calls.count("clip1") == 2
    assert read_video(tmp_path / "renders" / "heldout" / "clip0.mp4").shape == (12, 64, 96, 3)
    log = [json.loads(l) for l in (tmp_path / "renders" / "render-log-0000.jsonl").read_text().splitlines()]
    assert sum("error" in e for e in log) == 2 and sum("seconds" in e for e in log) == 2
    assert not list((tmp_path / "renders").rglob("*.tmp.mp4"))
    with pytest.raises(ValueError):
        write_video(tmp_path / "x.mp4", np.zeros((2, 4, 4), np.uint8))
