"""Evaluation metrics and pairwise ratings."""
import torch

from solarwm_b200.eval import metrics, ratings


def test_metrics_identity_and_degradation():
    torch.manual_seed(0)
    truth = torch.rand(4, 3, 32, 32)
    assert metrics.ssim(truth, truth) > 0.999 and metrics.psnr(truth, truth) > 100
    noisy = (truth + 0.1 * torch.randn_like(truth)).clamp(0, 1)
    assert metrics.ssim(noisy, truth) < 0.95 and 15 < metrics.psnr(noisy, truth) < 25
    assert metrics.flicker(noisy, truth) > 0 and abs(metrics.flicker(truth, truth)) < 1e-9
    cond = torch.zeros(2, 3, 32, 32)
    cond[:, :, :, 16:] = 1.0                       # one vertical edge
    e_same = metrics.edge_errors(cond, cond)
    assert e_same == {"missed": 0.0, "extra": 0.0}
    shifted = torch.roll(cond, 1, dims=3)          # within tolerance
    assert metrics.edge_errors(shifted, cond)["missed"] < 0.2
    blank = torch.zeros_like(cond)
    assert metrics.edge_errors(blank, cond)["missed"] == 1.0


def test_pair_verdict_and_bradley_terry():
    assert ratings.pair_verdict("1", "2", "a", "b") == "a"      # a wins in both orders
    assert ratings.pair_verdict("1", "1", "a", "b") is None     # the answer followed the slot, not the content
    games = [("a", "b", "a")] * 8 + [("a", "b", "b")] * 2 + [("b", "c", "b")] * 7 + [("b", "c", None)] * 3 + \
            [("a", "c", "a")] * 9 + [("a", "c", "c")]
    r = ratings.fit_bradley_terry(games)
    assert r["a"] > r["b"] > r["c"] and abs(sum(r.values()) / 3 - 1000) < 1e-6
    wr = ratings.win_rates(games)
    assert wr["a"] > wr["b"] > wr["c"]


def test_benchmark_cases_judge_debiasing_and_intervals(tmp_path):
    import json

    from solarwm_b200.eval import benchmark as bm

    root = tmp_path / "data"
    (root / "benchmark" / "hard").mkdir(parents=True)
    (root / "benchmark" / "heldout").mkdir(parents=True)
    rows = []
    for seg in range(4):
        for look in range(3):
            cid = f"seg{seg}__look{look}"
            (root / f"{cid}.txt").write_text(f" prompt {cid} \n")
            rows.append({"case_id": cid, "files": {"prompt.txt": f"{cid}.txt", "condition.mp4": f"{cid}.c.mp4", "first_frame.png": f"{cid}.png"},
                         "tags": ["t"], "condition": "depth"})
    (root / "benchmark" / "hard" / "cases.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (root / "benchmark" / "heldout" / "cases.jsonl").write_text(json.dumps(
        {"clip_id": "clipA", "prompt": "p", "files": {"condition.mp4": "c.mp4", "first_frame.png": "f.png"}, "ground_truth": "gt.mp4"}))
    cases = bm.load_cases(root)
    assert len(cases) == 13 and cases[0].prompt == "prompt seg0__look0" and cases[-1].ground_truth.endswith("gt.mp4")
    assert len(bm.load_cases(root, "heldout")) == 1 and cases[0].key == "hard/seg0__look0"
    ra, rb = tmp_path / "ra", tmp_path / "rb"
    for c in cases[:12]:
        for r in (ra, rb):
            c.render(r).parent.mkdir(parents=True, exist_ok=True)
            c.render(r).write_bytes(b"x")

    def judge(case, pos_a, pos_b, questions):            # prefers method "ra" on quality; always says "A" on bias
        return {"quality": "A" if "/ra/" in pos_a else "B", "bias": "A", "half": "A" if "/ra/" in pos_a else "tie"}

    out = bm.judge_pairs(cases, ra, rb, judge, ["quality", "bias", "half"], a="ra", b="rb")
    assert len(out) == 12 and all(r["quality"] == "ra" and r["bias"] == "tie" and r["half"] == "ra" for r in out)
    net = bm.net_preference(out, "quality", "ra", "rb")
    assert net["net"] == 1.0 and net["lo"] == 1.0 and net["wins"] == 12
    assert bm.net_preference(out, "bias", "ra", "rb")["net"] == 0.0
    # grouped resampling is wider than independent resampling when a whole segment agrees
    xs = [1, 1, 1, -1, -1, -1, 1, 1, 1, -1, -1, -1]
    groups = [bm.structure_segment(r["case"]) for r in out]
    _, lo_g, hi_g = bm.bootstrap_ci(xs, groups)
    _, lo_i, hi_i = bm.bootstrap_ci(xs)
    assert hi_g - lo_g > hi_i - lo_i
    assert bm.debiased_verdict({"q": "A"}, {"q": "A"}, "q", "m1", "m2") == "tie"      # each order picked position A
