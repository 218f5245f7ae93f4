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
