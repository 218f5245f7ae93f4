"""Streaming ViT decoder: latent-by-latent equals the windowed oracle, window shift, tiles, compensation."""
import torch

from solarwm_b200.models.vit_decoder import (CompensationTable, StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder,
                                             blend_tiles, tile_plan)


def _model():
    return ViTVideoDecoder(ViTDecoderConfig.tiny(), device="cpu", dtype=torch.float32, seed=0)


def test_streaming_equals_window_oracle_across_a_shift():
    m = _model()
    c = m.cfg
    torch.manual_seed(0)
    lat = torch.randn(12, c.latent_channels, 3, 4)
    dec = StreamingViTDecoder(m, (3, 4))
    outs = [dec.push(lat[i]) for i in range(12)]
    assert [o.shape[1] for o in outs] == [1, 4, 4, 4, 4, 1, 4, 4, 4, 4, 1, 4]
    F = c.frames_per_latent
    w0 = m.decode_window(lat[0:7].permute(1, 0, 2, 3).unsqueeze(0))[0]             # [3, 7*F, H, W]
    for i in range(7):
        want = w0[:, i * F:(i + 1) * F]
        want = want[:, -1:] if i % c.stride == 0 else want
        assert torch.allclose(outs[i], want, atol=1e-5), i
    w1 = m.decode_window(lat[5:12].permute(1, 0, 2, 3).unsqueeze(0))[0]            # window that starts at latent 5
    for i in range(7, 12):
        s = i - 5
        want = w1[:, s * F:(s + 1) * F]
        want = want[:, -1:] if i % c.stride == 0 else want
        assert torch.allclose(outs[i], want, atol=1e-5), i


def test_tile_plan_blend_and_tiled_streaming():
    plan = tile_plan(6, 8, tile=4, overlap=2)
    assert (0, 0) in plan and (2, 4) in plan and all(y + 4 <= 6 and x + 4 <= 8 for y, x in plan)
    # blending a constant field gives the constant (weights sum to one)
    tiles = [torch.full((3, 2, 8, 8), 0.7) for _ in plan]
    out = blend_tiles(tiles, plan, 6, 8, 4, 2, patch=2)
    assert out.shape == (3, 2, 12, 16) and torch.allclose(out, torch.full_like(out, 0.7), atol=1e-6)
    m = _model()
    dec = StreamingViTDecoder(m, (6, 8), tile=4, overlap=2)
    x = dec.push(torch.randn(m.cfg.latent_channels, 6, 8))
    assert x.shape == (3, 1, 12, 16) and torch.isfinite(x).all()


def test_compensation_table():
    t = CompensationTable.zeros(7, 4)
    t.a[2, 1, :] = 0.1
    t.b[2, 0, :] = 0.5
    t.c[0, :, 3] = 2.0
    x = torch.ones(3, 4, 2, 2)
    y = t.apply(x, slot=2, first_of_stream=False)
    assert torch.allclose(y[0], torch.full((4, 2, 2), 0.5)) and torch.allclose(y[1], torch.full((4, 2, 2), 0.9))
    first = t.apply(torch.ones(3, 1, 2, 2), slot=0, first_of_stream=True)
    assert torch.allclose(first, torch.full((3, 1, 2, 2), -1.0))


def test_compensation_folds_into_the_pixel_affine():
    t = CompensationTable.zeros(7, 4)
    t.a[3] = torch.rand(3, 4) * 0.1
    t.b[3] = torch.rand(3, 4) * 0.2
    mean, std = torch.tensor([0.4, 0.5, 0.6]), torch.tensor([0.2, 0.25, 0.3])
    x = torch.randn(3, 4, 5, 6)
    want = t.apply(x, slot=3, first_of_stream=False) * std.view(3, 1, 1, 1) + mean.view(3, 1, 1, 1)
    for f in range(4):
        s2, m2 = t.folded_affine(3, f, mean, std)
        got = x[:, f] * s2.view(3, 1, 1) + m2.view(3, 1, 1)
        assert torch.allclose(got, want[:, f], atol=1e-6)
