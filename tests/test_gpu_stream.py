"""GPU checks of the streaming paths: H3 chunk evaluation under CUDA-graph replay equals eager, the ViT
decoder streams the same frames as its windowed oracle, teacher forcing matches the CPU fp32 model."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_h3_stream_graph_replay_equals_eager():
    from solarwm_b200 import ops
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.serve.h3_stream import H3StreamConfig, H3StreamingGenerator

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    g = torch.Generator().manual_seed(0)
    text, anchor = torch.randn(64, cfg.text_dim, generator=g), torch.randn(24, 1, 8, 16, generator=g)
    outs = {}
    for graph in (False, True):
        gen = H3StreamingGenerator(model, H3StreamConfig(grid_hw=(4, 8), chunk_latents=2, window_chunks=2,
                                                         denoise_steps=2, use_cuda_graph=graph, seed=3))
        gen.start(text, anchor, torch.eye(4))
        chunks = []
        for i in range(6):
            cams = torch.eye(4).repeat(2, 1, 1)
            cams[:, 0, 3] = 0.02 * i
            chunks.append(gen.next_chunk(cams).float().cpu())
        outs[graph] = chunks
        assert [t.graph for t in gen.timings] == [False, False] + [graph] * 4
    ops.check_status()
    for a, b in zip(outs[False], outs[True]):
        assert torch.isfinite(a).all() and torch.equal(a, b)


def test_vit_decoder_streaming_matches_window_oracle_on_gpu():
    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder

    cfg = ViTDecoderConfig(latent_channels=8, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256, registers=8, patch=2)
    m = ViTVideoDecoder(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    lat = torch.randn(9, 8, 8, 8, generator=torch.Generator().manual_seed(1)).cuda()
    dec = StreamingViTDecoder(m, (8, 8))
    outs = [dec.push(lat[i]) for i in range(9)]
    F = cfg.frames_per_latent
    w0 = m.decode_window(lat[0:7].permute(1, 0, 2, 3).unsqueeze(0))[0].float()
    w1 = m.decode_window(lat[5:9].permute(1, 0, 2, 3).unsqueeze(0))[0].float()
    for i, o in enumerate(outs):
        src, s = (w0, i) if i < 7 else (w1, i - 5)
        want = src[:, s * F:(s + 1) * F]
        want = want[:, -1:] if i % cfg.stride == 0 else want
        err = (o - want).abs().max() / want.abs().max().clamp_min(1e-6)
        assert err < 3e-2, (i, float(err))


def test_wan_teacher_forcing_matches_cpu_fp32():
    from solarwm_b200.models import wan_tf
    from solarwm_b200.models.wan import WanConfig, WanDiT

    cfg = WanConfig(model_type="ti2v", in_dim=16, out_dim=16, dim=256, ffn_dim=512, num_heads=2, num_layers=2,
                    text_dim=64, text_len=16, freq_dim=64)
    ref = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        ref.get_parameter("head.head.weight").normal_(0, 0.05)
    gpu = WanDiT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    gpu.load_state_dict({k: v for k, v in ref.state_dict().items()})
    g = torch.Generator().manual_seed(0)
    clean, noisy = torch.randn(1, 16, 4, 16, 16, generator=g), torch.randn(1, 16, 4, 16, 16, generator=g)
    t = torch.tensor([[800.0, 800.0, 250.0, 250.0]])
    ctx = torch.randn(1, 16, 64, generator=g)
    want = wan_tf.forward_teacher_forcing(ref, clean, noisy, t, ctx, chunk_frames=2, window_chunks=1)
    got = wan_tf.forward_teacher_forcing(gpu, clean.cuda(), noisy.cuda(), t.cuda(), ctx.cuda(), chunk_frames=2,
                                         window_chunks=1).float().cpu()
    assert ((got - want).norm() / want.norm()) < 3e-2
