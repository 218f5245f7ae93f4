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


def test_vit_qkv_kernel_matches_unfused_composition():
    from solarwm_b200.models.vit_decoder import _head_rms, apply_rope
    from solarwm_b200.ops import functional as F_

    g = torch.Generator().manual_seed(0)
    for heads, dh in ((2, 64), (3, 128), (2, 32)):
        B, N, rows, lo = 3, 37, 100, 11
        a = heads * dh
        qkv = torch.randn(B, N, 3 * a, generator=g).cuda().bfloat16()
        qw, kw = (torch.rand(dh, generator=g) + 0.5).cuda(), (torch.rand(dh, generator=g) + 0.5).cuda()
        ang = torch.rand(N, dh, generator=g) * 6.0
        cos, sin = torch.cos(ang).cuda(), torch.sin(ang).cuda()
        for use_rope in (True, False):
            kc = torch.zeros(B, rows, a, device="cuda", dtype=torch.bfloat16)
            vc = torch.zeros_like(kc)
            q = F_.vit_qkv_to_cache(qkv, qw, kw, cos if use_rope else None, sin if use_rope else None, kc, vc, lo,
                                    heads=heads, eps=1e-6)
            q_ref = _head_rms(qkv[..., :a], qw, heads, 1e-6)
            k_ref = _head_rms(qkv[..., a:2 * a], kw, heads, 1e-6)
            if use_rope:
                q_ref, k_ref = apply_rope(q_ref, cos, sin, heads), apply_rope(k_ref, cos, sin, heads)
            assert (q.float() - q_ref.float()).abs().max() < 4e-2
            assert (kc[:, lo:lo + N].float() - k_ref.float()).abs().max() < 4e-2
            assert torch.equal(vc[:, lo:lo + N], qkv[..., 2 * a:])
            assert kc[:, :lo].abs().sum() == 0 and kc[:, lo + N:].abs().sum() == 0 and vc[:, lo + N:].abs().sum() == 0


def test_tile_blend_kernel_matches_reference_blend_and_compensation():
    from solarwm_b200.models.vit_decoder import CompensationTable, blend_tiles, tile_plan
    from solarwm_b200.ops import functional as F_

    g = torch.Generator().manual_seed(0)
    h, w, tile, overlap, patch, F = 6, 10, 4, 2, 4, 4
    plan = tile_plan(h, w, tile, overlap)
    tiles = torch.randn(len(plan), 3, F, tile * patch, tile * patch, generator=g).cuda().bfloat16()
    table = CompensationTable(torch.randn(7, 3, F, generator=g) * 0.1, torch.randn(7, 3, F, generator=g) * 0.1,
                              torch.randn(7, 3, F, generator=g) * 0.1)
    offs = [(y * patch, x * patch) for (y, x) in plan]
    for n_frames, first in ((F, False), (1, True), (F, True)):
        t = tiles[:, :, -n_frames:]
        want = blend_tiles([t[j] for j in range(t.shape[0])], plan, h, w, tile, overlap, patch)
        plain = F_.tile_blend(t, offs, h * patch, w * patch, overlap * patch, None)
        assert (plain - want).abs().max() < 1e-5
        got = F_.tile_blend(t, offs, h * patch, w * patch, overlap * patch, table.coefficients(3, n_frames, first))
        assert (got - table.apply(want, 3, first)).abs().max() < 1e-5


def test_vit_decoder_tiled_streaming_runs_fused_kernels():
    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
    from solarwm_b200.ops import _lib

    cfg = ViTDecoderConfig(latent_channels=8, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256, registers=8, patch=2)
    m = ViTVideoDecoder(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    lat = torch.randn(3, 8, 8, 12, generator=torch.Generator().manual_seed(1)).cuda()
    dec = StreamingViTDecoder(m, (8, 12), tile=8, overlap=4)
    before = dict(_lib.COUNTERS)
    outs = [dec.push(lat[i]) for i in range(3)]
    after = _lib.COUNTERS
    assert after.get("tile_blend", 0) - before.get("tile_blend", 0) == 3
    assert after.get("vit_qkv", 0) > before.get("vit_qkv", 0)
    assert outs[0].shape == (3, 1, 16, 24) and outs[1].shape == (3, cfg.frames_per_latent, 16, 24)
    assert all(torch.isfinite(o).all() for o in outs)


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


def test_causal_renderer_stream_equals_training_document_on_the_device():
    """The chunk stream and the one-pass training document agree on a GPU too (bf16, this package's attention kernels
    over concatenated key spans of uneven lengths), and both stay close to the CPU fp32 model."""
    from solarwm_b200 import ops
    from solarwm_b200.backends.minimax_h3.layout import patchify_latents
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.renderer.causal import CLEAN_LEVEL, CausalRenderer, ChunkKVCache, chunk_spans, teacher_forcing_prediction
    from solarwm_b200.renderer.cli import _sample

    cfg = h3_preset("tiny")
    gpu = H3DiT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    cpu = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    gpu.load_state_dict({k: v for k, v in cpu.state_dict().items()})       # the seeded initialisation depends on the device
    s = _sample(cfg, 3, frames=6, size=8)
    C, F, H, W = s["shape"]
    per = (H // 2) * (W // 2)
    g = torch.Generator().manual_seed(9)
    noisy = torch.randn(F * per, C * 4, generator=g)
    t_chunks = torch.tensor([0.3, 0.5, 0.7])
    before = ops.total_launches()
    with torch.no_grad():
        doc = teacher_forcing_prediction(gpu, s, noisy.cuda(), t_chunks, chunk=2, window=2).float().cpu()
        ref = teacher_forcing_prediction(cpu, s, noisy, t_chunks, chunk=2, window=2)
        r, cache = CausalRenderer(gpu, chunk=2, window=2, steps=2), ChunkKVCache(2)
        prompt, anchor_rows = s["prompt_embeds"].cuda().bfloat16(), patchify_latents(s["anchor_latents"]).cuda().bfloat16()
        s_rows, clean = patchify_latents(s["structure_latents"]).cuda().bfloat16(), patchify_latents(s["target_latents"]).cuda().bfloat16()
        parts = []
        for j, (a, b) in enumerate(chunk_spans(F, 2)):
            kw = dict(prompt=prompt, anchor_rows=anchor_rows, structure_rows=s_rows[a * per:b * per], frames=(a, b), total_frames=F,
                      grid_hw=(H // 2, W // 2), cameras=s["camera_w2c"])
            parts.append(r._evaluate(cache, target_rows=noisy[a * per:b * per].cuda().bfloat16(), t=float(t_chunks[j]), commit=False, **kw).float().cpu())
            r._evaluate(cache, target_rows=clean[a * per:b * per], t=CLEAN_LEVEL, commit=True, **kw)
        stream = torch.cat(parts)
        out = r.render(s, seed=1)
    ops.check_status()
    assert ops.total_launches() > before                              # the native kernels ran
    scale = float(ref.abs().max())
    assert float((stream - doc).abs().max()) < 4e-2 * scale           # same function, bf16 rounding apart
    assert float((doc - ref).abs().max()) < 8e-2 * scale
    assert out.shape == (C, F, H, W) and bool(torch.isfinite(out.float()).all())


def test_memory_session_engine_on_the_device(tmp_path):
    from solarwm_b200 import ops
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.serve.h3_stream import H3StreamConfig
    from solarwm_b200.serve.memory_engine import MemorySessionEngine

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    scfg = H3StreamConfig(grid_hw=(4, 8), chunk_latents=5, window_chunks=2, denoise_steps=2, use_cuda_graph=False, memory_latents=2)
    eng = MemorySessionEngine(model, scfg, run_dir=tmp_path, top_k=2)
    eng.set_condition(text=torch.randn(16, cfg.text_dim), anchor_latent=torch.randn(24, 1, 8, 16), scene_id="gpu-scene")
    eng.start(seed=3)
    for j in range(5):
        eng.advance_camera([["w"] if j < 3 else ["s"]] * (4 if j == 0 else 5))
        chunk, ms = eng.generate()
        assert chunk.is_cuda and chunk.shape == (24, 5, 8, 16) and bool(torch.isfinite(chunk.float()).all())
    assert [len(r["memory_latent_indices"]) for r in eng.records] == [0, 0, 0, 2, 2]
    assert eng.stop()["chunks"] == 5
    ops.check_status()
