"""Block-causal execution on CPU: a chunked rollout against the KV cache equals one dense forward
with the block-causal mask, the window shift keeps the most recent frames, and the teacher-forcing
segment plan equals dense-mask attention."""
import torch

from solarwm_b200.models.wan import WanDiT, wan_preset
from solarwm_b200.models.wan_causal import (CausalWanRunner, allocate_kv_cache, teacher_forcing_attention,
                                            teacher_forcing_mask)
from solarwm_b200.ops import reference as R


def _model():
    m = WanDiT(wan_preset("tiny"), device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator().manual_seed(1))
    return m


def test_cached_chunks_equal_full_causal_recompute():
    m = _model()
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 16, 4, 8, 8, generator=g)
    ctx = torch.randn(1, 32, 256, generator=g)
    runner = CausalWanRunner(m)
    cache = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=2, window_frames=8, sink_frames=0)
    runner.encode_text(cache, ctx)
    t = torch.zeros(1, 2)
    first = runner.forward_chunk(cache, x[:, :, :2], t, commit=True)
    peek = runner.forward_chunk(cache, x[:, :, 2:], t + 500.0, commit=False)     # leaves the cache alone
    assert cache.committed_frames == 2
    second = runner.forward_chunk(cache, x[:, :, 2:], t + 500.0, commit=True)
    assert torch.equal(peek, second) and cache.committed_frames == 4
    # oracle: chunk 2 attends to [chunk 1 | chunk 2]; chunk 1 alone equals the bidirectional model on 2 frames
    alone = m(x[:, :, :2], t, ctx)
    assert torch.allclose(first, alone, atol=1e-4, rtol=1e-4)
    again = CausalWanRunner(m)
    cache2 = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=2, window_frames=8, sink_frames=0)
    again.encode_text(cache2, ctx)
    again.forward_chunk(cache2, x[:, :, :2], t, commit=True)
    assert torch.allclose(again.forward_chunk(cache2, x[:, :, 2:], t + 500.0, commit=True), second, atol=1e-5)


def test_window_shift_keeps_sink_and_recent_frames():
    m = _model()
    runner = CausalWanRunner(m)
    cache = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=1, window_frames=3, sink_frames=1)
    assert cache.window_frames == 2                  # window counts frames besides the sink
    runner.encode_text(cache, torch.randn(1, 32, 256))
    seen = []
    for i in range(5):
        x = torch.full((1, 16, 1, 8, 8), float(i + 1))
        runner.forward_chunk(cache, x, torch.zeros(1, 1), commit=True)
        seen.append(cache.layers[0].k[(min(i, 2)) * 16].clone())
    assert cache.committed_frames == 3 and cache.total_frames == 5
    k = cache.layers[0].k
    # slot 0 = sink (frame 0), slots 1..2 = the two most recent frames (3 and 4)
    runner2 = CausalWanRunner(m)
    c2 = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=1, window_frames=3, sink_frames=1)
    runner2.encode_text(c2, torch.randn(1, 32, 256))
    runner2.forward_chunk(c2, torch.full((1, 16, 1, 8, 8), 1.0), torch.zeros(1, 1), commit=True)
    assert torch.allclose(k[:16], c2.layers[0].k[:16])


def test_teacher_forcing_segments_equal_dense_mask():
    torch.manual_seed(0)
    F_, ft, cf, W, H, D = 6, 4, 2, 1, 2, 16
    L = F_ * ft
    mk = lambda: torch.randn(1, L, H, D)
    qc, kc, vc, qn, kn, vn = mk(), mk(), mk(), mk(), mk(), mk()
    oc, on = teacher_forcing_attention(qc, kc, vc, qn, kn, vn, frame_tokens=ft, chunk_frames=cf, window_chunks=W)
    mask = teacher_forcing_mask(F_, ft, cf, W)
    dense = R.attention(torch.cat([qc, qn], 1), torch.cat([kc, kn], 1), torch.cat([vc, vn], 1), mask=mask.view(1, 1, 2 * L, 2 * L))
    assert torch.allclose(torch.cat([oc, on], 1), dense, atol=1e-5)
    assert mask[L:, L:].sum() == F_ // cf * (cf * ft) ** 2           # noisy tokens see only their own noisy chunk


def test_streaming_generator_runs_on_cpu():
    from solarwm_b200.serve.streaming import StreamingConfig, StreamingGenerator

    m = _model()
    gen = StreamingGenerator(m, StreamingConfig(chunk_frames=1, window_frames=3, sink_frames=1, denoise_timesteps=(1000.0, 500.0)))
    gen.start(torch.randn(1, 32, 256), grid_hw=(4, 4))
    chunks = [gen.next_chunk() for _ in range(4)]
    assert all(c.shape == (1, 16, 1, 8, 8) and torch.isfinite(c).all() for c in chunks)
    assert gen.cache.total_frames == 4 and gen.cache.committed_frames == 3


def test_cache_runner_camera_prope_matches_bidirectional_first_chunk():
    import torch

    from solarwm_b200.models.wan import WanConfig, WanDiT
    from solarwm_b200.models.wan_causal import CausalWanRunner, allocate_kv_cache

    cfg = WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=256, ffn_dim=256, num_heads=2, num_layers=2, text_dim=32,
                    text_len=8, freq_dim=32)
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    g = torch.Generator().manual_seed(0)
    x, ctx = torch.randn(1, 4, 2, 4, 4, generator=g), torch.randn(1, 8, 32, generator=g)
    t = torch.tensor([[400.0, 400.0]])
    q, _ = torch.linalg.qr(torch.randn(2, 3, 3, generator=g))
    view = torch.eye(4).repeat(1, 2, 1, 1)
    view[0, :, :3, :3] = q
    view[0, :, :3, 3] = torch.randn(2, 3, generator=g) * 0.3
    Ks = torch.eye(3).repeat(1, 2, 1, 1)
    Ks[0, :, 0, 0], Ks[0, :, 1, 1] = 0.7, 1.1
    cam = {"viewmats": view, "Ks": Ks}
    want = m(x, t, ctx, y_camera=cam)
    runner = CausalWanRunner(m)
    cache = allocate_kv_cache(m, grid_hw=(2, 2), chunk_frames=2, window_frames=4, sink_frames=0)
    runner.encode_text(cache, ctx)
    got = runner.forward_chunk(cache, x, t, commit=True, y_camera=cam)
    assert torch.allclose(got, want, atol=1e-4)
    # a second chunk sees the first through its own cached camera; identity cameras reproduce the camera-free path
    plain_cache = allocate_kv_cache(m, grid_hw=(2, 2), chunk_frames=2, window_frames=4, sink_frames=0)
    runner.encode_text(plain_cache, ctx)
    runner.forward_chunk(plain_cache, x, t, commit=True)
    ident = {"viewmats": torch.eye(4).repeat(1, 2, 1, 1), "Ks": None}
    id_cache = allocate_kv_cache(m, grid_hw=(2, 2), chunk_frames=2, window_frames=4, sink_frames=0)
    runner.encode_text(id_cache, ctx)
    runner.forward_chunk(id_cache, x, t, commit=True, y_camera=ident)
    x2 = torch.randn(1, 4, 2, 4, 4, generator=g)
    a = runner.forward_chunk(plain_cache, x2, t, commit=False)
    b = runner.forward_chunk(id_cache, x2, t, commit=False, y_camera=ident)
    assert torch.allclose(a, b, atol=1e-4)
    c = runner.forward_chunk(cache, x2, t, commit=False, y_camera=cam)
    assert not torch.allclose(a, c, atol=1e-3)


def test_camera_length_rollout():
    import torch

    from solarwm_b200.models.wan import WanConfig, WanDiT
    from solarwm_b200.serve.streaming import StreamingConfig, camera_rollout

    cfg = WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=256, ffn_dim=256, num_heads=2, num_layers=1, text_dim=32,
                    text_len=8, freq_dim=32)
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    scfg = StreamingConfig(chunk_frames=2, window_frames=4, sink_frames=0, denoise_timesteps=(1000.0, 500.0), use_cuda_graphs=False, seed=3)
    view = torch.eye(4).repeat(1, 7, 1, 1)
    view[0, :, 0, 3] = torch.linspace(0, 0.6, 7)
    ctx = torch.randn(1, 8, 32)
    first = torch.randn(1, 4, 1, 4, 4)
    out = camera_rollout(m, ctx, (2, 2), view, None, cfg=scfg, first_frame=first)
    assert out.shape == (1, 4, 7, 4, 4) and torch.isfinite(out).all() and torch.equal(out[:, :, :1], first)
    still = camera_rollout(m, ctx, (2, 2), torch.eye(4).repeat(1, 7, 1, 1), None, cfg=scfg, first_frame=first)
    assert not torch.allclose(out[:, :, 3:], still[:, :, 3:], atol=1e-4)          # the camera path matters


def test_wan_codec_adapters_btchw_contract_and_streaming_chunks():
    import pytest
    import torch

    from solarwm_b200.backends.wan22.codec import Wan5BVAE, WanA14BVAE, WanVideoCodec, flow_to_x0
    from solarwm_b200.errors import BackendContractError
    from solarwm_b200.models.vae import VAEConfig, VideoVAE

    torch.manual_seed(0)
    codec = WanVideoCodec(VideoVAE(VAEConfig(z_dim=4, base=8, temporal_ups=(True, False)), [0.1] * 4, [2.0] * 4))
    video = torch.rand(1, 5, 3, 16, 16) * 2 - 1
    z = codec.encode(video)
    assert z.shape == (1, 3, 4, 4, 4)                                   # 1 + (5 - 1) / 2 latent frames, 4x spatial
    full = codec.decode(z)
    assert full.shape == (1, 5, 3, 16, 16) and full.abs().max() <= 1.0
    pieces = list(codec.decode_streaming_chunks(z, chunk_latent_frames=2))
    assert [p.shape[1] for p in pieces] == [3, 2] and all(p.device.type == "cpu" for p in pieces)
    assert torch.allclose(torch.cat(pieces, 1), full, atol=1e-5)
    with pytest.raises(BackendContractError):
        list(codec.decode_streaming_chunks(torch.cat([z, z]), chunk_latent_frames=2))
    with pytest.raises(BackendContractError):
        list(codec.decode_streaming_chunks(torch.full_like(z, float("nan"))))
    with pytest.raises(BackendContractError):
        codec.decode(z[:, :, :3])
    with pytest.raises(BackendContractError):
        Wan5BVAE.build([0.0] * 16, [1.0] * 16)
    a14 = WanA14BVAE.build(base=8)
    assert a14.vae.cfg.z_dim == 16 and abs(float(a14.vae.std.flatten()[0]) - 2.8184) < 1e-6
    x_t, v = torch.randn(2, 3, 4, dtype=torch.bfloat16), torch.randn(2, 3, 4, dtype=torch.bfloat16)
    x0 = flow_to_x0(x_t, v, torch.tensor([0.25, 0.5]))
    assert x0.dtype == torch.bfloat16
    assert torch.allclose(x0.float(), (x_t.double() - torch.tensor([0.25, 0.5]).view(2, 1, 1).double() * v.double()).float(), atol=2e-2)


def test_rotated_key_cache_equals_rope_at_read_over_a_long_rollout():
    """Keys cached after RoPE and re-based by one delta rotation per chunk give the same predictions as the original
    form (un-rotated keys, RoPE over the whole window at every read), through the fill phase, the sliding window with a
    sink, and -- with a larger position cap (block-relative RoPE) -- through the stretch where positions are still
    absolute and the point where they saturate."""
    m = _model()
    g = torch.Generator().manual_seed(3)
    ctx = torch.randn(1, 32, 256, generator=g)
    chunks = [torch.randn(1, 16, 2, 8, 8, generator=g) for _ in range(8)]
    for cap in (None, 11):
        outs = {}
        for at_read in (True, False):
            runner = CausalWanRunner(m, rope_at_read=at_read)
            cache = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=2, window_frames=6, sink_frames=2,
                                      position_cap=None if at_read else cap)
            runner.encode_text(cache, ctx)
            got = []
            for i, x in enumerate(chunks):
                t = torch.full((1, 2), 300.0 + 50 * i)
                got.append(runner.forward_chunk(cache, x, t, commit=False))      # a denoise step leaves the cache alone
                runner.forward_chunk(cache, x, torch.zeros(1, 2), commit=True)
            outs[at_read] = got
            assert cache.committed_frames == 6 and cache.total_frames == 16
        if cap is None:
            for a, b in zip(outs[True], outs[False]):
                assert torch.allclose(a, b, atol=2e-4, rtol=1e-4)
        else:
            # with the larger cap positions differ from the window-relative ones once the window slides, but stay equal
            # while nothing has been evicted (first three chunks) ...
            for a, b in zip(outs[True][:3], outs[False][:3]):
                assert torch.allclose(a, b, atol=2e-4, rtol=1e-4)
            # ... and the newest position ends clamped at cap - 1
            assert cache.newest_pos == 11 - 1 - 2 and cache.positions_saturated


def test_block_relative_positions_follow_the_rule():
    m = _model()
    cache = allocate_kv_cache(m, grid_hw=(4, 4), chunk_frames=3, window_frames=9, sink_frames=3, position_cap=21)
    first = []
    for _ in range(9):
        first.append(CausalWanRunner.chunk_first_position(cache, 3))
        cache.total_frames += 3
    # absolute positions until the newest frame would pass cap - 1 = 20, then clamped (top-aligned)
    assert first == [0, 3, 6, 9, 12, 15, 18, 18, 18]


def _camera_pair(g, frames):
    import torch

    q, _ = torch.linalg.qr(torch.randn(frames, 3, 3, generator=g))
    view = torch.eye(4).repeat(1, frames, 1, 1)
    view[0, :, :3, :3] = q
    view[0, :, :3, 3] = torch.randn(frames, 3, generator=g) * 0.3
    Ks = torch.eye(3).repeat(1, frames, 1, 1)
    Ks[0, :, 0, 0], Ks[0, :, 1, 1] = 0.7, 1.1
    return {"viewmats": view, "Ks": Ks}


def test_parallel_camera_branch_is_zero_at_init_matches_its_oracle_and_streams():
    """``camera_attention_mode = "parallel"``: a second self-attention per block that knows positions only through the
    cameras.  At initialisation it changes nothing; with a trained output projection its contribution is the plain
    formula (own projections, q/k RMS norm, P^T / P^-1 / P on every 4-vector, softmax attention); the cache runner,
    which keeps the branch's keys and values in a cache of their own, reproduces the full forward chunk by chunk."""
    import torch

    from solarwm_b200.models import camera_prope
    from solarwm_b200.models.wan import WanConfig, WanDiT
    from solarwm_b200.models.wan_causal import CausalWanRunner, allocate_kv_cache

    cfg = WanConfig(model_type="t2v", in_dim=4, out_dim=4, dim=32, ffn_dim=64, num_heads=2, num_layers=2, text_dim=32,
                    text_len=8, freq_dim=32, camera_attention_mode="parallel")
    m = WanDiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    names = {n for n, _ in m.named_parameters()}
    assert {"blocks.0.cam_self_attn.q_proj.weight", "blocks.1.cam_self_attn.out_proj.bias",
            "blocks.0.cam_self_attn.norm_k.weight"} <= names
    with torch.no_grad():
        m.get_parameter("head.head.weight").normal_(0, 0.05)
    g = torch.Generator().manual_seed(0)
    x, ctx = torch.randn(1, 4, 2, 4, 4, generator=g), torch.randn(1, 8, 32, generator=g)
    t = torch.tensor([[400.0, 400.0]])
    cam = _camera_pair(g, 2)
    assert float(m.get_parameter("blocks.0.cam_self_attn.out_proj.weight").detach().abs().max()) == 0.0
    assert torch.equal(m(x, t, ctx, y_camera=cam), m(x, t, ctx))                       # zero-initialised branch
    with torch.no_grad():
        for b in m.blocks:
            b._p("cam_self_attn.out_proj.weight").normal_(0, 0.2, generator=g)
            b._p("cam_self_attn.out_proj.bias").normal_(0, 0.1, generator=g)
    with_cam = m(x, t, ctx, y_camera=cam)
    assert not torch.allclose(with_cam, m(x, t, ctx), atol=1e-4)

    # the branch of one block against the formula
    blk, D, H = m.blocks[0], 32, 2
    xm = torch.randn(8, D, generator=g)                                    # 2 frames x 4 tokens
    mats = camera_prope.prope_matrices(cam["viewmats"][0], cam["Ks"][0], transform="linear")
    rows = tuple(camera_prope.per_row(mm, 4) for mm in mats)
    got = blk.camera_attention(xm, rows, B=1, sp=__import__("solarwm_b200.models.wan", fromlist=["_NoSP"])._NoSP())

    def lin(v, n):
        return v @ blk._p(f"cam_self_attn.{n}.weight").T + blk._p(f"cam_self_attn.{n}.bias")

    def rms(v, n):
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * blk._p(f"cam_self_attn.{n}.weight")

    def lift(v, mm):                                                        # every 4-vector of a row times its matrix
        return torch.einsum("rij,rnj->rni", mm, v.view(v.shape[0], -1, 4)).reshape(v.shape)

    q, k, v = lift(rms(lin(xm, "q_proj"), "norm_q"), rows[0]), lift(rms(lin(xm, "k_proj"), "norm_k"), rows[1]), \
        lift(lin(xm, "v_proj"), rows[1])
    hd = D // H
    att = torch.softmax(torch.einsum("qhd,khd->hqk", q.view(8, H, hd), k.view(8, H, hd)) / hd ** 0.5, -1)
    o = torch.einsum("hqk,khd->qhd", att, v.view(8, H, hd)).reshape(8, D)
    assert torch.allclose(got, lin(lift(o, rows[2]), "out_proj"), atol=1e-5)

    # chunked generation with the branch's own cache == the full forward (one chunk), and a second chunk attends the
    # first through cached camera-space keys
    runner = CausalWanRunner(m)
    cache = allocate_kv_cache(m, grid_hw=(2, 2), chunk_frames=2, window_frames=4, sink_frames=0)
    assert cache.layers[0].cam_k is not None and cache.layers[0].cam_k.shape == cache.layers[0].k.shape
    runner.encode_text(cache, ctx)
    assert torch.allclose(runner.forward_chunk(cache, x, t, commit=True, y_camera=cam), with_cam, atol=1e-4)
    x2, cam2 = torch.randn(1, 4, 2, 4, 4, generator=g), _camera_pair(g, 2)
    both = {"viewmats": torch.cat([cam["viewmats"], cam2["viewmats"]], 1), "Ks": torch.cat([cam["Ks"], cam2["Ks"]], 1)}
    second = runner.forward_chunk(cache, x2, t, commit=False, y_camera=cam2)
    # oracle: the 4-frame causal forward, second chunk's rows (chunk 1 attends chunk 0 and itself)
    from solarwm_b200.models.wan_tf import forward_window

    with torch.no_grad():
        want = forward_window(m, torch.cat([x, x2], 2), torch.cat([t, t], 1), ctx, first_frame=0, current_frames=2,
                              chunk_frames=2, window_chunks=4, y_camera=both)
    assert torch.allclose(second, want, atol=1e-4)
    assert torch.isfinite(second).all() and not torch.allclose(second, runner.forward_chunk(cache, x2, t, commit=False), atol=1e-4)
