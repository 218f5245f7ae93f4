"""H3 streaming generator: cache bookkeeping, window sliding by delta rotation, camera matrices (CPU)."""
import pytest
import torch

from solarwm_b200.models.h3 import H3DiT, h3_preset, mm_rope_tables, prope_row_matrices
from solarwm_b200.ops import reference as R
from solarwm_b200.serve.h3_stream import H3StreamConfig, H3StreamingGenerator


def _gen(window=2):
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=2, window_chunks=window, denoise_steps=2, use_cuda_graph=False)
    g = H3StreamingGenerator(model, scfg)
    torch.manual_seed(0)
    g.start(torch.randn(6, cfg.text_dim), torch.randn(24, 1, 4, 6), torch.eye(4))
    return g, cfg


def test_delta_rotation_rebases_keys():
    pos = torch.zeros(5, 3, dtype=torch.float64)
    pos[:, 0] = torch.tensor([20.0, 21.5, 30.0, 31.0, 40.0])
    pos[:, 1:] = torch.rand(5, 2, dtype=torch.float64) * 30
    x = torch.randn(5, 2 * 128)
    cos, sin = mm_rope_tables(pos)
    k = R.head_norm_rope_prope(x, None, cos, sin, None, heads=2)
    delta = torch.zeros(5, 3, dtype=torch.float64)
    delta[:, 0] = -7.25
    dc, ds = mm_rope_tables(delta)
    moved = R.head_norm_rope_prope(k, None, dc, ds, None, heads=2)
    pos2 = pos.clone()
    pos2[:, 0] -= 7.25
    c2, s2 = mm_rope_tables(pos2)
    direct = R.head_norm_rope_prope(x, None, c2, s2, None, heads=2)
    assert torch.allclose(moved, direct, atol=1e-4)


def test_closed_form_camera_matrices_match_inverse():
    g, _ = _gen()
    q, _ = torch.linalg.qr(torch.randn(3, 3, 3))
    view = torch.eye(4).repeat(3, 1, 1)
    view[:, :3, :3] = q
    view[:, :3, 3] = torch.randn(3, 3) * 0.1
    a = g._camera_mats(view)
    b = prope_row_matrices(view, g.cfg.fx, g.cfg.fy)
    for x, y in zip(a, b):
        assert torch.allclose(x, y, atol=1e-5)


def test_streaming_rollout_window_and_shapes():
    g, cfg = _gen(window=2)
    n_cond = g.n_cond
    outs = []
    for i in range(4):
        cams = torch.eye(4).repeat(2, 1, 1)
        cams[:, 0, 3] = 0.05 * i
        out = g.next_chunk(cams)
        assert out.shape == (24, 2, 4, 6) and torch.isfinite(out).all()
        outs.append(out)
        assert g.hist_chunks == min(i + 1, 2)
    assert g.chunk_index == 4 and len(g.timings) == 4
    # the condition rows' keys are never touched by sliding
    k0 = g.kv[0].k[:n_cond].clone()
    g.next_chunk(None)
    assert torch.equal(k0, g.kv[0].k[:n_cond])
    assert not torch.equal(outs[0], outs[1])


def test_same_seed_same_stream():
    a, _ = _gen()
    b, _ = _gen()
    for _ in range(3):
        assert torch.equal(a.next_chunk(None), b.next_chunk(None))


def test_memory_rows_change_the_stream_and_can_be_cleared():
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)

    def run(mem):
        scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=2, window_chunks=2, denoise_steps=2, use_cuda_graph=False,
                              memory_latents=3)
        g = H3StreamingGenerator(model, scfg)
        torch.manual_seed(0)
        g.start(torch.randn(6, cfg.text_dim), torch.randn(24, 1, 4, 6), torch.eye(4))
        first = g.next_chunk(None)
        if mem == "set":
            g.set_memory(torch.randn(24, 2, 4, 6, generator=torch.Generator().manual_seed(9)), torch.eye(4).repeat(2, 1, 1))
        elif mem == "set-clear":
            g.set_memory(torch.randn(24, 2, 4, 6, generator=torch.Generator().manual_seed(9)), None)
            g.set_memory(None)
        return first, g.next_chunk(None), g

    f0, plain, _ = run("none")
    f1, with_mem, g = run("set")
    f2, cleared, _ = run("set-clear")
    assert torch.equal(f0, f1) and torch.equal(f0, f2)
    assert g.mem_rows == 2 * 6 and not torch.allclose(plain, with_mem)
    assert torch.equal(plain, cleared)


def test_full_length_generation_with_memory_and_streaming_decode(tmp_path):
    import json

    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
    from solarwm_b200.serve.h3_full_inference import generate_full_length

    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    vcfg = ViTDecoderConfig(latent_channels=24, dim=64, depth=1, heads=2, dim_head=32, ffn_dim=128, registers=2, patch=2)
    dec = StreamingViTDecoder(ViTVideoDecoder(vcfg, device="cpu", dtype=torch.float32), (4, 6))
    n_chunks, k = 8, 2
    c2w = torch.eye(4).repeat(1 + n_chunks * k, 1, 1)
    xs = torch.cat([torch.linspace(0, 12, 9), torch.linspace(12, 0, 8)])          # walk away and come back
    c2w[:, 0, 3] = xs
    K = torch.tensor([[0.5, 0, 0.5], [0, 0.9, 0.5], [0, 0, 1.0]]).repeat(1 + n_chunks * k, 1, 1)
    frames = []
    scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=k, window_chunks=2, denoise_steps=1, use_cuda_graph=False,
                          memory_latents=2)
    torch.manual_seed(0)
    man = generate_full_length(model, text=torch.randn(6, cfg.text_dim), anchor_latent=torch.randn(24, 1, 4, 6), c2w=c2w,
                               intrinsics=K, stream_cfg=scfg, decoder=dec, frame_sink=frames.append, use_memory=True,
                               top_k=2, out_dir=tmp_path)
    assert man["chunks"] == n_chunks and man["frames"] == sum(f.shape[1] for f in frames) > 0
    assert all(torch.isfinite(f).all() for f in frames) and frames[0].shape[-2:] == (8, 12)
    assert man["memory"]["retrieved"][0] == [] and len(man["memory"]["retrieved"][-1]) == 2
    assert json.loads((tmp_path / "manifest.json").read_text())["latents"] == n_chunks * k


def test_memory_adapter_bank_is_active_only_while_memory_rows_are_installed():
    cfg = h3_preset("tiny")
    model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
    model.add_adapter("memory", rank=4, seed=3)
    with torch.no_grad():                       # a zero B would make the bank a no-op
        for n, p in model.named_parameters():
            if n.endswith("lora_B__memory"):
                p.normal_(0, 0.05, generator=torch.Generator().manual_seed(p.numel()))
    assert len(model.adapter_state("memory")) == 2 * sum(1 for _ in model.modules() if type(_).__name__ == "LoRALinear")
    mem = torch.randn(24, 2, 4, 6, generator=torch.Generator().manual_seed(9))

    def run(adapter):
        scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=2, window_chunks=2, denoise_steps=2, use_cuda_graph=False,
                              memory_latents=3, memory_adapter=adapter)
        g = H3StreamingGenerator(model, scfg)
        torch.manual_seed(0)
        g.start(torch.randn(6, cfg.text_dim), torch.randn(24, 1, 4, 6), torch.eye(4))
        first = g.next_chunk(None)
        g.set_memory(mem, None)
        active = getattr(model, "active_adapter", None)
        second = g.next_chunk(None)
        g.set_memory(None)
        third = g.next_chunk(None)
        return first, second, third, active, getattr(model, "active_adapter", None)

    a = run(None)
    b = run("memory")
    assert a[3] is None and b[3] == "memory" and b[4] is None           # switched on with the rows, off with them
    assert torch.equal(a[0], b[0])                                        # before any memory: the same stream
    assert not torch.allclose(a[1], b[1])                                 # memory rows served by the Memory adapter
    with pytest.raises(KeyError):
        model.set_adapter("nope")


def test_fused_qkv_projection_changes_nothing_and_yields_to_adapter_banks():
    """``fuse_qkv``: the three projection weights of a block become views of one buffer and the generator issues one
    GEMM; the stream is the same as with three GEMMs, the per-projection modules still work, and a block whose adapter
    bank is switched on goes back to them."""
    cfg = h3_preset("tiny")
    outs = {}
    for fuse in (False, True):
        model = H3DiT(cfg, device="cpu", dtype=torch.float32, seed=0)
        scfg = H3StreamConfig(grid_hw=(2, 3), chunk_latents=2, window_chunks=2, denoise_steps=2, use_cuda_graph=False, fuse_qkv=fuse)
        g = H3StreamingGenerator(model, scfg)
        torch.manual_seed(0)
        g.start(torch.randn(6, cfg.text_dim), torch.randn(24, 1, 4, 6), torch.eye(4))
        outs[fuse] = torch.stack([g.next_chunk(None) for _ in range(3)])
        blk = model.blocks[0]
        if fuse:
            a = blk.to_q.weight.shape[0]
            assert blk.qkv_weight.shape[0] == 3 * a and blk.to_k.weight.data_ptr() == blk.qkv_weight[a:].data_ptr()
            x = torch.randn(5, cfg.hidden_size)
            assert torch.allclose(blk.to_v(x), x @ blk.qkv_weight[2 * a:].t(), atol=1e-5)
            assert model.fuse_qkv_() == 0                                  # nothing left to fuse
        else:
            assert getattr(blk, "qkv_weight", None) is None
    assert torch.allclose(outs[True], outs[False], atol=1e-5)
    lora = H3DiT(h3_preset("tiny").__class__(**{**h3_preset("tiny").__dict__, "lora_rank": 2}), device="cpu", dtype=torch.float32, seed=0)
    assert lora.fuse_qkv_() == 0                                           # trainable adapters: left alone
