"""Multi-GPU checks (skipped with fewer devices): the fused NVLink Ulysses path (forward AND backward exchanges
inside the kernels) against the NCCL collective path -- same forward output and the same parameter gradients, on 2
ranks and, where the box has them, on 4 / 8 ranks with 31 frames split unevenly --, the peer-memory runtime's
push / flag protocol including a bounded wait that is made to run out, the ZeRO-sharded AdamW with overlapped peer
reduce / single-launch push against its NCCL form, and the whole training step replayed as one CUDA graph against
the same step run eagerly."""
import os
from datetime import timedelta

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")


def _worker(rank, world, port, out_path):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=120),
                            device_id=torch.device("cuda", rank))
    from solarwm_b200 import ops
    from solarwm_b200.models.wan import WanConfig, WanDiT
    from solarwm_b200.parallel.fused_ulysses import FusedUlysses
    from solarwm_b200.parallel.symm import SymmetricHeap
    from solarwm_b200.parallel.ulysses import UlyssesCollective

    result = {}
    # ---- runtime: push + flags, then a wait nobody satisfies (bounded, reports a status)
    heap = SymmetricHeap(1 << 20, None)
    buf, off = heap.alloc((world, 1024), torch.float32)
    slot = heap.new_flag()
    src = torch.full((1024,), float(rank + 1), device="cuda")
    lib = heap.lib
    import ctypes

    rc = lib.solar_comm_push(ctypes.c_void_p(src.data_ptr()), heap.peer_ptr_array(off), ctypes.c_int(world),
                             ctypes.c_longlong(rank * 4096), ctypes.c_longlong(4096), heap.flag_ptrs(slot),
                             heap.counter_ptr(slot), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    heap.wait(slot)
    torch.cuda.synchronize()
    result["push_ok"] = bool(all(torch.all(buf[r] == r + 1).item() for r in range(world)))
    # the small all-sum kernel (used for the gradient norm): twice, so that both table parities are exercised
    allsum = heap.new_allsum(2)
    got = torch.zeros(2, device="cuda")
    for rnd in range(3):
        allsum(torch.tensor([float(rank + 1 + rnd), 1.0], device="cuda"), got)
        torch.cuda.synchronize()
        result[f"allsum_{rnd}"] = got.tolist() == [float(sum(r + 1 + rnd for r in range(world))), float(world)]
    heap.wait(slot, limit_seconds=0.3)       # no producer: must give up by itself
    torch.cuda.synchronize()
    from solarwm_b200.ops.functional import status_word

    result["raw_status"] = int(status_word(heap.device).item())
    result["raw_flag"] = int(heap._bytes[4 * slot:4 * slot + 4].view(torch.int32).item())
    try:
        ops.check_status(heap.device)
        result["timeout_reported"] = False
    except ops.NativeError as exc:
        result["timeout_reported"] = "code 5" in str(exc)
    dist.barrier()

    # ---- fused vs collective Ulysses on a small DiT
    cfg = WanConfig(model_type="t2v", in_dim=16, out_dim=16, dim=256, ffn_dim=512, num_heads=2, num_layers=2,
                    text_dim=128, text_len=64, freq_dim=64)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 16, 5, 16, 16, generator=g).cuda()
    ctx = torch.randn(1, 64, 128, generator=g).cuda()
    t = torch.tensor([[50.0, 300.0, 500.0, 700.0, 950.0]]).cuda()
    tgt = torch.randn(1, 16, 5, 16, 16, generator=g).cuda()
    outs = {}
    fused = FusedUlysses(None, max_tokens=5 * 64, dim=256, num_heads=2)
    for name, sp in (("nccl", UlyssesCollective(None)), ("fused", fused)):
        for mode in ("none", "selective"):
            model = WanDiT(cfg, device="cuda", dtype=torch.bfloat16, seed=3)
            with torch.no_grad():
                model.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator(device="cuda").manual_seed(1))
            model.sp = sp
            model.checkpointing = mode
            model.ensure_grads()
            ops.reset_counters()
            out = model(x, t, ctx)
            ((out.float() - tgt) ** 2).mean().backward()
            model.finalize_grads()
            sp.sum_gradients_([gr for u in model.units() for gr in (u.grad, u.grad_v)])
            torch.cuda.synchronize()
            ops.check_status()
            outs[(name, mode)] = (out.detach().float().cpu(),
                                  {n: p.main_grad.float().cpu() for n, p in model.named_parameters()},
                                  dict(ops.COUNTERS))
    with torch.no_grad():
        model.sp = fused
        outs["fused_infer"] = model(x, t, ctx).float().cpu()
    ref_out, ref_grads, _ = outs[("nccl", "none")]
    worst = 0.0
    for key in (("fused", "none"), ("fused", "selective"), ("nccl", "selective")):
        o, gr, counters = outs[key]
        result[f"out_{key[0]}_{key[1]}"] = ((o - ref_out).norm() / ref_out.norm()).item()
        for n, r in ref_grads.items():
            if r.norm() > 1e-6:
                worst = max(worst, ((gr[n] - r).norm() / r.norm()).item())
        if key[0] == "fused":
            result[f"fused_kernels_{key[1]}"] = (counters.get("gemm_scatter", 0), counters.get("attn_fwd_scatter", 0),
                                                 counters.get("attn_bwd_scatter", 0))
    result["worst_grad_rel"] = worst
    result["infer_rel"] = ((outs["fused_infer"] - ref_out).norm() / ref_out.norm()).item()
    # ---- ZeRO-sharded AdamW: fused peer reduce / push against the NCCL collectives
    from solarwm_b200.parallel.flat import FlatUnit
    from solarwm_b200.parallel.zero import ZeroAdamW

    specs = [("a.weight", (512, 256), False), ("a.bias", (512,), False), ("n.weight", (256,), True)]

    def make_unit():
        u = FlatUnit(specs, "cuda", dtype=torch.bfloat16, pad_to=world)
        for n, _, _ in specs:
            u.parameter(n)
        gg = torch.Generator(device="cuda").manual_seed(5)
        u.flat.copy_(torch.randn(u.numel_m, generator=gg, device="cuda") * 0.1)
        u.flat_v.copy_(torch.randn(u.numel_v, generator=gg, device="cuda"))
        u.ensure_grads()
        return u

    zheap = SymmetricHeap(8 << 20, None)
    u_c, u_f = make_unit(), make_unit()
    z_c = ZeroAdamW([u_c], None, transport="collective", lr=1e-2, weight_decay=0.1, ema_decay=0.9)
    z_f = ZeroAdamW([u_f], None, transport="fused", heap=zheap, lr=1e-2, weight_decay=0.1, ema_decay=0.9)
    norms = []
    for step in range(3):
        gg = torch.Generator(device="cuda").manual_seed(100 * step + rank)
        gm = torch.randn(u_c.numel_m, generator=gg, device="cuda")
        gv = torch.randn(u_c.numel_v, generator=gg, device="cuda")
        for u in (u_c, u_f):
            u.grad.copy_(gm)
            u.grad_v.copy_(gv)
            for prm in u.params.values():
                prm.grad_live = True                # written this step: finalize_grads must not clear them
        norms.append((float(z_c.sharded_step(1.0)), float(z_f.sharded_step(1.0))))
        torch.cuda.synchronize()
        dist.barrier()
    ops.check_status()
    result["zero_norms"] = norms
    result["zero_param_diff"] = float((u_c.flat.float() - u_f.flat.float()).abs().max())
    result["zero_vec_diff"] = float((u_c.flat_v - u_f.flat_v).abs().max())
    result["zero_ema_diff"] = float((z_c.state[0]["m"]["ema"] - z_f.state[0]["m"]["ema"]).abs().max())
    gathered = [torch.empty_like(u_f.flat) for _ in range(world)]
    dist.all_gather(gathered, u_f.flat)
    result["zero_ranks_agree"] = bool(all(torch.equal(gathered[0], t) for t in gathered))
    # ---- tile-parallel streaming decode: tiles dealt to the ranks, gathered on the device, blended on rank 0
    from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder

    vcfg = ViTDecoderConfig(latent_channels=8, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256, registers=8, patch=2)
    vit = ViTVideoDecoder(vcfg, device="cuda", dtype=torch.bfloat16, seed=0)
    lat = torch.randn(3, 8, 8, 16, generator=torch.Generator().manual_seed(1)).cuda()
    par = StreamingViTDecoder(vit, (8, 16), tile=8, overlap=4, distributed=True)       # three tiles over two ranks
    outs = [par.push(lat[i]) for i in range(3)]
    if rank == 0:
        one = StreamingViTDecoder(vit, (8, 16), tile=8, overlap=4)
        want = [one.push(lat[i]) for i in range(3)]
        result["tile_parallel_diff"] = max(float((a - b).abs().max()) for a, b in zip(outs, want))
    else:
        result["tile_parallel_diff"] = 0.0 if all(o is None for o in outs) else 1e9
    torch.save(result, f"{out_path}.{rank}")
    zheap.close()
    fused.close()
    heap.close()
    dist.destroy_process_group()


def test_fused_ulysses_matches_collective_on_two_gpus(tmp_path):
    _need_two()
    import torch.multiprocessing as mp

    out = str(tmp_path / "res")
    mp.spawn(_worker, args=(2, 29541, out), nprocs=2, join=True)
    for rank in range(2):
        r = torch.load(f"{out}.{rank}", weights_only=True)
        assert r["push_ok"] and r["timeout_reported"] and r["allsum_0"] and r["allsum_1"] and r["allsum_2"], r
        assert r["out_fused_none"] < 2e-2 and r["out_fused_selective"] < 2e-2 and r["out_nccl_selective"] < 1e-6, r
        assert r["infer_rel"] < 2e-2 and r["worst_grad_rel"] < 6e-2, r
        # per layer: forward QKV GEMM scatter + backward dO GEMM scatter; attention forward scatter; three backward kernels
        assert r["fused_kernels_none"] == (4, 2, 6) and r["fused_kernels_selective"] == (6, 2, 6), r
        assert r["zero_ranks_agree"] and r["zero_param_diff"] < 1e-2 and r["zero_vec_diff"] < 1e-5, r
        assert r["tile_parallel_diff"] < 1e-5, r
        assert r["zero_ema_diff"] < 1e-5 and all(abs(a - b) < 1e-3 * max(a, 1.0) for a, b in r["zero_norms"]), r


def _wide_worker(rank, world, port, out_path):
    """4 or 8 ranks, 31 latent frames (uneven whole-frame split), one head per rank: forward bit-identity and
    gradients of the fused exchanges against the NCCL path; then trainer steps eager against graph replay."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=180),
                            device_id=torch.device("cuda", rank))
    from solarwm_b200 import ops
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer
    from solarwm_b200.models.wan import WanConfig, WanDiT
    from solarwm_b200.parallel.fused_ulysses import FusedUlysses
    from solarwm_b200.parallel.symm import SymmetricHeap
    from solarwm_b200.parallel.ulysses import UlyssesCollective

    result = {}
    heads = world
    cfg = WanConfig(model_type="ti2v", in_dim=16, out_dim=16, dim=128 * heads, ffn_dim=512, num_heads=heads, num_layers=3,
                    text_dim=128, text_len=64, freq_dim=64)
    F, H, W = 31, 8, 12                                     # 24 tokens per frame, 744 tokens, frames split unevenly
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, 16, F, H, W, generator=g).cuda()
    ctx = torch.randn(1, 64, 128, generator=g).cuda()
    t = (torch.rand(1, F, generator=g) * 1000).cuda()
    tgt = torch.randn(1, 16, F, H, W, generator=g).cuda()
    tokens = F * (H // 2) * (W // 2)
    fused = FusedUlysses(None, max_tokens=tokens, dim=cfg.dim, num_heads=heads, max_frame_tokens=64)
    outs = {}
    for name, sp in (("nccl", UlyssesCollective(None)), ("fused", fused)):
        model = WanDiT(cfg, device="cuda", dtype=torch.bfloat16, seed=3)
        with torch.no_grad():
            model.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator(device="cuda").manual_seed(1))
        model.sp = sp
        model.ensure_grads()
        out = model(x, t, ctx)
        ((out.float() - tgt) ** 2).mean().backward()
        model.finalize_grads()
        UlyssesCollective.sum_gradients_(sp, [gr for u in model.units() for gr in (u.grad, u.grad_v)])
        torch.cuda.synchronize()
        ops.check_status()
        outs[name] = (out.detach().float().cpu(), {n: p.main_grad.float().cpu() for n, p in model.named_parameters()})
    result["forward_identical"] = bool(torch.equal(outs["nccl"][0], outs["fused"][0]))
    worst, worst_name = 0.0, ""
    # Every gradient is measured against its own norm, with a floor of a thousandth of the largest gradient; a key bias
    # (a column sum whose terms largely cancel) additionally against the gradient of the matching query bias.
    ref = outs["nccl"][1]
    floor = 1e-3 * max(float(r.norm()) for r in ref.values())
    for n, r in ref.items():
        scale = max(float(r.norm()), floor)
        if n.endswith(".k.bias"):
            scale = max(scale, float(ref[n[:-len("k.bias")] + "q.bias"].norm()))
        rel = float((outs["fused"][1][n] - r).norm()) / scale
        if rel > worst:
            worst, worst_name = rel, n
        top = sorted(result.get("grad_rel_top", []) + [(rel, n)], reverse=True)[:3]
        result["grad_rel_top"] = [(float(a), str(b)) for a, b in top]
    result["worst_grad_rel"], result["worst_grad_name"] = worst, worst_name
    fused.close()
    del model, outs
    # ---- trainer: fused transports, eager steps against the captured-graph replay of the same steps
    batch = {"latents": torch.randn(1, F, 16, H, W, generator=g).to(torch.bfloat16).pin_memory(),
             "text": torch.randn(1, 64, 128, generator=g).to(torch.bfloat16).pin_memory()}
    from solarwm_b200.parallel.zero import fused_heap_bytes

    runs = {}
    for mode in ("eager", "graph", "sharded", "sharded_graph"):
        sharded = mode.startswith("sharded")
        sp = FusedUlysses(None, max_tokens=tokens, dim=cfg.dim, num_heads=heads, max_frame_tokens=64)
        model = WanDiT(cfg, device="cuda", dtype=torch.bfloat16, seed=3, shard_pad=2 * world)
        with torch.no_grad():
            model.get_parameter("head.head.weight").normal_(0, 0.05, generator=torch.Generator(device="cuda").manual_seed(1))
        heap = SymmetricHeap(fused_heap_bytes(model.units(), world, [b.unit for b in model.blocks] if sharded else ()), None)
        opts = Stage0p5Options(lr=1e-3, seed=0, zero=True, zero_transport="fused", cuda_graph=mode.endswith("graph"),
                               graph_warmup_steps=1, max_grad_norm=1.0, shard_params=sharded)
        tr = WanStage0p5Trainer(cfg, "cuda", opts, sp=sp, model=model, heap=heap)
        ops.reset_counters()
        losses = []
        for _ in range(5):
            losses.append(float(tr.train_step(batch).item()))
        torch.cuda.synchronize()
        ops.check_status()
        if sharded:
            weights = model.param_provider.materialize(model)
            probe = weights["blocks.1.ffn.0.weight"].float()
            full = {n: v for n, v in weights.items()}
            # round trip: the full mapping loads back into the shards and gathers to the same values
            model.param_provider.load_state(model, full)
            again = model.param_provider.materialize(model)["blocks.2.self_attn.q.weight"].float()
            result[f"{mode}_roundtrip"] = bool(torch.equal(again, weights["blocks.2.self_attn.q.weight"].float()))
        else:
            probe = model.get_parameter("blocks.1.ffn.0.weight").detach().float().cpu().clone()
        runs[mode] = (losses, probe, float(tr.last_grad_norm.item()), ops.total_launches(),
                      ops.COUNTERS.get("param_gather", 0))
        dist.barrier()
        sp.close()
        heap.close()
        del tr, model
    result["losses"] = {m: r[0] for m, r in runs.items()}
    result["param_diff"] = {m: float((runs["eager"][1] - r[1]).abs().max()) for m, r in runs.items()}
    result["norms"] = {m: r[2] for m, r in runs.items()}
    result["launches"] = {m: r[3] for m, r in runs.items()}
    result["gathers"] = {m: r[4] for m, r in runs.items()}
    torch.save(result, f"{out_path}.{rank}")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchanges_uneven_frames_and_graph_replay(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    import torch.multiprocessing as mp

    out = str(tmp_path / "wide")
    mp.spawn(_wide_worker, args=(world, 29560 + world, out), nprocs=world, join=True)
    for rank in range(world):
        r = torch.load(f"{out}.{rank}", weights_only=True)
        assert r["forward_identical"], r
        # Both transports round the upstream gradients to bf16 in a different summation order.  The bias of the (normed)
        # cross-attention keys is a column sum over 64 text rows whose terms largely cancel, so it amplifies that rounding:
        # with eight ranks (93 tokens each) it differs by 1.9-2.0 % (deterministic, measured twice), every other parameter
        # by less than 1 %; worlds 2 and 4 stay under 1 % throughout.
        assert r["worst_grad_rel"] < (1e-2 if world <= 4 else 3e-2), r
        le = r["losses"]["eager"]
        for mode in ("graph", "sharded", "sharded_graph"):
            assert all(abs(a - b) <= 1e-3 * max(abs(a), 1.0) for a, b in zip(le, r["losses"][mode])), (mode, r)
            assert r["param_diff"][mode] < 1e-2, (mode, r)
        assert le[-1] < le[0], r
        assert r["launches"]["eager"] == r["launches"]["graph"] > 0, r
        assert r["launches"]["sharded"] == r["launches"]["sharded_graph"] > r["launches"]["eager"], r
        # 3 blocks, 5 steps: every block is gathered once in forward; backward re-uses the two resident blocks and
        # fetches the third again; the two whole-model reads of the check above gather every block once each
        assert r["gathers"]["eager"] == 0 and r["gathers"]["sharded"] == 5 * 4 + 2 * 3, r
        assert r["sharded_roundtrip"] and r["sharded_graph_roundtrip"], r


def _stream_worker(rank, world, port, out_path):
    """Block-causal streaming at SP = world: the fused head exchange (k / v appended straight into the peers' KV
    caches, graph replay once the window is full) against the NCCL all-to-all form of the same generator."""
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, timeout=timedelta(seconds=180),
                            device_id=torch.device("cuda", rank))
    from solarwm_b200 import ops
    from solarwm_b200.models.h3 import H3Config, H3DiT
    from solarwm_b200.parallel.ulysses import UlyssesCollective
    from solarwm_b200.serve.h3_stream import H3StreamConfig, H3StreamingGenerator

    cfg = H3Config(num_attention_heads=2 * world, attention_head_dim=128, hidden_size=256, num_layers=2, num_refiner_layers=1,
                   ffn_dim=512, text_dim=64, time_embed_hidden_dim=64, time_embed_dim=128)
    model = H3DiT(cfg, device="cuda", dtype=torch.bfloat16, seed=0)
    g = torch.Generator().manual_seed(0)
    text, anchor = torch.randn(40, cfg.text_dim, generator=g), torch.randn(24, 1, 8, 12, generator=g)
    result, outs = {}, {}
    for mode in ("collective", "fused"):
        scfg = H3StreamConfig(grid_hw=(4, 6), chunk_latents=2, window_chunks=2, denoise_steps=2, sp_exchange=mode,
                              max_text_tokens=64, use_cuda_graph=mode == "fused", seed=5)
        gen = H3StreamingGenerator(model, scfg, sp=UlyssesCollective(None))
        gen.start(text, anchor, torch.eye(4))
        ops.reset_counters()
        chunks = []
        for i in range(5):
            cams = torch.eye(4).repeat(2, 1, 1)
            cams[:, 0, 3] = 0.02 * i
            chunks.append(gen.next_chunk(cams).float().cpu())
        torch.cuda.synchronize()
        ops.check_status()
        outs[mode] = chunks
        result[f"{mode}_graph"] = [t.graph for t in gen.timings]
        result[f"{mode}_scatter"] = ops.COUNTERS.get("scatter_cols", 0)
        dist.barrier()
        if gen.fx is not None:
            gen.fx.close()
    result["max_rel"] = max(((a - b).norm() / b.norm()).item() for a, b in zip(outs["fused"], outs["collective"]))
    result["finite"] = bool(all(torch.isfinite(c).all() for c in outs["fused"]))
    torch.save(result, f"{out_path}.{rank}")
    dist.destroy_process_group()


def test_fused_stream_exchange_matches_collective_and_replays_as_a_graph(tmp_path):
    _need_two()
    import torch.multiprocessing as mp

    out = str(tmp_path / "stream")
    mp.spawn(_stream_worker, args=(2, 29577, out), nprocs=2, join=True)
    for rank in range(2):
        r = torch.load(f"{out}.{rank}", weights_only=True)
        assert r["finite"] and r["max_rel"] < 2e-2, r
        assert r["fused_graph"] == [False, False, True, True, True] and not any(r["collective_graph"]), r
        assert r["fused_scatter"] > 0 and r["collective_scatter"] == 0, r
