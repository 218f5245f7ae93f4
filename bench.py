"""Headline benchmark: Wan2.2 TI2V-5B-shaped DiT flow-matching training, tokens/s per box.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...      # the unmodified reference installed in baseline/_ref

Config (the headline benchmark shape): 30 blocks, dim 3072, 24 heads, FFN 14336, 48 latent channels, patch
1x2x2; one sample of latent [1,48,31,44,80] (27,280 tokens), text embedding [1,512,4096], bf16,
logit-normal sigmas with shift 5; Ulysses SP = N over the N GPUs (the one sample is split, so
scaling is strong), gradients summed over the SP group, AdamW update inside the timed region.
Synthetic data, random-init weights.

Two timed regions, each of exactly K steps bracketed by barrier + synchronize and timed with
CUDA events (max over ranks): (1) device-resident inputs -> ``value``; (2) end to end through
``WanStage0p5Trainer.train_step`` with the host->device copy of the step's inputs from pinned
memory and a device->host read of the loss every step -> ``e2e``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
BASELINE_TOKENS_PER_S = None  # the reference publishes no tokens/s figure


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "baseline"],
                    help="reference: the unmodified reference package (Wan 5B shape only); baseline: THIS model code on "
                         "library kernels -- cuBLAS GEMMs, cuDNN SDPA attention, NCCL all-to-all / reduce-scatter / "
                         "all-gather, eager -- the NCCL+library arm for shapes the reference cannot run offline")
    ap.add_argument("--model", default="ti2v_5b", choices=["ti2v_5b", "ltx_2b", "small", "i2v_a14b", "i2v_small"],
                    help="ltx_2b: LTX-Video-2B shape (its 6,144-token clip [128,16,16,24] is the default geometry); "
                         "i2v_a14b: Wan2.2 A14B-shaped TWO-expert training (high- / low-noise experts switched at sigma "
                         "0.875, 75,600-token clip [16,21,90,160] + I2V conditioning; needs 8 GPUs); i2v_small: the same "
                         "program on a small architecture")
    ap.add_argument("--mode", default="train", choices=["train", "realtime", "infer"],
                    help="train: the headline training step; realtime: H3-shaped block-causal streaming (FPS); infer: "
                         "8-step flow-matching sampling of one clip (seconds per sample; BASELINE config 4 with "
                         "--model ltx_2b)")
    ap.add_argument("--sample-steps", type=int, default=8, help="infer mode: solver steps per sample")
    ap.add_argument("--h3", default="h3_33b", choices=["h3_33b", "tiny"], help="realtime mode: model preset")
    ap.add_argument("--prompt-tokens", type=int, default=512)
    ap.add_argument("--geometry", default="baseline", choices=["baseline", "reference"],
                    help="realtime mode: 'baseline' = chunks of 3 latent frames against a KV cache of 60 latent frames "
                         "(20 chunks: 19 committed + the current one); 'reference' = the reference deployment's 5-latent "
                         "chunks with 5 committed chunks of history.  Both run 4 denoise + 1 commit evaluation per chunk")
    ap.add_argument("--decode", default="vit", choices=["vit", "none"],
                    help="realtime mode: decode every generated latent to RGB8 frames with the streaming ViT decoder "
                         "(tiles dealt to the ranks) inside the timed region")
    ap.add_argument("--frames", type=int, default=None, help="latent frames (default: the model's benchmark clip)")
    ap.add_argument("--height", type=int, default=None)
    ap.add_argument("--width", type=int, default=None)
    ap.add_argument("--checkpointing", default="auto", choices=["auto", "none", "full", "selective"])
    ap.add_argument("--zero", default="fused", choices=["off", "collective", "fused"],
                    help="N > 1: shard optimizer state and gradient reduction over the ranks (own FSDP); "
                         "fused = NVLink peer reduce + AdamW + parameter push kernels")
    ap.add_argument("--keep-blocks", type=int, default=-1,
                    help="blocks exempt from recompute under checkpointing (-1: sized from free HBM)")
    ap.add_argument("--lean", default="auto", choices=["auto", "on", "off"],
                    help="resident blocks drop their norm outputs and FFN hidden activation and rebuild them in "
                         "backward (auto: on only when not every block would fit resident as it is)")
    ap.add_argument("--phase-times", action="store_true",
                    help="after the timed region, run one more step under the phase timer and add the forward / "
                         "backward / optimizer split (CUDA events) to the JSON line")
    ap.add_argument("--attention", default=None, choices=[None, "native", "library"])
    ap.add_argument("--fsdp", default="optimizer", choices=["params", "optimizer"],
                    help="N > 1 with --zero fused: 'params' also shards every block's bf16 parameters and fp32 gradient "
                         "buffers (just-in-time gathers over NVLink, reduce-scatter under backward); 'optimizer' shards "
                         "the optimizer state only")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="capture the whole training step in one CUDA graph and replay it (auto: on with the fused "
                         "transports at N > 1, where the step contains no library collective)")
    ap.add_argument("--sp-transport", default="fused", choices=["fused", "nccl"],
                    help="Ulysses exchange: fused into the kernels over NVLink peer memory, or NCCL all-to-all")
    args = ap.parse_args()
    f, h, w = GEOMETRY[args.model]
    args.frames = f if args.frames is None else args.frames
    args.height = h if args.height is None else args.height
    args.width = w if args.width is None else args.width
    return args


class ClockSampler:
    """Samples SM clock and throttle reasons of this rank's GPU with nvidia-smi during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx = float(s[1])
            except ValueError:
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx,
                "reasons": sorted(reasons), "samples": len(sm)}


GEOMETRY = {"ti2v_5b": (31, 44, 80), "small": (31, 44, 80), "ltx_2b": (16, 16, 24), "i2v_a14b": (21, 90, 160),
            "i2v_small": (6, 16, 24)}


def model_config(args):
    from solarwm_b200.models.wan import WanConfig, wan_preset

    if args.model == "i2v_a14b":
        return wan_preset("i2v_a14b")
    if args.model == "i2v_small":
        return WanConfig(model_type="i2v", in_dim=36, out_dim=16, dim=1024, ffn_dim=2048, num_heads=8, num_layers=3,
                         text_dim=4096, text_len=512)
    if args.model == "small":
        return WanConfig(model_type="ti2v", in_dim=48, out_dim=48, dim=512, ffn_dim=2048, num_heads=8,
                         num_layers=4, text_dim=4096, text_len=512)
    return wan_preset("ltx_video_2b" if args.model == "ltx_2b" else "ti2v_5b")


def n_tokens(cfg, args) -> int:
    pt, ph, pw = cfg.patch_size
    return (args.frames // pt) * (args.height // ph) * (args.width // pw)


def make_batch(cfg, args, pinned=True):
    import torch

    g = torch.Generator().manual_seed(1234)
    lat = torch.randn(1, args.frames, cfg.out_dim if cfg.model_type == "i2v" else cfg.in_dim, args.height, args.width,
                      generator=g).to(torch.bfloat16)
    txt = torch.randn(1, cfg.text_len, cfg.text_dim, generator=g).to(torch.bfloat16)
    batch = {"latents": lat, "text": txt}
    if cfg.model_type == "i2v":          # I2V conditioning: 4-channel first-frame mask + the first frame's latent
        y = torch.zeros(1, args.frames, cfg.in_dim - cfg.out_dim, args.height, args.width, dtype=torch.bfloat16)
        y[:, 0, :4] = 1.0
        y[:, 0, 4:] = lat[:, 0]
        batch["y"] = y
    if pinned:
        batch = {k: v.pin_memory() for k, v in batch.items()}
    return batch


def timed_region(steps, fn, dist, torch):
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    timed_region.host_enqueue_ms = (time.perf_counter() - t0) * 1e3 / steps    # host time to issue one step
    stop.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    ms = torch.tensor([start.elapsed_time(stop)], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def resident_block_plan(cfg, tokens, world, total_memory, *, zero_on, checkpointing, keep_blocks=-1, lean_mode="auto"):
    """How many blocks keep their activations (the rest are recomputed under selective checkpointing) and whether
    the resident ones run lean.  Calibrated on the 5B shape (peak_allocated with 11 / 13 / 15 / 19 resident blocks):
    an un-checkpointed block keeps ~14.5 [S, dim] and 1 [S, ffn] bf16 tensors (the GELU output is rebuilt in
    backward); a checkpointed one its input and the two attention outputs; 18 GB covers those plus workspace at
    S = 27,280.  Lean blocks drop three [S, dim] norm outputs and the [S, ffn] hidden activation and rebuild them
    in backward; ``auto`` turns that on only when not every block would fit resident as it is."""
    lean = lean_mode == "on"
    if keep_blocks >= 0:
        return keep_blocks, lean
    if checkpointing != "selective":
        return 0, lean
    s_local = tokens / world
    per_block = s_local * (14.5 * cfg.dim + cfg.ffn_dim) * 2
    n_params = cfg.num_layers * (8 * cfg.dim * cfg.dim + 2 * cfg.dim * cfg.ffn_dim)
    fixed = (6.0 + 12.0 / (world if zero_on else 1)) * n_params      # bf16 weight + fp32 grad + fp32 master / m / v
    budget = max(0.0, 0.88 * total_memory - fixed - 18e9 / world)
    keep = int(budget // per_block)
    if keep < cfg.num_layers and lean_mode == "auto":
        lean = True
    if lean:
        per_block -= s_local * (3 * cfg.dim + cfg.ffn_dim) * 2
        keep = int(budget // per_block)
    return min(keep, cfg.num_layers), lean


def run_ours(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dist = None
    sp = None
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
        # the fused transports need peer access between every pair of GPUs; all ranks agree on the answer before
        # any symmetric buffer is exchanged, and fall back to the NCCL forms together otherwise
        can = all(torch.cuda.can_device_access_peer(local, d) for d in range(world) if d != local)
        agree = torch.tensor([1 if can else 0], device=f"cuda:{local}")
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            args.sp_transport, args.zero = "nccl", ("collective" if args.zero == "fused" else args.zero)
        if args.sp_transport == "fused":
            from solarwm_b200.parallel.fused_ulysses import FusedUlysses

            mc = model_config(args)
            sp = FusedUlysses(None, max_tokens=n_tokens(mc, args), dim=mc.dim,
                              num_heads=mc.num_heads)
        else:
            from solarwm_b200.parallel.ulysses import UlyssesCollective

            sp = UlyssesCollective(None)

    from solarwm_b200 import ops
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer

    if args.attention:
        ops.set_backend(args.attention)
    cfg = model_config(args)
    ckpt = args.checkpointing
    if ckpt == "auto":
        ckpt = "selective" if (args.model == "ti2v_5b" and world < 4) else "none"
    keep, lean = resident_block_plan(cfg, n_tokens(cfg, args), world, torch.cuda.get_device_properties(local).total_memory,
                                     zero_on=world > 1 and args.zero != "off", checkpointing=ckpt,
                                     keep_blocks=args.keep_blocks, lean_mode=args.lean)
    zero = world > 1 and args.zero != "off"
    graph = args.graph == "on" or (args.graph == "auto" and world > 1 and args.sp_transport == "fused"
                                   and args.zero == "fused")
    opts = Stage0p5Options(lr=1e-4, timestep_shift=5.0, sigma_sampling="logit_normal", checkpointing=ckpt,
                           keep_blocks=keep, lean_kept=lean, max_grad_norm=1.0, seed=0, zero=zero,
                           zero_transport=args.zero, cuda_graph=graph,
                           shard_params=zero and args.zero == "fused" and args.fsdp == "params")
    model = heap = None
    if zero:
        from solarwm_b200.models.wan import WanDiT

        model = WanDiT(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, seed=0, shard_pad=world)
        if args.zero == "fused":
            from solarwm_b200.parallel.symm import SymmetricHeap

            from solarwm_b200.parallel.zero import fused_heap_bytes

            heap = SymmetricHeap(fused_heap_bytes(model.units(), world,
                                                  [b.unit for b in model.blocks] if args.fsdp == "params" else ()), None)
    trainer = WanStage0p5Trainer(cfg, f"cuda:{local}", opts, sp=sp, model=model, heap=heap)
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()            # construction transients (the un-sharded model) are not the step
    with torch.no_grad():  # a zero head would zero every upstream gradient; keep the step representative
        trainer.model.get_parameter("head.head.weight").normal_(0, 0.02)
    batch = make_batch(cfg, args)
    dev_batch = {k: v.to(f"cuda:{local}") for k, v in batch.items()}
    tokens = n_tokens(cfg, args)
    h2d = sum(v.numel() * v.element_size() for v in batch.values())

    def step_device():
        trainer.train_step(dev_batch)

    losses = []

    def step_e2e():
        loss = trainer.train_step(batch)
        losses.append(float(loss.item()))  # device -> host read of the step's result

    for _ in range(args.warmup):
        step_e2e()
    ops.check_status(f"cuda:{local}")
    sampler = ClockSampler(local)
    sampler.start()
    ops.reset_counters()
    ms = timed_region(args.steps, step_device, dist, torch)
    host_ms = round(timed_region.host_enqueue_ms, 2)
    launches = ops.total_launches()
    counters = dict(ops.COUNTERS)
    ms_e2e = timed_region(args.steps, step_e2e, dist, torch)
    clocks = sampler.stop()
    phases = None
    if args.phase_times:
        from solarwm_b200.utils.trace import PhaseTimer

        timer = PhaseTimer(f"cuda:{local}")
        with timer.installed():
            step_device()
        phases = {k: v["total_ms"] for k, v in timer.summary().items() if not k.startswith("block.")}
    ops.check_status(f"cuda:{local}")
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30
    # the symmetric heap (parameters, gradients, exchange buffers of the fused transports) is allocated outside the
    # caching allocator: report it, and the device's own view of used memory, next to the allocator's peak
    free_b, total_b = torch.cuda.mem_get_info()
    heap_gib = sum(h.nbytes for h in (heap, getattr(sp, "heap", None)) if h is not None) / 2 ** 30
    used_gib = (total_b - free_b) / 2 ** 30
    utilization = {}
    try:        # model FLOPs (no recompute counted) against the measured sustained cuBLAS rate of this pool
        from solarwm_b200.utils.roofline import step_utilization

        utilization = {"utilization": dict(step_utilization(cfg, tokens, ms / args.steps, world))}
    except Exception as exc:  # noqa: BLE001 - a reporting extra must never cost the measurement
        utilization = {"utilization": {"error": f"{type(exc).__name__}: {exc}"[:120]}}
    if rank == 0:
        value = tokens * args.steps / (ms / 1e3)
        e2e = tokens * args.steps / (ms_e2e / 1e3)
        out = {
            "metric": "DiT train tokens/s/box (Wan2.2 TI2V-5B-shaped flow-matching step)" if args.model != "ltx_2b"
            else "DiT train tokens/s/box (LTX-Video-2B-shaped flow-matching step)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None if BASELINE_TOKENS_PER_S is None else value / BASELINE_TOKENS_PER_S,
            "dtype": "bf16", "data": "synthetic latents/text of the named shapes, random-init weights",
            "impl": args.impl,
            "config": {"model": {"ti2v_5b": "wan22_ti2v_5b-shaped", "ltx_2b": "ltx_video_2b-shaped"}.get(args.model, "small-debug"),
                       "gemm_backend": "library (cuBLAS)" if args.impl == "baseline" else "native",
                       "global_batch": 1, "seq_len": tokens, "parallelism": f"sp{world}", "sp_transport": args.sp_transport if world > 1 else "none",
                       "optimizer_sharding": (f"zero-{args.zero}" if zero else "none"),
                       "cuda_graph_step": bool(graph),
                       "parameter_sharding": ("blocks sharded 1/N, gathered just in time" if opts.shard_params else "none"),
                       "latent": [1, cfg.in_dim, args.frames, args.height, args.width],
                       "text": [1, cfg.text_len, cfg.text_dim], "activation_checkpointing": ckpt, "keep_blocks": keep,
                       "lean_resident_blocks": lean,
                       "attention_backend": ops.get_backend(), "optimizer": "AdamW fp32 master (in timed region)",
                       "l2": "no flush: per-step working set (>=10 GB of weights) exceeds the 126 MB L2",
                       "peak_allocated_gib": round(peak_gib, 2), "symmetric_heap_gib": round(heap_gib, 2),
                       "device_memory_in_use_gib": round(used_gib, 2)},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "launch_counters": counters, "host_enqueue_ms_per_step": host_ms,
            **({"phase_ms": phases} if phases is not None else {}),
            **utilization,
            "final_loss": losses[-1] if losses else None,
        }
        print(json.dumps(out))
    if dist is not None:
        if hasattr(sp, "close"):
            sp.close()
        dist.destroy_process_group()


def run_infer(args):
    """Seconds per ``--sample-steps``-step flow-matching sample of one clip (BASELINE config 4: LTX-Video-2B shape,
    8 steps), through the LTX backend's public sampler, at SP = N.  A timed sample includes the host -> device copy of
    the text embedding from pinned memory and the device -> host read of the finished latent."""
    import torch

    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    torch.cuda.set_device(local)
    dist = sp = None
    cfg = model_config(args)
    tokens = n_tokens(cfg, args)
    if world > 1:
        import torch.distributed as dist_mod

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
        if args.sp_transport == "fused":
            from solarwm_b200.parallel.fused_ulysses import FusedUlysses

            sp = FusedUlysses(None, max_tokens=tokens, dim=cfg.dim, num_heads=cfg.num_heads,
                              max_frame_tokens=max(tokens // args.frames, 64))
        else:
            from solarwm_b200.parallel.ulysses import UlyssesCollective

            sp = UlyssesCollective(None)
    from solarwm_b200 import ops
    from solarwm_b200.backends.ltx25.backend import sample
    from solarwm_b200.models.wan import WanDiT

    if args.attention:
        ops.set_backend(args.attention)
    model = WanDiT(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, seed=0)
    with torch.no_grad():
        model.get_parameter("head.head.weight").normal_(0, 0.02)
    if sp is not None:
        model.sp = sp
    text_host = torch.randn(1, cfg.text_len, cfg.text_dim, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).pin_memory()
    out_host = torch.empty(1, cfg.out_dim, args.frames, args.height, args.width, dtype=torch.bfloat16).pin_memory()

    # the network evaluation is replayed from a CUDA graph unless a library collective sits inside it
    graph_state = {} if (args.graph != "off" and (world == 1 or args.sp_transport == "fused")) else None

    def one_sample():
        text = text_host.to(f"cuda:{local}", non_blocking=True)
        with torch.no_grad():
            x = sample(model, text, frames=args.frames, height=args.height, width=args.width, steps=args.sample_steps,
                       seed=3, graph=graph_state)
        out_host.copy_(x, non_blocking=True)

    for _ in range(max(args.warmup, 3)):
        one_sample()
    torch.cuda.synchronize()
    ops.check_status(f"cuda:{local}")
    sampler = ClockSampler(local)
    sampler.start()
    ops.reset_counters()
    ms = timed_region(args.steps, one_sample, dist, torch)
    launches = ops.total_launches()
    clocks = sampler.stop()
    ops.check_status(f"cuda:{local}")
    if rank == 0:
        per_sample = ms / args.steps / 1e3
        print(json.dumps({
            "metric": f"seconds per {args.sample_steps}-step flow-matching sample ({args.model}-shaped DiT)", "value": per_sample,
            "unit": "s/sample", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic text embedding and seed noise of the named shapes, random-init weights",
            "impl": args.impl,
            "config": {"model": args.model, "solver": f"Euler, {args.sample_steps} steps, linear sigma grid", "seq_len": tokens,
                       "latent": [1, cfg.out_dim, args.frames, args.height, args.width], "text": [1, cfg.text_len, cfg.text_dim],
                       "parallelism": f"sp{world}", "sp_transport": args.sp_transport if world > 1 else "none",
                       "attention_backend": ops.get_backend(), "cuda_graph_forward": graph_state is not None,
                       "gemm_backend": "library (cuBLAS)" if args.impl == "baseline" else "native",
                       "l2": "no flush: 2 B parameters (4 GB) are re-read every solver step"},
            "clocks": clocks,
            "e2e": {"value": per_sample, "unit": "s/sample", "h2d_bytes_per_step": int(text_host.numel() * 2),
                    "d2h_bytes_per_step": int(out_host.numel() * 2)},
            "gpu_launches": launches, "tokens_per_s": tokens * args.sample_steps * args.steps / (ms / 1e3)}))
    if dist is not None:
        if hasattr(sp, "close"):
            sp.close()
        dist.destroy_process_group()


def run_two_expert(args):
    """BASELINE config 3: A14B-shaped two-expert training.  Both experts (40 blocks, dim 5120, 40 heads each) live
    on the N GPUs with their parameters, gradient reductions and optimizer state sharded 1 / N (fused transports);
    every step draws sigma, picks the expert by the 0.875 boundary and trains it on the 75,600-token clip."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus or world < 2:
        raise SystemExit("the two-expert benchmark needs N >= 2 GPUs launched with torch.distributed.run "
                         "(two 14 B experts with AdamW state do not fit one device)")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from solarwm_b200 import ops
    from solarwm_b200.backends.wan22.experts import TwoExpertTrainer
    from solarwm_b200.backends.wan22.stage0p5 import Stage0p5Options, WanStage0p5Trainer
    from solarwm_b200.models.wan import WanDiT
    from solarwm_b200.parallel.fused_ulysses import FusedUlysses
    from solarwm_b200.parallel.symm import SymmetricHeap
    from solarwm_b200.parallel.zero import fused_heap_bytes

    cfg = model_config(args)
    tokens = n_tokens(cfg, args)
    frame_tokens = tokens // args.frames
    sp = FusedUlysses(None, max_tokens=tokens, dim=cfg.dim, num_heads=cfg.num_heads, max_frame_tokens=frame_tokens)
    # two 14B experts: selective recompute keeps one expert's activations near 20 GiB per rank at 8 ranks
    ckpt = ("selective" if args.model == "i2v_a14b" else "none") if args.checkpointing == "auto" else args.checkpointing
    graph = args.graph != "off"
    trainers, need = {}, 1 << 20
    models = {}
    for i, name in enumerate(("high_noise", "low_noise")):
        models[name] = WanDiT(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, seed=i, shard_pad=2 * world)
        with torch.no_grad():
            models[name].get_parameter("head.head.weight").normal_(0, 0.02)
        need += fused_heap_bytes(models[name].units(), world, [b.unit for b in models[name].blocks])
    heap = SymmetricHeap(need, None)
    for name in ("high_noise", "low_noise"):
        opts = Stage0p5Options(lr=1e-4, timestep_shift=5.0, sigma_sampling="logit_normal", checkpointing=ckpt,
                               max_grad_norm=1.0, seed=0, zero=True, zero_transport="fused", cuda_graph=graph,
                               shard_params=True, ti2v_first_frame_clean=False)
        trainers[name] = WanStage0p5Trainer(cfg, f"cuda:{local}", opts, sp=sp, model=models[name], heap=heap)
        torch.cuda.empty_cache()
    pair = TwoExpertTrainer(trainers["high_noise"], trainers["low_noise"], boundary=0.875, shift=5.0, seed=0)
    batch = make_batch(cfg, args)
    dev_batch = {k: v.to(f"cuda:{local}") for k, v in batch.items()}
    h2d = sum(v.numel() * v.element_size() for v in batch.values())
    losses = []
    # warm-up must take BOTH experts past their eager steps and their graph capture
    warm_sigmas = [0.95, 0.5] * max(args.warmup, 4)
    for s_ in warm_sigmas:
        losses.append(float(pair.train_step(batch, sigma=torch.tensor([s_])).item()))
    ops.check_status(f"cuda:{local}")
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(local)
    sampler.start()
    ops.reset_counters()
    pair.steps = {"high_noise": 0, "low_noise": 0}
    ms = timed_region(args.steps, lambda: pair.train_step(dev_batch), dist, torch)
    launches, counters = ops.total_launches(), dict(ops.COUNTERS)
    per_expert = dict(pair.steps)

    def step_e2e():
        losses.append(float(pair.train_step(batch).item()))

    ms_e2e = timed_region(args.steps, step_e2e, dist, torch)
    clocks = sampler.stop()
    ops.check_status(f"cuda:{local}")
    free_b, total_b = torch.cuda.mem_get_info()
    if rank == 0:
        value = tokens * args.steps / (ms / 1e3)
        print(json.dumps({
            "metric": "DiT train tokens/s/box (Wan2.2 A14B-shaped two-expert flow-matching step)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": len(warm_sigmas),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic latents / I2V conditioning / text of the named shapes, random-init weights",
            "impl": "ours",
            "config": {"model": f"{args.model}: two experts x {cfg.num_layers} blocks, dim {cfg.dim}, {cfg.num_heads} heads, "
                                f"ffn {cfg.ffn_dim}", "expert_boundary_sigma": 0.875, "steps_per_expert": per_expert,
                       "global_batch": 1, "seq_len": tokens, "parallelism": f"sp{world}", "sp_transport": "fused",
                       "optimizer_sharding": "zero-fused", "parameter_sharding": "blocks sharded 1/N, gathered just in time",
                       "cuda_graph_step": graph, "latent": [1, cfg.out_dim, args.frames, args.height, args.width],
                       "i2v_condition": [1, cfg.in_dim - cfg.out_dim, args.frames, args.height, args.width],
                       "text": [1, cfg.text_len, cfg.text_dim], "activation_checkpointing": ckpt,
                       "optimizer": "AdamW fp32 master per expert (in timed region)",
                       "l2": "no flush: per-step working set exceeds the 126 MB L2",
                       "peak_allocated_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2),
                       "symmetric_heap_gib": round((heap.nbytes + sp.heap.nbytes) / 2 ** 30, 2),
                       "device_memory_in_use_gib": round((total_b - free_b) / 2 ** 30, 2)},
            "clocks": clocks,
            "e2e": {"value": tokens * args.steps / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d + 4, "d2h_bytes_per_step": 4},
            "gpu_launches": launches, "launch_counters": counters, "final_loss": losses[-1]}))
    sp.close()
    dist.destroy_process_group()


def run_realtime(args):
    """H3-shaped realtime streaming: W warm chunks (the window fills, CUDA graphs are captured), then K timed
    chunks.  One chunk = 4 denoise evaluations + 1 commit evaluation of 5 latent frames (20 pixel frames)."""
    import torch

    from solarwm_b200 import ops
    from solarwm_b200.models.h3 import H3DiT, h3_preset
    from solarwm_b200.serve.h3_stream import H3StreamConfig, H3StreamingGenerator

    rank, local, world = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("LOCAL_RANK", 0), ("WORLD_SIZE", 1)))
    torch.cuda.set_device(local)
    dist = sp = None
    if world > 1:
        import torch.distributed as dist_mod

        from solarwm_b200.parallel.ulysses import UlyssesCollective

        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist, sp = dist_mod, UlyssesCollective(None)
    cfg = h3_preset(args.h3)
    model = H3DiT(cfg, device=f"cuda:{local}", dtype=torch.bfloat16, seed=0)
    scfg = H3StreamConfig() if args.h3 == "h3_33b" else H3StreamConfig(grid_hw=(8, 16))
    # the chunk evaluation is graph-captured on one GPU and, with the fused head exchange (no library collective inside
    # the evaluation), at SP > 1 too; the NCCL form runs eagerly (a captured run with NCCL all-to-alls did not finish
    # on this pool: collectives enqueued from a capture need every rank's capture to reach them in step, which the
    # eager warm-up chunks of the generator do not guarantee; not retried)
    if args.sp_transport != "fused":
        scfg.sp_exchange = "collective"
    scfg.use_cuda_graph = args.graph != "off" and (world == 1 or scfg.sp_exchange == "fused")
    gen = H3StreamingGenerator(model, scfg, sp=sp)
    g = torch.Generator().manual_seed(0)
    text = torch.randn(args.prompt_tokens, cfg.text_dim, generator=g).pin_memory()
    anchor = torch.randn(scfg.latent_channels, 1, 2 * scfg.grid_hw[0], 2 * scfg.grid_hw[1], generator=g).pin_memory()
    gen.start(text, anchor, torch.eye(4))
    cams = torch.eye(4).repeat(scfg.chunk_latents, 1, 1).pin_memory()
    warm = max(args.warmup, scfg.window_chunks + 2)
    for i in range(warm):
        gen.next_chunk(cams)
    ops.check_status(f"cuda:{local}")
    sampler = ClockSampler(local)
    sampler.start()
    ops.reset_counters()
    host = torch.empty(scfg.latent_channels, scfg.chunk_latents, 2 * scfg.grid_hw[0], 2 * scfg.grid_hw[1],
                       dtype=torch.bfloat16).pin_memory()
    dec = frames_host = None
    lh, lw = 2 * scfg.grid_hw[0], 2 * scfg.grid_hw[1]
    if args.decode == "vit":
        from solarwm_b200.models.vit_decoder import StreamingViTDecoder, ViTDecoderConfig, ViTVideoDecoder
        from solarwm_b200.ops import functional as F_

        vcfg = ViTDecoderConfig(latent_channels=scfg.latent_channels) if args.h3 == "h3_33b" else \
            ViTDecoderConfig(latent_channels=scfg.latent_channels, dim=128, depth=2, heads=2, dim_head=64, ffn_dim=256)
        vit = ViTVideoDecoder(vcfg, device=f"cuda:{local}", dtype=torch.bfloat16, seed=1)
        tiled = lh > 16 and lw > 16
        dec = StreamingViTDecoder(vit, (lh, lw), tile=16 if tiled else None, overlap=4 if tiled else 0,
                                  distributed=world > 1)
        if rank == 0:
            frames_host = torch.empty(scfg.chunk_latents * vcfg.frames_per_latent, lh * vcfg.patch, lw * vcfg.patch, 3,
                                      dtype=torch.uint8).pin_memory()
    dit_ev, dec_ev, emitted = [], [], []

    def decode(latents):
        """latents [C, n, H, W] -> RGB8 frames in pinned host memory on rank 0."""
        n_out = 0
        for j in range(latents.shape[1]):
            fr = dec.push(latents[:, j])
            if fr is None:
                continue
            fr = fr.to(torch.bfloat16)
            for f in range(fr.shape[1]):
                rgb, _ = F_.rgb8(fr[:, f], mean=(0.5, 0.5, 0.5), std=(0.5, 0.5, 0.5))
                frames_host[n_out % frames_host.shape[0]].copy_(rgb, non_blocking=True)
                n_out += 1
        return n_out

    if dec is not None:                                          # the decoder's first window, outside the timed region
        decode(torch.zeros(scfg.latent_channels, 7, lh, lw, device=f"cuda:{local}", dtype=torch.bfloat16))
        torch.cuda.synchronize()

    def chunk():
        cams[:, 0, 3] += 0.01                                   # a moving camera, copied from pinned memory
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        lat = gen.next_chunk(cams)
        host.copy_(lat)                                         # the generated latent chunk is read back
        e[1].record()
        if dec is not None:
            emitted.append(decode(lat))
        e[2].record()
        dit_ev.append((e[0], e[1]))
        dec_ev.append((e[1], e[2]))

    ms = timed_region(args.steps, chunk, dist, torch)
    dit_ms = sum(a.elapsed_time(b) for a, b in dit_ev[-args.steps:]) / args.steps
    dec_ms = sum(a.elapsed_time(b) for a, b in dec_ev[-args.steps:]) / args.steps
    launches = ops.total_launches()
    clocks = sampler.stop()
    ops.check_status(f"cuda:{local}")
    if rank == 0:
        # with the decoder on, count the frames it actually emitted (a latent that opens a group yields one)
        frames = emitted[-1] if emitted else 4 * scfg.chunk_latents
        fps = frames * args.steps / (ms / 1e3)
        print(json.dumps({
            "metric": "realtime generation FPS (H3-shaped block-causal streaming"
                      + (", DiT + streaming ViT decode to RGB8)" if dec is not None else ", DiT only)"), "value": fps,
            "unit": "frames/s", "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic prompt/anchor/cameras, random-init weights", "impl": args.impl,
            "config": {"model": args.h3, "geometry": args.geometry, "chunk_latents": scfg.chunk_latents,
                       "window_chunks": scfg.window_chunks,
                       "kv_cache_latents": (scfg.window_chunks + 1) * scfg.chunk_latents,
                       "sp_exchange": scfg.sp_exchange if world > 1 else "none",
                       "gemm_backend": "library (cuBLAS)" if args.impl == "baseline" else "native",
                       "attention_backend": ops.get_backend(),
                       "denoise_steps": scfg.denoise_steps, "rows_per_latent": gen.rows_per_latent,
                       "frames_per_chunk": frames,
                       "prompt_tokens": args.prompt_tokens, "parallelism": f"sp{world}",
                       "cuda_graph": bool(gen.timings[-1].graph),
                       "decode": "streaming ViT decoder, 16 x 16 latent tiles dealt to the ranks, RGB8 frames to "
                                 "pinned host memory" if dec is not None else "not included"},
            "clocks": clocks, "chunk_latency_ms": {"total": ms / args.steps, "dit": dit_ms, "decode": dec_ms},
            "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": int(cams.numel() * 4),
                    "d2h_bytes_per_step": int(host.numel() * 2 + (frames_host.numel() if frames_host is not None else 0))},
            "gpu_launches": launches}))
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "baseline":
        # same model, library kernels and collectives: the baseline arm
        args.attention, args.sp_transport, args.graph, args.fsdp = "library", "nccl", "off", "optimizer"
        args.zero = "collective" if args.zero == "fused" else args.zero
        from solarwm_b200 import ops as _ops

        _ops.set_gemm_backend("library")
    if args.mode == "realtime" and args.impl in ("ours", "baseline"):
        run_realtime(args)
        return 0
    if args.mode == "infer":
        run_infer(args)
        return 0
    if args.model in ("i2v_a14b", "i2v_small"):
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference trains one A14B expert and shards nothing over the SP group (its FSDP group is "
                              "the logical-DP group, size 1 at SP=8): 14 B parameters with fp32 gradients and AdamW state do "
                              "not fit one 180 GB device, and it has no two-expert training step"}))
            return 0
        run_two_expert(args)
        return 0
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline"))
        try:
            import reference_arm
        except Exception as exc:  # noqa: BLE001
            print(json.dumps({"impl": "reference", "unavailable": f"reference arm import failed: {exc!r}"[:300]}))
            return 0
        return reference_arm.run(args)
    run_ours(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
