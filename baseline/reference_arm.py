"""Reference arm of bench.py: the UNMODIFIED reference package installed under ``baseline/_ref``.

The same metric and config as the main arm (Wan2.2 TI2V-5B-shaped flow-matching training step,
one 27,280-token sample, bf16 compute, Ulysses SP = N, AdamW inside the timed region), driven
through the reference's own classes and functions:

  * model        ``solar.backends.wan22.runtime.modeling.causal_model.CausalWanModel`` (5B dims,
                 camera branch and control adapter off: the benchmark config has no camera input)
  * parallelism  ``init_sequence_parallel``, ``wrap_transformer_fsdp`` (FSDP1, param bf16 /
                 reduce fp32), ``apply_wan_activation_checkpointing``,
                 ``sync_sequence_parallel_gradients``
  * step         ``WanDiffusion`` + ``FlowMatchScheduler.add_noise/training_target/training_weight``,
                 ``weighted_masked_mse``, ``first_frame_loss_mask``, ``torch.optim.AdamW`` --
                 the sequence of calls of ``Wan5BStage0p5Runtime.train_microbatch`` /
                 ``prepare_optimizer_step`` / ``optimizer_step`` without its dataset reader
                 (no dataset or checkpoint can be downloaded here, so inputs are synthetic and
                 weights keep the reference's own random initialisation).

``diffusers`` is not installed in the image; ``baseline/shims/diffusers`` provides the three
base-class names the reference model imports.  None of this repository's models, kernels or
engine is on this path.
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why[:300]}))
    return 0


def run(args) -> int:
    if not (HERE / "_ref" / "solar").exists():
        return _unavailable("reference package is not installed under baseline/_ref")
    for p in (str(HERE / "shims"), str(HERE / "_ref")):
        if p not in sys.path:
            sys.path.insert(0, p)
    try:
        import torch
        import torch.distributed as dist
        from solar.backends.wan22.objectives import first_frame_loss_mask, weighted_masked_mse
        from solar.backends.wan22.runtime.components import WanDiffusion
        from solar.backends.wan22.runtime.distributed import apply_wan_activation_checkpointing, wrap_transformer_fsdp
        from solar.backends.wan22.runtime.modeling.causal_model import CausalWanAttentionBlock, CausalWanModel
        from solar.backends.wan22.runtime.sequence_parallel import (
            broadcast_sequence_parallel_tensor, get_fsdp_process_group, init_sequence_parallel,
            sync_sequence_parallel_gradients)
        from solar.backends.wan22.runtime.stage0p5 import expand_timesteps_to_tokens
        from solar.runtime.topology import Topology
    except Exception as exc:  # noqa: BLE001
        return _unavailable(f"reference import failed: {exc!r}")
    if not torch.cuda.is_available():
        return _unavailable("no CUDA device")

    sys.path.insert(0, str(HERE.parent))
    from bench import ClockSampler, make_batch, timed_region

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", "0")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    init_sequence_parallel(sp_size=world)
    topology = Topology.from_environ(world) if world > 1 else Topology(1, 0, 1, 0, 1)

    frame_tokens = (args.height // 2) * (args.width // 2)
    if args.model == "small":
        dims = dict(dim=512, ffn_dim=2048, num_heads=8, num_layers=4)
    else:
        dims = dict(dim=3072, ffn_dim=14336, num_heads=24, num_layers=30)
    torch.manual_seed(0)
    with torch.device(device):
        model = CausalWanModel(model_type="ti2v", patch_size=(1, 2, 2), text_len=512, in_dim=48, out_dim=48,
                               freq_dim=256, text_dim=4096, local_attn_size=12, sink_size=3, qk_norm=True,
                               cross_attn_norm=True, eps=1e-6, add_control_adapter=False,
                               cam_self_attn_layers=[], frame_seq_length=frame_tokens, **dims)
    with torch.no_grad():  # keep gradients non-trivial, as in the main arm
        model.head.head.weight.normal_(0, 0.02)
    model.train().requires_grad_(True)
    ckpt = args.checkpointing
    if ckpt == "auto":
        ckpt = "full" if (args.model == "ti2v_5b" and world < 4) else "none"
    fsdp_cfg = {"strategy": "FULL_SHARD", "param_dtype": "bfloat16", "reduce_dtype": "float32",
                "buffer_dtype": "bfloat16", "activation_checkpointing": ckpt == "full"}
    if world > 1:
        module = wrap_transformer_fsdp(model, {"train": {"fsdp": fsdp_cfg}}, topology)
    else:
        # wrap_transformer_fsdp returns the bare fp32 module at world size 1; to keep the named
        # bf16 compute dtype the same FSDP1 wrap (identical arguments) is applied on one rank.
        import functools

        from torch.distributed.fsdp import BackwardPrefetch, FullyShardedDataParallel, MixedPrecision, ShardingStrategy
        from torch.distributed.fsdp.wrap import transformer_auto_wrap_policy

        module = FullyShardedDataParallel(
            model,
            auto_wrap_policy=functools.partial(transformer_auto_wrap_policy,
                                               transformer_layer_cls={CausalWanAttentionBlock}),
            process_group=get_fsdp_process_group(), sharding_strategy=ShardingStrategy.FULL_SHARD,
            mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                           buffer_dtype=torch.bfloat16, cast_root_forward_inputs=True),
            device_id=local, use_orig_params=True, forward_prefetch=True,
            backward_prefetch=BackwardPrefetch.BACKWARD_PRE, sync_module_states=False, limit_all_gathers=True)
        if ckpt == "full":
            apply_wan_activation_checkpointing(module)
    diffusion = WanDiffusion(module, timestep_shift=5.0, frame_sequence_length=frame_tokens,
                             num_output_frames=args.frames)
    optimizer = torch.optim.AdamW(module.parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)

    class _Cfg:  # make_batch reads these three fields
        in_dim, text_len, text_dim = 48, 512, 4096

    batch = make_batch(_Cfg, args)
    dev_batch = {k: v.to(device) for k, v in batch.items()}
    tokens = args.frames * frame_tokens
    h2d = sum(v.numel() * v.element_size() for v in batch.values())
    sched = diffusion.scheduler
    sp = world

    def train_step(b):
        clean = b["latents"].to(device, non_blocking=True)
        prompt = {"prompt_embeds": b["text"].to(device, non_blocking=True)}
        B, F = clean.shape[:2]
        dropped = torch.zeros(B, dtype=torch.bool, device=device)
        tidx = torch.randint(0, 1000, (B, 1), device=device, dtype=torch.long).expand(B, F).contiguous()
        if sp > 1:
            broadcast_sequence_parallel_tensor(tidx)
        timestep = sched.timesteps.to(device=device, dtype=torch.float32)[tidx]
        timestep[~dropped, 0] = 0.0
        noise = torch.randn_like(clean)
        if sp > 1:
            broadcast_sequence_parallel_tensor(noise)
        noisy = sched.add_noise(clean.flatten(0, 1).float(), noise.flatten(0, 1).float(),
                                timestep.flatten(0, 1)).unflatten(0, (B, F)).to(clean.dtype)
        noisy[~dropped, 0] = clean[~dropped, 0]
        t_tokens = expand_timesteps_to_tokens(timestep, frame_tokens)
        pred = diffusion(noisy, prompt, None, t_tokens, sequence_length=F * frame_tokens)
        target = sched.training_target(clean, noise, timestep)
        weight = sched.training_weight(timestep).view(B, F, 1, 1, 1)
        mask = first_frame_loss_mask(B, F, dropped)
        loss = weighted_masked_mse(pred, target, mask, weight)
        (loss / sp).backward()
        sync_sequence_parallel_gradients(module)
        module.clip_grad_norm_(1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return loss

    losses = []

    def step_device():
        train_step(dev_batch)

    def step_e2e():
        losses.append(float(train_step(batch).item()))

    try:
        for _ in range(args.warmup):
            step_e2e()
        sampler = ClockSampler(local)
        sampler.start()
        ms = timed_region(args.steps, step_device, dist, torch)
        ms_e2e = timed_region(args.steps, step_e2e, dist, torch)
        clocks = sampler.stop()
    except torch.OutOfMemoryError as exc:
        if rank == 0:
            _unavailable(f"reference step ran out of device memory at N={world}: {str(exc)[:120]}")
        dist.destroy_process_group()
        return 0
    peak_gib = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        value = tokens * args.steps / (ms / 1e3)
        e2e = tokens * args.steps / (ms_e2e / 1e3)
        print(json.dumps({
            "metric": "DiT train tokens/s/box (Wan2.2 TI2V-5B-shaped flow-matching step)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic latents/text of the named shapes, random-init weights",
            "impl": "reference",
            "config": {"model": "wan22_ti2v_5b-shaped" if args.model == "ti2v_5b" else "small-debug",
                       "global_batch": 1, "seq_len": tokens, "parallelism": f"sp{world}",
                       "latent": [1, 48, args.frames, args.height, args.width], "text": [1, 512, 4096],
                       "activation_checkpointing": ckpt, "fsdp": "FSDP1 param bf16 / reduce fp32 (reference stock)",
                       "attention_backend": "reference stock (flash_attn 2 when importable, else SDPA)",
                       "optimizer": "torch.optim.AdamW (in timed region)",
                       "l2": "no flush: per-step working set (>=10 GB of weights) exceeds the 126 MB L2",
                       "peak_allocated_gib": round(peak_gib, 2)},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "final_loss": losses[-1] if losses else None,
        }))
    dist.destroy_process_group()
    return 0
