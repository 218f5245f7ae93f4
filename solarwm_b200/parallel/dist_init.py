"""Process-group bootstrap: one process per GPU (NCCL) or per CPU rank (gloo), SP/DP subgroups.

``initialize(sp_size)`` reads the torchrun environment, initialises ``torch.distributed`` if the
world is larger than one, creates the sequence-parallel group of this rank (adjacent raw ranks)
and the data-parallel group (stride ``sp_size``), and returns the rank algebra plus an SP context
(collective transport; the fused NVLink transport is swapped in by ``parallel.fused_ulysses``).
Rendezvous always uses the MASTER_ADDR from the environment (127.0.0.1 on one node).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from datetime import timedelta
from typing import Optional

import torch
import torch.distributed as dist

from ..runtime.topology import Topology


@dataclass
class DistContext:
    topology: Topology
    device: torch.device
    sp: Optional[object]
    sp_group: Optional[object]
    dp_group: Optional[object]
    owns_process_group: bool


def initialize(sp_size: int = 1, *, timeout: timedelta = timedelta(hours=1), device: Optional[str] = None) -> DistContext:
    from .ulysses import UlyssesCollective

    if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
        topo = Topology.from_environ(sp_size)
    else:
        topo = Topology(1, 0, 1, 0, 1)
    use_cuda = torch.cuda.is_available() and device != "cpu"
    dev = torch.device("cuda", topo.local_rank) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(dev)
    owns = False
    if topo.raw_world_size > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if use_cuda:
            dist.init_process_group("nccl", timeout=timeout, device_id=dev)
        else:
            dist.init_process_group("gloo", timeout=timeout)
        owns = True
    sp_ctx = sp_group = dp_group = None
    if topo.raw_world_size > 1:
        # every rank must create every group, in the same order
        for d in range(topo.dp_size):
            g = dist.new_group(list(topo.sp_group_ranks(d)))
            if d == topo.dp_rank:
                sp_group = g
        for s in range(topo.sp_size):
            g = dist.new_group(list(topo.dp_group_ranks(s)))
            if s == topo.sp_rank:
                dp_group = g
        if topo.sp_size > 1:
            sp_ctx = UlyssesCollective(sp_group)
    return DistContext(topo, dev, sp_ctx, sp_group, dp_group, owns)


def shutdown(ctx: DistContext) -> None:
    if ctx.owns_process_group and dist.is_initialized():
        dist.destroy_process_group()
