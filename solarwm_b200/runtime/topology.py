"""Rank algebra: ``raw_rank = dp_rank * sp_size + sp_rank``; SP peers are adjacent raw ranks, so an
SP group never leaves a node while ``sp_size <= local_world_size``
(reference: solar/runtime/topology.py:12-79)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Mapping, Optional

from ..errors import ConfigurationError


@dataclass(frozen=True)
class Topology:
    raw_world_size: int
    raw_rank: int
    local_world_size: int
    local_rank: int
    sp_size: int

    def __post_init__(self):
        if self.raw_world_size < 1 or not 0 <= self.raw_rank < self.raw_world_size:
            raise ConfigurationError(f"invalid raw rank {self.raw_rank} of {self.raw_world_size}")
        if self.local_world_size < 1 or not 0 <= self.local_rank < self.local_world_size:
            raise ConfigurationError(f"invalid local rank {self.local_rank} of {self.local_world_size}")
        if self.sp_size < 1 or self.raw_world_size % self.sp_size != 0:
            raise ConfigurationError(f"sequence_parallel_size {self.sp_size} must divide world size {self.raw_world_size}")
        if self.raw_world_size % self.local_world_size != 0:
            raise ConfigurationError("world size must be a multiple of the local world size")

    @classmethod
    def from_environ(cls, sp_size: int, environ: Optional[Mapping[str, str]] = None) -> "Topology":
        env = os.environ if environ is None else environ
        try:
            world, rank = int(env["WORLD_SIZE"]), int(env["RANK"])
            local_world = int(env.get("LOCAL_WORLD_SIZE", world))
            local_rank = int(env.get("LOCAL_RANK", rank % local_world))
        except (KeyError, ValueError) as exc:
            raise ConfigurationError("torchrun environment (WORLD_SIZE/RANK/LOCAL_RANK) is incomplete") from exc
        return cls(world, rank, local_world, local_rank, int(sp_size))

    @property
    def dp_size(self) -> int:
        return self.raw_world_size // self.sp_size

    @property
    def dp_rank(self) -> int:
        return self.raw_rank // self.sp_size

    @property
    def sp_rank(self) -> int:
        return self.raw_rank % self.sp_size

    @property
    def node_rank(self) -> int:
        return self.raw_rank // self.local_world_size

    @property
    def num_nodes(self) -> int:
        return self.raw_world_size // self.local_world_size

    def sp_group_ranks(self, dp_rank: Optional[int] = None) -> tuple:
        d = self.dp_rank if dp_rank is None else dp_rank
        return tuple(range(d * self.sp_size, (d + 1) * self.sp_size))

    def dp_group_ranks(self, sp_rank: Optional[int] = None) -> tuple:
        s = self.sp_rank if sp_rank is None else sp_rank
        return tuple(range(s, self.raw_world_size, self.sp_size))

    @property
    def is_main(self) -> bool:
        return self.raw_rank == 0
