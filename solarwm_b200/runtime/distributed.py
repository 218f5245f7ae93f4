"""Fail-closed, fail-together distributed control flow.

* ``propagate_collective_error`` / ``collective_call`` / ``collective_rank_zero_call``: every rank
  runs its rank-local phase, then all ranks exchange ``(rank, error text)`` and raise the SAME
  rank-sorted message before the next collective can be entered.  Only strings cross ranks.
* ``DataReadiness``: slow or failing batch reads are agreed upon over a separate gloo group so the
  NCCL watchdog never observes storage latency.
* SP identity fingerprints: sequence-parallel peers must have consumed identical samples / RNG.

The ``dist`` handle is a parameter so the logic is testable with a fake process group
(reference: solar/runtime/distributed.py:17-254).
"""
from __future__ import annotations

import hashlib
import time
from datetime import timedelta
from typing import Any, Callable, Mapping, Optional, Sequence, TypeVar

from ..config.loader import canonical_json
from ..errors import BackendContractError

T = TypeVar("T")


def _coordinates(dist, rank, world_size):
    live = bool(dist is not None and dist.is_initialized())
    r = int(rank) if rank is not None else (int(dist.get_rank()) if live else 0)
    w = int(world_size) if world_size is not None else (int(dist.get_world_size()) if live else 1)
    if w < 1 or not 0 <= r < w:
        raise BackendContractError("collective failure propagation got an invalid rank/world_size")
    if live and (r, w) != (int(dist.get_rank()), int(dist.get_world_size())):
        raise BackendContractError("collective failure propagation rank/world_size differs from the process group")
    return r, w, live


def propagate_collective_error(local_error: Optional[str], *, dist, label: str, rank=None, world_size=None,
                               error_type=BackendContractError) -> None:
    r, w, live = _coordinates(dist, rank, world_size)
    mine = (r, str(local_error or ""))
    records = [mine]
    if live and w > 1:
        records = [None] * w
        dist.all_gather_object(records, mine)
    seen: dict[int, str] = {}
    for rec in records:
        if not isinstance(rec, (tuple, list)) or len(rec) != 2 or isinstance(rec[0], bool):
            raise error_type(f"{label} failure exchange returned a malformed rank record")
        try:
            peer = int(rec[0])
        except (TypeError, ValueError) as exc:
            raise error_type(f"{label} failure exchange returned a malformed rank value") from exc
        if not 0 <= peer < w:
            raise error_type(f"{label} failure exchange returned an out-of-range rank")
        seen[peer] = str(rec[1] or "")
    if len(records) != w or set(seen) != set(range(w)):
        raise error_type(f"{label} failure exchange did not cover every raw rank")
    failed = [(peer, text) for peer, text in sorted(seen.items()) if text]
    if failed:
        raise error_type(f"{label} failed collectively: " + " | ".join(f"rank {p}: {t}" for p, t in failed))


def collective_call(call: Callable[[], T], *, dist, label: str, rank=None, world_size=None,
                    error_type=BackendContractError) -> T:
    result, caught, text = None, None, ""
    try:
        result = call()
    except Exception as exc:  # noqa: BLE001 - the text is exchanged, the instance never leaves the rank
        caught, text = exc, f"{type(exc).__name__}: {exc}"
    try:
        propagate_collective_error(text, dist=dist, label=label, rank=rank, world_size=world_size,
                                   error_type=error_type)
    except Exception as exc:
        if caught is not None:
            raise exc from caught
        raise
    return result


def collective_rank_zero_call(call: Callable[[], T], *, dist, label: str, rank=None, world_size=None,
                              error_type=BackendContractError) -> T:
    r, w, live = _coordinates(dist, rank, world_size)
    value = collective_call(call if r == 0 else (lambda: None), dist=dist, label=label, rank=r, world_size=w,
                            error_type=error_type)
    box = [value if r == 0 else None]
    if live and w > 1:
        dist.broadcast_object_list(box, src=0)
    return box[0]


def raise_if_device_wait_failed(code: int, *, dist, label: str = "fused transport", rank=None, world_size=None) -> None:
    """``code``: this rank's bounded-wait status word (0 = every device-side wait completed).  All ranks exchange their
    codes and, when any is non-zero, raise the SAME message before the next optimizer update or checkpoint: a wait that
    gave up means a consumer kernel ran on a half-filled receive buffer, so the step's result must not be kept."""
    text = "" if int(code) == 0 else f"a device-side bounded wait gave up (status code {int(code)})"
    propagate_collective_error(text, dist=dist, label=label, rank=rank, world_size=world_size)


class DataReadiness:
    """All ranks finish (or fail) their batch read together, on a CPU-side gloo group."""

    def __init__(self, *, enabled: bool, timeout: timedelta = timedelta(hours=2)):
        self.group = None
        if not enabled:
            return
        import torch
        import torch.distributed as dist

        if not dist.is_initialized() or dist.get_world_size() == 1:
            return
        self.torch, self.dist = torch, dist
        self.group = dist.new_group(backend="gloo", timeout=timeout)

    def read(self, call: Callable[[], T]) -> T:
        if self.group is None:
            return call()
        t0 = time.monotonic()
        result, err = None, None
        try:
            result = call()
        except Exception as exc:  # noqa: BLE001
            err = exc
        rank, world = self.dist.get_rank(), self.dist.get_world_size()
        flag = self.torch.tensor([rank if err is not None else world], dtype=self.torch.int64)
        self.dist.all_reduce(flag, op=self.dist.ReduceOp.MIN, group=self.group)
        first_failed = int(flag.item())
        if first_failed != world:
            box = [f"{type(err).__name__}: {err}" if rank == first_failed else ""]
            self.dist.broadcast_object_list(box, src=first_failed, group=self.group)
            raise BackendContractError(f"training data read failed on rank {first_failed}: {box[0]}") from err
        waited = time.monotonic() - t0
        if waited >= 30:
            print(f"[data-readiness][rank{rank}] all batches ready after {waited:.1f}s", flush=True)
        return result


def identity_fingerprint(value: Mapping[str, Any]) -> str:
    return hashlib.blake2s(canonical_json(value)).hexdigest()


def assert_peer_fingerprints(values: Sequence[str]) -> str:
    if not values or any(not v for v in values):
        raise BackendContractError("SP peer fingerprints are missing")
    if len(set(values)) != 1:
        raise BackendContractError(f"SP peers loaded different sample/RNG identities: {list(values)}")
    return values[0]


def gather_and_assert_sp_identity(value: Mapping[str, Any], *, sp_size: int, group=None, dist=None) -> str:
    mine = identity_fingerprint(value)
    if sp_size == 1:
        return mine
    if dist is None:
        import torch.distributed as dist  # noqa: PLC0415
    if not dist.is_initialized():
        raise BackendContractError("SP identity check requires initialized torch.distributed")
    peers = [None] * sp_size
    dist.all_gather_object(peers, mine, group=group)
    return assert_peer_fingerprints([str(p or "") for p in peers])
