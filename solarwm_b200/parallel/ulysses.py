"""Ulysses sequence parallelism: sequence-sharded activations, head-sharded attention.

Tokens are sharded over the SP group as whole latent frames (uneven shards allowed: with F
frames and P ranks the first ``F % P`` ranks hold one frame more).  Around attention one
exchange turns ``[B, S_local, H, D]`` into ``[B, S, H/P, D]`` and a second one turns the
attention output back.  q, k and v travel in ONE all-to-all (the reference issues three,
solar/backends/wan22/runtime/sequence_parallel.py:446-475) and the packing copies are a single
index permutation on each side.

Two transports implement the same interface:

* ``UlyssesCollective``  -- ``torch.distributed.all_to_all_single`` (NCCL on GPUs, gloo on CPU).
  This is the baseline arm and the CPU/gloo test path.
* ``parallel.fused_ulysses.FusedUlysses`` -- the exchange is done by this library's own kernels
  with peer-to-peer stores into symmetric buffers over NVLink (see that module).

Gradient semantics follow the reference (sequence_parallel.py:562-622): every SP rank
evaluates the same full-sequence loss, the backward of the final sequence all-gather sums the
P identical upstream gradients, so the loss is pre-divided by ``sp_size`` and parameter
gradients are summed over the SP group.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def frame_split(num_frames: int, size: int):
    """Per-rank (first_frame, num_frames) for whole-frame sharding."""
    base, rem = divmod(num_frames, size)
    out = []
    start = 0
    for r in range(size):
        n = base + int(r < rem)
        out.append((start, n))
        start += n
    return out


def balanced_lengths(total_rows: int, size: int):
    """Balanced, descending row counts of a contiguous partition: the first ``total % size`` ranks hold one row
    more (reference: deploy/solar_wm/.../attention/collectives.py:13-31)."""
    if total_rows < size:
        raise ValueError("every rank needs one row")
    return [(total_rows + size - 1 - r) // size for r in range(size)]


def balanced_bounds(total_rows: int, size: int, rank: int):
    lengths = balanced_lengths(total_rows, size)
    start = sum(lengths[:rank])
    return start, start + lengths[rank]


class _AllToAll(torch.autograd.Function):
    """all_to_all_single with explicit split sizes; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.group, ctx.in_splits, ctx.out_splits = group, in_splits, out_splits
        x = x.contiguous()
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g, ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


class _AllGatherSeq(torch.autograd.Function):
    """Concatenate uneven sequence shards; backward sums the upstream gradients over the group
    and returns this rank's slice (reduce-scatter semantics)."""

    @staticmethod
    def forward(ctx, x, sizes, group):
        ctx.group, ctx.sizes = group, sizes
        rank = dist.get_rank(group)
        ctx.rank = rank
        # shards may be uneven: pad to the largest, gather equal blocks, drop the padding
        biggest = max(sizes)
        x = x.contiguous()
        if x.shape[0] < biggest:
            x = torch.cat([x, x.new_zeros((biggest - x.shape[0],) + tuple(x.shape[1:]))], 0)
        outs = [torch.empty_like(x) for _ in sizes]
        dist.all_gather(outs, x, group=group)
        return torch.cat([o[:n] for o, n in zip(outs, sizes)], 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        start = sum(ctx.sizes[:ctx.rank])
        return g[start:start + ctx.sizes[ctx.rank]].clone(), None, None


class UlyssesCollective:
    """Sequence-parallel context backed by torch.distributed collectives."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._layout = None

    def set_layout(self, B: int, num_frames: int, frame_tokens: int) -> None:
        splits = frame_split(num_frames, self.size)
        self._layout = (B, [n * frame_tokens for _, n in splits])

    def set_layout_rows(self, B: int, lengths) -> None:
        """Arbitrary per-rank row counts (e.g. ``balanced_lengths``) instead of whole frames."""
        if len(lengths) != self.size:
            raise ValueError("one length per rank is required")
        self._layout = (B, [int(n) for n in lengths])

    # [B, S_local, H, D] x3 -> [B, S, H/P, D] x3 -------------------------------------------
    def scatter_heads(self, q, k, v, contiguous: bool = True):
        """``contiguous=False`` returns strided views of the exchange buffer (unit stride on D, sequence stride
        3 * hp * D): the attention kernels read them through their tensor maps and a cache write is one strided
        copy, so the three packing copies are saved."""
        B, seq = self._layout
        P, r = self.size, self.rank
        Sl, H, D = q.shape[1], q.shape[2], q.shape[3]
        if H % P != 0:
            raise ValueError(f"num_heads={H} must be divisible by sp_size={P}")
        hp = H // P
        # pack [P, S_local, 3, B, hp, D]: destination-major so each peer's block is contiguous
        x = torch.stack([q, k, v], 0).view(3, B, Sl, P, hp, D).permute(3, 2, 0, 1, 4, 5).reshape(P * Sl, 3, B, hp, D)
        out = _AllToAll.apply(x, [Sl] * P, list(seq), self.group)   # [S, 3, B, hp, D]
        out = out.permute(1, 2, 0, 3, 4)                            # [3, B, S, hp, D]
        if not contiguous:
            return out[0], out[1], out[2]
        return out[0].contiguous(), out[1].contiguous(), out[2].contiguous()

    # [B, S, H/P, D] -> [B, S_local, H, D] --------------------------------------------------
    def gather_heads(self, o):
        B, seq = self._layout
        P, r = self.size, self.rank
        S, hp, D = o.shape[1], o.shape[2], o.shape[3]
        Sl = seq[r]
        x = o.permute(1, 0, 2, 3).reshape(S, B, hp, D)              # sequence-major: peers' slices contiguous
        out = _AllToAll.apply(x, list(seq), [Sl] * P, self.group)   # [P*Sl, B, hp, D], source-major
        out = out.view(P, Sl, B, hp, D).permute(2, 1, 0, 3, 4).reshape(B, Sl, P * hp, D)
        return out.contiguous()

    # [B*S_local, dim] -> [B*S, dim] --------------------------------------------------------
    def gather_sequence(self, x, B: int):
        _, seq = self._layout
        Sl = seq[self.rank]
        xs = x.view(B, Sl, -1).transpose(0, 1).contiguous()         # [S_local, B, dim]
        full = _AllGatherSeq.apply(xs, list(seq), self.group)       # [S, B, dim]
        return full.transpose(0, 1).reshape(B * sum(seq), -1)

    def broadcast_(self, *tensors, src: int = 0):
        """SP peers must consume identical samples: broadcast sampled tensors from SP rank 0."""
        gsrc = dist.get_global_rank(self.group, src) if self.group is not None else src
        for t in tensors:
            dist.broadcast(t, src=gsrc, group=self.group)

    def sum_gradients_(self, flat_grads) -> None:
        """Sum flat gradient buffers over the SP group (one collective per buffer)."""
        for g in flat_grads:
            dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)
