"""Structured attention in ONE kernel call: per-row key ranges and the tile lists the masked kernels walk.

A ``SegmentMask`` says, for runs of consecutive query rows, which key ranges they attend (at most three ``[lo, hi)``
ranges per row): a block-causal window with a sink, the ``[clean | noisy]`` teacher-forcing rule, the prefix + window +
own-chunk rule of six-chunk context.  From the runs it derives what ``csrc/attention.cu`` / ``attention_bwd.cu`` read:

  ``row_ranges``            int32 ``[Sq, 6]``
  forward                   per block of 256 queries, the 128-key tiles some query of the block sees
  backward, dK / dV mode    per block of 128 keys, the 64-query tiles that see any key of the block
  backward, dQ mode         per block of 128 queries, the 64-key tiles they see

with bit 30 set on a tile that contains a masked (query, key) pair -- only there do the kernels test elements.  Tiles
nobody sees are never loaded, so the cost follows the mask's density (27 % for the six-chunk window of 10 + 10 chunks).

``masked_attention(q, k, v, mask)`` is the autograd op ([B, S, H, D] tensors); on CPU it evaluates the same mask densely
and serves as the oracle.  The reference builds FlexAttention block masks for the Wan teacher-forcing path and runs one
library call per segment for six-chunk context (solar/backends/wan22/runtime/modeling/causal_model.py:245-534,
solar/backends/minimax_h3/w6_attention.py:92-188).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

PARTIAL = 1 << 30
Range = Tuple[int, int]


@dataclass(frozen=True)
class Run:
    """Query rows ``[q_lo, q_hi)`` attend the union of ``ranges`` (up to three ``[lo, hi)`` key ranges)."""
    q_lo: int
    q_hi: int
    ranges: Tuple[Range, ...]


def _merge(ranges: Sequence[Range]) -> Tuple[Range, ...]:
    """Sorted, non-empty, non-overlapping (touching ranges are joined)."""
    out: List[List[int]] = []
    for lo, hi in sorted((int(a), int(b)) for a, b in ranges if int(b) > int(a)):
        if out and lo <= out[-1][1]:
            out[-1][1] = max(out[-1][1], hi)
        else:
            out.append([lo, hi])
    return tuple((a, b) for a, b in out)


class SegmentMask:
    def __init__(self, Sq: int, Sk: int, runs: Sequence[Run]):
        self.Sq, self.Sk = int(Sq), int(Sk)
        cleaned = []
        cursor = 0
        for run in sorted(runs, key=lambda r: r.q_lo):
            if run.q_lo != cursor or run.q_hi <= run.q_lo:
                raise ValueError("runs must tile the query rows without gaps or overlaps")
            merged = _merge(run.ranges)
            if not merged:
                raise ValueError(f"query rows [{run.q_lo}, {run.q_hi}) see no key")
            if len(merged) > 3:
                raise ValueError("a row may attend at most three disjoint key ranges")
            if merged[-1][1] > self.Sk or merged[0][0] < 0:
                raise ValueError("key range outside the key sequence")
            cleaned.append(Run(run.q_lo, run.q_hi, merged))
            cursor = run.q_hi
        if cursor != self.Sq:
            raise ValueError("runs must cover every query row")
        self.runs: Tuple[Run, ...] = tuple(cleaned)
        self._device: Dict[str, dict] = {}

    # -- oracles ----------------------------------------------------------------------------------------------------
    def dense(self) -> torch.Tensor:
        """Boolean ``[Sq, Sk]`` (True = visible)."""
        m = torch.zeros(self.Sq, self.Sk, dtype=torch.bool)
        for run in self.runs:
            for lo, hi in run.ranges:
                m[run.q_lo:run.q_hi, lo:hi] = True
        return m

    def density(self) -> float:
        seen = sum((r.q_hi - r.q_lo) * sum(hi - lo for lo, hi in r.ranges) for r in self.runs)
        return seen / float(self.Sq * self.Sk)

    # -- tables -----------------------------------------------------------------------------------------------------
    def row_ranges(self) -> np.ndarray:
        table = np.zeros((self.Sq, 6), dtype=np.int32)
        for run in self.runs:
            flat = [v for rng in run.ranges for v in rng] + [0] * (6 - 2 * len(run.ranges))
            table[run.q_lo:run.q_hi] = flat
        return table

    def _tiles_over_keys(self, q_block: int, k_tile: int):
        """For every block of ``q_block`` query rows: the key tiles of ``k_tile`` keys that some row sees."""
        n_blocks = -(-self.Sq // q_block)
        n_tiles = -(-self.Sk // k_tile)
        lists = []
        for b in range(n_blocks):
            a0, a1 = b * q_block, min((b + 1) * q_block, self.Sq)
            mine = [r for r in self.runs if r.q_lo < a1 and r.q_hi > a0]
            entries = []
            for t in range(n_tiles):
                t0, t1 = t * k_tile, min((t + 1) * k_tile, self.Sk)
                touch = [any(lo < t1 and hi > t0 for lo, hi in r.ranges) for r in mine]
                if not any(touch):
                    continue
                whole = all(any(lo <= t0 and hi >= t1 for lo, hi in r.ranges) for r in mine)
                entries.append(t | (0 if whole else PARTIAL))
            lists.append(entries)
        return lists

    def _tiles_over_queries(self, k_block: int, q_tile: int):
        """For every block of ``k_block`` keys: the query tiles of ``q_tile`` rows that see some key of the block."""
        n_blocks = -(-self.Sk // k_block)
        n_tiles = -(-self.Sq // q_tile)
        lists = []
        for b in range(n_blocks):
            k0, k1 = b * k_block, min((b + 1) * k_block, self.Sk)
            entries = []
            for t in range(n_tiles):
                a0, a1 = t * q_tile, min((t + 1) * q_tile, self.Sq)
                mine = [r for r in self.runs if r.q_lo < a1 and r.q_hi > a0]
                if not any(any(lo < k1 and hi > k0 for lo, hi in r.ranges) for r in mine):
                    continue
                whole = all(any(lo <= k0 and hi >= k1 for lo, hi in r.ranges) for r in mine)
                entries.append(t | (0 if whole else PARTIAL))
            lists.append(entries)
        return lists

    @staticmethod
    def _pack(lists, what: str):
        if any(len(e) == 0 for e in lists):
            raise ValueError(f"a {what} block interacts with nothing (every row and key must take part)")
        stride = max(len(e) for e in lists)
        table = np.zeros((len(lists), stride), dtype=np.int32)
        for i, e in enumerate(lists):
            table[i, :len(e)] = e
        return table, np.asarray([len(e) for e in lists], dtype=np.int32), stride

    def tables(self, device) -> dict:
        """Device copies of all tables (built once per device)."""
        key = str(device)
        if key not in self._device:
            fwd = self._pack(self._tiles_over_keys(256, 128), "query")
            dq = self._pack(self._tiles_over_keys(128, 64), "query")
            dkv = self._pack(self._tiles_over_queries(128, 64), "key")
            to = lambda a: torch.from_numpy(a).to(device)          # noqa: E731
            # launch order of the CTAs: heaviest stationary tile first (CTAs are dispatched in index order, so the
            # launch then ends with its lightest tiles instead of its longest ones)
            order = lambda counts: to(np.argsort(-counts.astype(np.int64), kind="stable").astype(np.int32))   # noqa: E731
            self._device[key] = {
                "row_ranges": to(self.row_ranges()),
                "fwd": (to(fwd[0]), to(fwd[1]), fwd[2]), "dq": (to(dq[0]), to(dq[1]), dq[2]),
                "dkv": (to(dkv[0]), to(dkv[1]), dkv[2]),
                "fwd_order": order(fwd[1]), "dq_order": order(dq[1]), "dkv_order": order(dkv[1]),
                "tiles_visited": int(fwd[1].sum()), "tiles_dense": len(fwd[1]) * (-(-self.Sk // 128)),
            }
        return self._device[key]


# ---------------------------------------------------------------------------------------------------------------------
# mask constructors for the rules the models use
# ---------------------------------------------------------------------------------------------------------------------
def block_causal_mask(L: int, chunk: int, window_chunks: int, sink: int = 0) -> SegmentMask:
    """Chunk i of ``chunk`` rows sees the sink rows and chunks ``max(0, i - W) .. i`` of the same sequence."""
    runs = []
    for i in range(-(-L // chunk)):
        lo, hi = max(0, i - window_chunks) * chunk, min((i + 1) * chunk, L)
        runs.append(Run(i * chunk, hi, ((0, sink if lo > 0 else 0), (lo, hi))))
    return SegmentMask(L, L, runs)


def teacher_forcing_segment_mask(L: int, chunk: int, window_chunks: int, sink: int = 0, prefix: int = 0) -> SegmentMask:
    """Rows ``[prefix | clean L | noisy L]``.  Prefix rows see the prefix; clean chunk i sees prefix + sink + clean
    chunks ``max(0, i - W) .. i``; noisy chunk i sees prefix + sink + clean chunks ``max(0, i - W) .. i - 1`` + its own
    noisy chunk (``prefix = 0`` is the Wan rule, ``sink = 0`` with a prefix the six-chunk-context rule)."""
    c0, n0 = prefix, prefix + L
    runs = []
    if prefix:
        runs.append(Run(0, prefix, ((0, prefix),)))
    clean, noisy = [], []
    for i in range(-(-L // chunk)):
        lo, hi = max(0, i - window_chunks) * chunk, min((i + 1) * chunk, L)
        head = (0, prefix + (sink if lo > 0 else 0)) if (prefix or (sink and lo > 0)) else (0, 0)
        clean.append(Run(c0 + i * chunk, c0 + hi, (head, (c0 + lo, c0 + hi))))
        noisy.append(Run(n0 + i * chunk, n0 + hi, (head, (c0 + lo, c0 + i * chunk), (n0 + i * chunk, n0 + hi))))
    S = prefix + 2 * L
    return SegmentMask(S, S, runs + clean + noisy)


# ---------------------------------------------------------------------------------------------------------------------
# the op
# ---------------------------------------------------------------------------------------------------------------------
def _dense_reference(q, k, v, mask: SegmentMask, scale: float):
    m = mask.dense().to(q.device)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    s = s.masked_fill(~m, float("-inf"))
    return torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, dim=-1), v.float()).to(q.dtype)


class _MaskedAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, scale):
        from . import _lib
        from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
        from .attention_native import _bshd
        from .functional import status_word

        q, k, v = _bshd(q), _bshd(k), _bshd(v)
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        t = mask.tables(q.device)
        o = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device)
        lst, cnt, stride = t["fwd"]
        rc = _lib.load().solar_attn_fwd_masked(
            ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(B), c_int(Sq), c_int(Sk), c_int(H), c_int(D),
            c_ll(q.stride(1)), c_ll(q.stride(0)), c_ll(k.stride(1)), c_ll(k.stride(0)), c_ll(v.stride(1)), c_ll(v.stride(0)),
            c_ll(o.stride(1)), c_ll(o.stride(0)), c_float(scale), ptr(status_word(q.device)), stream_handle(),
            ptr(t["row_ranges"]), ptr(lst), ptr(cnt), c_int(stride), ptr(t["fwd_order"]))
        check(rc, "solar_attn_fwd_masked")
        count("attn_fwd_masked")
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.mask, ctx.scale = mask, scale
        return o

    @staticmethod
    def backward(ctx, do):
        from . import _lib
        from ._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
        from .attention_bwd_native import ensure_tail_overlap_default
        from .attention_native import _bshd
        from .functional import status_word

        ensure_tail_overlap_default()
        q, k, v, o, lse = ctx.saved_tensors
        do = _bshd(do.contiguous())
        B, Sq, H, D = q.shape
        Sk = k.shape[1]
        t = ctx.mask.tables(q.device)
        dq = torch.empty((B, Sq, H, D), dtype=q.dtype, device=q.device)
        dk = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
        dv = torch.empty((B, Sk, H, D), dtype=q.dtype, device=q.device)
        scratch = torch.empty(2 * B * H * ((Sq + 127) // 128 * 128), dtype=torch.float32, device=q.device)
        (kl, kc, ks), (ql, qc, qs) = t["dkv"], t["dq"]
        rc = _lib.load().solar_attn_bwd_masked(
            ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(dq), ptr(dk), ptr(dv), ptr(scratch), c_int(B), c_int(Sq),
            c_int(Sk), c_int(H), c_int(D), c_ll(q.stride(1)), c_ll(q.stride(0)), c_ll(k.stride(1)), c_ll(k.stride(0)),
            c_ll(v.stride(1)), c_ll(v.stride(0)), c_ll(o.stride(1)), c_ll(o.stride(0)), c_ll(do.stride(1)), c_ll(do.stride(0)),
            c_float(ctx.scale), ptr(status_word(q.device)), stream_handle(), ptr(t["row_ranges"]), ptr(kl), ptr(kc),
            c_int(ks), ptr(ql), ptr(qc), c_int(qs), ptr(t["dkv_order"]), ptr(t["dq_order"]))
        check(rc, "solar_attn_bwd_masked")
        count("attn_bwd_masked", 3)
        return dq, dk, dv, None, None


def masked_attention(q, k, v, mask: SegmentMask, *, scale=None):
    """softmax(scale q k^T + mask) v for ``[B, S, H, D]`` tensors with the structured ``mask`` (one kernel forward, the
    two backward kernels; tiles nobody sees are skipped)."""
    from . import _lib
    from .attention import get_backend

    scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.shape[1] != mask.Sq or k.shape[1] != mask.Sk:
        raise ValueError(f"mask is for {mask.Sq} x {mask.Sk}, tensors are {q.shape[1]} x {k.shape[1]}")
    native = q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] in (64, 128) and get_backend() == "native" \
        and _lib.available()
    if not native:
        return _dense_reference(q, k, v, mask, scale)
    return _MaskedAttentionFn.apply(q, k, v, mask, scale)
