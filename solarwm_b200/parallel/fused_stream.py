"""Head / sequence exchanges of block-causal streaming inference as this library's own NVLink kernels.

At SP = P every rank runs the projections and per-head transforms on its rows of the chunk and attention on its
heads over the whole window.  Per layer that takes two exchanges; here neither is a library collective:

  q | k | v   ``solar_comm_scatter_cols``: one launch stores column block ``d`` (rank d's heads) of the local q, k
              and v rows into rank d's memory -- q into an exchange buffer, k and v STRAIGHT INTO RANK d's KV CACHE at
              the rows of the current chunk, so the cache append is the exchange and no copy follows it;
  output      the flash-attention epilogue (``solar_attn_fwd_scatter``) stores every output row into the token
              owner's ``[rows_local, heads * head_dim]`` buffer.

Each producer's last CTA bumps a flag on every rank; consumers are preceded by a bounded device-side wait whose round
counter lives on the device.  The evaluation is therefore a FIXED launch sequence with no host value in it, which is
what lets the serving layer capture it in a CUDA graph at SP > 1 exactly as it does on one GPU.  Buffers alternate by
layer parity (a layer's wait implies that every peer has consumed the previous layer's buffers).

The KV caches live in the symmetric heap.  A peer writes only the rows of the chunk being evaluated, and only after
its previous exchange round, which every rank enters after it finished the previous evaluation; ``barrier`` is the
extra round the generator needs after it moved cache rows itself (window slide).

Reference: the realtime deployment runs the same exchanges as NCCL all-to-alls scheduled around the GEMMs inside
captured graphs (deploy/solar_wm/backends/standard/acceleration/graph/resident.py:101-190,
operators/schedule.py:287-390).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from ..ops.functional import status_word
from .symm import SymmetricHeap
from .ulysses import balanced_lengths


class FusedHeadExchange:
    fused = True

    def __init__(self, group: Optional[dist.ProcessGroup], *, heads: int, head_dim: int, layers: int, cache_rows: int,
                 max_rows: int, out_width: int, dtype=torch.bfloat16):
        self.group = group
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        P = self.size
        if heads % P:
            raise ValueError(f"heads={heads} must be divisible by the sequence-parallel size {P}")
        self.heads, self.hd, self.hl = heads, head_dim, heads // P
        self.a_local, self.a_full = self.hl * head_dim, heads * head_dim
        self.max_rows, self.cache_rows, self.layers = int(max_rows), int(cache_rows), int(layers)
        self.max_local = (self.max_rows + P - 1) // P
        self.out_width = int(out_width)
        need = (2 * self.max_rows * self.a_local + 2 * self.max_local * self.a_full + self.max_rows * self.out_width
                + 2 * layers * self.cache_rows * self.a_local) * 2 + (1 << 20)
        self.heap = SymmetricHeap(need, group)
        self.lib = _lib.load()
        h = self.heap

        def pair(shape):
            ts, offs = [], []
            for _ in range(2):
                t, off = h.alloc(shape, dtype)
                ts.append(t)
                offs.append(off)
            return ts, offs

        self.qbuf, self.qbuf_off = pair((self.max_rows, self.a_local))
        self.obuf, self.obuf_off = pair((self.max_local, self.a_full))
        self.seqbuf, self.seqbuf_off = h.alloc((self.max_rows, self.out_width), dtype)
        self.k_cache, self.v_cache, self.k_off, self.v_off = [], [], [], []
        for _ in range(layers):
            k, ko = h.alloc((self.cache_rows, self.a_local), dtype)
            v, vo = h.alloc((self.cache_rows, self.a_local), dtype)
            self.k_cache.append(k)
            self.v_cache.append(v)
            self.k_off.append(ko)
            self.v_off.append(vo)
        self.o_local = torch.empty(self.max_rows, self.a_local, dtype=dtype, device=h.device)   # the kernel's local copy
        self.flag_qkv = [h.new_flag() for _ in range(2)]
        self.flag_o = [h.new_flag() for _ in range(2)]
        self.flag_seq = h.new_flag()
        self.flag_sync = h.new_flag()
        self._parity = 0
        self._rows = None

    # -- layout -----------------------------------------------------------------------------------------------------
    def set_rows(self, n_rows: int) -> None:
        """The next exchanges move a segment of ``n_rows`` rows, dealt to the ranks in balanced contiguous ranges."""
        if n_rows == self._rows:
            return
        if n_rows > self.max_rows:
            raise ValueError(f"{n_rows} rows exceed the exchange buffers ({self.max_rows})")
        lengths = balanced_lengths(n_rows, self.size)
        starts = [0]
        for n in lengths:
            starts.append(starts[-1] + n)
        self._rows, self._starts = n_rows, starts
        self._starts_c = (ctypes.c_int * (self.size + 1))(*starts)

    def local_bounds(self):
        return self._starts[self.rank], self._starts[self.rank + 1]

    def next_parity(self) -> int:
        self._parity ^= 1
        return self._parity

    # -- exchanges --------------------------------------------------------------------------------------------------
    def exchange_qkv(self, q, k, v, layer: int, key_base: int, parity: int) -> torch.Tensor:
        """q, k, v: this rank's rows ``[rows_local, heads * head_dim]``.  Returns q of this rank's heads for all rows
        ``[n_rows, heads_local * head_dim]``; k and v of the segment are then in rows ``[key_base, key_base + n_rows)`` of
        EVERY rank's layer cache (each rank holding its own heads)."""
        h, P = self.heap, self.size
        a0 = self._starts[self.rank]
        rows_local = q.shape[0]
        srcs = (ctypes.c_void_p * 3)(q.data_ptr(), k.data_ptr(), v.data_ptr())
        src_ld = (ctypes.c_longlong * 3)(q.stride(0), k.stride(0), v.stride(0))
        dst = (ctypes.c_void_p * (3 * P))(*([p + self.qbuf_off[parity] for p in h.ptrs]
                                            + [p + self.k_off[layer] for p in h.ptrs]
                                            + [p + self.v_off[layer] for p in h.ptrs]))
        dst_ld = (ctypes.c_longlong * 3)(self.a_local, self.a_local, self.a_local)
        dst_row = (ctypes.c_longlong * 3)(a0, key_base + a0, key_base + a0)
        dst_col = (ctypes.c_longlong * 3)(0, 0, 0)
        slot = self.flag_qkv[parity]
        check(self.lib.solar_comm_scatter_cols(c_int(3), srcs, src_ld, c_ll(rows_local), c_int(self.a_local), dst, dst_ld,
                                               dst_row, dst_col, c_int(P), h.flag_ptrs(slot), h.counter_ptr(slot),
                                               c_int(0), stream_handle()), "solar_comm_scatter_cols")
        count("scatter_cols")
        h.wait(slot, P)
        return self.qbuf[parity][:self._rows]

    def attention(self, q, layer: int, key_lo: int, key_hi: int, scale: float, parity: int) -> torch.Tensor:
        """Attention of the segment's queries (this rank's heads) over cache rows ``[key_lo, key_hi)``; returns the
        output of this rank's ROWS for all heads ``[rows_local, heads * head_dim]`` (pushed there by every rank's
        attention epilogue)."""
        h = self.heap
        n_rows, n_keys = self._rows, key_hi - key_lo
        kc, vc = self.k_cache[layer][key_lo:key_hi], self.v_cache[layer][key_lo:key_hi]
        slot = self.flag_o[parity]
        check(self.lib.solar_attn_fwd_scatter(ptr(q), ptr(kc), ptr(vc), ptr(self.o_local), ptr(None), c_int(n_rows),
                                              c_int(n_keys), c_int(self.hl), c_int(self.hd), c_ll(q.stride(0)),
                                              c_ll(self.a_local), c_ll(self.a_local), c_ll(self.a_local), c_float(scale),
                                              ptr(status_word(q.device)), stream_handle(),
                                              h.peer_ptr_array(self.obuf_off[parity]), h.flag_ptrs(slot),
                                              h.counter_ptr(slot), c_int(self.size), c_ll(self.a_full),
                                              c_ll(self.max_local), self._starts_c, c_int(self.rank * self.a_local)),
              "solar_attn_fwd_scatter")
        count("attn_fwd_scatter")
        h.wait(slot, self.size)
        a, b = self.local_bounds()
        return self.obuf[parity][:b - a]

    def gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's output rows ``[rows_local, out_width]`` -> all rows of the segment on every rank."""
        h = self.heap
        x = x.contiguous()
        a, _ = self.local_bounds()
        check(self.lib.solar_comm_push(ptr(x), h.peer_ptr_array(self.seqbuf_off), c_int(self.size),
                                       c_ll(a * self.out_width * 2), c_ll(x.numel() * 2), h.flag_ptrs(self.flag_seq),
                                       h.counter_ptr(self.flag_seq), stream_handle()), "solar_comm_push")
        count("comm_push")
        h.wait(self.flag_seq, self.size)
        return self.seqbuf[:self._rows]

    def barrier(self) -> None:
        """A flag round with no data: every rank's work enqueued so far (e.g. a window slide that moved cache rows)
        is complete before any rank's later kernels run."""
        self.heap.signal(self.flag_sync)
        self.heap.wait(self.flag_sync, self.size)

    def close(self) -> None:
        self.heap.close()
