"""Ulysses exchanges fused into the producing kernels in BOTH directions (NVLink peer stores, no NCCL in the layer).

Forward of one attention layer at SP = P, tokens sharded by whole frames, heads by rank:

  1. QKV projection GEMM (tcgen05).  Its epilogue stores the V columns straight into the receive buffer of the rank
     that owns each head (``solar_gemm_bf16_scatter``); Q and K columns stay local because Wan normalises them over
     the full width first.
  2. full-width RMSNorm + RoPE of Q and of K (row kernel) whose output stage is the same column scatter
     (``solar_rmsnorm_rope_scatter``).  Every rank now holds ``[S, q_loc | k_loc | v_loc]``.
  3. flash attention over the local heads and the whole sequence; its epilogue stores each output row into the token
     owner's ``[S_local, dim]`` buffer (``solar_attn_fwd_scatter``).
  4. the out-projection GEMM reads that buffer.

Backward runs the same exchanges in reverse, again from inside the producing kernels:

  4'. the out-projection dgrad GEMM ``dY W_o`` leaves through the column scatter: every rank receives
      ``dO [S, heads_local * hd]`` for its heads (``solar_gemm_bf16_scatter``, NN layout);
  3'. the attention backward kernels store every row of dQ / dK / dV into the token owner's ``[S_local, 3 * dim]``
      buffer at this rank's head columns (``solar_attn_bwd_scatter``); nothing is written locally;
  2'. RMSNorm + RoPE backward of the q and k column blocks in place, then the QKV dgrad and wgrad GEMMs read the
      buffer as it is.

Each producer kernel's last CTA adds 1 to a flag word on every rank; consumers are preceded on the stream by a bounded
device-side wait whose round counter lives on the device (``SymmetricHeap.wait``), so the whole layer is a fixed launch
sequence that a CUDA graph can replay.  Buffers are double-buffered by layer parity, which is sufficient because every
wait of a layer depends on every peer having finished the previous layer's consumer kernels (stream order).

The reference performs the forward as three ``nn.Linear`` + two norms + RoPE + three ``all_to_all_single`` with packing
copies and one more all-to-all after attention, and the backward as the reverse all-to-alls
(solar/backends/wan22/runtime/modeling/causal_model.py:878-1027, sequence_parallel.py:407-541).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib, functional as F_
from ..ops._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from ..ops.functional import status_word
from ..utils.trace import span
from .symm import SymmetricHeap
from .ulysses import UlyssesCollective


class _GatherSeqFused(torch.autograd.Function):
    """Sequence all-gather as peer pushes.  Every rank then evaluates the SAME head and loss on the full sequence,
    so the upstream gradient is identical on all ranks; the reduce-scatter of the collective form (a sum of ``P``
    identical tensors, then this rank's slice) is therefore the local slice times ``P``, exactly, with no traffic."""

    @staticmethod
    def forward(ctx, x, sp):
        ctx.sp = sp
        return sp._push_rows(x)

    @staticmethod
    def backward(ctx, g):
        sp = ctx.sp
        a, b = sp._row_start[sp.rank], sp._row_start[sp.rank + 1]
        return g[a:b] * float(sp.size), None


class FusedUlysses(UlyssesCollective):
    fused = True

    def __init__(self, group: Optional[dist.ProcessGroup], *, max_tokens: int, dim: int, num_heads: int,
                 max_frame_tokens: int = 4096):
        super().__init__(group)
        P = self.size
        if num_heads % P:
            raise ValueError(f"num_heads={num_heads} must be divisible by sp_size={P}")
        self.dim, self.heads, self.hd = dim, num_heads, dim // num_heads
        self.dl = dim // P                       # columns of one rank's head block
        self.max_tokens = int(max_tokens)
        # whole-frame sharding: a rank holds at most ceil(F / P) frames, i.e. at most one frame more than the mean
        self.max_local = (self.max_tokens + P - 1) // P + int(max_frame_tokens)
        ml, mt = self.max_local, self.max_tokens
        need = 2 * (mt * 3 * self.dl + ml * dim + mt * self.dl + ml * 3 * dim) * 2 + mt * dim * 2 + (1 << 16)
        self.heap = SymmetricHeap(need, group)

        def pair(shape):
            tensors, offsets = [], []
            for _ in range(2):
                t, off = self.heap.alloc(shape)
                tensors.append(t)
                offsets.append(off)
            return tensors, offsets

        self.recv, self.recv_off = pair((mt, 3 * self.dl))          # forward: q | k | v of this rank's heads
        self.obuf, self.obuf_off = pair((ml, dim))                  # forward: attention output of this rank's tokens
        self.dobuf, self.dobuf_off = pair((mt, self.dl))            # backward: dO of this rank's heads
        self.dqkv, self.dqkv_off = pair((ml, 3 * dim))              # backward: dq | dk | dv of this rank's tokens
        self.seqbuf, self.seqbuf_off = self.heap.alloc((mt, dim))   # final sequence gather
        self.flag_qkv = [self.heap.new_flag() for _ in range(2)]
        self.flag_o = [self.heap.new_flag() for _ in range(2)]
        self.flag_do = [self.heap.new_flag() for _ in range(2)]
        self.flag_dqkv = [self.heap.new_flag() for _ in range(2)]
        self.flag_seq = self.heap.new_flag()
        self._parity = 0
        self._bwd_parity = 0
        self._row_start = None

    # layout -------------------------------------------------------------------------------
    def set_layout(self, B: int, num_frames: int, frame_tokens: int) -> None:
        super().set_layout(B, num_frames, frame_tokens)
        if B != 1:
            raise ValueError("the fused Ulysses path handles one sample per step (B == 1)")
        _, seq = self._layout
        starts = [0]
        for n in seq:
            starts.append(starts[-1] + n)
        if starts[-1] > self.max_tokens:
            raise ValueError("sequence longer than the symmetric receive buffers")
        if max(seq) > self.max_local:
            # the attention epilogues store a rank's rows into per-rank buffers of max_local rows: refuse a layout
            # whose largest shard does not fit instead of writing past the buffer in a peer's memory
            raise ValueError(f"a rank would own {max(seq)} tokens but the per-rank buffers hold {self.max_local}; "
                             f"build FusedUlysses with max_frame_tokens >= {frame_tokens}")
        self._row_start = starts
        self._row_start_c = (ctypes.c_int * (self.size + 1))(*starts)

    def next_parity(self) -> int:
        self._parity ^= 1
        return self._parity

    def next_bwd_parity(self) -> int:
        """Backward layers alternate their own buffer pair, counted at backward time: with recomputed blocks the
        forward parity a layer was (re)run with says nothing about which backward layer came just before it."""
        self._bwd_parity ^= 1
        return self._bwd_parity

    # step 1 + 2 ---------------------------------------------------------------------------
    def qkv_exchange(self, xm, w_qkv, b_qkv, nq_w, nk_w, rope, eps, parity):
        """Returns (qkv_local [Sl, 3*dim] with q,k columns valid, rstd_q, rstd_k, recv view [S, 3*dl])."""
        lib = _lib.load()
        D, dl, P = self.dim, self.dl, self.size
        Sl = xm.shape[0]
        S = self._row_start[-1]
        row_off = self._row_start[self.rank]
        heap = self.heap
        slot = self.flag_qkv[parity]
        dst = heap.peer_ptr_array(self.recv_off[parity])
        flags = heap.flag_ptrs(slot)
        counter = heap.counter_ptr(slot)
        qkv = torch.empty((Sl, 3 * D), dtype=xm.dtype, device=xm.device)
        xm = F_._rowmajor(xm)
        rc = lib.solar_gemm_bf16_scatter(ptr(xm), ptr(w_qkv), ptr(qkv), ptr(b_qkv), c_int(Sl), c_int(3 * D), c_int(D),
                                         c_ll(xm.stride(0)), c_ll(w_qkv.stride(0)), c_ll(3 * D), c_int(F_.NT), c_int(0),
                                         ptr(status_word(xm.device)), c_int(0), stream_handle(), dst, flags, counter,
                                         c_int(P), c_ll(3 * dl), c_int(D), c_int(dl), c_int(row_off), c_int(2 * D),
                                         c_int(0))
        check(rc, "solar_gemm_bf16_scatter")
        count("gemm_scatter")
        rstd = []
        for i, w in enumerate((nq_w, nk_w)):
            r = torch.empty((Sl,), dtype=torch.float32, device=xm.device)
            x = qkv[:, i * D:(i + 1) * D]
            rc = lib.solar_rmsnorm_rope_scatter(ptr(x), c_ll(x.stride(0)), ptr(w), ptr(rope), c_int(rope.shape[1]), ptr(r),
                                                c_ll(Sl), c_int(D), c_float(eps), c_int(0), stream_handle(), dst, flags,
                                                counter, c_int(P), c_ll(3 * dl), c_int(dl), c_int(row_off), c_int(i * dl))
            check(rc, "solar_rmsnorm_rope_scatter")
            count("rmsnorm_rope_scatter")
            rstd.append(r)
        heap.wait(slot, 3 * P)
        return qkv, rstd[0], rstd[1], self.recv[parity][:S]

    # step 3 -------------------------------------------------------------------------------
    def attention_exchange(self, recv, scale, parity):
        """recv [S, 3*dl] -> (o_heads [1,S,hp,hd], lse, o_tokens view [Sl, dim])."""
        lib = _lib.load()
        S = recv.shape[0]
        hp, hd, dl = self.heads // self.size, self.hd, self.dl
        q, k, v = recv[:, :dl], recv[:, dl:2 * dl], recv[:, 2 * dl:]
        o = torch.empty((1, S, hp, hd), dtype=recv.dtype, device=recv.device)
        lse = torch.empty((1, hp, S), dtype=torch.float32, device=recv.device)
        slot = self.flag_o[parity]
        heap = self.heap
        rc = lib.solar_attn_fwd_scatter(ptr(q), ptr(k), ptr(v), ptr(o), ptr(lse), c_int(S), c_int(S), c_int(hp), c_int(hd),
                                        c_ll(3 * dl), c_ll(3 * dl), c_ll(3 * dl), c_ll(hp * hd), c_float(scale),
                                        ptr(status_word(recv.device)), stream_handle(),
                                        heap.peer_ptr_array(self.obuf_off[parity]), heap.flag_ptrs(slot),
                                        heap.counter_ptr(slot), c_int(self.size), c_ll(self.dim), c_ll(self.max_local),
                                        self._row_start_c, c_int(self.rank * dl))
        check(rc, "solar_attn_fwd_scatter")
        count("attn_fwd_scatter")
        heap.wait(slot, self.size)
        Sl = self._row_start[self.rank + 1] - self._row_start[self.rank]
        return o, lse, self.obuf[parity][:Sl]

    # step 4' ------------------------------------------------------------------------------
    def dgrad_exchange(self, dy, w_o, parity):
        """dy [Sl, dim] (gradient of the out-projection output) -> dO view [S, dl] for this rank's heads: the dgrad
        GEMM ``dy @ W_o`` whose epilogue stores each 64-column chunk into the head owner's buffer."""
        lib = _lib.load()
        D, dl, P = self.dim, self.dl, self.size
        dy = F_._rowmajor(dy)
        Sl = dy.shape[0]
        heap = self.heap
        slot = self.flag_do[parity]
        rc = lib.solar_gemm_bf16_scatter(ptr(dy), ptr(w_o), ptr(dy), ptr(None), c_int(Sl), c_int(D), c_int(w_o.shape[0]),
                                         c_ll(dy.stride(0)), c_ll(w_o.stride(0)), c_ll(dy.stride(0)), c_int(F_.NN), c_int(0),
                                         ptr(status_word(dy.device)), c_int(0), stream_handle(),
                                         heap.peer_ptr_array(self.dobuf_off[parity]), heap.flag_ptrs(slot),
                                         heap.counter_ptr(slot), c_int(P), c_ll(dl), c_int(D), c_int(dl),
                                         c_int(self._row_start[self.rank]), c_int(0), c_int(0))
        check(rc, "solar_gemm_bf16_scatter")
        count("gemm_scatter")
        return slot

    # step 3' ------------------------------------------------------------------------------
    def attention_bwd_exchange(self, recv, o, lse, do, scale, parity):
        """Attention backward over this rank's heads; dq | dk | dv rows land in the token owners' buffers.
        Returns the local ``[Sl, 3 * dim]`` view (valid after the wait enqueued here)."""
        from ..ops.attention_bwd_native import ensure_tail_overlap_default

        ensure_tail_overlap_default()
        lib = _lib.load()
        S = recv.shape[0]
        hp, hd, dl, D = self.heads // self.size, self.hd, self.dl, self.dim
        q, k, v = recv[:, :dl], recv[:, dl:2 * dl], recv[:, 2 * dl:]
        sq_pad = (S + 127) // 128 * 128
        scratch = torch.empty(2 * hp * sq_pad, dtype=torch.float32, device=recv.device)
        heap = self.heap
        slot = self.flag_dqkv[parity]
        col = self.rank * dl
        rc = lib.solar_attn_bwd_scatter(ptr(q), ptr(k), ptr(v), ptr(o), ptr(do), ptr(lse), ptr(scratch), c_int(S), c_int(hp),
                                        c_int(hd), c_ll(3 * dl), c_ll(hp * hd), c_ll(do.stride(0)), c_float(scale),
                                        ptr(status_word(recv.device)), stream_handle(),
                                        heap.peer_ptr_array(self.dqkv_off[parity]), heap.flag_ptrs(slot),
                                        heap.counter_ptr(slot, 0), heap.counter_ptr(slot, 1), c_int(self.size),
                                        c_ll(3 * D), c_ll(self.max_local), self._row_start_c, c_int(col), c_int(D + col),
                                        c_int(2 * D + col))
        check(rc, "solar_attn_bwd_scatter")
        count("attn_bwd_scatter", 3)
        heap.wait(slot, 2 * self.size)                 # the dK/dV kernel and the dQ kernel of every rank
        Sl = self._row_start[self.rank + 1] - self._row_start[self.rank]
        return self.dqkv[parity][:Sl]

    # final sequence gather ------------------------------------------------------------------
    def _push_rows(self, x):
        lib = _lib.load()
        x = x.contiguous()
        heap, slot = self.heap, self.flag_seq
        S = self._row_start[-1]
        off = self._row_start[self.rank] * self.dim * 2
        rc = lib.solar_comm_push(ptr(x), heap.peer_ptr_array(self.seqbuf_off), c_int(self.size), c_ll(off),
                                 c_ll(x.numel() * 2), heap.flag_ptrs(slot), heap.counter_ptr(slot), stream_handle())
        check(rc, "solar_comm_push")
        count("comm_push")
        heap.wait(slot, self.size)
        return self.seqbuf[:S].clone()

    def gather_sequence(self, x, B: int):
        if not (x.is_cuda and B == 1 and x.dtype == torch.bfloat16 and x.shape[1] == self.dim):
            return super().gather_sequence(x, B)
        return _GatherSeqFused.apply(x, self)

    def close(self) -> None:
        self.heap.close()


class FusedSelfAttention(torch.autograd.Function):
    """Modulated input ``xm [Sl, dim]`` -> out-projection output ``[Sl, dim]`` of one self-attention layer; the four
    exchanges of the layer (two forward, two backward) ride on the kernels listed in the module docstring.
    Parameter gradients go to the flat ``main_grad`` buffers."""

    @staticmethod
    def forward(ctx, xm, w, b, nq_w, nk_w, rope, w_o, b_o, eps, scale, sp, parity, memo):
        grads_on = any(ctx.needs_input_grad)
        with span("sa.fwd.qkv_exchange"):
            qkv, rstd_q, rstd_k, recv = sp.qkv_exchange(xm, w, b, nq_w, nk_w, rope, eps, parity)
        cached = None if memo is None else memo[0].pop(memo[1], None)
        if cached is not None:                      # recompute under selective checkpointing: attention is carried
            o, lse, tokens = cached
        else:
            with span("sa.fwd.attention_exchange"):
                o, lse, view = sp.attention_exchange(recv, scale, parity)
            # the receive buffers are reused two layers later: what backward needs is copied out of them
            storing = memo is not None and memo[0].get("__store__", False)
            tokens = view.clone() if (grads_on or storing) else view
            if storing:
                memo[0][memo[1]] = (o, lse, tokens)
        y = F_.gemm(tokens, w_o, F_.NT, bias=b_o) if F_._forward_needed(w_o) else tokens.new_empty((tokens.shape[0], w_o.shape[0]))
        if grads_on:
            ctx.save_for_backward(xm, qkv, rstd_q, rstd_k, rope, nq_w, nk_w, recv.clone(), o, lse, tokens)
            ctx.misc = (w, b, w_o, b_o, sp, eps, scale)
        return y

    @staticmethod
    def backward(ctx, dy):
        xm, qkv, rstd_q, rstd_k, rope, nq_w, nk_w, recv, o, lse, tokens = ctx.saved_tensors
        w, b, w_o, b_o, sp, eps, scale = ctx.misc
        parity = sp.next_bwd_parity()
        D, dl = sp.dim, sp.dl
        hp, hd = sp.heads // sp.size, sp.hd
        Sl, S = xm.shape[0], recv.shape[0]
        lib = _lib.load()
        dy = F_._rowmajor(dy)
        # 4': dO leaves through the dgrad GEMM's epilogue; the weight / bias gradients run while it lands
        with span("sa.bwd.dgrad_exchange"):
            slot_do = F_.wgrad_beside(dy, tokens, w_o, lambda: sp.dgrad_exchange(dy, w_o, parity))
            if b_o is not None:
                F_.accumulate_main_grad(b_o, F_.colsum(dy))
            sp.heap.wait(slot_do, sp.size)
        do = sp.dobuf[parity][:S]
        # 3': attention backward, gradients scattered to the token owners
        with span("sa.bwd.attention_exchange"):
            g = sp.attention_bwd_exchange(recv, o, lse, do, scale, parity)      # [Sl, 3D]: dq | dk | dv, all heads
        # 2': norm + RoPE backward of the q and k blocks in place (the kernel reads a row completely before it writes)
        dws = []
        for i, (nw, rstd) in enumerate(((nq_w, rstd_q), (nk_w, rstd_k))):
            gi = g[:, i * D:(i + 1) * D]
            x = qkv[:, i * D:(i + 1) * D]
            splits = F_._splits_for(D, 1)
            part = torch.empty((splits, D), dtype=torch.float32, device=xm.device)
            rc = lib.solar_rmsnorm_rope_bwd(ptr(gi), c_ll(gi.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(gi),
                                            c_ll(gi.stride(0)), ptr(nw), ptr(rope), c_int(rope.shape[1]), ptr(rstd),
                                            ptr(part), c_int(splits), c_ll(Sl), c_int(D), c_int(0), stream_handle())
            check(rc, "solar_rmsnorm_rope_bwd")
            count("rmsnorm_rope_bwd")
            dws.append(part.sum(0))
        dxm = F_.wgrad_beside(g, xm, w, lambda: F_.gemm(g, w, F_.NN))
        F_.accumulate_main_grad(b, F_.colsum(g))
        return dxm, None, None, dws[0], dws[1], None, None, None, None, None, None, None, None
