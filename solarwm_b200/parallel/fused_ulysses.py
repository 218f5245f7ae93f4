"""Ulysses exchanges fused into the producing kernels (NVLink peer stores, no NCCL on the forward path).

Forward of one attention layer at SP = P, tokens sharded by whole frames, heads by rank:

  1. QKV projection GEMM (tcgen05).  Its epilogue stores the V columns straight into the receive
     buffer of the rank that owns each head (``solar_gemm_bf16_scatter``); Q and K columns stay local
     because Wan normalises them over the full width first.
  2. full-width RMSNorm + RoPE of Q and of K (row kernel) whose output stage is the same column
     scatter (``solar_rmsnorm_rope_scatter``).  Every rank now holds ``[S, q_loc | k_loc | v_loc]``.
  3. flash attention over the local heads and the whole sequence; its epilogue stores each output
     row into the token owner's ``[S_local, dim]`` buffer (``solar_attn_fwd_scatter``).
  4. the out-projection GEMM reads that buffer.

Each producer kernel's last CTA adds 1 to a flag word on every rank; consumers are preceded on the
stream by a bounded device-side wait for ``3 * P`` (step 2) or ``P`` (step 3) new signals.  Receive
buffers are double-buffered by layer parity, which is sufficient because every layer's wait depends
on every peer having finished the previous layer's consumer.

The backward pass exchanges gradients with the collective transport of the parent class (the
reverse all-to-all), and so does everything on CPU.  The reference performs steps 1-3 as three
``nn.Linear`` + two norms + RoPE + three ``all_to_all_single`` with packing copies, and one more
all-to-all after attention (solar/backends/wan22/runtime/modeling/causal_model.py:878-1027,
sequence_parallel.py:446-524).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib, functional as F_
from ..ops._lib import c_float, c_int, c_ll, check, count, ptr, stream_handle
from ..ops.functional import status_word
from .symm import SymmetricHeap
from .ulysses import UlyssesCollective, _AllToAll


class FusedUlysses(UlyssesCollective):
    fused = True

    def __init__(self, group: Optional[dist.ProcessGroup], *, max_tokens: int, dim: int, num_heads: int):
        super().__init__(group)
        P = self.size
        if num_heads % P:
            raise ValueError(f"num_heads={num_heads} must be divisible by sp_size={P}")
        self.dim, self.heads, self.hd = dim, num_heads, dim // num_heads
        self.dl = dim // P                       # columns of one rank's head block
        self.max_tokens = int(max_tokens)
        max_local = (self.max_tokens + P - 1) // P + 4096
        need = 2 * self.max_tokens * 3 * self.dl * 2 + 2 * max_local * dim * 2 + 4096
        self.heap = SymmetricHeap(need, group)
        self.recv, self.recv_off, self.obuf, self.obuf_off = [], [], [], []
        for _ in range(2):
            t, off = self.heap.alloc((self.max_tokens, 3 * self.dl))
            self.recv.append(t)
            self.recv_off.append(off)
        for _ in range(2):
            t, off = self.heap.alloc((max_local, dim))
            self.obuf.append(t)
            self.obuf_off.append(off)
        self.flag_qkv = [self.heap.new_flag() for _ in range(2)]
        self.flag_o = [self.heap.new_flag() for _ in range(2)]
        self._parity = 0
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
        self._row_start = starts
        self._row_start_c = (ctypes.c_int * (self.size + 1))(*starts)

    def next_parity(self) -> int:
        self._parity ^= 1
        return self._parity

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
        heap.wait(slot, heap.expect(slot, 3 * P))
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
                                        heap.counter_ptr(slot), c_int(self.size), c_ll(self.dim), self._row_start_c,
                                        c_int(self.rank * dl))
        check(rc, "solar_attn_fwd_scatter")
        count("attn_fwd_scatter")
        heap.wait(slot, heap.expect(slot, self.size))
        Sl = self._row_start[self.rank + 1] - self._row_start[self.rank]
        return o, lse, self.obuf[parity][:Sl]

    # reverse exchanges for the backward pass (collective transport) -------------------------
    def heads_to_tokens_grad(self, d_recv):
        """d_recv [S, 3*dl] (this rank's heads, all tokens) -> [Sl, 3, dim] (this rank's tokens, all heads)."""
        _, seq = self._layout
        P, hp, hd = self.size, self.heads // self.size, self.hd
        Sl = seq[self.rank]
        x = d_recv.reshape(-1, 3, hp, hd)
        out = _AllToAll.apply(x, list(seq), [Sl] * P, self.group)          # [P*Sl, 3, hp, hd], source-major
        return out.view(P, Sl, 3, hp * hd).permute(1, 2, 0, 3).reshape(Sl, 3, P * hp * hd)

    def tokens_to_heads_grad(self, d_tokens):
        """d_tokens [Sl, dim] -> [S, dl] (gradient of the attention output in head layout)."""
        _, seq = self._layout
        P, dl = self.size, self.dl
        Sl = d_tokens.shape[0]
        x = d_tokens.view(Sl, P, dl).permute(1, 0, 2).reshape(P * Sl, dl)
        return _AllToAll.apply(x, [Sl] * P, list(seq), self.group)        # [S, dl]

    def close(self) -> None:
        self.heap.close()


class FusedQKV(torch.autograd.Function):
    """xm -> received [S, q_loc|k_loc|v_loc]; forward = steps 1-2 above, backward = reverse all-to-all,
    RMSNorm/RoPE backward, dgrad and wgrad GEMMs (gradients go to the flat ``main_grad`` buffers)."""

    @staticmethod
    def forward(ctx, xm, w, b, nq_w, nk_w, rope, eps, sp, parity, anchors):
        qkv, rstd_q, rstd_k, recv = sp.qkv_exchange(xm, w, b, nq_w, nk_w, rope, eps, parity)
        # with autograd the receive buffer (reused two layers later) cannot be the saved tensor
        out = recv.clone() if any(ctx.needs_input_grad) else recv
        ctx.save_for_backward(xm, qkv, rstd_q, rstd_k, rope, nq_w, nk_w)
        ctx.misc = (w, b, sp, eps, anchors)
        return out

    @staticmethod
    def backward(ctx, d_recv):
        xm, qkv, rstd_q, rstd_k, rope, nq_w, nk_w = ctx.saved_tensors
        w, b, sp, eps, anchors = ctx.misc
        D = sp.dim
        Sl = xm.shape[0]
        g = sp.heads_to_tokens_grad(d_recv.contiguous())                    # [Sl, 3, D]
        dqkv = torch.empty((Sl, 3 * D), dtype=xm.dtype, device=xm.device)
        lib = _lib.load()
        dws = []
        for i, (nw, rstd) in enumerate(((nq_w, rstd_q), (nk_w, rstd_k))):
            dy = g[:, i].contiguous()
            x = qkv[:, i * D:(i + 1) * D]
            dx = dqkv[:, i * D:(i + 1) * D]
            splits = F_._splits_for(D, 1)
            part = torch.empty((splits, D), dtype=torch.float32, device=xm.device)
            rc = lib.solar_rmsnorm_rope_bwd(ptr(dy), c_ll(dy.stride(0)), ptr(x), c_ll(x.stride(0)), ptr(dx),
                                            c_ll(dx.stride(0)), ptr(nw), ptr(rope), c_int(rope.shape[1]), ptr(rstd),
                                            ptr(part), c_int(splits), c_ll(Sl), c_int(D), c_int(0), stream_handle())
            check(rc, "solar_rmsnorm_rope_bwd")
            count("rmsnorm_rope_bwd")
            dws.append(part.sum(0))
        dqkv[:, 2 * D:] = g[:, 2]
        dxm = F_.gemm(dqkv, w, F_.NN)
        F_.gemm(dqkv, xm, F_.TN, out=w.main_grad, accumulate=F_._grad_is_live(w))
        F_._mark_grad_live(w)
        F_.accumulate_main_grad(b, F_.colsum(dqkv))
        return dxm, None, None, dws[0], dws[1], None, None, None, None, None


class FusedAttention(torch.autograd.Function):
    """received q|k|v -> attention output in token layout [Sl, dim]; forward = step 3, backward =
    reverse all-to-all of the output gradient + the attention backward kernels."""

    @staticmethod
    def forward(ctx, recv, scale, sp, parity, memo):
        cached = None if memo is None else memo[0].pop(memo[1], None)
        if cached is not None:
            o, lse, tokens = cached
        else:
            o, lse, view = sp.attention_exchange(recv, scale, parity)
            tokens = view.clone() if any(ctx.needs_input_grad) else view
            if memo is not None and memo[0].get("__store__", False):
                memo[0][memo[1]] = (o, lse, tokens)
        ctx.save_for_backward(recv, o, lse)
        ctx.misc = (scale, sp)
        return tokens

    @staticmethod
    def backward(ctx, d_tokens):
        from ..ops.attention_native import attn_bwd

        recv, o, lse = ctx.saved_tensors
        scale, sp = ctx.misc
        S = recv.shape[0]
        hp, hd, dl = sp.heads // sp.size, sp.hd, sp.dl
        do = sp.tokens_to_heads_grad(d_tokens.contiguous()).view(1, S, hp, hd)
        q = recv[:, :dl].view(1, S, hp, hd)
        k = recv[:, dl:2 * dl].view(1, S, hp, hd)
        v = recv[:, 2 * dl:].view(1, S, hp, hd)
        dq, dk, dv = attn_bwd(q, k, v, o, lse, do, scale)
        d_recv = torch.cat([dq.reshape(S, dl), dk.reshape(S, dl), dv.reshape(S, dl)], dim=1)
        return d_recv, None, None, None, None
