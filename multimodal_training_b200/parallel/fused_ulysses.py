"""Ulysses (sequence <-> heads) exchange of the vision encoder's full-attention layers over peer memory.

``to_heads`` stores this rank's rows, head group by head group, straight into the owning peer's
[T_all, parts * W] buffer at the row's IMAGE-MAJOR position, so what arrives is already in the order
attention wants; ``to_tokens`` stores attention rows back into the token owner's [T_loc, parts * C]
buffer.  One kernel + one bounded flag wait each, instead of an NCCL all-to-all between two row
permutation passes (``models/vision.py``, library path) or the reference's six all-to-alls per layer
(modeling_qwen2_5_vl.py:628-640,744-746).  Rotary embedding is applied before the exchange, so
neither cos/sin nor masks travel.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch

from ..ops import functional as F
from ..ops import native as nv
from .fused import FusedComm, GemmCommC, PeerSetC

_P, _I, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_long
nv.declare("mmt_ulysses_to_heads", _I, [_P, _P, ctypes.POINTER(PeerSetC), _P, _I, _L, _I, _I, _I, _P])
nv.declare("mmt_ulysses_to_tokens", _I, [_P, _P, _P, ctypes.POINTER(PeerSetC), _P, _I, _L, _I, _I, _I, _I, _P])


class UlyssesFused:
    def __init__(self, fc: FusedComm):
        self.fc = fc
        m = fc.mesh
        self.sp, self.sp_rank = m.sp, m.sp_rank
        self.ranks = [m.vdp_rank * m.sp + i for i in range(m.sp)]     # heap ranks of my sequence-parallel group
        self._dummies: dict[int, torch.Tensor] = {}
        # full-attention layers as one autograd node with the exchanges inside the GEMMs (ops/ulysses_block.py)
        self.one_node = os.environ.get("MMT_ULYSSES_BLOCK", "1") == "1"

    def _routes(self, plan, device):
        r = getattr(plan, "_ulysses", None)
        if r is None:
            off = np.concatenate([[0], np.cumsum(plan.rank_tokens)])
            inv = plan.to_rank_major.numpy()            # exchange-order row -> image-major position
            fwd = plan.to_image_major.numpy()           # image-major position -> exchange-order row
            me = self.sp_rank
            dst_row = inv[off[me]:off[me + 1]].astype(np.int32)
            owner = (np.searchsorted(off, fwd, side="right") - 1).astype(np.int32)
            row_local = (fwd - off[owner]).astype(np.int32)
            r = {"dst_row": torch.from_numpy(dst_row).to(device), "owner": torch.from_numpy(owner).to(device),
                 "row_local": torch.from_numpy(row_local).to(device), "t_all": int(off[-1]),
                 "t_loc_max": int(max(plan.rank_tokens))}
            plan._ulysses = r
        return r

    def rope_tables(self, plan, device):
        """cos / sin [T_all, head_dim] of every row of the gathered sequence (image-major order = window order of all
        patches): the head owner rotates rows that the QKV epilogue delivered un-rotated."""
        t = getattr(plan, "_ulysses_rope", None)
        if t is None:
            from .sp import rope_table
            cos, sin = rope_table(plan.all_pos, plan.head_dim)
            t = (cos.to(device), sin.to(device))
            plan._ulysses_rope = t
        return t

    # ------------------------------------------------------------------ exchanges fused into GEMMs
    def gemm_scatter(self, a: torch.Tensor, w: torch.Tensor, bias, parts: int, routes, name: str, b_mn: bool = False):
        """``a @ w^T (+ bias)`` whose epilogue stores column block r of each of the ``parts`` output blocks straight
        into rank r's [T_all, parts * W] buffer at the row's image-major position (sequence -> heads exchange inside
        the GEMM).  Returns this rank's buffer once every peer's rows have landed."""
        fc, ctx = self.fc, self.fc.ctx
        N = w.shape[1] if b_mn else w.shape[0]
        C = N // parts
        W = C // self.sp
        off, local = fc._region(name, (routes["t_all"], parts * W))
        slot = ctx.slot(name)
        epoch = ctx.next_epoch(slot)
        c = GemmCommC()
        c.rs_rows, c.rs_self, c.rs_ranks, c.rs_epoch = 0, self.sp_rank, self.sp, epoch
        c.rs_counter = ctx.counter_addr(slot)
        for i, r in enumerate(self.ranks):
            c.rs_base[i] = ctx.heap.ptrs[r] + off
            c.rs_flag[i] = ctx.flag_addr(r, slot, self.sp_rank)
        c.sc_row, c.sc_part, c.sc_w = routes["dst_row"].data_ptr(), C, W
        c.sc_ld, c.sc_rows_dst = parts * W, routes["t_all"]
        dummy = self._dummies.get(N)
        if dummy is None:
            dummy = self._dummies[N] = torch.empty(8, N, device=a.device, dtype=torch.bfloat16)
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(a, w, b_mn=b_mn, bias=bias, out=dummy)          # C itself is not written
        nv.call("mmt_wait_flags", ctx.local_flags(slot), self.sp, -1, epoch, nv.stream())
        return local

    def to_tokens_nowait(self, src: torch.Tensor, W: int, routes, name: str):
        """heads -> sequence exchange of [T_all, W] rows without the wait: returns (this rank's [T_loc_max, sp * W]
        buffer, flag words, epoch) for a GEMM that consumes the buffer's K slices behind the flags."""
        fc, ctx = self.fc, self.fc.ctx
        off, local = fc._region(name, (routes["t_loc_max"], W * self.sp))
        slot = ctx.slot(name)
        epoch = ctx.next_epoch(slot)
        ps = ctx.peerset(off, self.ranks, slot, self.sp_rank)
        src = src.contiguous()
        nv.call("mmt_ulysses_to_tokens", src.data_ptr(), routes["owner"].data_ptr(), routes["row_local"].data_ptr(),
                ctypes.byref(ps), ctx.counter_addr(slot), epoch, src.shape[0], 1, self.sp, self.sp_rank, W, nv.stream())
        return local, ctx.local_flags(slot), epoch

    def gemm_k_slices(self, a: torch.Tensor, w: torch.Tensor, bias, residual, flags_ptr: int, epoch: int, W: int):
        """``a @ w^T (+ bias + residual)`` where columns [s * W, (s + 1) * W) of ``a`` were written by rank s: the GEMM
        starts on its own slice and waits per source before it loads a peer's (heads -> sequence exchange as the
        GEMM's prologue)."""
        c = GemmCommC()
        c.rs_rows = 0
        c.kf_flags, c.kf_epoch, c.kf_w, c.kf_self, c.kf_ranks = flags_ptr, epoch, W, self.sp_rank, self.sp
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        return F.gemm(a, w, bias=bias, residual=residual)

    def _exchange(self, kind: str, src: torch.Tensor, parts: int, W: int, routes, name: str) -> torch.Tensor:
        fc, ctx = self.fc, self.fc.ctx
        C = W * self.sp
        if kind == "heads":
            shape = (routes["t_all"], parts * W)
        else:
            shape = (routes["t_loc_max"], parts * C)
        off, local = fc._region(name, shape)
        slot = ctx.slot(name)
        epoch = ctx.next_epoch(slot)
        ps = ctx.peerset(off, self.ranks, slot, self.sp_rank)
        src = src.contiguous()
        if kind == "heads":
            nv.call("mmt_ulysses_to_heads", src.data_ptr(), routes["dst_row"].data_ptr(), ctypes.byref(ps),
                    ctx.counter_addr(slot), epoch, src.shape[0], parts, self.sp, W, nv.stream())
        else:
            nv.call("mmt_ulysses_to_tokens", src.data_ptr(), routes["owner"].data_ptr(),
                    routes["row_local"].data_ptr(), ctypes.byref(ps), ctx.counter_addr(slot), epoch, src.shape[0],
                    parts, self.sp, self.sp_rank, W, nv.stream())
        nv.call("mmt_wait_flags", ctx.local_flags(slot), self.sp, -1, epoch, nv.stream())
        return local

    def ulysses_attention(self, qkv: torch.Tensor, plan, full_seq, n_heads: int, dim: int) -> torch.Tensor:
        hl = n_heads // self.sp
        x = _ToHeads.apply(qkv, 3, hl * dim, plan, self)                 # [T_all, 3*hl*dim], image-major
        a = F.attention(x, hl, hl, dim, full_seq, causal=False)         # [T_all, hl*dim]
        return _ToTokens.apply(a, 1, hl * dim, plan, self)              # [T_loc, n_heads*dim]


class _ToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, parts, W, plan, uf: UlyssesFused):
        routes = uf._routes(plan, x.device)
        out = uf._exchange("heads", x, parts, W, routes, f"ul_heads{parts}")
        ctx.misc = (parts, W, plan, uf, x.shape[0])
        return out if uf.fc.checkpointed else out.clone()

    @staticmethod
    def backward(ctx, dy):
        parts, W, plan, uf, t_loc = ctx.misc
        routes = uf._routes(plan, dy.device)
        back = uf._exchange("tokens", dy, parts, W, routes, f"ul_tokens{parts}_bwd")
        return back[:t_loc].clone(), None, None, None, None


class _ToTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, parts, W, plan, uf: UlyssesFused):
        routes = uf._routes(plan, a.device)
        t_loc = plan.rank_tokens[uf.sp_rank]
        out = uf._exchange("tokens", a, parts, W, routes, f"ul_tokens{parts}")[:t_loc]
        ctx.misc = (parts, W, plan, uf)
        return out if uf.fc.checkpointed else out.clone()

    @staticmethod
    def backward(ctx, dy):
        parts, W, plan, uf = ctx.misc
        routes = uf._routes(plan, dy.device)
        back = uf._exchange("heads", dy, parts, W, routes, f"ul_heads{parts}_bwd")
        return back.clone(), None, None, None, None
