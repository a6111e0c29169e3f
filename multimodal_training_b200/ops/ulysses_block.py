"""One full-attention vision layer under sequence parallelism as ONE autograd node, with the Ulysses exchanges
inside the GEMMs (GPU, sequence-parallel size > 1).

    qkv_h = scatter( rmsnorm(x) @ Wqkv^T + b )     QKV projection whose epilogue stores every head group's columns
                                                   straight into the owning rank's [T_all, 3 * W] buffer at the
                                                   row's image-major position (sequence -> heads)
    a_h   = attention( rope(qkv_h) )               over all rows, this rank's heads; the owner rotates
    a_tok = to_tokens(a_h)                         rows back into the token owner's [T_loc, C] buffer (no wait)
    x1    = x + a_tok @ Wproj^T + b                output projection that starts on its own K slice and waits per
                                                   source rank before it loads a peer's (heads -> sequence)
    y     = x1 + mlp(rmsnorm(x1))                  as in ops/blocks.py

Backward walks the chain by hand: the output projection's input gradient is again a GEMM with the scatter epilogue
(one column block), the attention backward runs on the head owner, the q|k|v gradient goes back through the
heads -> sequence kernel.  Replaces, per layer, the reference's six all-to-alls in and one out with their padded
buffers (python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:628-640, 744-746) and this package's per-op graph for
these layers (models/vision.py::_block).
"""
from __future__ import annotations

import torch

from . import functional as F
from .attention import SeqInfo
from .blocks import (BlockSpec, _attn_bwd, _attn_fwd, _grad_into, _linear_bwd, _rmsnorm_bwd, _rmsnorm_fwd, _rope_,
                     _swiglu_bwd, _swiglu_fwd)


def _forward_chain(uf, x, s: BlockSpec, sh: BlockSpec, plan, seq, P, keep: bool):
    """``s`` describes all heads (local rows), ``sh`` this rank's heads (all rows)."""
    ln1_w, qkv_w, qkv_b, proj_w, proj_b, ln2_w, gu_w, gu_b, down_w, down_b = P
    routes = uf._routes(plan, x.device)
    cos, sin = uf.rope_tables(plan, x.device)
    W = sh.n_q * sh.head_dim
    t_loc = x.shape[0]
    h1, rstd1 = _rmsnorm_fwd(x, ln1_w, s.eps)
    qkv_h = uf.gemm_scatter(h1, qkv_w, qkv_b, 3, routes, "ul_heads3")
    _rope_(qkv_h, cos, sin, sh.rope_heads, sh.head_dim, False)
    if keep:
        qkv_h = qkv_h.clone()            # the region is rewritten by the next full-attention layer
    a_h, lse = _attn_fwd(qkv_h, sh, seq)
    a_tok, flags, epoch = uf.to_tokens_nowait(a_h, W, routes, "ul_tokens1")
    a_tok = a_tok[:t_loc]
    x1 = uf.gemm_k_slices(a_tok, proj_w, proj_b, x, flags, epoch, W)
    if keep:
        a_tok = a_tok.clone()
    h2, rstd2 = _rmsnorm_fwd(x1, ln2_w, s.eps)
    gu = F.gemm(h2, gu_w, bias=gu_b)
    m = _swiglu_fwd(gu)
    y = F.gemm(m, down_w, bias=down_b, residual=x1)
    return y, (h1, rstd1, qkv_h, a_h, lse, a_tok, x1, h2, rstd2, gu, m)


class _UlyssesBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec, spec_h, plan, seq, recompute, uf, *params):
        x = x if x.is_contiguous() else x.contiguous()
        y, kept = _forward_chain(uf, x, spec, spec_h, plan, seq, params, keep=not recompute)
        extra = ()
        if not recompute:
            h1, rstd1, qkv_h, a_h, lse, a_tok, x1, h2, rstd2, gu, m = kept
            extra = (rstd1, qkv_h, a_h, lse, a_tok, x1, rstd2, gu)      # h1, h2, m are rebuilt (cheap kernels)
        ctx.n_extra = len(extra)
        ctx.save_for_backward(x, *extra, *[p for p in params if p is not None])
        ctx.has = [p is not None for p in params]
        ctx.misc = (spec, spec_h, plan, seq, uf)
        return y

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        x = saved[0]
        extra = saved[1:1 + ctx.n_extra]
        it = iter(saved[1 + ctx.n_extra:])
        P = tuple(next(it) if h else None for h in ctx.has)
        s, sh, plan, seq, uf = ctx.misc
        ln1_w, qkv_w, qkv_b, proj_w, proj_b, ln2_w, gu_w, gu_b, down_w, down_b = P
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if ctx.n_extra:
            rstd1, qkv_h, a_h, lse, a_tok, x1, rstd2, gu = extra
            h1, _ = _rmsnorm_fwd(x, ln1_w, s.eps)
            h2, _ = _rmsnorm_fwd(x1, ln2_w, s.eps)
            m = _swiglu_fwd(gu)
        else:
            # recomputation repeats the forward chain, exchanges included, on every rank alike; the heap views it
            # returns are read below before this layer's backward exchanges let any peer move on
            _, (h1, rstd1, qkv_h, a_h, lse, a_tok, x1, h2, rstd2, gu, m) = _forward_chain(uf, x, s, sh, plan, seq, P,
                                                                                          keep=False)
        routes = uf._routes(plan, x.device)
        cos, sin = uf.rope_tables(plan, x.device)
        W = sh.n_q * sh.head_dim
        t_loc = x.shape[0]
        # MLP half
        dm = _linear_bwd(dy, m, down_w, down_b)
        dgu = _swiglu_bwd(dm, gu)
        dh2 = _linear_bwd(dgu, h2, gu_w, gu_b)
        dx1 = _rmsnorm_bwd(dh2, x1, ln2_w, rstd2, dy)
        # output projection: weight / bias gradients read the gathered attention rows, the input gradient leaves
        # through the scatter epilogue (one column block) towards the head owners
        _grad_into(proj_w, lambda out, acc: F.gemm(dx1, a_tok, a_mn=True, b_mn=True, out=out, accumulate=acc))
        if proj_b is not None:
            _grad_into(proj_b, lambda out, acc: F.colsum(dx1, out=out, accumulate=acc))
        da_h = uf.gemm_scatter(dx1, proj_w, None, 1, routes, "ul_heads1_bwd", b_mn=True)
        dqkv_h = _attn_bwd(qkv_h, a_h, da_h, lse, sh, seq)
        _rope_(dqkv_h, cos, sin, sh.rope_heads, sh.head_dim, True)
        dqkv = uf._exchange("tokens", dqkv_h, 3, W, routes, "ul_tokens3_bwd")[:t_loc]
        dh1 = _linear_bwd(dqkv, h1, qkv_w, qkv_b)
        dx = _rmsnorm_bwd(dh1, x, ln1_w, rstd1, dx1)
        return (dx, None, None, None, None, None, None) + (None,) * len(ctx.has)


def ulysses_block(x: torch.Tensor, spec: BlockSpec, plan, seq: SeqInfo, uf, params: tuple,
                  recompute: bool = True) -> torch.Tensor:
    """``params`` as in :func:`ops.blocks.local_block`; ``x`` is this rank's [T_loc, C] rows; ``seq`` describes the
    gathered (image-major) sequence; ``uf`` the process's :class:`parallel.fused_ulysses.UlyssesFused`.  Every rank of
    the sequence-parallel group must call this for the same layer at the same point of its stream order."""
    hl = spec.n_q // uf.sp
    spec_h = BlockSpec(n_q=hl, n_kv=hl, head_dim=spec.head_dim, rope_heads=2 * hl, causal=False, eps=spec.eps,
                       scale=spec.scale)
    return _UlyssesBlockFn.apply(x, spec, spec_h, plan, seq, bool(recompute), uf, *params)
