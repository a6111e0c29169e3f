"""One tensor-parallel decoder layer as ONE autograd node over the fused peer-memory paths (GPU, TP > 1).

The layer works on token shards (sequence-parallel tensor parallelism):

    x1 = x  + reduce_scatter( attention(rope(all_gather(rmsnorm(x))  @ Wqkv^T + b)) @ Wo^T )
    y  = x1 + reduce_scatter( swiglu(all_gather(rmsnorm(x1)) @ Wgu^T)               @ Wd^T )

with every all-gather fused into the GEMM that consumes it and every reduce-scatter fused into the epilogue of the
GEMM that produces it (``parallel/fused.py``).  Built from the per-op autograd functions under an activation
checkpoint this is about forty graph nodes per layer and two passes through the autograd engine; here the same
kernels and exchanges are issued directly, forward and backward, exactly as ``ops/blocks.py`` does for layers without
communication.  The per-op path (``models/text.py::_layer``) stays the oracle: the 2-GPU test trains with both and
compares the losses.

Order matters in backward: a weight-gradient GEMM that reads a gathered input runs BEFORE the exchange that lets the
peers move on, because the gathered input lives in a heap region that a peer overwrites in its next forward.

Replaces the reference's DTensor plan for the decoder layer (python/ray/text.py:1165-1177: replicated activations,
an all-reduce after o_proj and down_proj, up to five all-reduces of input gradients in backward).
"""
from __future__ import annotations

import torch

from . import functional as F
from .attention import SeqInfo
from .blocks import (BlockSpec, _attn_bwd, _attn_fwd, _grad_into, _rmsnorm_bwd, _rope_, _swiglu_bwd, _swiglu_fwd)


def _col_fwd(fc, x_shard, norm_w, eps, w, b, role, keep: bool):
    """(RMSNorm ->) all-gather -> GEMM.  Returns (y, gathered input, rstd); the gathered input is a private copy
    when it has to outlive the heap region (activations kept for backward)."""
    if fc.fused_ag:
        y, gathered, rstd = fc.ag_gemm(x_shard, norm_w, eps, w, role=role, bias=b)
    else:
        rows = x_shard.shape[0]
        gathered, rstd, flags, epoch = fc.push_gather(x_shard, norm_w, eps, role)
        y = fc.gemm_gathered(gathered, flags, epoch, rows, w, bias=b)
    return y, (gathered.clone() if keep else gathered), rstd


def _row_bwd(fc, dy_shard, a, w, role):
    """Backward of ``reduce_scatter(a @ w^T)``: gather the output gradient, input gradient through the gathered
    GEMM, weight gradient from the same gathered rows."""
    if fc.fused_ag:
        da, gathered, _ = fc.ag_gemm(dy_shard, None, 0.0, w, role=role + "_bwd", b_mn=True)
    else:
        rows = dy_shard.shape[0]
        gathered, _, flags, epoch = fc.push_gather(dy_shard, None, 0.0, role + "_bwd")
        da = fc.gemm_gathered(gathered, flags, epoch, rows, w, b_mn=True)
    _grad_into(w, lambda out, acc: F.gemm(gathered, a, a_mn=True, b_mn=True, out=out, accumulate=acc))
    return da


def _col_bwd(fc, dy, gathered, w, b, role):
    """Backward of ``all_gather(h) @ w^T + b``: weight / bias gradients first (they read the gathered input), then
    the input gradient reduce-scattered back to token shards."""
    _grad_into(w, lambda out, acc: F.gemm(dy, gathered, a_mn=True, b_mn=True, out=out, accumulate=acc))
    if b is not None:
        _grad_into(b, lambda out, acc: F.colsum(dy, out=out, accumulate=acc))
    return fc.gemm_reduce_scatter(dy, w, b_mn=True, residual=None, role=role + "_bwd")


def _forward_chain(fc, x, s: BlockSpec, cos, sin, seq, P, keep: bool):
    ln1_w, qkv_w, qkv_b, o_w, ln2_w, gu_w, down_w = P
    qkv, g1, rstd1 = _col_fwd(fc, x, ln1_w, s.eps, qkv_w, qkv_b, "qkv", keep)
    _rope_(qkv, cos, sin, s.rope_heads, s.head_dim, False)
    a, lse = _attn_fwd(qkv, s, seq)
    x1 = fc.gemm_reduce_scatter(a, o_w, b_mn=False, residual=x, role="o")
    gu, g2, rstd2 = _col_fwd(fc, x1, ln2_w, s.eps, gu_w, None, "mlp", keep)
    m = _swiglu_fwd(gu)
    y = fc.gemm_reduce_scatter(m, down_w, b_mn=False, residual=x1, role="down")
    return y, (g1, rstd1, qkv, a, lse, x1, g2, rstd2, gu, m)


class _TPBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec, cos, sin, seq, recompute, fc, *params):
        # recompute: True = keep only the layer input (activation checkpointing: backward repeats the forward chain,
        # exchanges included, on every rank alike); False = keep what backward needs, with private copies of the two
        # gathered inputs (the heap regions they arrived in are reused by the next layer)
        x = x if x.is_contiguous() else x.contiguous()
        y, kept = _forward_chain(fc, x, spec, cos, sin, seq, params, keep=not recompute)
        extra = ()
        if not recompute:
            g1, rstd1, qkv, a, lse, x1, g2, rstd2, gu, m = kept
            extra = (g1, rstd1, qkv, a, lse, x1, g2, rstd2, gu)          # m is rebuilt from gu (one cheap kernel)
        ctx.n_extra = len(extra)
        ctx.save_for_backward(x, cos, sin, *extra, *[p for p in params if p is not None])
        ctx.has = [p is not None for p in params]
        ctx.spec, ctx.seq, ctx.fc = spec, seq, fc
        return y

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        x, cos, sin = saved[0], saved[1], saved[2]
        extra = saved[3:3 + ctx.n_extra]
        it = iter(saved[3 + ctx.n_extra:])
        P = tuple(next(it) if h else None for h in ctx.has)
        s, seq, fc = ctx.spec, ctx.seq, ctx.fc
        ln1_w, qkv_w, qkv_b, o_w, ln2_w, gu_w, down_w = P
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if ctx.n_extra:
            g1, rstd1, qkv, a, lse, x1, g2, rstd2, gu = extra
            m = _swiglu_fwd(gu)
        else:
            _, (g1, rstd1, qkv, a, lse, x1, g2, rstd2, gu, m) = _forward_chain(fc, x, s, cos, sin, seq, P, keep=False)
        # MLP half
        dm = _row_bwd(fc, dy, m, down_w, "down")
        dgu = _swiglu_bwd(dm, gu)
        dh2 = _col_bwd(fc, dgu, g2, gu_w, None, "mlp")
        dx1 = _rmsnorm_bwd(dh2, x1, ln2_w, rstd2, dy)
        # attention half
        da = _row_bwd(fc, dx1, a, o_w, "o")
        dqkv = _attn_bwd(qkv, a, da, lse, s, seq)
        _rope_(dqkv, cos, sin, s.rope_heads, s.head_dim, True)
        dh1 = _col_bwd(fc, dqkv, g1, qkv_w, qkv_b, "qkv")
        dx = _rmsnorm_bwd(dh1, x, ln1_w, rstd1, dx1)
        return (dx, None, None, None, None, None, None) + (None,) * len(ctx.has)


def tp_block(x_shard: torch.Tensor, spec: BlockSpec, cos: torch.Tensor, sin: torch.Tensor, seq: SeqInfo, fc,
             params: tuple, recompute: bool = True) -> torch.Tensor:
    """``params`` = (ln1_w, qkv_w, qkv_b, o_w, ln2_w, gate_up_w, down_w) of this rank's shard; ``x_shard`` is the
    [T/tp, H] token shard (bf16, GPU); ``fc`` the process's :class:`parallel.fused.FusedComm`.  ``spec`` counts the
    LOCAL heads.  Every rank of the tensor-parallel group must call this for the same layer at the same point of its
    stream order (the exchanges inside are collective)."""
    return _TPBlockFn.apply(x_shard, spec, cos, sin, seq, bool(recompute), fc, *params)
