"""One transformer block as ONE autograd node with a hand-written backward (GPU path).

A pre-norm block without communication inside it,

    x1 = x  + proj(attention(rope(qkv(rmsnorm(x)))))
    y  = x1 + down(swiglu(gate_up(rmsnorm(x1))))

is what the vision encoder runs in its window-attention layers at any sequence-parallel size (and in its
full-attention layers when one rank holds the whole image) and what the text decoder runs when it is not
tensor parallel.  Built from the per-op autograd functions of :mod:`.functional` under an activation
checkpoint, such a block costs about forty graph nodes and two passes through the autograd engine per step,
and on a B200 the HOST then needs as long to enqueue a training step as the GPU needs to run it.  This module
issues the same kernels directly:

* forward keeps the block input only (activation checkpointing) or, when memory allows, also the GEMM and
  attention results;
* backward recomputes what was not kept and walks the chain by hand, writing weight gradients straight into
  the parameters' ``main_grad`` views of the flat gradient buffer.

The arithmetic, kernel by kernel, is identical to the per-op path, which stays in use on the CPU, for blocks
with communication inside (Ulysses layers, tensor-parallel layers) and as the oracle of the tests.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import functional as F
from . import native as nv
from .attention import SeqInfo


@dataclass(frozen=True)
class BlockSpec:
    n_q: int
    n_kv: int
    head_dim: int
    rope_heads: int          # leading heads of the fused q|k|v buffer that are rotated (q and k heads)
    causal: bool
    eps: float
    scale: float


def _rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float):
    rows, cols = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    nv.call("mmt_rmsnorm_fwd", x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, eps, nv.stream())
    return y, rstd


def _rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, rstd: torch.Tensor,
                 extra: torch.Tensor) -> torch.Tensor:
    """Gradient of the norm's input plus ``extra`` (the gradient arriving through the residual connection)."""
    rows, cols = x.shape
    dx = torch.empty_like(x)
    parts = nv.lib().mmt_rmsnorm_bwd_parts(rows)
    scratch = F._scratch_f32(parts * cols, x.device, "rmsnorm")

    def run(out, acc):
        nv.call("mmt_rmsnorm_bwd_add", dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), extra.data_ptr(),
                dx.data_ptr(), out.data_ptr(), scratch.data_ptr(), rows, cols, int(acc), nv.stream())

    _grad_into(w, run)
    return dx


def _grad_into(p: torch.Tensor, compute) -> None:
    """Parameter gradient: into ``main_grad`` (flat buffer) when the parameter has one, else accumulated in .grad."""
    g = F._write_param_grad(p, compute)
    if g is not None:
        p.grad = g if p.grad is None else p.grad + g


def _rope_(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int, dim: int, inverse: bool) -> None:
    nv.call("mmt_rope", t.data_ptr(), cos.data_ptr(), sin.data_ptr(), t.shape[0], heads, dim, t.stride(0),
            int(inverse), nv.stream())


def _attn_fwd(qkv: torch.Tensor, s: BlockSpec, seq: SeqInfo):
    T = qkv.shape[0]
    lo, hi = seq.bounds()
    out = torch.empty(T, s.n_q * s.head_dim, device=qkv.device, dtype=qkv.dtype)
    lse = torch.empty(s.n_q, T, device=qkv.device, dtype=torch.float32)
    nv.call("mmt_attn_fwd", qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), lo.data_ptr(), hi.data_ptr(), T, s.n_q,
            s.n_kv, s.head_dim, qkv.stride(0), int(s.causal), s.scale, nv.stream())
    return out, lse


def _attn_bwd(qkv, out, dout, lse, s: BlockSpec, seq: SeqInfo) -> torch.Tensor:
    from .attention import _sm_count
    T = qkv.shape[0]
    lo, hi = seq.bounds()
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(s.n_q, T, device=qkv.device, dtype=torch.float32)
    ws = None
    if s.n_q > s.n_kv and ((T + 127) // 128) * s.n_kv < 2 * _sm_count():
        ws = torch.empty(2 * s.n_q * T * s.head_dim, device=qkv.device, dtype=torch.float32)
    nv.call("mmt_attn_bwd", qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(), delta.data_ptr(),
            dqkv.data_ptr(), lo.data_ptr(), hi.data_ptr(), T, s.n_q, s.n_kv, s.head_dim, qkv.stride(0), int(s.causal),
            s.scale, nv.ptr(ws), nv.stream())
    return dqkv


def _swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    rows, two_i = gu.shape
    out = torch.empty(rows, two_i // 2, device=gu.device, dtype=gu.dtype)
    nv.call("mmt_swiglu_fwd", gu.data_ptr(), out.data_ptr(), rows, two_i // 2, nv.stream())
    return out


def _swiglu_bwd(dout: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    dgu = torch.empty_like(gu)
    nv.call("mmt_swiglu_bwd", dout.data_ptr(), gu.data_ptr(), dgu.data_ptr(), gu.shape[0], gu.shape[1] // 2,
            nv.stream())
    return dgu


def _linear_bwd(dy: torch.Tensor, x: torch.Tensor, w: torch.Tensor, b) -> torch.Tensor:
    """Weight / bias gradients of ``y = x w^T + b`` into the parameters, returns dx."""
    _grad_into(w, lambda out, acc: F.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=acc))
    if b is not None:
        _grad_into(b, lambda out, acc: F.colsum(dy, out=out, accumulate=acc))
    return F.gemm(dy, w, b_mn=True)


def _forward_chain(x, s: BlockSpec, cos, sin, seq, P, keep: bool):
    """The block's kernels in order; with ``keep`` every intermediate the backward needs is returned."""
    ln1_w, qkv_w, qkv_b, proj_w, proj_b, ln2_w, gu_w, gu_b, down_w, down_b = P
    h1, rstd1 = _rmsnorm_fwd(x, ln1_w, s.eps)
    qkv = F.gemm(h1, qkv_w, bias=qkv_b)
    _rope_(qkv, cos, sin, s.rope_heads, s.head_dim, False)
    a, lse = _attn_fwd(qkv, s, seq)
    x1 = F.gemm(a, proj_w, bias=proj_b, residual=x)
    h2, rstd2 = _rmsnorm_fwd(x1, ln2_w, s.eps)
    gu = F.gemm(h2, gu_w, bias=gu_b)
    m = _swiglu_fwd(gu)
    y = F.gemm(m, down_w, bias=down_b, residual=x1)
    if keep:
        return y, (h1, rstd1, qkv, a, lse, x1, h2, rstd2, gu, m)
    return y, None


class _LocalBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, spec, cos, sin, seq, recompute, *params):
        # recompute: 2 = keep only the block input, 1 = also keep what is expensive to rebuild (GEMM and attention
        # results; the element-wise intermediates are recomputed from them), 0 = keep every intermediate
        x = x if x.is_contiguous() else x.contiguous()
        y, kept = _forward_chain(x, spec, cos, sin, seq, params, keep=recompute < 2)
        extra = ()
        if recompute < 2:
            h1, rstd1, qkv, a, lse, x1, h2, rstd2, gu, m = kept
            extra = (qkv, a, lse, x1, gu) if recompute == 1 else (qkv, a, lse, x1, gu, h1, rstd1, h2, rstd2, m)
        ctx.n_extra = len(extra)
        ctx.save_for_backward(x, cos, sin, *extra, *[p for p in params if p is not None])
        ctx.has = [p is not None for p in params]
        ctx.spec, ctx.seq = spec, seq
        return y

    @staticmethod
    def backward(ctx, dy):
        saved = ctx.saved_tensors
        x, cos, sin = saved[0], saved[1], saved[2]
        extra = saved[3:3 + ctx.n_extra]
        it = iter(saved[3 + ctx.n_extra:])
        P = tuple(next(it) if h else None for h in ctx.has)
        s, seq = ctx.spec, ctx.seq
        ln1_w, qkv_w, qkv_b, proj_w, proj_b, ln2_w, gu_w, gu_b, down_w, down_b = P
        dy = dy if dy.is_contiguous() else dy.contiguous()
        if ctx.n_extra == 10:
            qkv, a, lse, x1, gu, h1, rstd1, h2, rstd2, m = extra
        elif ctx.n_extra:
            qkv, a, lse, x1, gu = extra
            h1, rstd1 = _rmsnorm_fwd(x, ln1_w, s.eps)
            h2, rstd2 = _rmsnorm_fwd(x1, ln2_w, s.eps)
            m = _swiglu_fwd(gu)
        else:
            _, (h1, rstd1, qkv, a, lse, x1, h2, rstd2, gu, m) = _forward_chain(x, s, cos, sin, seq, P, keep=True)
        # MLP half
        dm = _linear_bwd(dy, m, down_w, down_b)
        dgu = _swiglu_bwd(dm, gu)
        dh2 = _linear_bwd(dgu, h2, gu_w, gu_b)
        dx1 = _rmsnorm_bwd(dh2, x1, ln2_w, rstd2, dy)
        # attention half
        da = _linear_bwd(dx1, a, proj_w, proj_b)
        dqkv = _attn_bwd(qkv, a, da, lse, s, seq)
        _rope_(dqkv, cos, sin, s.rope_heads, s.head_dim, True)
        dh1 = _linear_bwd(dqkv, h1, qkv_w, qkv_b)
        dx = _rmsnorm_bwd(dh1, x, ln1_w, rstd1, dx1)
        return (dx, None, None, None, None, None) + (None,) * len(ctx.has)


def local_block(x: torch.Tensor, spec: BlockSpec, cos: torch.Tensor, sin: torch.Tensor, seq: SeqInfo, params: tuple,
                recompute: bool = True, keep_elementwise: bool = False):
    """``params`` = (ln1_w, qkv_w, qkv_b, proj_w, proj_b, ln2_w, gate_up_w, gate_up_b, down_w, down_b); biases may
    be None.  x is [T, C] bf16 on the GPU; the result has the same shape.  ``recompute``: keep only the block input
    and rebuild everything in backward (activation checkpointing); else keep the GEMM / attention results and, with
    ``keep_elementwise``, the normalised inputs and the SwiGLU output as well."""
    level = 2 if recompute else (0 if keep_elementwise else 1)
    return _LocalBlockFn.apply(x, spec, cos, sin, seq, level, *params)


def usable(x: torch.Tensor) -> bool:
    """The fused block needs the GPU path and a gradient-carrying input (it is its own activation checkpoint)."""
    return x.is_cuda and x.dtype == torch.bfloat16
