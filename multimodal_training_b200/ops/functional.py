"""Differentiable ops of the training step.

Every op has two implementations behind one name:

* CUDA tensors (bf16): the hand-written sm_100a kernels of ``csrc/`` through
  :mod:`.native`, wrapped in ``torch.autograd.Function`` so forward and
  backward both run native code.  There is no PyTorch fallback on the GPU.
* CPU tensors (any float dtype): plain PyTorch, which is the numerical oracle
  of the tests and the gloo-parallel reference path.

Weight gradients on the GPU path are written straight into the parameter's
``main_grad`` view of the flat gradient buffer (see ``parallel/zero.py``) when
the parameter has one, with the kernel's accumulate flag instead of a separate
add pass.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from . import native as nv

_scratch: dict[tuple, torch.Tensor] = {}


def _scratch_f32(numel: int, device: torch.device, tag: str = "") -> torch.Tensor:
    """Reusable fp32 scratch buffer (grown on demand, one per device and tag)."""
    key = (device, tag)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < numel:
        buf = torch.empty(max(numel, 1 << 16), dtype=torch.float32, device=device)
        _scratch[key] = buf
    return buf


def _native(t: torch.Tensor) -> bool:
    if not t.is_cuda:
        return False
    if t.dtype != torch.bfloat16:
        raise TypeError(f"the sm_100a path is bf16 only, got {t.dtype}")
    return True


def _c(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


# --------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False, bias=None, residual=None,
         act: int = 0, out: torch.Tensor | None = None, accumulate: bool = False, out_f32: bool = False,
         alpha: float = 1.0) -> torch.Tensor:
    """``C[M,N] = alpha * A @ B^T (+bias, act, +residual)`` with the tcgen05 kernel.

    A is logically [M,K]: pass it as [M,K] (``a_mn=False``) or as [K,M] (``a_mn=True``); likewise B
    logically [N,K], passed as [N,K] or [K,N].  All 2-D, bf16; row strides are taken from the tensors.
    """
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, (a.shape, b.shape, a_mn, b_mn)
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=torch.float32 if out_f32 else torch.bfloat16)
    assert out.stride(1) == 1
    if M == 0:
        return out
    nv.call("mmt_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), nv.ptr(bias), nv.ptr(residual), M, N, K,
            a.stride(0), b.stride(0), out.stride(0), residual.stride(0) if residual is not None else 0,
            int(a_mn), int(b_mn), act, int(accumulate), int(out_f32), alpha, 0, nv.stream())
    return out


def _write_param_grad(p: torch.Tensor, compute) -> torch.Tensor | None:
    """Run ``compute(out, accumulate)`` into the parameter's flat-buffer gradient view if it has one."""
    mg = getattr(p, "main_grad", None)
    if mg is None:
        out = torch.empty_like(p)
        compute(out, False)
        return out
    compute(mg, bool(getattr(p, "grad_written", False)))
    p.grad_written = True
    return None


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, residual):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8:
            x2 = x2.contiguous()
        res2 = None
        if residual is not None:
            res2 = _c(residual.reshape(-1, w.shape[0]))
        y = gemm(x2, w, bias=b, residual=res2)
        ctx.save_for_backward(x2, w)
        ctx.has_bias = b is not None
        ctx.has_res = residual is not None
        ctx.bias_ref = b
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = _c(dy.reshape(-1, w.shape[0]))
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view(ctx.xshape)
        if ctx.needs_input_grad[1]:
            dw = _write_param_grad(w, lambda out, acc: gemm(dy2, x2, a_mn=True, b_mn=True, out=out, accumulate=acc))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            b = ctx.bias_ref
            db = _write_param_grad(b, lambda out, acc: colsum(dy2, out=out, accumulate=acc))
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


def linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None,
           residual: torch.Tensor | None = None) -> torch.Tensor:
    """``y = x @ w^T + b (+ residual)``; w is [out, in] like ``nn.Linear``."""
    if _native(x):
        return _LinearFn.apply(x, w, b, residual)
    y = F.linear(x, w, b)
    return y if residual is None else y + residual


def colsum(x2: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    rows, cols = x2.shape
    if out is None:
        out = torch.empty(cols, device=x2.device, dtype=torch.bfloat16)
    parts = nv.lib().mmt_colsum_parts(rows)
    scratch = _scratch_f32(parts * cols, x2.device, "colsum")
    nv.call("mmt_colsum", x2.data_ptr(), out.data_ptr(), scratch.data_ptr(), rows, cols, x2.stride(0),
            int(accumulate), nv.stream())
    return out


# --------------------------------------------------------------------------------------
# RMSNorm
# --------------------------------------------------------------------------------------
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        x2 = _c(x.reshape(-1, x.shape[-1]))
        rows, cols = x2.shape
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        nv.call("mmt_rmsnorm_fwd", x2.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols, eps,
                nv.stream())
        ctx.save_for_backward(x2, w, rstd)
        ctx.xshape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        rows, cols = x2.shape
        dy2 = _c(dy.reshape(rows, cols))
        dx = torch.empty_like(x2)
        parts = nv.lib().mmt_rmsnorm_bwd_parts(rows)
        scratch = _scratch_f32(parts * cols, x2.device, "rmsnorm")

        def run(out, acc):
            nv.call("mmt_rmsnorm_bwd", dy2.data_ptr(), x2.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                    out.data_ptr(), scratch.data_ptr(), rows, cols, int(acc), nv.stream())

        dw = _write_param_grad(w, run)
        return dx.view(ctx.xshape), dw, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if _native(x):
        return _RMSNormFn.apply(x, w, eps)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


# --------------------------------------------------------------------------------------
# Rotary embedding (rotate-half) on the leading `heads` heads of a fused [T, n*dim] buffer
# --------------------------------------------------------------------------------------
class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, heads, dim):
        y = x.clone()
        nv.call("mmt_rope", y.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.shape[0], heads, dim, y.stride(0), 0,
                nv.stream())
        ctx.save_for_backward(cos, sin)
        ctx.hd = (heads, dim)
        return y

    @staticmethod
    def backward(ctx, dy):
        cos, sin = ctx.saved_tensors
        heads, dim = ctx.hd
        dx = dy.clone()
        nv.call("mmt_rope", dx.data_ptr(), cos.data_ptr(), sin.data_ptr(), dx.shape[0], heads, dim, dx.stride(0), 1,
                nv.stream())
        return dx, None, None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    """Rotate the first ``heads`` heads (``dim`` columns each) of every row of x [T, W]; cos/sin are [T, dim] fp32."""
    if _native(x):
        assert x.dim() == 2 and x.is_contiguous() and cos.dtype == torch.float32 and cos.is_contiguous()
        return _RopeFn.apply(x, cos, sin, heads, dim)
    T = x.shape[0]
    xr = x[:, : heads * dim].reshape(T, heads, dim).float()
    c, s = cos.float().unsqueeze(1), sin.float().unsqueeze(1)
    half = dim // 2
    rot = torch.cat((-xr[..., half:], xr[..., :half]), dim=-1)
    out = (xr * c + rot * s).to(x.dtype).reshape(T, heads * dim)
    return torch.cat((out, x[:, heads * dim:]), dim=1)


# --------------------------------------------------------------------------------------
# Activations
# --------------------------------------------------------------------------------------
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        rows, two_i = gu.shape
        inter = two_i // 2
        out = torch.empty(rows, inter, device=gu.device, dtype=gu.dtype)
        nv.call("mmt_swiglu_fwd", gu.data_ptr(), out.data_ptr(), rows, inter, nv.stream())
        ctx.save_for_backward(gu)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        rows, two_i = gu.shape
        dgu = torch.empty_like(gu)
        nv.call("mmt_swiglu_bwd", _c(dout).data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, two_i // 2, nv.stream())
        return dgu


def swiglu(gu: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` on a fused [rows, 2*I] = gate|up buffer."""
    if _native(gu):
        assert gu.dim() == 2 and gu.is_contiguous()
        return _SwiGLUFn.apply(gu)
    g, u = gu.chunk(2, dim=-1)
    return F.silu(g) * u


class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        y = torch.empty_like(x)
        nv.call("mmt_gelu_fwd", x.data_ptr(), y.data_ptr(), x.numel(), nv.stream())
        ctx.save_for_backward(x)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        dx = torch.empty_like(x)
        nv.call("mmt_gelu_bwd", _c(dy).data_ptr(), x.data_ptr(), dx.data_ptr(), x.numel(), nv.stream())
        return dx


def gelu(x: torch.Tensor) -> torch.Tensor:
    if _native(x):
        return _GeluFn.apply(_c(x))
    return F.gelu(x)


# --------------------------------------------------------------------------------------
# Row gather / scatter (embedding, window permutation, splice)
# --------------------------------------------------------------------------------------
def gather_rows_raw(src: torch.Tensor, idx: torch.Tensor, lo: int = 0, hi: int | None = None,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    hi = lo + src.shape[0] if hi is None else hi
    if out is None:
        out = torch.empty(idx.numel(), src.shape[1], device=src.device, dtype=src.dtype)
    nv.call("mmt_gather_rows", src.data_ptr(), idx.data_ptr(), out.data_ptr(), idx.numel(), src.shape[1], lo, hi,
            src.stride(0), out.stride(0), nv.stream())
    return out


def scatter_rows_raw(src: torch.Tensor, idx: torch.Tensor, dst: torch.Tensor, lo: int = 0, hi: int | None = None,
                     add: bool = False) -> torch.Tensor:
    hi = lo + dst.shape[0] if hi is None else hi
    nv.call("mmt_scatter_rows", src.data_ptr(), idx.data_ptr(), dst.data_ptr(), idx.numel(), src.shape[1], lo, hi,
            src.stride(0), dst.stride(0), int(add), nv.stream())
    return dst


class _GatherRowsFn(torch.autograd.Function):
    """out[r] = src[idx[r]]; idx is a permutation or a subset without repeats (window order, splice)."""

    @staticmethod
    def forward(ctx, src, idx):
        ctx.save_for_backward(idx)
        ctx.n = src.shape[0]
        return gather_rows_raw(src, idx)

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        dsrc = torch.zeros(ctx.n, dout.shape[1], device=dout.device, dtype=dout.dtype)
        scatter_rows_raw(_c(dout), idx, dsrc)
        return dsrc, None


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    if _native(src):
        return _GatherRowsFn.apply(_c(src), idx)
    return src.index_select(0, idx)


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table, lo):
        ctx.save_for_backward(ids)
        ctx.table = table
        ctx.lo = lo
        return gather_rows_raw(table, ids, lo, lo + table.shape[0])

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        table, lo = ctx.table, ctx.lo
        dout = _c(dout)

        def run(out, acc):
            if not acc:
                out.zero_()
            scatter_rows_raw(dout, ids, out, lo, lo + table.shape[0], add=True)

        return None, _write_param_grad(table, run), None


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_lo: int = 0) -> torch.Tensor:
    """Rows of a (vocab-sharded) table; ids outside [vocab_lo, vocab_lo + rows) give zero rows."""
    if _native(table):
        return _EmbeddingFn.apply(ids, table, vocab_lo)
    local = ids - vocab_lo
    ok = (local >= 0) & (local < table.shape[0])
    out = F.embedding(local.clamp(0, table.shape[0] - 1), table)
    return out * ok.unsqueeze(-1).to(out.dtype)


# --------------------------------------------------------------------------------------
# Attention (varlen, packed)
# --------------------------------------------------------------------------------------
def attention_reference(q, k, v, cu_seqlens: list[int], causal: bool, scale: float) -> torch.Tensor:
    """Plain-PyTorch packed attention.  q [T,Hq,D], k/v [T,Hkv,D]; returns [T,Hq,D]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    out = torch.empty_like(q)
    for i in range(len(cu_seqlens) - 1):
        s, e = cu_seqlens[i], cu_seqlens[i + 1]
        if e == s:
            continue
        qi = q[s:e].transpose(0, 1).float()
        ki = k[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        vi = v[s:e].transpose(0, 1).float().repeat_interleave(rep, dim=0)
        att = torch.matmul(qi, ki.transpose(1, 2)) * scale
        if causal:
            L = e - s
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            att = att.masked_fill(~mask, float("-inf"))
        p = att.softmax(-1)
        out[s:e] = torch.matmul(p, vi).transpose(0, 1).to(q.dtype)
    return out


def attention(qkv: torch.Tensor, n_q: int, n_kv: int, dim: int, cu_seqlens, causal: bool,
              scale: float | None = None, max_seqlen: int | None = None) -> torch.Tensor:
    """Packed varlen attention on a fused [T, (n_q + 2 n_kv) * dim] q|k|v buffer -> [T, n_q * dim].

    ``cu_seqlens`` is a :class:`SeqInfo` (host list + device int32 tensor) or a plain python list.
    """
    from .attention import SeqInfo, flash_attention  # local import: keeps CPU-only use free of ctypes

    scale = 1.0 / math.sqrt(dim) if scale is None else scale
    info = cu_seqlens if isinstance(cu_seqlens, SeqInfo) else SeqInfo.from_list(list(cu_seqlens), qkv.device)
    if _native(qkv):
        return flash_attention(qkv, n_q, n_kv, dim, info, causal, scale)
    T = qkv.shape[0]
    q = qkv[:, : n_q * dim].reshape(T, n_q, dim)
    k = qkv[:, n_q * dim: (n_q + n_kv) * dim].reshape(T, n_kv, dim)
    v = qkv[:, (n_q + n_kv) * dim:].reshape(T, n_kv, dim)
    return attention_reference(q, k, v, info.host, causal, scale).reshape(T, n_q * dim)


# --------------------------------------------------------------------------------------
# Fused lm_head + (vocab-parallel) cross-entropy
# --------------------------------------------------------------------------------------
def _all_reduce(t: torch.Tensor, op, group) -> None:
    if group is not None and torch.distributed.get_world_size(group) > 1:
        torch.distributed.all_reduce(t, op=op, group=group)


class _LMHeadCEFn(torch.autograd.Function):
    """loss = mean over valid rows of CE(hidden @ W^T, labels); gradients are produced in forward.

    The logits of a row chunk live only in a bf16 workspace: statistics kernel -> (tiny cross-rank
    reductions for vocab parallelism) -> in-place gradient kernel -> dgrad / wgrad GEMMs, so neither
    fp32 logits nor a softmax copy of the whole sequence is ever materialised.
    """

    @staticmethod
    def forward(ctx, hidden, weight, labels, vocab_lo, group, chunk_rows, smoothing=0.0, vocab_total=0):
        T, H = hidden.shape
        V = weight.shape[0]
        dev = hidden.device
        valid = (labels >= 0)
        n_valid = valid.sum().to(torch.float32).clamp_(min=1.0)
        inv = (1.0 / n_valid).reshape(1)
        dhidden = torch.empty_like(hidden)
        loss_sum = torch.zeros((), device=dev, dtype=torch.float32)
        ws = torch.empty(min(chunk_rows, T), V, device=dev, dtype=torch.bfloat16)
        ReduceOp = torch.distributed.ReduceOp
        need_w = weight.requires_grad
        mg = getattr(weight, "main_grad", None)
        if need_w:
            if mg is None:
                dw = torch.zeros_like(weight)
                acc0 = False
            else:
                dw = mg
                acc0 = bool(getattr(weight, "grad_written", False))
        for c0 in range(0, T, chunk_rows):
            c1 = min(T, c0 + chunk_rows)
            rows = c1 - c0
            h = hidden[c0:c1]
            lab = labels[c0:c1]
            logits = ws[:rows]
            gemm(h, weight, out=logits)
            st = torch.empty(3, rows, device=dev, dtype=torch.float32)
            nv.call("mmt_ce_stats", logits.data_ptr(), lab.data_ptr(), st[0].data_ptr(), st[1].data_ptr(),
                    st[2].data_ptr(), rows, V, logits.stride(0), vocab_lo, nv.stream())
            if group is not None and torch.distributed.get_world_size(group) > 1:
                lmax = st[0].clone()
                _all_reduce(st[0], ReduceOp.MAX, group)
                st[1].mul_(torch.exp(lmax - st[0]))
                _all_reduce(st[1:3], ReduceOp.SUM, group)
            if smoothing > 0.0:
                # label smoothing (rare path, plain tensor ops around the kernels): the loss also needs the mean
                # logit over the whole vocabulary, the gradient moves `smoothing` of the target's mass to all ids
                zsum = logits.sum(-1, dtype=torch.float32)
                _all_reduce(zsum, ReduceOp.SUM, group)
                row_loss = (torch.log(st[1]) + st[0] - (1.0 - smoothing) * st[2] - smoothing * zsum / vocab_total) \
                    * valid[c0:c1]
            else:
                row_loss = (torch.log(st[1]) + st[0] - st[2]) * valid[c0:c1]
            loss_sum += row_loss.sum()
            nv.call("mmt_ce_grad", logits.data_ptr(), lab.data_ptr(), st[0].data_ptr(), st[1].data_ptr(),
                    inv.data_ptr(), rows, V, logits.stride(0), vocab_lo, nv.stream())
            if smoothing > 0.0:
                scale = (inv[0] * valid[c0:c1]).to(logits.dtype)                       # [rows]
                logits.sub_((smoothing / vocab_total) * scale.unsqueeze(1))
                local = lab - vocab_lo
                mine = (local >= 0) & (local < V) & valid[c0:c1]
                logits.view(-1).index_add_(0, (torch.arange(rows, device=dev) * logits.stride(0)
                                               + local.clamp(0, V - 1))[mine], (smoothing * scale)[mine])
            gemm(logits, weight, b_mn=True, out=dhidden[c0:c1])
            if need_w:
                gemm(logits, h, a_mn=True, b_mn=True, out=dw, accumulate=acc0 or c0 > 0)
        if need_w and mg is not None:
            weight.grad_written = True
        ctx.save_for_backward(dhidden, dw if (need_w and mg is None) else None)
        ctx.need_w = need_w
        return loss_sum * inv[0]

    @staticmethod
    def backward(ctx, dloss):
        dhidden, dw = ctx.saved_tensors
        # dloss is 1 for a loss that is the root of backward; scale otherwise
        dh = dhidden * dloss.to(dhidden.dtype)
        if dw is not None:
            dw = dw * dloss.to(dw.dtype)
        return dh, dw, None, None, None, None, None, None


def lm_head_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor, vocab_lo: int = 0,
                          group=None, chunk_rows: int = 4096, label_smoothing: float = 0.0) -> torch.Tensor:
    """Mean CE over rows with ``labels >= 0``.  ``weight`` is this rank's [V_local, H] vocab shard starting at
    ``vocab_lo``; with a group, max / sum-exp / target logit are reduced over it
    (Megatron-style, reference: python/tensor_parallel/cross_entropy.py:41-236).

    ``labels`` are already shifted (row t holds the id to predict at t) and use -100 (any negative) to ignore.
    On the GPU path, the weight gradient assumes ``dloss == 1`` when it is written into ``main_grad``.

    ``label_smoothing`` = a in (0, 1): the target keeps 1 - a of the probability mass and the other ids of the WHOLE
    vocabulary share a (the reference's option, python/tensor_parallel/cross_entropy.py:185-202,223-230, which takes
    the mean over the local shard only): with s = a V / (V - 1), loss = (1 - s) nll - s mean_v(log p_v).
    """
    multi = group is not None and torch.distributed.get_world_size(group) > 1
    vocab_total = weight.shape[0] * (torch.distributed.get_world_size(group) if multi else 1)
    if not 0.0 <= label_smoothing < 1.0:
        raise ValueError("label_smoothing must be in [0, 1)")
    smoothing = label_smoothing * vocab_total / (vocab_total - 1) if label_smoothing > 0 else 0.0
    if _native(hidden):
        return _LMHeadCEFn.apply(_c(hidden), weight, labels, vocab_lo, group, chunk_rows, smoothing, vocab_total)
    logits = F.linear(hidden, weight).float()
    V = weight.shape[0]
    ReduceOp = torch.distributed.ReduceOp
    m = logits.max(dim=-1).values.detach()
    if multi:
        _all_reduce(m, ReduceOp.MAX, group)
    z = logits - m.unsqueeze(-1)
    local = labels - vocab_lo
    ok = (local >= 0) & (local < V)
    tgt = z.gather(1, local.clamp(0, V - 1).unsqueeze(1)).squeeze(1) * ok
    se = z.exp().sum(-1)
    if multi:
        from ..parallel.comm import all_reduce_sum_autograd
        tgt = all_reduce_sum_autograd(tgt, group)
        se = all_reduce_sum_autograd(se, group)
    valid = labels >= 0
    if smoothing > 0.0:
        zsum = z.sum(-1)
        if multi:
            zsum = all_reduce_sum_autograd(zsum, group)
        row = (se.log() - (1.0 - smoothing) * tgt - smoothing * zsum / vocab_total) * valid
    else:
        row = (se.log() - tgt) * valid
    return row.sum() / valid.sum().clamp(min=1)


# --------------------------------------------------------------------------------------
# Optimizer-side kernels
# --------------------------------------------------------------------------------------
def adamw_step(p, g, master, m, v, *, n_decay: int, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, step: int, grad_scale: torch.Tensor | None = None) -> None:
    """Fused AdamW over flat buffers; elements [0, n_decay) get weight decay.

    With ``master`` (fp32 copy of the weights) the moments are fp32 too and ``p`` receives the rounded master.
    ``master=None`` is the optimizer of a bf16 model without a master copy (what ``torch.optim.AdamW`` does on bf16
    parameters, the reference's setting): the moments have ``p``'s dtype, an element is updated in fp32 and weight
    and moments are rounded when stored."""
    if p.is_cuda:
        if master is None:
            nv.call("mmt_adamw_bf16", p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), n_decay, lr,
                    beta1, beta2, eps, weight_decay, step, nv.ptr(grad_scale), nv.stream())
            return
        nv.call("mmt_adamw", p.data_ptr(), g.data_ptr(), master.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(),
                n_decay, lr, beta1, beta2, eps, weight_decay, step, nv.ptr(grad_scale), nv.stream())
        return
    gf = g.float()
    if grad_scale is not None:
        gf = gf * grad_scale
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    if master is None:
        mf = m.float().mul_(beta1).add_(gf, alpha=1 - beta1)
        vf = v.float().mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
        upd = (mf / bc1) / ((vf / bc2).sqrt() + eps)
        w = p.float()
        wd = torch.zeros_like(w)
        wd[:n_decay] = weight_decay
        p.copy_((w - lr * (upd + wd * w)).to(p.dtype))
        m.copy_(mf.to(m.dtype))
        v.copy_(vf.to(v.dtype))
        return
    m.mul_(beta1).add_(gf, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(gf, gf, value=1 - beta2)
    upd = (m / bc1) / ((v / bc2).sqrt() + eps)
    wd = torch.zeros_like(master)
    wd[:n_decay] = weight_decay
    master.sub_(lr * (upd + wd * master))
    p.copy_(master.to(p.dtype))


def sum_squares(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[0] += sum(x^2) in fp32 (no host sync)."""
    if x.is_cuda:
        nv.call("mmt_sumsq", x.data_ptr(), x.numel(), out.data_ptr(), nv.stream())
    else:
        out += x.float().pow(2).sum()
    return out
