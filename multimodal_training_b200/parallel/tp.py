"""Tensor parallelism: sequence-parallel activations for the text decoder, replicated activations for the vision
encoder's optional tensor-parallel mode (``copy_to_tp`` / ``reduce_from_tp``).

Activations between layers are sharded along the token axis (T/tp rows per rank).  A
column-parallel linear all-gathers its input rows and multiplies by its slice of the output
features; a row-parallel linear multiplies its slice of the input features and reduce-scatters
the partial sums back to token shards.  The reference's DTensor plan instead keeps activations
replicated and all-reduces (python/ray/text.py:448-512,1165-1177).

Two implementations sit behind each function: NCCL/gloo collectives from :mod:`.comm` plus the
GEMM op, and the fused peer-memory kernels of :mod:`.fused` (all-gather->GEMM and
GEMM->reduce-scatter in one kernel each) when a symmetric heap is attached to the context.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import functional as F
from . import comm


@dataclass
class TPContext:
    group: object = None          # torch.distributed group of the tensor-parallel ranks
    size: int = 1
    rank: int = 0
    fused: object = None          # parallel.fused.FusedTP when peer-memory kernels are in use

    @classmethod
    def single(cls) -> "TPContext":
        return cls()


def column_parallel_linear(x_shard: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, ctx: TPContext,
                           norm_w: torch.Tensor | None = None, eps: float = 1e-6, role: str = "qkv") -> torch.Tensor:
    """[T/tp, K] token shard -> (RMSNorm with ``norm_w``) -> all-gather rows -> ``x @ w^T + b`` with the local
    weight slice -> [T, N/tp].  ``role`` names the peer-memory buffers of the fused path."""
    if ctx.size > 1 and ctx.fused is not None and x_shard.is_cuda:
        return ctx.fused.ag_linear(x_shard, w, b, norm_w=norm_w, eps=eps, role=role)
    h = x_shard if norm_w is None else F.rmsnorm(x_shard, norm_w, eps)
    if ctx.size == 1:
        return F.linear(h, w, b)
    return F.linear(comm.all_gather(h, ctx.group), w, b)


def row_parallel_linear(x: torch.Tensor, w: torch.Tensor, residual_shard: torch.Tensor | None, ctx: TPContext,
                        role: str = "o") -> torch.Tensor:
    """[T, K/tp] -> [T/tp, N]: partial ``x @ w^T`` summed over ranks and scattered by token rows (+ residual)."""
    if ctx.size == 1:
        return F.linear(x, w, None, residual_shard)
    if ctx.fused is not None and x.is_cuda:
        return ctx.fused.linear_rs(x, w, residual_shard, role=role)
    y = comm.reduce_scatter(F.linear(x, w), ctx.group)
    return y if residual_shard is None else y + residual_shard


def copy_to_tp(x: torch.Tensor, ctx: TPContext) -> torch.Tensor:
    """Input of a column-parallel linear on replicated activations: identity, gradient summed over the group."""
    return x if ctx.size == 1 else comm.copy_to_group(x, ctx.group)


def reduce_from_tp(x: torch.Tensor, ctx: TPContext) -> torch.Tensor:
    """Output of a row-parallel linear on replicated activations: summed over the group, gradient passes through."""
    return x if ctx.size == 1 else comm.all_reduce_sum_autograd(x, ctx.group)


def shard_rows(full: torch.Tensor, size: int, rank: int) -> torch.Tensor:
    n = full.shape[0] // size
    return full[rank * n:(rank + 1) * n]


def shard_cols(full: torch.Tensor, size: int, rank: int) -> torch.Tensor:
    n = full.shape[1] // size
    return full[:, rank * n:(rank + 1) * n]


def vocab_range(vocab_size: int, size: int, rank: int) -> tuple[int, int]:
    """[lo, hi) of the vocabulary rows owned by ``rank`` (reference: python/tensor_parallel/embedding.py:15-35)."""
    per = vocab_size // size
    if per * size != vocab_size:
        raise ValueError(f"vocab_size {vocab_size} is not divisible by the tensor-parallel size {size}")
    return rank * per, (rank + 1) * per
