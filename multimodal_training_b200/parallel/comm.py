"""Differentiable collectives over ``torch.distributed`` (NCCL on GPUs, gloo on CPU).

These are the library ("lib") versions of every exchange in the step; the fused
peer-memory kernels in :mod:`.fused` replace them on NVLink-connected GPUs.  Each
function degenerates to the identity for a group of one, so single-GPU runs issue
no communication at all.

Reference call sites being replaced: DeepSpeed ``_SeqAllToAll``
(modeling_qwen2_5_vl.py:628-640,744-746), the ragged all-gather
(modeling_qwen2_5_vl.py:110-189) and DTensor's row/column-parallel all-reduces
(python/ray/text.py:1165-1177).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


# ---------------------------------------------------------------------------
# all-gather along dim 0 (equal shards)  <->  reduce-scatter along dim 0
# ---------------------------------------------------------------------------
def _all_gather_raw(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out


def _reduce_scatter_raw(x: torch.Tensor, group) -> torch.Tensor:
    n = group_size(group)
    assert x.shape[0] % n == 0
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x.contiguous(), op=dist.ReduceOp.SUM, group=group)
    else:
        # gloo has no reduce_scatter: all-reduce then slice
        tmp = x.contiguous().clone()
        dist.all_reduce(tmp, op=dist.ReduceOp.SUM, group=group)
        r = group_rank(group)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
    return out


class _AllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_raw(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _reduce_scatter_raw(dy, ctx.group), None


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_raw(x, group)

    @staticmethod
    def backward(ctx, dy):
        return _all_gather_raw(dy, ctx.group), None


def all_gather(x: torch.Tensor, group) -> torch.Tensor:
    """Concatenate equal shards along dim 0; the backward pass is a reduce-scatter (sum)."""
    if group_size(group) == 1:
        return x
    return _AllGather.apply(x, group)


def reduce_scatter(x: torch.Tensor, group) -> torch.Tensor:
    """Sum over the group and keep this rank's dim-0 shard; the backward pass is an all-gather."""
    if group_size(group) == 1:
        return x
    return _ReduceScatter.apply(x, group)


def all_gather_ragged(x: torch.Tensor, rows: list[int], group) -> list[torch.Tensor]:
    """Every rank's ``[rows[p], ...]`` tensor on every rank (no autograd); shorter ones travel padded."""
    n = group_size(group)
    if n == 1:
        return [x]
    width = max(rows)
    mine = x.contiguous()
    if mine.shape[0] < width:
        mine = torch.cat([mine, mine.new_zeros((width - mine.shape[0],) + tuple(mine.shape[1:]))], 0)
    parts = [torch.empty_like(mine) for _ in range(n)]
    dist.all_gather(parts, mine, group=group)
    return [p[:r] for p, r in zip(parts, rows)]


# ---------------------------------------------------------------------------
# all-reduce variants
# ---------------------------------------------------------------------------
class _AllReduceSum(torch.autograd.Function):
    """Sum over the group in forward, identity in backward (every rank holds the same upstream gradient)."""

    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


class _CopyToGroup(torch.autograd.Function):
    """Identity in forward, sum over the group in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, dy):
        y = dy.contiguous().clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=ctx.group)
        return y, None


def all_reduce_sum_autograd(x: torch.Tensor, group) -> torch.Tensor:
    if group_size(group) == 1:
        return x
    return _AllReduceSum.apply(x, group)


def copy_to_group(x: torch.Tensor, group) -> torch.Tensor:
    if group_size(group) == 1:
        return x
    return _CopyToGroup.apply(x, group)


# ---------------------------------------------------------------------------
# all-to-all with per-rank row counts
# ---------------------------------------------------------------------------
def _all_to_all_rows_raw(x: torch.Tensor, send_rows: list[int], recv_rows: list[int], group) -> torch.Tensor:
    out = torch.empty((sum(recv_rows),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    x = x.contiguous()
    if x.is_cuda:
        dist.all_to_all_single(out, x, output_split_sizes=recv_rows, input_split_sizes=send_rows, group=group)
    else:
        # gloo: all_to_all_single is unsupported; exchange with point-to-point ops in a fixed order
        n, r = group_size(group), group_rank(group)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(n))
        so = [0]
        for s in send_rows:
            so.append(so[-1] + s)
        ro = [0]
        for s in recv_rows:
            ro.append(ro[-1] + s)
        out[ro[r]:ro[r + 1]].copy_(x[so[r]:so[r + 1]])
        ops = []
        for p in range(n):
            if p == r:
                continue
            if send_rows[p] > 0:
                ops.append(dist.P2POp(dist.isend, x[so[p]:so[p + 1]].contiguous(), ranks[p], group=group))
            if recv_rows[p] > 0:
                ops.append(dist.P2POp(dist.irecv, out[ro[p]:ro[p + 1]], ranks[p], group=group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
    return out


class _AllToAllRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send_rows, recv_rows, group):
        ctx.meta = (send_rows, recv_rows, group)
        return _all_to_all_rows_raw(x, send_rows, recv_rows, group)

    @staticmethod
    def backward(ctx, dy):
        send_rows, recv_rows, group = ctx.meta
        return _all_to_all_rows_raw(dy, recv_rows, send_rows, group), None, None, None


def all_to_all_rows(x: torch.Tensor, send_rows: list[int], recv_rows: list[int], group) -> torch.Tensor:
    """Send ``send_rows[p]`` leading-dim rows to peer p (in order) and receive ``recv_rows[p]`` from it."""
    if group_size(group) == 1:
        return x
    return _AllToAllRows.apply(x, list(send_rows), list(recv_rows), group)
