"""Activation checkpointing for blocks built from this package's ops.

The reference turns on HF ``gradient_checkpointing_enable()`` per block
(python/ray/trainer.py:257-267).  Here a block is a plain function of tensors; the
forward pass runs without a graph and keeps only the block inputs, the backward pass
recomputes the block and back-propagates through the recomputed graph.  Weight gradients
are written by the ops themselves (``main_grad``) or accumulate into ``.grad`` as usual.
"""
from __future__ import annotations

import torch
import torch.distributed


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensors, *args):
        ctx.fn = fn
        tensors = args[:n_tensors]
        ctx.extra = args[n_tensors:]
        ctx.save_for_backward(*tensors)
        ctx.req = [t.requires_grad for t in tensors]
        with torch.no_grad():
            out = fn(*tensors, *ctx.extra)
        return out

    @staticmethod
    def backward(ctx, *douts):
        tensors = [t.detach().requires_grad_(r) for t, r in zip(ctx.saved_tensors, ctx.req)]
        with torch.enable_grad():
            out = ctx.fn(*tensors, *ctx.extra)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, douts) if isinstance(o, torch.Tensor) and o.requires_grad]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        grads = tuple(t.grad if r else None for t, r in zip(tensors, ctx.req))
        return (None, None) + grads + (None,) * len(ctx.extra)


def checkpoint(fn, tensors: tuple, extra: tuple = (), enabled: bool = True):
    """``fn(*tensors, *extra)`` with recomputation in backward.

    ``tensors`` are the differentiable inputs (saved); ``extra`` are non-tensor or constant
    arguments; parameters are reached through ``fn``'s closure and receive gradients in backward.
    """
    if not enabled or not torch.is_grad_enabled():
        return fn(*tensors, *extra)
    return _Checkpoint.apply(fn, len(tensors), *tensors, *extra)


_DECISIONS: dict = {}


def bucket_tokens(n: int) -> int:
    """Token count rounded up to a quarter of an octave (1024, 1280, 1536, 1792, 2048, 2560, ...).

    ``decide`` caches one decision per size; with images of varying sizes nearly every batch has a new token count,
    and every new size costs a collective and a host synchronisation.  Buckets bound the number of sizes (and make
    the estimate an upper bound)."""
    n = max(int(n), 1)
    if n <= 1024:
        return 1024
    top = 1 << (n - 1).bit_length()
    step = top // 8
    return -(-n // step) * step


def decide(mode, need_bytes: int, device=None, headroom: float = 0.5, group=None, key=None) -> bool:
    """Should a stack of blocks recompute its activations in backward?

    ``mode`` is the config value: True / False, or ``"auto"``: keep the activations (no recomputation, about a
    quarter less work per step) when ``need_bytes`` of them fit into ``headroom`` of the memory that is free right
    now on ``device``, recompute otherwise.  The reference always checkpoints (it was sized for 80 GB GPUs,
    python/ray/trainer.py:257-267); on a 180 GB B200 the 7B model's activations at the benchmark's sequence
    lengths fit many times over.
    """
    if isinstance(mode, str):
        if mode.lower() != "auto":
            return mode.lower() not in ("false", "0", "off", "no")
        if device is None or torch.device(device).type != "cuda":
            return False
        # Ranks that exchange activations inside the blocks (sequence / tensor parallel peers) must all take the
        # same branch, or the ones that recompute would wait for exchanges the others never start.  The decision is
        # therefore the OR over ``group`` and is taken once per (key, size): later steps with the same shapes reuse it
        # without a collective or a host synchronisation.  Callers must pass a ``need_bytes`` that is the SAME on
        # every rank of ``group`` (derived from the largest rank's token count, not from the local one): the cache
        # decides who enters the collective, so peers with different sizes would enter it in different steps.
        ck = (key, int(need_bytes))
        hit = _DECISIONS.get(ck)
        if hit is not None:
            return hit
        free, _ = torch.cuda.mem_get_info(device)
        free += torch.cuda.memory_reserved(device) - torch.cuda.memory_allocated(device)
        recompute = need_bytes > headroom * free
        if group is not None and torch.distributed.is_initialized() and torch.distributed.get_world_size(group) > 1:
            flag = torch.tensor([1 if recompute else 0], device=device, dtype=torch.int32)
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MAX, group=group)
            recompute = bool(flag.item())
        _DECISIONS[ck] = recompute
        return recompute
    return bool(mode)
