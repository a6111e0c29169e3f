"""Flat-buffer ZeRO-1 AdamW.

All parameters of a trainer live in ONE flat buffer (and their gradients in another); every
``nn.Parameter`` is a view.  That gives: weight-gradient kernels that write straight into the flat
gradient (``main_grad``), a single reduce-scatter per step, one fused AdamW launch over the owned
shard (fp32 master weights and moments exist only for that shard) and a single all-gather of the
updated bf16 parameters.  With a group of one this is simply a fused multi-tensor AdamW.

Replaces DeepSpeed ZeRO-1 around an external ``torch.optim.Adam`` in the reference
(python/ray/trainer.py:479-577,675-849, python/ray/vision.py:228-294).  Differences on purpose:
decoupled weight decay (AdamW), fp32 master weights and moments, gradients summed over ranks that
split tokens (sequence parallel) and averaged over data-parallel replicas.

Layout of the flat buffer: [decayed | decayed, replicated over the tensor-parallel group |
non-decayed, replicated (among them the sequence-parallel ones whose gradient is a partial sum over
that group) | non-decayed], each parameter padded to 128 elements, the total padded so that all
shards are equal and 1024-aligned.  The replicated range is contiguous: the gradient norm counts it
once per tensor-parallel group.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..ops import functional as F
from . import comm

ALIGN = 128


def default_no_decay(name: str) -> bool:
    """The reference's rule (python/ray/trainer.py:469-477): bias / norm / ln_ parameters are not decayed."""
    n = name.lower()
    return "bias" in n or "norm" in n or "ln_" in n or n.endswith("_b") or "ln1" in n or "ln2" in n


class ZeroAdamW:
    def __init__(self, named_params, *, group=None, lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, no_decay_fn=default_no_decay, grad_divisor: float = 1.0,
                 partial_grad_group=None, fused=None, master_weights: bool = True):
        named = [(n, p) for n, p in named_params if p.requires_grad]
        seen, uniq = set(), []
        for n, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                uniq.append((n, p))
        self.group = group
        self.gsize = comm.group_size(group)
        self.grank = comm.group_rank(group)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.grad_divisor = grad_divisor
        self.partial_grad_group = partial_grad_group
        self.fused = fused
        self.step_count = 0
        # False: no fp32 master copy, moments in the parameters' dtype (torch.optim.AdamW on a bf16 model, the
        # reference's optimizer: half the optimizer traffic and a third of its memory, bf16 rounding of every update)
        self.master_weights = bool(master_weights)

        def replicated(p):
            return getattr(p, "sequence_parallel", False) or getattr(p, "tensor_replicated", False)

        for n, p in uniq:
            if getattr(p, "sequence_parallel", False) and not no_decay_fn(n):
                raise ValueError(f"{n}: a parameter with partial-sum gradients must be in the non-decayed set")
        decay = [(n, p) for n, p in uniq if not no_decay_fn(n) and not replicated(p)]
        decay_rep = [(n, p) for n, p in uniq if not no_decay_fn(n) and replicated(p)]
        nodecay_rep = [(n, p) for n, p in uniq if no_decay_fn(n) and replicated(p)]
        nodecay = [(n, p) for n, p in uniq if no_decay_fn(n) and not replicated(p)]
        self.names, self.params, offsets = [], [], []
        off = 0
        marks = {}
        for tag, seg in (("decay", decay), ("decay_rep", decay_rep), ("nodecay_rep", nodecay_rep),
                         ("nodecay", nodecay)):
            marks[tag] = off
            for n, p in seg:
                self.names.append(n)
                self.params.append(p)
                offsets.append(off)
                off += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.n_decay = marks["nodecay_rep"]            # [0, n_decay) gets weight decay
        # [rep_start, rep_end): identical on every rank of the tensor-parallel group (counted once in the norm);
        # its non-decayed part [partial_start, partial_end) is what ``partial_grad_group`` all-reduces
        self.rep_start, self.rep_end = marks["decay_rep"], marks["nodecay"]
        self.partial_start, self.partial_end = marks["nodecay_rep"], marks["nodecay"]
        quantum = self.gsize * 1024
        self.total = (off + quantum - 1) // quantum * quantum if off else quantum
        self.shard = self.total // self.gsize
        self.offsets = offsets
        p0 = self.params[0]
        self.device, self.dtype = p0.device, p0.dtype
        self.native = p0.is_cuda

        self.fz = None
        if fused is not None and self.native and self.gsize > 1 and self.gsize <= 8 and self.master_weights:
            from .fused import FusedZero
            self.fz = FusedZero(group, self.total, self.device)
            self.flat_param, self.flat_grad = self.fz.flat_param, self.fz.flat_grad
        else:
            self.flat_param = torch.zeros(self.total, dtype=self.dtype, device=self.device)
            self.flat_grad = torch.zeros(self.total, dtype=self.dtype, device=self.device)
        for p, o in zip(self.params, offsets):
            n = p.numel()
            self.flat_param[o:o + n].copy_(p.data.reshape(-1))
            p.data = self.flat_param[o:o + n].view(p.shape)
            gview = self.flat_grad[o:o + n].view(p.shape)
            if self.native:
                p.main_grad = gview
                p.grad_written = False
            else:
                p.grad = gview
        lo = self.grank * self.shard
        self.shard_lo = lo
        if self.master_weights:
            self.master = self.flat_param[lo:lo + self.shard].to(torch.float32, copy=True)
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
        else:
            self.master = None
            self.exp_avg = torch.zeros(self.shard, dtype=self.dtype, device=self.device)
            self.exp_avg_sq = torch.zeros(self.shard, dtype=self.dtype, device=self.device)
        self._normsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._coef = torch.ones(1, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ gradients
    def zero_grad(self, set_to_none: bool = False) -> None:
        """GPU path: the first gradient write of a step overwrites, so only the flags are reset.
        CPU path: autograd accumulates into the ``.grad`` views, which are zeroed here."""
        if self.native:
            for p in self.params:
                p.grad_written = False
                p.grad = None
        else:
            self.flat_grad.zero_()
            for p, o in zip(self.params, self.offsets):
                p.grad = self.flat_grad[o:o + p.numel()].view(p.shape)

    def _finish_grads(self) -> None:
        """Parameters that took no gradient this step must contribute zeros, not stale data."""
        if not self.native:
            return
        for p, o in zip(self.params, self.offsets):
            if not p.grad_written:
                if p.grad is not None:   # came through autograd accumulation
                    p.main_grad.copy_(p.grad)
                    p.grad = None
                else:
                    p.main_grad.zero_()
                p.grad_written = True

    def reduce_gradients(self) -> torch.Tensor:
        """Partial-sum all-reduce for sequence-parallel parameters, then reduce-scatter over the ZeRO group.
        Returns this rank's gradient shard (a view of the flat gradient)."""
        self._finish_grads()
        if self.partial_grad_group is not None and self.partial_end > self.partial_start and \
                comm.group_size(self.partial_grad_group) > 1:
            dist.all_reduce(self.flat_grad[self.partial_start:self.partial_end], group=self.partial_grad_group)
        lo = self.shard_lo
        shard = self.flat_grad[lo:lo + self.shard]
        if self.gsize > 1:
            if self.native:
                dist.reduce_scatter_tensor(shard, self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
            else:
                dist.all_reduce(self.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
        return shard

    def grad_norm_sq_local(self, shard: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """(sum of squares of TP-sharded parameters' gradients, same for TP-replicated ones) in this shard,
        after ``reduce_gradients`` and including the ``grad_divisor`` scaling."""
        lo, hi = self.shard_lo, self.shard_lo + self.shard
        ps, pe = max(self.rep_start, lo), min(self.rep_end, hi)
        total = torch.zeros(1, dtype=torch.float32, device=self.device)
        F.sum_squares(shard, total)
        rep = torch.zeros(1, dtype=torch.float32, device=self.device)
        if pe > ps:
            seg = self.flat_grad[ps:pe]
            if self.native and (seg.numel() % 8 or seg.data_ptr() % 16):
                rep += seg.float().pow(2).sum()
            else:
                F.sum_squares(seg, rep)
        d2 = self.grad_divisor ** 2
        return (total - rep) / d2, rep / d2

    # ------------------------------------------------------------------ update
    def step(self, lr: float | None = None, grad_scale: torch.Tensor | float | None = None,
             shard: torch.Tensor | None = None) -> None:
        """AdamW on the owned shard, then all-gather the updated parameters.

        ``grad_scale`` (device scalar or float) multiplies gradients on the fly (clipping); the
        ``grad_divisor`` (data-parallel mean) is folded into it."""
        self.step_count += 1
        lr = self.lr if lr is None else lr
        if isinstance(grad_scale, torch.Tensor):
            scale_t = grad_scale.to(torch.float32).reshape(1) / self.grad_divisor
        else:
            s = (1.0 if grad_scale is None else float(grad_scale)) / self.grad_divisor
            scale_t = None if s == 1.0 else torch.full((1,), s, dtype=torch.float32, device=self.device)
        lo = self.shard_lo
        n_decay_local = min(max(self.n_decay - lo, 0), self.shard)
        if shard is None and self.fz is not None:
            # one kernel: pull the peers' gradient shards, AdamW, push the parameters to every peer
            self._finish_grads()
            if self.partial_grad_group is not None and self.partial_end > self.partial_start and \
                    comm.group_size(self.partial_grad_group) > 1:
                dist.all_reduce(self.flat_grad[self.partial_start:self.partial_end], group=self.partial_grad_group)
            self.fz.step(self.master, self.exp_avg, self.exp_avg_sq, lo, self.shard, n_decay_local, lr, self.betas[0],
                         self.betas[1], self.eps, self.weight_decay, self.step_count, scale_t, None)
            return
        if shard is None:
            shard = self.reduce_gradients()
        p_shard = self.flat_param[lo:lo + self.shard]
        F.adamw_step(p_shard, shard, self.master, self.exp_avg, self.exp_avg_sq, n_decay=n_decay_local, lr=lr,
                     beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=self.weight_decay,
                     step=self.step_count, grad_scale=scale_t)
        if self.gsize > 1:
            dist.all_gather_into_tensor(self.flat_param, p_shard.clone() if not self.native else p_shard,
                                        group=self.group)

    # ------------------------------------------------------------------ (de)serialisation of the optimizer shard
    def state_dict(self) -> dict:
        return {"step": self.step_count, "master": None if self.master is None else self.master.cpu(),
                "exp_avg": self.exp_avg.cpu(),
                "exp_avg_sq": self.exp_avg_sq.cpu(), "shard_lo": self.shard_lo, "total": self.total,
                "names": list(self.names)}

    def load_state_dict(self, sd: dict) -> None:
        if sd["total"] != self.total or sd["shard_lo"] != self.shard_lo:
            raise ValueError("optimizer shard layout does not match the checkpoint")
        self.step_count = int(sd["step"])
        if (sd.get("master") is None) != (self.master is None):
            raise ValueError("the checkpoint's optimizer was saved with a different training.optimizer_master_weights")
        if self.master is not None:
            self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])

    def refresh_master_from_params(self) -> None:
        """After loading model weights into the parameter views."""
        lo = self.shard_lo
        if self.master is not None:
            self.master.copy_(self.flat_param[lo:lo + self.shard].float())


def lr_at(step: int, *, base_lr: float, total_steps: int, warmup_steps: int = 0, kind: str = "cosine",
          min_ratio: float = 0.0) -> float:
    """Learning rate of optimizer step ``step`` (0-based): linear warmup then cosine / linear / constant.
    Mirrors ``transformers.get_scheduler`` as used by the reference (python/ray/trainer.py:579-623)."""
    if warmup_steps > 0 and step < warmup_steps:
        return base_lr * step / max(1, warmup_steps)
    if kind in ("constant", "constant_with_warmup"):
        return base_lr
    prog = (step - warmup_steps) / max(1, total_steps - warmup_steps)
    prog = min(max(prog, 0.0), 1.0)
    if kind == "linear":
        return base_lr * max(min_ratio, 1.0 - prog)
    if kind == "cosine":
        return base_lr * max(min_ratio, 0.5 * (1.0 + math.cos(math.pi * prog)))
    raise ValueError(f"unknown lr_scheduler_type '{kind}'")
