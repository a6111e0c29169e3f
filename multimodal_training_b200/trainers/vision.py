"""Vision trainer: one sequence-parallel rank of the vision encoder.

Step API of the reference's ``QwenVisionTrainer`` (python/ray/vision.py:433-580): ``forward_step``
encodes this rank's slice of every image of its replica and returns the merged tokens (kept attached
to the autograd graph for ``backward_step``); ``backward_step`` takes the gradient of those tokens
from the text trainer.  Parameters are replicated over all vision ranks and optimised with ZeRO-1
over the whole world: gradients are summed over sequence-parallel ranks (they split the tokens) and
the data-parallel mean is already part of the incoming gradient.

With ``vision.parallelism: tensor`` the ranks of the group split heads and MLP columns instead of tokens (see
``models/vision.py``): every rank encodes all images of its replica, hands its window-aligned share of the
(replicated) output to the text side exactly as a sequence-parallel rank would, and in backward the shares'
gradients are all-gathered so that every rank back-propagates the full gradient.  ZeRO-1 then runs over the ranks
that hold the same shard (one per replica).
"""
from __future__ import annotations

import torch

from ..models.vision import SPContext, VisionEncoder
from ..ops import attention as attn_mod
from ..parallel import comm
from ..parallel.sp import build_vision_plan
from ..parallel.tp import TPContext
from .context import StagingRing, local_pixels
from .trainer import Trainer


class _OutputShare(torch.autograd.Function):
    """Rows ``rows[rank]`` of a tensor that is replicated over ``group``; backward gathers every rank's gradient
    rows into the full gradient (each row belongs to exactly one rank)."""

    @staticmethod
    def forward(ctx, full, rows, rank, group):
        ctx.rows, ctx.group, ctx.n = rows, group, full.shape[0]
        return full.index_select(0, rows[rank])

    @staticmethod
    def backward(ctx, g):
        parts = comm.all_gather_ragged(g, [int(r.numel()) for r in ctx.rows], ctx.group)
        out = g.new_empty((ctx.n,) + tuple(g.shape[1:]))
        for rows, part in zip(ctx.rows, parts):
            out.index_copy_(0, rows, part)
        return out, None, None, None


class VisionTrainer(Trainer):
    kind = "vision"
    norm_type = "sequence"

    def build_model(self) -> bool:
        mesh = self._ensure_mesh()
        cfg = self._model_cfg()
        dev, dt = self._get_device(), self._dtype()
        if self.config.get("attention_backend") == "flash_attention_2" and self.config.get("library_attention"):
            attn_mod.set_backend("lib")
        self.tensor_parallel = self.config.get("parallelism") == "tensor" and mesh.sp > 1
        cfg.vision.sequence_parallel = mesh.sp > 1 and not self.tensor_parallel
        ulysses = None
        if (self.state.fused is not None and mesh.sp > 1 and not self.tensor_parallel
                and self.config.get("fused_ulysses", True)):
            from ..parallel.fused_ulysses import UlyssesFused
            ulysses = UlyssesFused(self.state.fused)
            self.state.fused.ulysses = True
        if self.tensor_parallel:
            # the mesh's vision group is the tensor-parallel group; nothing is sequence parallel inside the model
            self.norm_type = "tensor"
            sp, tp = SPContext(), TPContext(mesh.sp_group, mesh.sp, mesh.sp_rank)
        else:
            sp, tp = SPContext(mesh.sp_group, mesh.sp, mesh.sp_rank, fused=ulysses), None
        self.model = VisionEncoder(cfg.vision, sp, dtype=dt, device=dev, seed=self.seed, tp=tp,
                                   activation_checkpointing=self.config.get("activation_checkpointing", True))
        pre = self.config.get("pretrained_checkpoint_dir")
        if pre:
            self._load_pretrained(pre)
        if self.tensor_parallel:
            zero_group = mesh.vdp_group if mesh.vdp > 1 else None      # the ranks that hold the same shard
        else:
            zero_group = mesh.vision_zero_group if mesh.world > 1 else None
        self._build_optimizer(self.model.named_parameters(), zero_group, grad_divisor=float(mesh.tdp))
        self._pending = []
        self._staging = StagingRing(pin=dev.type == "cuda")
        return True

    def _load_pretrained(self, directory: str) -> None:
        import os
        path = os.path.join(directory, "vision_model.pt")
        if not os.path.exists(path):
            import logging
            logging.getLogger("mmt_b200").warning("pretrained vision weights %s not found; keeping random init", path)
            return
        payload = torch.load(path, map_location="cpu", weights_only=False)
        self.model.load_reference_state_dict(payload["model"])

    def _load_model_state(self, sd: dict, sharded: bool) -> None:
        self.model.load_reference_state_dict(sd, sharded=sharded and self.tensor_parallel)

    def _tensor_parallel_views(self, ctx):
        """The plan over ALL tokens of this replica's images, and for every rank of the group the rows of the full
        merged stream that form its window-aligned share (in that share's own order)."""
        hit = getattr(ctx, "_vision_tp_views", None)
        if hit is not None:
            return hit
        mesh, v = self._ensure_mesh(), self._model_cfg().vision
        grids = [g for i in ctx.vision_samples for g in ctx.samples[i].grid_thw]
        kw = dict(spatial_merge_size=v.spatial_merge_size, window_size=v.window_size, patch_size=v.patch_size,
                  head_dim=v.head_dim)
        full = build_vision_plan(grids, sp=1, rank=0, **kw)
        inverse = torch.empty_like(full.local_merged_ids)
        inverse[full.local_merged_ids] = torch.arange(inverse.numel())
        rows = [inverse[build_vision_plan(grids, sp=mesh.sp, rank=r, **kw).local_merged_ids] for r in range(mesh.sp)]
        ctx._vision_tp_views = (full, rows)
        return full, rows

    def forward_step(self, iteration: int) -> dict:
        t0 = self._timer_start()
        ctx = self.step_context(iteration)
        dev = self._get_device()
        if self.state.fused is not None:
            self.state.fused.begin_step(ctx.sizes)
        plan, rows = ctx.vision_plan, None
        if plan is None:
            # no image in this replica's share of the batch: nothing to encode, nothing to hand over
            self._pending.append(None)
            return {"vision_embeddings": None, "sample_index": [ctx.samples[i].sample_index
                                                                for i in ctx.vision_samples],
                    "iteration": iteration}
        if self.tensor_parallel:
            plan, rows = self._tensor_parallel_views(ctx)
        if dev.type == "cuda":
            n, d = plan.local_patch_index.numel(), self._model_cfg().vision.patch_dim
            host = local_pixels(ctx, out=self._staging.acquire(n, d, torch.bfloat16), plan=plan)
            pixels = host.to(dev, non_blocking=True)
            self._staging.copied()
            self.h2d_bytes = host.numel() * host.element_size()
        else:
            pixels = local_pixels(ctx, plan=plan).to(self._dtype())
            self.h2d_bytes = 0
        merged = self.model(pixels, plan)
        if rows is not None:
            mesh = self._ensure_mesh()
            merged = _OutputShare.apply(merged, [r.to(dev) for r in rows], mesh.sp_rank, mesh.sp_group)
        self._pending.append(merged)
        out = {"vision_embeddings": merged.detach(), "sample_index": [ctx.samples[i].sample_index
                                                                      for i in ctx.vision_samples],
               "iteration": iteration}
        ms = self._timer_stop(t0)
        if ms is not None:
            out["forward_time_ms"] = ms
        return out

    def backward_step(self, grad) -> dict:
        t0 = self._timer_start()
        if isinstance(grad, dict):
            grad = grad["grad"]
        merged = self._pending.pop(0)
        if merged is None or grad is None:
            return {}
        if grad.dim() == merged.dim() + 1:
            grad = grad.squeeze(0)
        merged.backward(gradient=grad.to(device=merged.device, dtype=merged.dtype))
        out = {}
        ms = self._timer_stop(t0)
        if ms is not None:
            out["backward_time_ms"] = ms
        return out


QwenVisionTrainer = VisionTrainer
