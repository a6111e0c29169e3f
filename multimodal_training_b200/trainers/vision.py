"""Vision trainer: one sequence-parallel rank of the vision encoder.

Step API of the reference's ``QwenVisionTrainer`` (python/ray/vision.py:433-580): ``forward_step``
encodes this rank's slice of every image of its replica and returns the merged tokens (kept attached
to the autograd graph for ``backward_step``); ``backward_step`` takes the gradient of those tokens
from the text trainer.  Parameters are replicated over all vision ranks and optimised with ZeRO-1
over the whole world: gradients are summed over sequence-parallel ranks (they split the tokens) and
the data-parallel mean is already part of the incoming gradient.
"""
from __future__ import annotations

import torch

from ..models.vision import SPContext, VisionEncoder
from ..ops import attention as attn_mod
from .context import local_pixels
from .trainer import Trainer


class VisionTrainer(Trainer):
    kind = "vision"
    norm_type = "sequence"

    def build_model(self) -> bool:
        mesh = self._ensure_mesh()
        cfg = self._model_cfg()
        dev, dt = self._get_device(), self._dtype()
        if self.config.get("attention_backend") == "flash_attention_2" and self.config.get("library_attention"):
            attn_mod.set_backend("lib")
        cfg.vision.sequence_parallel = mesh.sp > 1
        ulysses = None
        if self.state.fused is not None and mesh.sp > 1 and self.config.get("fused_ulysses", True):
            from ..parallel.fused_ulysses import UlyssesFused
            ulysses = UlyssesFused(self.state.fused)
        sp = SPContext(mesh.sp_group, mesh.sp, mesh.sp_rank, fused=ulysses)
        self.model = VisionEncoder(cfg.vision, sp, dtype=dt, device=dev, seed=self.seed,
                                   activation_checkpointing=self.config.get("activation_checkpointing", True))
        pre = self.config.get("pretrained_checkpoint_dir")
        if pre:
            self._load_pretrained(pre)
        self._build_optimizer(self.model.named_parameters(), mesh.vision_zero_group if mesh.world > 1 else None,
                              grad_divisor=float(mesh.tdp))
        self._pending = []
        self._staging = None
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
        self.model.load_reference_state_dict(sd)

    def forward_step(self, iteration: int) -> dict:
        t0 = self._timer_start()
        ctx = self.step_context(iteration)
        dev = self._get_device()
        plan = ctx.vision_plan
        if dev.type == "cuda":
            n, d = plan.local_patch_index.numel(), self._model_cfg().vision.patch_dim
            if self._staging is None or self._staging.shape[0] < n:
                self._staging = torch.empty(n, d, dtype=torch.bfloat16).pin_memory()
            host = local_pixels(ctx, out=self._staging[:n])
            pixels = host.to(dev, non_blocking=True)
            self.h2d_bytes = host.numel() * host.element_size()
        else:
            pixels = local_pixels(ctx).to(self._dtype())
            self.h2d_bytes = 0
        merged = self.model(pixels, plan)
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
        if grad.dim() == merged.dim() + 1:
            grad = grad.squeeze(0)
        merged.backward(gradient=grad.to(merged.dtype))
        out = {}
        ms = self._timer_stop(t0)
        if ms is not None:
            out["backward_time_ms"] = ms
        return out


QwenVisionTrainer = VisionTrainer
