"""Text trainer: one tensor-parallel rank of the decoder with sequence-parallel activations.

Step API of the reference's ``QwenTextTrainer`` (python/ray/text.py:697-1053): ``forward_step`` takes
the vision trainer's output, routes merged tokens to the rows of their image placeholders, runs the
decoder and the vocab-parallel loss; ``backward_step`` back-propagates and returns the gradient of
the vision tokens.  The desync guards of the reference are kept: iteration equality, sample-index
equality, placeholder count equals vision rows, labels ignored at image positions.
"""
from __future__ import annotations

import torch

from ..models.text import TextDecoder, mrope_cos_sin
from ..ops import attention as attn_mod
from ..ops.attention import SeqInfo
from ..parallel.handoff import exchange_vision_rows, splice_rows
from ..parallel.tp import TPContext
from .trainer import Trainer


class TextTrainer(Trainer):
    kind = "text"
    norm_type = "tensor"

    def build_model(self) -> bool:
        mesh = self._ensure_mesh()
        cfg = self._model_cfg()
        dev, dt = self._get_device(), self._dtype()
        if self.config.get("attention_backend") == "flash_attention_2" and self.config.get("library_attention"):
            attn_mod.set_backend("lib")
        tp = TPContext(mesh.tp_group, mesh.tp, mesh.tp_rank, fused=self.state.fused)
        self.model = TextDecoder(cfg.text, tp, dtype=dt, device=dev, seed=self.seed,
                                 activation_checkpointing=self.config.get("activation_checkpointing", True))
        self.model.tp_block = bool(self.config.get("tp_block", True))
        pre = self.config.get("pretrained_checkpoint_dir")
        if pre:
            self._load_pretrained(pre)
        self._build_optimizer(self.model.named_parameters(), mesh.tdp_group if mesh.tdp > 1 else None,
                              grad_divisor=float(mesh.tdp), partial_grad_group=mesh.tp_group if mesh.tp > 1 else None)
        self._loss = None
        self._vision_leaf = None
        return True

    def _load_pretrained(self, directory: str) -> None:
        import logging
        import os
        path = os.path.join(directory, "text_model.pt")
        if not os.path.exists(path):
            logging.getLogger("mmt_b200").warning("pretrained text weights %s not found; keeping random init", path)
            return
        payload = torch.load(path, map_location="cpu", weights_only=False)
        self.model.load_reference_state_dict(payload["model"], sharded=False)

    def _load_model_state(self, sd: dict, sharded: bool) -> None:
        self.model.load_reference_state_dict(sd, sharded=sharded)

    def forward_step(self, vision_out, iteration: int) -> dict:
        t0 = self._timer_start()
        mesh = self._ensure_mesh()
        cfg = self._model_cfg()
        ctx = self.step_context(iteration)
        dev = self._get_device()
        if self.state.fused is not None:
            self.state.fused.begin_step(ctx.sizes)
        tb = ctx.text_batch
        vis = None
        if vision_out is not None:
            if isinstance(vision_out, dict):
                if vision_out.get("iteration", iteration) != iteration:
                    raise RuntimeError(f"vision output is for iteration {vision_out['iteration']}, "
                                       f"text step is {iteration}")
                vis = vision_out["vision_embeddings"]
                # the vision half must have encoded exactly the samples that this step's context assigns to its
                # replica (same guard as the reference's sample-index check, python/ray/text.py:794-807; there both
                # halves see the whole batch, here the vision replica's share is the expected list)
                got = vision_out.get("sample_index")
                want = [ctx.samples[i].sample_index for i in ctx.vision_samples]
                if got is not None and list(got) != want:
                    raise RuntimeError(f"vision output covers samples {list(got)[:8]}..., this step expects "
                                       f"{want[:8]}... (the halves are out of step)")
            else:
                vis = vision_out
        # ---- guards (host metadata only, no device sync)
        n_rows = sum(len(r) for r in tb.image_rows)
        if n_rows and ctx.handoff is None:
            raise RuntimeError("image placeholders present but no handoff plan")
        img_rows = torch.from_numpy(__import__("numpy").concatenate(tb.image_rows)) if n_rows else None
        if img_rows is not None and bool((tb.shifted_labels[(img_rows - 1).clamp(min=0)] != -100).any()):
            # label of position t-1 predicts token t; image tokens must not be predicted
            raise RuntimeError("labels are not ignored at image placeholder positions")

        ids = tb.input_ids.to(dev, non_blocking=True)
        labels = tb.shifted_labels.to(dev, non_blocking=True)
        self.h2d_bytes = ids.numel() * 8 * 2 + tb.position_ids.numel() * 8
        x = self.model.embed(ids)                           # [T/tp, H] token shard
        if ctx.handoff is not None:
            plan = ctx.handoff
            if vis is None:
                raise RuntimeError("this batch has images but no vision output was passed")
            if vis.shape[0] != sum(plan.send_counts):
                raise RuntimeError(f"vision rows ({vis.shape[0]}) do not match the plan ({sum(plan.send_counts)})")
            # rows handed over by value from a vision actor in another process arrive as host tensors
            leaf = vis.detach().to(device=dev, dtype=x.dtype).requires_grad_(True)
            self._vision_leaf = leaf
            fused = self.state.fused
            if fused is not None and x.is_cuda:
                x = fused.handoff(leaf, x, plan)
            else:
                recv = exchange_vision_rows(leaf, plan, mesh)
                x = splice_rows(x, recv, plan.recv_rows.to(dev))
        cos, sin = mrope_cos_sin(tb.position_ids, cfg.text.head_dim, cfg.text.rope_theta, cfg.text.mrope_section,
                                 device=dev)
        seq = SeqInfo.from_list(tb.cu_seqlens, dev)
        h = self.model(x, cos, sin, seq)
        loss = self.model.loss(h, labels, chunk_rows=int(self.config.get("ce_chunk_rows", 4096)),
                               label_smoothing=float(self.config.get("label_smoothing", 0.0) or 0.0))
        self._loss = loss
        out = {"loss": loss.detach(), "sample_index": tb.sample_index, "iteration": iteration}
        if loss.is_cuda and bool(self.config.get("async_loss", True)):
            out["loss_async"] = self._loss_handle(loss)
        ms = self._timer_stop(t0)
        if ms is not None:
            out["forward_time_ms"] = ms
        return out

    def _loss_handle(self, loss: torch.Tensor):
        """The loss (and the device error word) on their way to pinned host memory, with an event behind the copies:
        whoever reads the loss later -- the actor runtime when it ships this step's result to the driver -- waits for
        that event only and learns at the same time whether a kernel reported a failed wait."""
        from ..engine import LossHandle
        from ..ops import native as nv
        ring = getattr(self, "_loss_ring", None)
        if ring is None:
            # the actor driver reads losses at logging points, at the latest after 8 optimizer steps; every
            # micro-batch of those steps holds a slot until then
            slots = max(32, 16 * int(getattr(self, "accumulation_steps", 1)))
            ring = self._loss_ring = [(torch.zeros(1, dtype=torch.float32, pin_memory=True),
                                       torch.zeros(4, dtype=torch.int32, pin_memory=True)) for _ in range(slots)]
            self._loss_i = 0
            self._err_dev = nv.error_word_tensor() if nv.available() else None
        host, err = ring[self._loss_i % len(ring)]
        self._loss_i += 1
        host.copy_(loss.detach().float().reshape(1), non_blocking=True)
        if self._err_dev is not None:
            err.copy_(self._err_dev, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return LossHandle(host, event, err if self._err_dev is not None else None)

    def backward_step(self) -> dict:
        t0 = self._timer_start()
        if self._loss is None:
            raise RuntimeError("backward_step called before forward_step")
        self._loss.backward()
        self._loss = None
        grad = None
        if self._vision_leaf is not None:
            grad = self._vision_leaf.grad
            self._vision_leaf = None
        out = {"grad": grad}
        ms = self._timer_stop(t0)
        if ms is not None:
            out["backward_time_ms"] = ms
        return out


QwenTextTrainer = TextTrainer
