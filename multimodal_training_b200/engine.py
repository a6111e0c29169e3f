"""SPMD training engine: one process per GPU runs both halves of the model.

This is the launch mode for ``torchrun``-style jobs (and ``bench.py``): every rank builds a
:class:`VisionTrainer` and a :class:`TextTrainer` in the same process and calls them in the order
of the reference's driver loop (python/train_ray.py:315-382): zero_grad, vision forward, text
forward, text backward, vision backward, gradient norm, two optimizer steps.  The actor runtime in
``runtime/`` drives the same trainers through ``ActorGroup.execute_all`` instead.
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from .trainers.text import TextTrainer
from .trainers.trainer import process_state
from .trainers.vision import VisionTrainer
from .utils import tracing


class DeviceStepError(RuntimeError):
    """A kernel of the step reported a failure (a bounded wait on a peer ran out, an access was out of range)."""


class LossHandle:
    """Loss of one step on its way to the host (see ``HybridEngine.train_step_async``), together with a copy of the
    device error word taken behind the step: reading the loss also tells whether the step's kernels all finished
    their exchanges, without an extra synchronisation."""

    __slots__ = ("host", "event", "err")

    def __init__(self, host: torch.Tensor, event, err: torch.Tensor | None = None):
        self.host, self.event, self.err = host, event, err

    def value(self) -> float:
        if self.event is not None:
            self.event.synchronize()
        if self.err is not None and int(self.err[0]) != 0:
            from .ops.native import format_error
            raise DeviceStepError(format_error(*[int(x) for x in self.err[:4]]))
        return float(self.host[0])


class HybridEngine:
    def __init__(self, vision_config: dict, text_config: dict, rank: int | None = None):
        import os
        rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.vision = VisionTrainer(vision_config, rank)
        self.text = TextTrainer(text_config, rank)
        self.vision.build_model()
        self.text.build_model()
        self.vision.initialize_trainer()
        self.text.initialize_trainer()
        self.mesh = process_state().mesh
        self.clip = bool(text_config.get("clip_grad_norm", False))
        self.max_norm = float(text_config.get("max_grad_norm", 1.0))
        self.step_index = 0
        self.accum = self.text.accumulation_steps
        self.last_grad_norm = None
        # pinned host slots for train_step_async (allocated here: the first pinned allocation of a process is slow)
        pin = torch.cuda.is_available()
        self._loss_ring = [torch.zeros(1, dtype=torch.float32, pin_memory=pin) for _ in range(8)]
        self._err_ring = [torch.zeros(4, dtype=torch.int32, pin_memory=pin) for _ in range(8)]
        self._err_dev = None
        self._loss_i = 0
        # single-GPU runs hold the whole optimizer state on one device (37 ms of AdamW per 7B step);
        # training.overlap_optimizer puts the text update on a side stream behind the next vision forward.  Off by
        # default: measured on a B200 it changes nothing (206.6 ms with, 204-209 ms without), because the update's
        # thread blocks fill every SM before the persistent GEMM CTAs of the vision forward can become resident.
        self._opt_stream = None
        self._text_opt_event = None
        if (torch.cuda.is_available() and self.mesh.world == 1
                and bool(text_config.get("overlap_optimizer", False))):
            self._opt_stream = torch.cuda.Stream()
        # bench.py sets this to time the optimizer phase (gradient reduction, AdamW, parameter all-gather) of every
        # step with a pair of CUDA events, so that a step time without the optimizer can be reported
        self.record_optimizer_time = False
        self._opt_events: list = []
        # device-timed phases (CUDA events, no host syncs) when training.trace is on
        self.timer = None
        if bool(text_config.get("trace", False)) or tracing.enabled():
            tracing.enable(True)
            self.timer = tracing.PhaseTimer()

    @classmethod
    def from_config(cls, cfg: dict) -> "HybridEngine":
        from .config.loader import trainer_configs
        v, t = trainer_configs(cfg)
        return cls(v, t)

    def _global_grad_scale(self):
        """Device-side global-norm clipping coefficient (no host sync)."""
        vo, to = self.vision.optimizer, self.text.optimizer
        vs, ts = vo.reduce_gradients(), to.reduce_gradients()
        self.vision._reduced_shard, self.text._reduced_shard = vs, ts
        va, vb = vo.grad_norm_sq_local(vs)
        ta, tb = to.grad_norm_sq_local(ts)
        # parts that are replicated inside a tensor-parallel group are counted once
        vtp = self.mesh.sp if getattr(self.vision, "tensor_parallel", False) else 1
        total = va + vb / vtp + ta + tb / max(self.mesh.tp, 1)
        if self.mesh.world > 1:
            dist.all_reduce(total, group=self.mesh.world_group)
        norm = total.sqrt()
        self.last_grad_norm = norm
        return torch.clamp(self.max_norm / (norm + 1e-6), max=1.0)

    def train_step(self, step: int | None = None) -> torch.Tensor:
        """One optimisation step (``gradient_accumulation_steps`` micro-batches of one global batch each); returns
        this rank's loss averaged over the micro-batches (device scalar)."""
        step = self.step_index if step is None else step
        ph = self.timer.phase if self.timer is not None else (lambda name: tracing.trace_range(name))
        self.vision.zero_grad()
        self.text.zero_grad()
        # gradient accumulation: micro-batches run back to back into the same flat gradient (the weight-gradient
        # kernels overwrite on the first write of a step and accumulate afterwards); one optimizer step follows
        loss = None
        for micro in range(self.accum):
            idx = self.text.data_index(step, micro)
            with ph("vision.forward"):
                v_out = self.vision.forward_step(idx)
            if self._text_opt_event is not None:
                # the text optimizer of the previous step ran on its own stream, behind this step's vision forward
                torch.cuda.current_stream().wait_event(self._text_opt_event)
                self._text_opt_event = None
            with ph("text.forward"):
                t_out = self.text.forward_step(v_out, idx)
            with ph("text.backward"):
                g = self.text.backward_step()
            with ph("vision.backward"):
                self.vision.backward_step(g)          # a no-op for a batch without images
            loss = t_out["loss"] if loss is None else loss + t_out["loss"]
        if self.accum > 1:
            loss = loss / self.accum
        opt_ev = None
        if self.record_optimizer_time and torch.cuda.is_available():
            opt_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            opt_ev[0].record()
        with ph("optimizer"):
            scale = self._global_grad_scale() if self.clip else None
            for tr in (self.text, self.vision):
                shard = getattr(tr, "_reduced_shard", None)
                tr._reduced_shard = None
                if tr is self.text and self._opt_stream is not None:
                    # The text update is pure HBM streaming (fp32 master weights and moments) and the next step's
                    # vision forward does not read text parameters: run the update on a side stream so the two
                    # overlap; the next text forward waits for it.
                    self._opt_stream.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(self._opt_stream):
                        tr.optimizer.step(lr=tr.current_lr(), grad_scale=scale, shard=shard)
                    self._text_opt_event = self._opt_stream.record_event()
                else:
                    tr.optimizer.step(lr=tr.current_lr(), grad_scale=scale, shard=shard)
                tr.global_step += 1
        if opt_ev is not None:
            self.join_streams()
            opt_ev[1].record()
            self._opt_events.append(opt_ev)
        if self.timer is not None:
            self.timer.end_step()
        fused = process_state().fused
        if fused is not None:
            fused.end_step()          # after a step that reserved or moved heap regions: all ranks compare layouts
        self.step_index = step + 1
        return loss

    def optimizer_ms(self) -> float:
        """Device time of the optimizer phases recorded since the last call (synchronises; see
        ``record_optimizer_time``)."""
        if not self._opt_events:
            return 0.0
        self._opt_events[-1][1].synchronize()
        total = sum(a.elapsed_time(b) for a, b in self._opt_events)
        self._opt_events = []
        return total

    def join_streams(self) -> None:
        """Make the current stream wait for work this engine put on its side stream (no host synchronisation)."""
        if self._text_opt_event is not None:
            torch.cuda.current_stream().wait_event(self._text_opt_event)
            self._text_opt_event = None

    def synchronize(self) -> None:
        """Wait for everything this engine has launched, including an optimizer update on the side stream (call
        before reading parameters from the host, e.g. for a checkpoint)."""
        self.join_streams()
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    def train_step_async(self, step: int | None = None) -> "LossHandle":
        """``train_step`` plus a non-blocking copy of the loss into pinned host memory.

        The host does not wait for the GPU: the returned handle's ``value()`` waits for that step's copy only, so
        a training loop that reads the loss of step s-1 after launching step s logs every loss without ever
        draining the launch queue.  At most ``len(ring)`` handles may be outstanding.
        """
        loss = self.train_step(step)
        host = self._loss_ring[self._loss_i % len(self._loss_ring)]
        err = None
        host.copy_(loss.detach().float().reshape(1), non_blocking=True)
        event = None
        if loss.is_cuda:
            from .ops import native as nv
            if nv.available():
                if self._err_dev is None:
                    self._err_dev = nv.error_word_tensor()
                err = self._err_ring[self._loss_i % len(self._err_ring)]
                err.copy_(self._err_dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        self._loss_i += 1
        return LossHandle(host, event, err)

    # ------------------------------------------------------------------ checkpoints (same layout as the actor driver)
    def save_checkpoint(self, checkpoint_dir: str, tag, config: dict | None = None, extra_meta: dict | None = None):
        """Every rank writes its vision and text shard under ``epoch_N`` (``tag`` an int) or the directory named
        ``tag``; rank 0 then writes ``metadata.json``, which marks the checkpoint complete."""
        from .checkpoint import write_metadata
        self.synchronize()
        # a device-side failure (checked inside the trainers' save) raises here, before metadata.json marks the
        # checkpoint complete
        self.vision.save_checkpoint(checkpoint_dir, tag)
        self.text.save_checkpoint(checkpoint_dir, tag)
        if self.mesh.world > 1:
            dist.barrier(group=self.mesh.world_group)
        name = self.text._ckpt_name(tag)
        if self.mesh.rank == 0:
            import os
            paths = {k: [os.path.join(checkpoint_dir, name, k, f"rank_{r}.pt") for r in range(self.mesh.world)]
                     for k in ("vision", "text")}
            write_metadata(checkpoint_dir, name, paths["vision"], paths["text"], config or {},
                           dict({"epoch": tag}, **(extra_meta or {})))
        if self.mesh.world > 1:
            dist.barrier(group=self.mesh.world_group)
        return name

    def load_checkpoint(self, checkpoint_dir: str, tag) -> bool:
        """True only if every rank loaded both of its shards."""
        ok = self.vision.load_checkpoint(checkpoint_dir, tag) and self.text.load_checkpoint(checkpoint_dir, tag)
        if self.mesh.world > 1:
            dev = next(self.text.model.parameters()).device
            flag = torch.tensor([1 if ok else 0], device=dev, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.mesh.world_group)
            ok = bool(flag.item())
        return ok

    def set_global_step(self, step: int) -> None:
        self.vision.set_global_step(step)
        self.text.set_global_step(step)
        self.step_index = int(step)

    def mean_loss(self, loss: torch.Tensor) -> float:
        """Mean over text replicas (every TP rank of a replica holds the same loss)."""
        t = loss.detach().float().clone().reshape(1)
        if self.mesh.world > 1:
            dist.all_reduce(t, group=self.mesh.world_group)
            t /= self.mesh.world
        return float(t.item())
