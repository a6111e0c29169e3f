"""Training driver for ``torchrun``-style launches: one process per GPU runs both halves of the model.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 -m multimodal_training_b200.train_spmd \
        --config-path configs --config-name sample training.parallel_size=8

Same configuration, data order, checkpoints (layout, resume rules, step-granular saves) and log lines as the actor
driver ``multimodal_training_b200.train`` (the reference's python/train_ray.py:141-459), without the actor runtime in
between: every rank builds a :class:`~multimodal_training_b200.engine.HybridEngine` and calls ``train_step`` in
lockstep.  The host never waits for the GPU between logging points: the loss of a step is copied to pinned memory
and read when it is logged (``training.log_interval``), so with a sparse log interval the launch queue stays full.
"""
from __future__ import annotations

import logging
import sys
import time

import torch.distributed as dist

from .checkpoint import plan_resume
from .config.loader import parse_cli
from .engine import HybridEngine
from .runtime.logger import setup_logging
from .trainers.trainer import init_distributed_comm

log = logging.getLogger("mmt_b200")


def main(cfg: dict) -> dict:
    setup_logging(force=True)
    tr = cfg["training"]
    # a rank that dies between steps makes the others' next collective fail after this long instead of waiting for
    # the library's default (ten minutes for NCCL)
    init_distributed_comm(tr.get("backend"), tr.get("dist_timeout_s"))
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    expected = int(tr["parallel_size"]) * int(tr.get("dp_size", 1))
    if world != expected:
        raise RuntimeError(f"launched with {world} ranks but training.parallel_size x dp_size = {expected}")
    if not bool(tr.get("collocate", True)) and rank == 0:
        log.warning("training.collocate=false is a placement of the actor driver (python -m multimodal_training_b200."
                    "train); this launcher runs one process per GPU with both halves in it")
    engine = HybridEngine.from_config(cfg)

    num_epochs, num_iterations = int(tr["num_epochs"]), int(tr["num_iterations"])
    warmup_steps = int(tr.get("warmup_steps", 0))
    log_interval = max(1, int(tr.get("log_interval", 1)))
    checkpoint_dir = tr.get("checkpoint_dir", "/tmp/checkpoints")
    use_ckpt = not bool(tr.get("no_checkpoint", True))
    save_every = int(tr.get("save_every_steps", 0) or 0)
    max_steps = int(tr.get("max_steps", 0) or 0)

    start_epoch, start_iteration = 0, 0
    plan = plan_resume(checkpoint_dir, num_iterations) if use_ckpt else None
    if plan is not None:
        tag, e, i = plan
        if engine.load_checkpoint(checkpoint_dir, tag):
            start_epoch, start_iteration = e, i
            if rank == 0:
                log.info("Resumed from %s (next: epoch %d, iteration %d)",
                         tag if isinstance(tag, str) else f"epoch {tag}", e, i)
        elif rank == 0:
            log.warning("Failed to load checkpoint %s; starting from scratch", tag)
    global_step = start_epoch * num_iterations + start_iteration
    if global_step:
        engine.set_global_step(global_step)

    losses, measured, measured_time = [], 0, 0.0
    pending = []                      # (epoch, iteration, step, handle) not logged yet
    t_mark, steps_since_mark = time.perf_counter(), 0
    stop = False

    def flush_log():
        """Read the loss of the newest pending step (one host wait), log it with the mean step time since the last
        logging point."""
        nonlocal t_mark, steps_since_mark, measured, measured_time
        if not pending:
            return
        epoch, iteration, step, handle = pending[-1]
        local = handle.value()                              # waits for that step only
        loss = local
        if world > 1:
            import torch
            t = torch.tensor([local], dtype=torch.float64)
            if dist.get_backend() == "nccl":
                t = t.cuda()
            dist.all_reduce(t)
            loss = float(t.item()) / world
        now = time.perf_counter()
        dt = (now - t_mark) / max(steps_since_mark, 1)
        for _, _, s, _ in pending:
            if s >= warmup_steps:
                measured += 1
                measured_time += dt
        losses.append(loss)
        if rank == 0:
            line = (f"Epoch {epoch + 1}/{num_epochs}, Iter {iteration + 1}/{num_iterations} "
                    f"({'warmup' if step < warmup_steps else 'training'}) - Loss: {loss:.4f}, "
                    f"Iteration time: {dt:.3f}s")
            if engine.last_grad_norm is not None:
                line += f", Grad norm: {float(engine.last_grad_norm):.4f}"
            vm, tm = engine.vision.get_memory_stats(), engine.text.get_memory_stats()
            line += f", Mem: {tm['allocated_mb']:.0f} MB (peak {max(vm['peak_mb'], tm['peak_mb']):.0f})"
            log.info(line)
        pending.clear()
        t_mark, steps_since_mark = time.perf_counter(), 0

    for epoch in range(start_epoch, num_epochs):
        for iteration in range(start_iteration if epoch == start_epoch else 0, num_iterations):
            handle = engine.train_step_async(global_step)
            pending.append((epoch, iteration, global_step, handle))
            steps_since_mark += 1
            global_step += 1
            if iteration % log_interval == 0 or len(pending) >= 6:
                flush_log()
            last_of_epoch = iteration + 1 == num_iterations
            if use_ckpt and save_every and global_step % save_every == 0 and not last_of_epoch:
                flush_log()
                engine.save_checkpoint(checkpoint_dir, f"step_{global_step}", cfg,
                                       {"epoch": epoch, "next_iteration": iteration + 1, "global_step": global_step})
                if rank == 0:
                    _prune_steps(checkpoint_dir, int(tr.get("keep_step_checkpoints", 2)))
                t_mark = time.perf_counter()
            if max_steps and global_step >= max_steps:
                stop = True
                break
        flush_log()
        if use_ckpt and global_step == (epoch + 1) * num_iterations:
            engine.save_checkpoint(checkpoint_dir, epoch, cfg)
            t_mark = time.perf_counter()
        if stop:
            break
    engine.synchronize()
    if engine.timer is not None:
        # training.trace: device time per phase, and a chrome://tracing file per rank when a path is given
        phases = engine.timer.summary()
        if rank == 0:
            log.info("Device time per phase (mean ms per step): %s",
                     ", ".join(f"{k} {v:.2f}" for k, v in phases.items()))
        if tr.get("trace_file"):
            engine.timer.chrome_trace(f"{tr['trace_file']}.rank{rank}.json", rank=rank)
    avg_t = measured_time / measured if measured else float("nan")
    if rank == 0:
        log.info("Training completed! %d epochs, %d total steps, %d measured steps (avg %.3fs/step)", num_epochs,
                 global_step, measured, avg_t)
        log.info("Average iteration time: %.3fs", avg_t)
    return {"losses": losses, "avg_step_s": avg_t, "steps": global_step}


def _prune_steps(checkpoint_dir: str, keep: int) -> None:
    import os
    import shutil

    from .checkpoint import _step_dirs
    if keep <= 0:
        return
    for old in sorted(_step_dirs(checkpoint_dir))[:-keep]:
        shutil.rmtree(os.path.join(checkpoint_dir, f"step_{old}"), ignore_errors=True)


def cli(argv: list[str] | None = None) -> int:
    cfg, _ = parse_cli(argv)
    main(cfg)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(cli())
