"""Driver: one process that steers the vision and text actor groups through a training run.

``python -m multimodal_training_b200.train --config-path=configs --config-name=sample key=value ...``

Loop and log lines follow the reference (python/train_ray.py:141-459): per iteration zero_grad on
both groups, vision ``forward_step`` (async), text ``forward_step`` fed with the vision refs, text
``backward_step``, vision ``backward_step`` fed with the text refs, optional global-norm clipping,
two optimizer steps, memory stats, one log line; per epoch a checkpoint; at the end the line
``Training completed! E epochs, S total steps, M measured steps (avg X.XXXs/step)`` that sweep
scripts grep.  Differences: the data-parallel replicas see different samples, the LR schedule spans
all epochs, and there is no hidden 100-iteration cap.
"""
from __future__ import annotations

import logging
import math
import sys
import time

from .checkpoint import load_epoch_checkpoint, plan_resume, save_epoch_checkpoint, save_step_checkpoint
from .config.loader import parse_cli, trainer_configs
from .runtime.actor_group import ActorGroup, get
from .runtime.logger import setup_logging

log = logging.getLogger("mmt_b200")


def get_vision_trainer_class(model_type: str):
    if model_type == "qwen2_5_vl":
        from .trainers.vision import QwenVisionTrainer
        return QwenVisionTrainer
    raise ValueError(f"Unsupported vision model type: {model_type}")


def get_text_trainer_class(model_type: str):
    if model_type == "qwen2_5_vl":
        from .trainers.text import QwenTextTrainer
        return QwenTextTrainer
    raise ValueError(f"Unsupported text model type: {model_type}")


def aggregate_grad_norms(vision_norms: list[dict], text_norms: list[dict], dp_size: int = 1,
                         parallel_size: int = 1) -> float:
    """Global gradient norm from the per-actor squared-norm pieces.

    Each piece is ``{"type", "sharded", "replicated", ...}`` computed after gradient reduction on the
    actor's ZeRO shard.  ZeRO shards are disjoint, so sharded parts add over all actors.  Parameters
    that are replicated inside a tensor-parallel group (norm weights) appear once per TP rank and are
    counted once: their part is divided by the TP degree.  (The reference samples actors per replica for
    the same purpose, python/train_ray.py:37-122.)
    """
    total = 0.0
    for n in vision_norms:
        vtp = max(1, int(n.get("tp_size", 1))) if n.get("type") == "tensor" else 1
        total += float(n.get("sharded", 0.0)) + float(n.get("replicated", 0.0)) / vtp
    tp = max(1, int(text_norms[0].get("tp_size", parallel_size))) if text_norms else 1
    for n in text_norms:
        total += float(n.get("sharded", 0.0)) + float(n.get("replicated", 0.0)) / tp
    return math.sqrt(max(total, 0.0))


def main(cfg: dict) -> dict:
    setup_logging(force=True)
    tr = cfg["training"]
    vision_config, text_config = trainer_configs(cfg)
    parallel_size, dp_size = int(tr["parallel_size"]), int(tr.get("dp_size", 1))
    num_actors = parallel_size * dp_size
    collocate = bool(tr.get("collocate", True))
    log.info("Creating %d vision and %d text actors (collocate=%s)", num_actors, num_actors, collocate)

    vision_cls = get_vision_trainer_class(cfg["vision"]["model_type"])
    text_cls = get_text_trainer_class(cfg["text"]["model_type"])
    vision_group = ActorGroup(vision_config, vision_cls, num_actors, collocate=collocate,
                              rpc_timeout_s=tr.get("rpc_timeout_s"))
    if collocate:
        # the halves share hosts (one process and one torch.distributed world per GPU): the handoff is an exchange
        # inside that world, or a peer store
        text_group = ActorGroup(text_config, text_cls, num_actors, collocate=True,
                                placement_group_handle=vision_group.placement_group_handle)
    else:
        # training.collocate: false -- the text half gets host processes (and, when the node has enough of them,
        # GPUs) of its own and a world of its own.  Vision actor i's rows travel to text actor i by value through
        # the driver (ActorGroup._localise), the text group exchanges them among its own ranks, and the gradient
        # comes back the same way (python/train_ray.py:257-260 moves these tensors with Ray's NCCL transport).
        offset = 0
        try:
            import torch
            if torch.cuda.is_available() and torch.cuda.device_count() >= 2 * num_actors:
                offset = num_actors
        except Exception:  # noqa: BLE001
            pass
        text_group = ActorGroup(text_config, text_cls, num_actors, collocate=False,
                                rpc_timeout_s=tr.get("rpc_timeout_s"), gpu_offset=offset)
        log.info("Text actors on hosts of their own (GPU offset %d)", offset)
    try:
        return _run(cfg, vision_group, text_group, num_actors, parallel_size, dp_size)
    finally:
        vision_group.shutdown()
        if not collocate:
            text_group.shutdown()


def _run(cfg, vision_group, text_group, num_actors, parallel_size, dp_size) -> dict:
    tr = cfg["training"]
    vision_group.execute_all("build_model")
    text_group.execute_all("build_model")
    vision_group.execute_all("initialize_trainer")
    text_group.execute_all("initialize_trainer")
    vision_group.execute_all("set_receiver_info", text_group.execute_all("get_physical_gpu_id"))

    num_epochs, num_iterations = int(tr["num_epochs"]), int(tr["num_iterations"])
    warmup_steps = int(tr.get("warmup_steps", 0))
    accum = max(1, int(tr.get("gradient_accumulation_steps", 1)))
    log_interval = max(1, int(tr.get("log_interval", 1)))
    clip = bool(tr.get("clip_grad_norm", False))
    profile_time = bool(tr.get("profile_time", False))
    checkpoint_dir = tr.get("checkpoint_dir", "/tmp/checkpoints")
    use_ckpt = not bool(tr.get("no_checkpoint", True))

    save_every = int(tr.get("save_every_steps", 0) or 0)
    keep_steps = int(tr.get("keep_step_checkpoints", 2))
    max_steps = int(tr.get("max_steps", 0) or 0)          # stop after this many optimizer steps (0 = run to the end)

    start_epoch, start_iteration = 0, 0
    plan = plan_resume(checkpoint_dir, num_iterations) if use_ckpt else None
    if plan is not None:
        tag, e, i = plan
        if load_epoch_checkpoint(checkpoint_dir, tag, vision_group, text_group):
            start_epoch, start_iteration = e, i
            log.info("Resumed from %s (next: epoch %d, iteration %d)", tag if isinstance(tag, str) else f"epoch {tag}",
                     e, i)
        else:
            log.warning("Failed to load checkpoint %s; starting from scratch", tag)

    global_step = start_epoch * num_iterations + start_iteration
    if global_step:
        # the learning-rate schedule continues where the saved run stopped
        vision_group.execute_all("set_global_step", global_step)
        text_group.execute_all("set_global_step", global_step)
    measured, measured_time, losses = 0, 0.0, []
    stop = False
    # Steps whose losses have not been read yet.  Reading a loss makes the driver wait for the devices, so with
    # training.log_interval > 1 it is done at the logging points only (and before checkpoints and at the end): in
    # between, the actors' hosts run ahead of their GPUs and the launch latency of a step hides behind the previous
    # step's kernels.  With log_interval = 1 every step is read at once, as in the reference's loop.
    pending: list[dict] = []
    t_mark = time.perf_counter()

    def flush(log_line: bool) -> None:
        nonlocal measured, measured_time, t_mark
        if not pending:
            return
        outs = [[get(refs) for refs in p["text_refs"]] for p in pending]       # waits for the newest step
        vmem = get(vision_group.execute_all_async("get_memory_stats"))
        tmem = get(text_group.execute_all_async("get_memory_stats"))
        dt = (time.perf_counter() - t_mark) / len(pending)
        for p, micro_outs in zip(pending, outs):
            loss = 0.0
            for text_out in micro_outs:
                step_losses = [float(o["loss"]) for o in text_out]
                loss += sum(step_losses) / len(step_losses) / accum
            p["loss"], p["text_out"] = loss, micro_outs[-1]
            losses.append(loss)
            if not p["is_warmup"]:
                measured += 1
                measured_time += dt
            for refs in p["text_refs"]:
                text_group.free(refs)
            for group, refs in p["acks"]:
                get(refs)
                group.free(refs)
            for group, refs in p["late_free"]:
                group.free(refs)
        p = pending[-1]
        if log_line:
            avg = lambda xs, k: sum(x[k] for x in xs) / len(xs)  # noqa: E731
            line = (f"Epoch {p['epoch'] + 1}/{num_epochs}, Iter {p['iteration'] + 1}/{num_iterations} "
                    f"({'warmup' if p['is_warmup'] else 'training'}) - Loss: {p['loss']:.4f}, "
                    f"Iteration time: {dt:.3f}s")
            if profile_time:
                line += (f", Vision fwd: {avg(p['vision_fwd'], 'forward_time_ms'):.1f}ms, "
                         f"Vision bwd: {avg(p['vision_bwd'], 'backward_time_ms'):.1f}ms, "
                         f"Text fwd: {avg(p['text_out'], 'forward_time_ms'):.1f}ms, "
                         f"Text bwd: {avg(p['text_bwd'], 'backward_time_ms'):.1f}ms")
            if p["global_norm"] is not None:
                line += f", Grad norm: {p['global_norm']:.4f}"
            line += (f", Vision mem: {avg(vmem, 'allocated_mb'):.0f} MB (peak {avg(vmem, 'peak_mb'):.0f}), "
                     f"Text mem: {avg(tmem, 'allocated_mb'):.0f} MB (peak {avg(tmem, 'peak_mb'):.0f})")
            log.info(line)
        pending.clear()
        t_mark = time.perf_counter()

    for epoch in range(start_epoch, num_epochs):
        for iteration in range(start_iteration if epoch == start_epoch else 0, num_iterations):
            is_warmup = global_step < warmup_steps
            # calls whose results the driver does not need are only queued (the hosts execute an actor's calls in
            # order); their acknowledgements are collected at the next logging point, where a failure would surface
            acks = [(vision_group, vision_group.execute_all_async("zero_grad")),
                    (text_group, text_group.execute_all_async("zero_grad"))]
            kept_text_refs = []
            log_now = iteration % log_interval == 0
            for micro in range(accum):
                if micro:
                    vision_group.free(vision_refs + vision_bwd_refs)
                    text_group.free(text_bwd_refs)
                idx = global_step * accum + micro
                vision_refs = vision_group.execute_all_async("forward_step", idx)
                text_refs = text_group.execute_all_async("forward_step", vision_refs, [idx] * num_actors)
                kept_text_refs.append(text_refs)
                text_bwd_refs = text_group.execute_all_async("backward_step")
                vision_bwd_refs = vision_group.execute_all_async("backward_step", text_bwd_refs)
                # the text half's result carries the gradient for the vision half: it stays in the actors' object
                # table (fetching it would copy it to the driver); waiting for the vision half covers both
                vision_bwd = get(vision_bwd_refs) if (log_now or clip or micro + 1 < accum) else None
                text_bwd = get(text_bwd_refs) if (profile_time and log_now) else None
            global_norm = None
            if clip:
                vn = vision_group.execute_all("compute_grad_norm_contribution")
                tn = text_group.execute_all("compute_grad_norm_contribution")
                global_norm = aggregate_grad_norms(vn, tn, dp_size, parallel_size)
            acks.append((text_group, text_group.execute_all_async("optimizer_step", global_norm)))
            acks.append((vision_group, vision_group.execute_all_async("optimizer_step", global_norm)))
            pending.append({"epoch": epoch, "iteration": iteration, "is_warmup": is_warmup, "text_refs": kept_text_refs,
                            "acks": acks, "late_free": [] if vision_bwd is not None else
                            [(vision_group, vision_refs + vision_bwd_refs), (text_group, text_bwd_refs)],
                            "global_norm": global_norm, "text_bwd": text_bwd, "vision_bwd": vision_bwd,
                            "vision_fwd": get(vision_refs) if (profile_time and log_now) else None})
            if log_now or len(pending) >= 8:
                flush(log_now)
            if vision_bwd is not None:            # otherwise freed at the next logging point, once the calls have run
                vision_group.free(vision_refs + vision_bwd_refs)
                text_group.free(text_bwd_refs)
            global_step += 1
            last_of_epoch = iteration + 1 == num_iterations
            if use_ckpt and save_every and global_step % save_every == 0 and not last_of_epoch:
                flush(False)
                save_step_checkpoint(checkpoint_dir, global_step, epoch, iteration + 1, vision_group, text_group, cfg,
                                     keep=keep_steps)
                t_mark = time.perf_counter()
            if max_steps and global_step >= max_steps:
                stop = True
                break
        flush(False)
        if use_ckpt and global_step == (epoch + 1) * num_iterations:       # the epoch ran to its end
            save_epoch_checkpoint(checkpoint_dir, epoch, vision_group, text_group, cfg)
            t_mark = time.perf_counter()
        if stop:
            log.info("Stopping after %d steps (training.max_steps)", global_step)
            break
    avg_t = measured_time / measured if measured else float("nan")
    log.info("Training completed! %d epochs, %d total steps, %d measured steps (avg %.3fs/step)", num_epochs,
             global_step, measured, avg_t)
    log.info("Average iteration time: %.3fs", avg_t)
    return {"losses": losses, "avg_step_s": avg_t, "steps": global_step}


def cli(argv: list[str] | None = None) -> int:
    cfg, _ = parse_cli(argv)
    main(cfg)
    return 0


if __name__ == "__main__":
    sys.exit(cli())
