"""Epoch checkpoints fanned out over both actor groups.

Layout of the reference (python/checkpoint.py:15-136), kept bit-for-bit at the path level::

    {checkpoint_dir}/epoch_{N}/vision/rank_{r}.pt   {"model": state_dict}
    {checkpoint_dir}/epoch_{N}/text/rank_{r}.pt     {"model": state_dict}
    {checkpoint_dir}/epoch_{N}/metadata.json        {epoch, timestamp, vision_checkpoints, text_checkpoints,
                                                     config_summary}

plus an optional superset written when ``training.save_optimizer`` is set
(``{vision,text}_optim/rank_{r}.pt``: optimizer shard, step counter, RNG state).  Files are written
to a temporary name and renamed, so a crash never leaves a half-written shard under the final name.
"""
from __future__ import annotations

import json
import logging
import os
import re
import time

log = logging.getLogger("mmt_b200")


def find_latest_checkpoint(checkpoint_dir: str) -> int | None:
    """Largest N such that ``epoch_N/metadata.json`` exists, or None."""
    if not os.path.isdir(checkpoint_dir):
        return None
    best = None
    for name in os.listdir(checkpoint_dir):
        m = re.fullmatch(r"epoch_(\d+)", name)
        if m and os.path.isfile(os.path.join(checkpoint_dir, name, "metadata.json")):
            n = int(m.group(1))
            best = n if best is None or n > best else best
    return best


def save_epoch_checkpoint(checkpoint_dir: str, epoch: int, vision_group, text_group, config: dict) -> str:
    return _save(checkpoint_dir, epoch, f"epoch_{epoch}", vision_group, text_group, config, {})


def _save(checkpoint_dir: str, tag, name: str, vision_group, text_group, config: dict, extra_meta: dict) -> str:
    """Fan ``save_checkpoint(checkpoint_dir, tag)`` out to every actor, then write ``{name}/metadata.json`` (last,
    so a directory without it is an interrupted save and is ignored by the finders)."""
    from .runtime.actor_group import get

    v_refs = vision_group.execute_all_async("save_checkpoint", checkpoint_dir, tag)
    t_refs = text_group.execute_all_async("save_checkpoint", checkpoint_dir, tag)
    v_paths, t_paths = get(v_refs), get(t_refs)
    return write_metadata(checkpoint_dir, name, v_paths, t_paths, config, dict({"epoch": tag}, **extra_meta))


def write_metadata(checkpoint_dir: str, name: str, v_paths: list, t_paths: list, config: dict,
                   extra_meta: dict) -> str:
    """``{name}/metadata.json`` for shards that are already on disk (atomic: temporary name, then rename)."""
    epoch_dir = os.path.join(checkpoint_dir, name)
    os.makedirs(epoch_dir, exist_ok=True)
    tr = config.get("training", {})
    epoch = extra_meta.get("epoch")
    meta = {
        "epoch": epoch,
        "timestamp": time.strftime("%Y-%m-%dT%H:%M:%S"),
        "vision_checkpoints": v_paths,
        "text_checkpoints": t_paths,
        "config_summary": {
            "vision_parallelism": config.get("vision", {}).get("parallelism"),
            "text_parallelism": config.get("text", {}).get("parallelism"),
            "batch_size": tr.get("batch_size"),
            "parallel_size": tr.get("parallel_size"),
            "dp_size": tr.get("dp_size", 1),
        },
    }
    meta.update(extra_meta)
    tmp = os.path.join(epoch_dir, "metadata.json.tmp")
    with open(tmp, "w") as f:
        json.dump(meta, f, indent=2)
    os.replace(tmp, os.path.join(epoch_dir, "metadata.json"))
    log.info("Saved checkpoint %s to %s", name, epoch_dir)
    return epoch_dir


# ---------------------------------------------------------------------------------------------------------------
# Step-granular checkpoints (``training.save_every_steps``): ``{checkpoint_dir}/step_{S}/`` with the layout of an
# epoch checkpoint; S is the number of optimizer steps done.  The reference only saves at epoch ends
# (python/train_ray.py:441-443); a run that dies inside a long epoch loses the whole epoch there.
# ---------------------------------------------------------------------------------------------------------------
def save_step_checkpoint(checkpoint_dir: str, global_step: int, epoch: int, iteration: int, vision_group, text_group,
                         config: dict, keep: int = 2) -> str:
    """``global_step`` optimizer steps are done; ``iteration`` is the next iteration of ``epoch`` to run."""
    name = f"step_{global_step}"
    out = _save(checkpoint_dir, name, name, vision_group, text_group, config,
                {"epoch": epoch, "next_iteration": iteration, "global_step": global_step})
    if keep > 0:
        import shutil
        steps = sorted(_step_dirs(checkpoint_dir))
        for old in steps[:-keep]:
            shutil.rmtree(os.path.join(checkpoint_dir, f"step_{old}"), ignore_errors=True)
    return out


def _step_dirs(checkpoint_dir: str) -> list[int]:
    if not os.path.isdir(checkpoint_dir):
        return []
    out = []
    for name in os.listdir(checkpoint_dir):
        m = re.fullmatch(r"step_(\d+)", name)
        if m and os.path.isfile(os.path.join(checkpoint_dir, name, "metadata.json")):
            out.append(int(m.group(1)))
    return out


def find_latest_step_checkpoint(checkpoint_dir: str) -> dict | None:
    """Metadata of the newest complete ``step_S`` checkpoint, or None."""
    steps = _step_dirs(checkpoint_dir)
    if not steps:
        return None
    with open(os.path.join(checkpoint_dir, f"step_{max(steps)}", "metadata.json")) as f:
        return json.load(f)


def load_step_checkpoint(checkpoint_dir: str, global_step: int, vision_group, text_group) -> bool:
    return load_epoch_checkpoint(checkpoint_dir, f"step_{global_step}", vision_group, text_group)


def load_epoch_checkpoint(checkpoint_dir: str, epoch: int, vision_group, text_group) -> bool:
    """True only if every actor of both groups loaded its shard."""
    from .runtime.actor_group import get

    v = get(vision_group.execute_all_async("load_checkpoint", checkpoint_dir, epoch))
    t = get(text_group.execute_all_async("load_checkpoint", checkpoint_dir, epoch))
    ok = all(v) and all(t)
    if not ok:
        log.warning("checkpoint %s could not be loaded on every actor (vision %s, text %s)", epoch, v, t)
    return ok


def plan_resume(checkpoint_dir: str, num_iterations: int) -> tuple | None:
    """What to load to continue a run: ``(tag, start_epoch, start_iteration)`` or None for a fresh start.
    A step checkpoint inside an unfinished epoch wins over the last finished epoch when it is newer."""
    latest = find_latest_checkpoint(checkpoint_dir)
    step_meta = find_latest_step_checkpoint(checkpoint_dir)
    epoch_steps = -1 if latest is None else (latest + 1) * num_iterations
    if step_meta is not None and int(step_meta["global_step"]) > epoch_steps:
        done = int(step_meta["global_step"])
        return f"step_{done}", done // num_iterations, done % num_iterations
    if latest is not None:
        return latest, latest + 1, 0
    return None
