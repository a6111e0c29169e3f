"""Merge per-rank vision and text training checkpoints into one Hugging Face style checkpoint.

    python -m multimodal_training_b200.cli.merge_checkpoint --checkpoint-dir ckpt/epoch_5 \
        --output-dir merged/epoch_5 --model-name Qwen/Qwen2.5-VL-7B-Instruct --parallel-size 4

Reads ``{vision,text}/rank_*.pt`` (``{"model": state_dict}`` each), merges the tensor-parallel
shards by key (embed_tokens / lm_head and q/k/v/gate/up along dim 0, o_proj / proj / down_proj along
dim 1, bit-equal tensors taken from rank 0), re-fuses the vision ``attn.{q,k,v}`` into HF's
``attn.qkv`` and writes ``pytorch_model.bin`` (keys ``visual.*`` / ``language_model.*`` /
``lm_head.*``), ``config.json`` and ``merge_metadata.json``.  Same command line and output layout as
the reference tool (scripts/merge_checkpoint.py:31-279), which leaves q/k/v split.
"""
from __future__ import annotations

import argparse
import json
import logging
import os
import re

import torch

from ..config.model_configs import get_model_config

log = logging.getLogger("mmt_b200.merge")

DIM0_PATTERNS = ("embed_tokens", "lm_head", "q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", ".q.", ".k.", ".v.",
                 "qkv", "mlp.0", "fc1")
DIM1_PATTERNS = ("o_proj", "down_proj", "attn.proj", "mlp.2", "fc2")
ALWAYS_DIM0 = ("embed_tokens", "lm_head", "q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", ".q.", ".k.", ".v.",
               "attn.qkv")
ALWAYS_DIM1 = ("o_proj", "down_proj", "attn.proj")


def merge_tensor(key: str, shards: list[torch.Tensor]) -> torch.Tensor:
    """One tensor from its per-rank shards."""
    first = shards[0]
    if len(shards) == 1:
        return first
    # layers that are always split by a tensor-parallel run are concatenated even when their shards happen to be
    # bit-equal (biases that are still zero)
    if any(p in key for p in ALWAYS_DIM0):
        return torch.cat(shards, dim=0)
    if any(p in key for p in ALWAYS_DIM1) and not key.endswith(".bias"):
        return torch.cat(shards, dim=1)
    if all(s.shape == first.shape and torch.equal(s, first) for s in shards[1:]):
        return first                                        # replicated
    if first.dim() == 1:
        if any(p in key for p in DIM0_PATTERNS):
            return torch.cat(shards, dim=0)                 # bias of a column-parallel layer
        return torch.stack([s.float() for s in shards]).mean(0).to(first.dtype)
    if any(p in key for p in DIM1_PATTERNS) and not key.endswith(".bias"):
        return torch.cat(shards, dim=1)
    if any(p in key for p in DIM0_PATTERNS):
        return torch.cat(shards, dim=0)
    if all(s.shape == first.shape for s in shards):
        log.warning("%s: shards differ but no rule matches; averaging", key)
        return torch.stack([s.float() for s in shards]).mean(0).to(first.dtype)
    return torch.cat(shards, dim=0)


def merge_state_dicts(rank_state_dicts: list[dict]) -> dict:
    keys = list(rank_state_dicts[0].keys())
    out = {}

    def local(t):
        return t.to_local() if hasattr(t, "to_local") else t

    # data-parallel replicas (no tensor parallelism in that half): every file holds the same full tensors
    first = rank_state_dicts[0]
    if all(all(local(sd[k]).shape == local(first[k]).shape and torch.equal(local(sd[k]), local(first[k]))
               for k in keys) for sd in rank_state_dicts[1:]):
        return {k: local(first[k]) for k in keys}
    for k in keys:
        shards = []
        for sd in rank_state_dicts:
            t = sd[k]
            if hasattr(t, "to_local"):       # DTensor values in checkpoints written by the reference
                t = t.to_local()
            shards.append(t)
        out[k] = merge_tensor(k, shards)
    return out


def load_and_merge_sharded_weights(checkpoint_dir: str, num_ranks: int, component: str, replicated: bool = False):
    sds = []
    for r in range(num_ranks):
        path = os.path.join(checkpoint_dir, f"rank_{r}.pt")
        if not os.path.exists(path):
            raise FileNotFoundError(f"Checkpoint not found: {path}")
        sds.append(torch.load(path, map_location="cpu", weights_only=False)["model"])
        if replicated:
            break
    log.info("loaded %d %s shard(s)", len(sds), component)
    return sds[0] if len(sds) == 1 else merge_state_dicts(sds)


def refuse_vision_qkv(sd: dict) -> dict:
    """``blocks.N.attn.{q,k,v}_proj.{weight,bias}`` (the reference's names, modeling_qwen2_5_vl.py:334-338; the
    shorter ``attn.{q,k,v}`` of earlier checkpoints of this package is accepted too) ->
    ``blocks.N.attn.qkv.{weight,bias}`` (HF layout)."""
    out = {}
    groups: dict[tuple[str, str], dict[str, torch.Tensor]] = {}
    for k, v in sd.items():
        m = re.fullmatch(r"(.*\.attn)\.([qkv])(?:_proj)?\.(weight|bias)", k)
        if m:
            groups.setdefault((m.group(1), m.group(3)), {})[m.group(2)] = v
        else:
            out[k] = v
    for (prefix, kind), parts in groups.items():
        out[f"{prefix}.qkv.{kind}"] = torch.cat([parts["q"], parts["k"], parts["v"]], dim=0)
    return out


def merge_checkpoint(checkpoint_dir: str, output_dir: str, model_name: str, parallel_size: int,
                     text_parallel_size: int | None = None, keep_split_qkv: bool = False,
                     vision_tensor_parallel: bool = False) -> str:
    # sequence-parallel vision ranks hold identical weights (rank 0 is read); tensor-parallel ones hold shards
    vision = load_and_merge_sharded_weights(os.path.join(checkpoint_dir, "vision"), parallel_size, "vision",
                                            replicated=not vision_tensor_parallel)
    text = load_and_merge_sharded_weights(os.path.join(checkpoint_dir, "text"), text_parallel_size or parallel_size,
                                          "text")
    if not keep_split_qkv:
        vision = refuse_vision_qkv(vision)
    merged = {}
    for k, v in vision.items():
        merged["visual." + k] = v
    for k, v in text.items():
        merged[k if k.startswith("lm_head.") else "language_model." + k] = v
    os.makedirs(output_dir, exist_ok=True)
    torch.save(merged, os.path.join(output_dir, "pytorch_model.bin"))
    try:
        cfg = get_model_config(model_name).to_dict()
    except KeyError:
        cfg = {"name": model_name}
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    meta = {"source": checkpoint_dir, "parallel_size": parallel_size, "num_tensors": len(merged),
            "vision_qkv": "split" if keep_split_qkv else "fused", "model_name": model_name}
    with open(os.path.join(output_dir, "merge_metadata.json"), "w") as f:
        json.dump(meta, f, indent=2)
    return output_dir


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--checkpoint-dir", required=True)
    ap.add_argument("--output-dir", required=True)
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--parallel-size", type=int, default=1)
    ap.add_argument("--text-parallel-size", type=int, default=None)
    ap.add_argument("--keep-split-qkv", action="store_true")
    ap.add_argument("--vision-tensor-parallel", action="store_true",
                    help="the run used vision.parallelism=tensor: merge the vision shards of --parallel-size ranks")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    merge_checkpoint(a.checkpoint_dir, a.output_dir, a.model_name, a.parallel_size, a.text_parallel_size,
                     a.keep_split_qkv, a.vision_tensor_parallel)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
