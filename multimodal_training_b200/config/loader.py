"""YAML training config: loader, Hydra-style command line, schema and validation.

Keeps the reference's schema (configs/sample.yaml:1-73) and command line
(``--config-path=... --config-name=... key=value``, python/train_ray.py:141 and
README.md:319-323) without Hydra/OmegaConf, which a no-network image lacks.
The sections are flattened per trainer the same way the reference does
(``vision|text`` + ``training`` + ``data`` + ``deepspeed``, python/train_ray.py:152-164).
"""
from __future__ import annotations

import argparse
import copy
from pathlib import Path
from typing import Any

import yaml

VISION_PARALLELISM = ("none", "tensor", "sequence", "deepspeed")
TEXT_PARALLELISM = ("none", "tensor", "deepspeed", "autotp")
DTYPES = ("float16", "bfloat16", "float32")
ATTN_BACKENDS = ("sdpa", "flash_attention_2", "eager", "sm100")

DEFAULTS: dict[str, Any] = {
    "debug": False,
    "vision": {
        "model_type": "qwen2_5_vl",
        "model_name": "Qwen/Qwen2.5-VL-7B-Instruct",
        "parallelism": "sequence",
        "dtype": "bfloat16",
        "attention_backend": "flash_attention_2",
        "activation_checkpointing": True,
        "autocast": True,
        "zero_stage": 1,
        "pretrained_checkpoint_dir": None,
    },
    "text": {
        "model_type": "qwen2_5_vl",
        "model_name": "Qwen/Qwen2.5-VL-7B-Instruct",
        "parallelism": "tensor",
        "dtype": "bfloat16",
        "attention_backend": "flash_attention_2",
        "activation_checkpointing": True,
        "autocast": True,
        "zero_stage": 1,
        "autotp_size": None,
        "tensor_parallel_size": None,
        "tp_overlap_comm": False,
        "use_vocab_parallel": True,
        "pretrained_checkpoint_dir": None,
    },
    "training": {
        "batch_size": 4,
        "learning_rate": 5e-5,
        "num_epochs": 1,
        "num_iterations": 20,
        "warmup_steps": 10,
        "warmup_ratio": 0.03,
        "lr_scheduler_type": "cosine",
        "weight_decay": 0.01,
        "gradient_accumulation_steps": 1,
        "seed": 42,
        "parallel_size": 1,
        "dp_size": 1,
        "collocate": True,
        "clip_grad_norm": False,
        "max_grad_norm": 1.0,
        "no_checkpoint": True,
        "save_every_steps": 0,          # also save step_{S}/ every this many optimizer steps (0 = epoch ends only)
        "keep_step_checkpoints": 2,
        "max_steps": 0,                 # stop after this many optimizer steps (0 = all epochs)
        "checkpoint_dir": "/tmp/checkpoints",
        "log_interval": 1,
        "profile_time": False,
        "trace": False,            # NVTX ranges + device-timed phases (utils/tracing.py)
        "dist_timeout_s": None,    # torch.distributed timeout of the torchrun-style driver (None = library default)
        "trace_file": None,        # with trace: prefix of the per-rank chrome://tracing files (train_spmd)
        "backend": None,           # torch.distributed backend: default nccl on GPU, gloo on CPU
        "runtime": "auto",         # actor runtime: auto | ray | builtin
        "label_smoothing": 0.0,    # cross-entropy label smoothing (python/tensor_parallel/cross_entropy.py:185-202)
        "fused_comm": "auto",      # peer-memory fused collectives: true | false | auto (on when every GPU can map
                                   # every other one; heap regions grow with the longest batch seen)
        # true: AdamW on fp32 master weights with fp32 moments; false: AdamW directly on the bf16 parameters with bf16
        # moments, as torch.optim.AdamW on a bf16 model (the reference's optimizer): half the optimizer's memory
        # traffic, a third of its memory, every update rounded to bf16
        "optimizer_master_weights": True,
        "overlap_optimizer": False,  # single-GPU engine: text AdamW on a side stream behind the next vision forward
        "symm_heap_mb": 8192,      # size of each GPU's symmetric heap (exchange buffers of the fused collectives)
    },
    "data": {
        "datasets": [],
        "data_registry": {},
        "num_workers": 4,
        "pin_memory": True,
        "data_flatten": True,
        "min_pixels": 802816,
        "max_pixels": 802816,
        "force_fixed_size": False,
        "model_max_length": 8192,
        "synthetic": None,         # {"image_size": 896, "text_tokens": 1024} -> no files needed
    },
    "deepspeed": {"reduce_bucket_size": 500000000},
}


class ConfigError(ValueError):
    pass


def _deep_update(base: dict, upd: dict) -> dict:
    for k, v in upd.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _deep_update(base[k], v)
        else:
            base[k] = v
    return base


def _parse_scalar(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def apply_overrides(cfg: dict, overrides: list[str]) -> dict:
    """Apply dotted ``a.b.c=value`` overrides (``+a.b=value`` adds a new key, ``~a.b`` deletes)."""
    for ov in overrides:
        if ov.startswith("~"):
            parts = ov[1:].split(".")
            node = cfg
            for p in parts[:-1]:
                node = node.get(p, {})
            node.pop(parts[-1], None)
            continue
        if "=" not in ov:
            raise ConfigError(f"override '{ov}' is not of the form key=value")
        key, val = ov.split("=", 1)
        add = key.startswith("+")
        key = key.lstrip("+")
        parts = key.split(".")
        node = cfg
        for p in parts[:-1]:
            if p not in node or not isinstance(node[p], dict):
                if not add and p not in node:
                    raise ConfigError(f"override '{ov}': unknown section '{p}' (prefix with + to add)")
                node[p] = {} if not isinstance(node.get(p), dict) else node[p]
            node = node[p]
        node[parts[-1]] = _parse_scalar(val)
    return cfg


def validate(cfg: dict) -> dict:
    """Check enumerations, types and cross-field constraints; returns cfg."""
    for sec in ("vision", "text", "training", "data"):
        if sec not in cfg or not isinstance(cfg[sec], dict):
            raise ConfigError(f"missing section '{sec}'")
    v, t, tr = cfg["vision"], cfg["text"], cfg["training"]
    if v["model_type"] != "qwen2_5_vl" or t["model_type"] != "qwen2_5_vl":
        raise ConfigError("only model_type 'qwen2_5_vl' is supported")
    if v["parallelism"] not in VISION_PARALLELISM:
        raise ConfigError(f"vision.parallelism must be one of {VISION_PARALLELISM}")
    if t["parallelism"] not in TEXT_PARALLELISM:
        raise ConfigError(f"text.parallelism must be one of {TEXT_PARALLELISM}")
    for sec in (v, t):
        if sec["dtype"] not in DTYPES:
            raise ConfigError(f"dtype must be one of {DTYPES}")
        if sec["attention_backend"] not in ATTN_BACKENDS:
            raise ConfigError(f"attention_backend must be one of {ATTN_BACKENDS}")
        if sec.get("zero_stage") not in (0, 1, 2, 3, None):
            raise ConfigError("zero_stage must be 0..3")
        # zero_stage matters only with parallelism: deepspeed (as in the reference, python/ray/text.py:99-106).
        # Stages 0-2 run as the flat-buffer ZeRO optimizer of parallel/zero.py: gradients are reduce-scattered, so
        # each rank reduces and keeps only its own partition (what stage 2 adds to stage 1), and optimizer states
        # are always sharded.  Stage 3 (parameters partitioned, gathered layer by layer) is not implemented:
        # sequence / tensor parallelism is how this framework splits a model that does not fit one GPU.
        if sec["parallelism"] == "deepspeed" and sec.get("zero_stage") == 3:
            raise ConfigError("parallelism: deepspeed with zero_stage: 3 (parameter partitioning) is not supported; "
                              "use zero_stage 1 or 2, or parallelism: tensor / sequence to shard the model")
    for k in ("batch_size", "num_epochs", "num_iterations", "parallel_size", "dp_size",
              "gradient_accumulation_steps"):
        if not isinstance(tr[k], int) or tr[k] < 1:
            raise ConfigError(f"training.{k} must be a positive integer")
    if float(tr["learning_rate"]) <= 0:
        raise ConfigError("training.learning_rate must be positive")
    return cfg


def load_config(path: str | Path | None = None, overrides: list[str] | None = None) -> dict:
    cfg = copy.deepcopy(DEFAULTS)
    if path is not None:
        with open(path) as f:
            _deep_update(cfg, yaml.safe_load(f) or {})
    if overrides:
        apply_overrides(cfg, overrides)
    cfg["training"]["learning_rate"] = float(cfg["training"]["learning_rate"])
    return validate(cfg)


def trainer_configs(cfg: dict) -> tuple[dict, dict]:
    """Flatten the sections into one dict per trainer (vision, text)."""
    tr = cfg["training"]
    shared = {**tr, **cfg["data"], **cfg.get("deepspeed", {})}
    vision = {**cfg["vision"], **shared}
    text = {**cfg["text"], **shared}
    ps, dp = tr["parallel_size"], tr.get("dp_size", 1)
    vision["sequence_parallel_size"] = ps
    vision["dp_size"] = dp
    text["autotp_size"] = cfg["text"].get("autotp_size") or ps
    text["tensor_parallel_size"] = cfg["text"].get("tensor_parallel_size") or ps
    text["dp_size"] = dp
    # mesh factors: sequence/tensor parallel degrees inside the world of ps*dp ranks
    sp = ps if cfg["vision"]["parallelism"] in ("sequence", "tensor") else 1
    if cfg["text"]["parallelism"] == "autotp":
        tp = text["autotp_size"]
    elif cfg["text"]["parallelism"] == "tensor":
        tp = text["tensor_parallel_size"]
    else:
        tp = 1
    for d in (vision, text):
        d["mesh_sp"], d["mesh_tp"] = int(sp), int(tp)
        d["world_size"] = int(ps * dp)
        d["vision_parallelism"] = cfg["vision"]["parallelism"]
        d["text_parallelism"] = cfg["text"]["parallelism"]
        d["vision_model_name"] = cfg["vision"]["model_name"]
        d["text_model_name"] = cfg["text"]["model_name"]
    return vision, text


def parse_cli(argv: list[str] | None = None) -> tuple[dict, argparse.Namespace]:
    """``--config-path DIR --config-name NAME key=value ...`` -> validated config."""
    ap = argparse.ArgumentParser(add_help=True)
    ap.add_argument("--config-path", default=str(Path(__file__).resolve().parents[2] / "configs"))
    ap.add_argument("--config-name", default="sample")
    ap.add_argument("overrides", nargs="*")
    ns = ap.parse_args(argv)
    name = ns.config_name if ns.config_name.endswith((".yaml", ".yml")) else ns.config_name + ".yaml"
    path = Path(ns.config_path) / name
    if not path.exists():
        raise ConfigError(f"config file {path} not found")
    return load_config(path, ns.overrides), ns
