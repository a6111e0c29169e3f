"""Runtime helpers: GPU identity, environment forwarding, runtime selection.

Counterpart of the reference's python/ray/utils.py:9-86.
"""
from __future__ import annotations

import os
import socket


def get_physical_gpu_id(device_index: int | None = None) -> str:
    """UUID of the CUDA device this process uses, or ``"cpu"``."""
    try:
        import torch
        if not torch.cuda.is_available():
            return "cpu"
        idx = torch.cuda.current_device() if device_index is None else device_index
        return str(torch.cuda.get_device_properties(idx).uuid)
    except Exception:
        return "cpu"


def prepare_runtime_environment() -> dict:
    """Environment variables that every actor process must inherit."""
    env = {}
    for k in ("WANDB_API_KEY", "RAY_TRAIN_LOG_FILE", "MMT_TRAIN_LOG_FILE", "NCCL_DEBUG", "NCCL_NVLS_ENABLE",
              "CUDA_VISIBLE_DEVICES"):
        if k in os.environ:
            env[k] = os.environ[k]
    return env


def ray_available() -> bool:
    try:
        import ray  # noqa: F401
        return True
    except Exception:
        return False


def select_runtime(requested: str = "auto") -> str:
    if requested == "ray":
        if not ray_available():
            raise RuntimeError("runtime 'ray' requested but ray is not installed")
        return "ray"
    if requested == "builtin":
        return "builtin"
    return "ray" if ray_available() else "builtin"


def initialize_ray() -> None:
    """``ray.init`` with the forwarded environment (python/ray/utils.py:42-45); no-op without ray."""
    if ray_available():
        import ray
        if not ray.is_initialized():
            ray.init(runtime_env={"env_vars": prepare_runtime_environment()})


def get_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def get_node_ip_addr() -> str:
    return os.environ.get("MMT_NODE_IP", "127.0.0.1")
