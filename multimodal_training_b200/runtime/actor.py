"""Actor base class and the torchrun-style rendezvous record.

Counterpart of the reference's python/ray/actor.py:11-62.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

from . import utils
from .logger import setup_logging


@dataclass
class TorchDistributedConfig:
    rank: int
    local_rank: int
    world_size: int
    local_world_size: int
    master_addr: str
    master_port: int
    backend: str = "nccl"


class RayActor:
    """Base of everything an :class:`ActorGroup` can host."""

    def __init__(self, *args, **kwargs):
        setup_logging()

    def setup_env_variables(self, cfg: TorchDistributedConfig) -> bool:
        """Mimic torchrun so that ``init_process_group`` can use the env:// rendezvous."""
        os.environ["LOCAL_RANK"] = str(cfg.local_rank)
        os.environ["WORLD_SIZE"] = str(cfg.world_size)
        os.environ["RANK"] = str(cfg.rank)
        os.environ["LOCAL_WORLD_SIZE"] = str(cfg.local_world_size)
        os.environ["MASTER_ADDR"] = cfg.master_addr
        os.environ["MASTER_PORT"] = str(cfg.master_port)
        os.environ["MMT_DIST_BACKEND"] = cfg.backend
        return True

    def get_node_ip_addr(self) -> str:
        return utils.get_node_ip_addr()

    def get_free_port(self) -> int:
        return utils.get_free_port()

    def get_rank(self) -> int:
        return getattr(self, "rank", 0)

    def get_physical_gpu_id(self) -> str:
        return utils.get_physical_gpu_id()
