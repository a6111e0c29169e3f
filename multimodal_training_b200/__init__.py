"""B200-native disaggregated hybrid-parallel VLM trainer: vision encoder sequence-parallel, text decoder
tensor-parallel, both on the same GPUs, hot ops as hand-written sm_100a kernels (see README.md)."""
__version__ = "0.1.0"

from .config.loader import load_config, trainer_configs  # noqa: F401
from .config.model_configs import get_model_config  # noqa: F401


def __getattr__(name):
    if name == "HybridEngine":
        from .engine import HybridEngine
        return HybridEngine
    if name == "ActorGroup":
        from .runtime.actor_group import ActorGroup
        return ActorGroup
    if name in ("VisionTrainer", "QwenVisionTrainer"):
        from .trainers.vision import VisionTrainer
        return VisionTrainer
    if name in ("TextTrainer", "QwenTextTrainer"):
        from .trainers.text import TextTrainer
        return TextTrainer
    raise AttributeError(name)
