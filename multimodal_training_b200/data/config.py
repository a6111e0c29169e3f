"""Data configuration (reference: python/data/config.py:8-29)."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class DataConfig:
    datasets: list[str] = field(default_factory=lambda: ["mscoco2017_train_captions"])
    data_registry: dict = field(default_factory=dict)   # name -> {"annotation_path", "data_path"}
    model_max_length: int = 8192
    padding_side: str = "right"
    use_fast_tokenizer: bool = False
    max_pixels: int = 50176
    min_pixels: int = 784
    force_fixed_size: bool = False
    num_workers: int = 4
    pin_memory: bool = True
    data_flatten: bool = True

    @classmethod
    def from_flat(cls, cfg: dict) -> "DataConfig":
        names = {f for f in cls.__dataclass_fields__}
        return cls(**{k: v for k, v in cfg.items() if k in names and v is not None})


DEFAULT_DATA_REGISTRY = {
    "mscoco2017_train_captions": {"annotation_path": "__PATH_TO_MSCOCO2017__/annotations/coco2017_train_qwen.json",
                                  "data_path": "__PATH_TO_MSCOCO2017__"},
    "mscoco2017_val_captions": {"annotation_path": "__PATH_TO_MSCOCO2017__/annotations/coco2017_val_qwen.json",
                                "data_path": "__PATH_TO_MSCOCO2017__"},
}
