from .collator import (DataCollatorForSupervisedDataset, FlattenedDataCollatorForSupervisedDataset,  # noqa: F401
                       VisionDataCollator)
from .config import DEFAULT_DATA_REGISTRY, DataConfig  # noqa: F401
from .preprocessing import IGNORE_INDEX, IMAGE_TOKEN_INDEX, preprocess_qwen_visual  # noqa: F401
from .rope_utils import get_rope_index_for_images  # noqa: F401

__all__ = ["LazySupervisedDataset", "build_dataloader", "DataCollatorForSupervisedDataset",
           "FlattenedDataCollatorForSupervisedDataset", "VisionDataCollator", "preprocess_qwen_visual",
           "get_rope_index_for_images", "DEFAULT_DATA_REGISTRY", "parse_sampling_rate", "get_dataset_configs",
           "DataConfig"]


def __getattr__(name):
    if name in ("LazySupervisedDataset", "build_dataloader", "parse_sampling_rate", "get_dataset_configs",
                "DatasetSource"):
        from . import dataset
        return getattr(dataset, name)
    raise AttributeError(name)
