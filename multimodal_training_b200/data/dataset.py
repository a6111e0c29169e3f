"""Lazy supervised dataset over LLaVA-style annotation files, plus the dataloader builder and the
batch source used by the trainers (reference: python/data/dataset.py:35-397).

* ``name%NN`` keeps NN percent of a dataset (``parse_sampling_rate``).
* A seeded shuffle fixes the sample order; all ranks build the same order so that the vision and
  the text half (and all tensor / sequence parallel ranks) agree on the global batch, while
  data-parallel replicas take DIFFERENT slices of it (``trainers/context.py``).
* ``modality`` in {"all", "image", "text"}: "image" drops the text keys, "text" drops the pixels.
* A sample that fails to load is retried 3 times, then its neighbours are tried (3 times each)
  before the error is raised.
"""
from __future__ import annotations

import json
import logging
import random
import re

import torch
from torch.utils.data import DataLoader, Dataset

from .collator import (DataCollatorForSupervisedDataset, FlattenedDataCollatorForSupervisedDataset,
                       VisionDataCollator)
from .config import DEFAULT_DATA_REGISTRY, DataConfig
from .preprocessing import preprocess_qwen_visual
from .rope_utils import get_rope_index_for_images
from .synthetic import Sample

log = logging.getLogger("mmt_b200")


def parse_sampling_rate(name: str) -> tuple[str, float]:
    m = re.fullmatch(r"(.+)%(\d+)", name)
    if m:
        return m.group(1), int(m.group(2)) / 100.0
    return name, 1.0


def get_dataset_configs(names: list[str], registry: dict | None = None) -> list[dict]:
    reg = dict(DEFAULT_DATA_REGISTRY)
    reg.update(registry or {})
    out = []
    for n in names:
        base, rate = parse_sampling_rate(n)
        if base not in reg:
            raise KeyError(f"dataset '{base}' is not in the data registry")
        out.append({**reg[base], "name": base, "sampling_rate": rate})
    return out


def read_jsonl(path: str) -> list[dict]:
    with open(path) as f:
        return [json.loads(line) for line in f if line.strip()]


def read_annotations(path: str) -> list[dict]:
    if path.endswith(".jsonl"):
        return read_jsonl(path)
    with open(path) as f:
        return json.load(f)


class LazySupervisedDataset(Dataset):
    def __init__(self, processor, data_config: DataConfig, modality: str = "all", seed: int = 42,
                 spatial_merge_size: int = 2, image_token_id: int = 151655, vision_start_token_id: int = 151652):
        if modality not in ("all", "image", "text"):
            raise ValueError(f"modality must be all|image|text, got {modality}")
        self.processor, self.cfg, self.modality = processor, data_config, modality
        self.merge, self.image_token_id, self.vision_start_token_id = spatial_merge_size, image_token_id, \
            vision_start_token_id
        rng = random.Random(seed)
        samples = []
        for ds in get_dataset_configs(data_config.datasets, data_config.data_registry):
            ann = read_annotations(ds["annotation_path"])
            if ds["sampling_rate"] < 1.0:
                ann = rng.sample(ann, int(len(ann) * ds["sampling_rate"]))
            for a in ann:
                a = dict(a)
                a["data_path"] = ds["data_path"]
                samples.append(a)
        rng.shuffle(samples)
        self.samples = samples

    def __len__(self) -> int:
        return len(self.samples)

    def __getitem__(self, i: int) -> dict:
        last = None
        for cand in (i, i + 1, i - 1):
            cand %= len(self.samples)
            for _ in range(3):
                try:
                    return self._get_item(cand)
                except Exception as e:  # unreadable image, broken annotation, ...
                    last = e
                    log.warning("sample %d failed to load: %s", cand, e)
        raise RuntimeError(f"sample {i} and its neighbours could not be loaded") from last

    def _get_item(self, i: int) -> dict:
        s = self.samples[i]
        item = preprocess_qwen_visual([s], self.processor, data_path=s.get("data_path", ""),
                                      max_pixels=self.cfg.max_pixels, min_pixels=self.cfg.min_pixels,
                                      force_fixed_size=self.cfg.force_fixed_size)
        ids = item["input_ids"]
        grid = item.get("image_grid_thw")
        pos, _ = get_rope_index_for_images(self.merge, ids, grid.tolist() if grid is not None else [],
                                           image_token_id=self.image_token_id,
                                           vision_start_token_id=self.vision_start_token_id)
        item["position_ids"] = pos
        item["attention_mask"] = [ids.shape[1]]
        item["sample_index"] = torch.tensor([i])
        if self.modality == "image":
            for k in ("input_ids", "labels", "position_ids", "attention_mask"):
                item.pop(k, None)
        elif self.modality == "text":
            item.pop("pixel_values", None)
        return item


def default_processor(model_name, model_cfg=None):
    """The model's own HF processor when its files are on this machine, else the in-tree image processor and
    chat template (``data/processor.py``) around the HF tokenizer if that is available, else around the byte
    tokenizer (synthetic and test runs)."""
    import logging
    from .processor import ByteTokenizer, Qwen2_5_VLImageProcessor, Qwen2_5_VLProcessor
    try:
        from transformers import AutoProcessor
        return AutoProcessor.from_pretrained(model_name, local_files_only=True)
    except Exception as e:  # no files / no network: say so once and continue with the in-tree one
        logging.getLogger("mmt_b200").warning("HF processor for %s unavailable (%s): using the in-tree processor",
                                              model_name, type(e).__name__)
    tok = None
    try:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(model_name, local_files_only=True)
    except Exception:
        tok = ByteTokenizer.for_config(model_cfg)
    v = getattr(model_cfg, "vision", None)
    ip = Qwen2_5_VLImageProcessor(patch_size=getattr(v, "patch_size", 14),
                                  temporal_patch_size=getattr(v, "temporal_patch_size", 2),
                                  merge_size=getattr(v, "spatial_merge_size", 2))
    return Qwen2_5_VLProcessor(ip, tok)


def build_dataloader(processor, data_config: DataConfig, batch_size: int, rank: int = 0, world_size: int = 1,
                     generator=None, worker_init_fn=None, drop_last: bool = True, modality: str = "all",
                     seed: int = 42, **dataset_kw) -> DataLoader:
    ds = LazySupervisedDataset(processor, data_config, modality=modality, seed=seed, **dataset_kw)
    if modality == "image":
        collate = VisionDataCollator()
    else:
        pad = getattr(getattr(processor, "tokenizer", None), "pad_token_id", 0) or 0
        cls = FlattenedDataCollatorForSupervisedDataset if data_config.data_flatten else \
            DataCollatorForSupervisedDataset
        collate = cls(pad_token_id=pad, model_max_length=data_config.model_max_length)
    sampler = None
    if world_size > 1:
        sampler = torch.utils.data.distributed.DistributedSampler(ds, num_replicas=world_size, rank=rank,
                                                                 shuffle=False, drop_last=drop_last)
    return DataLoader(ds, batch_size=batch_size, shuffle=False, sampler=sampler, collate_fn=collate,
                      num_workers=data_config.num_workers, pin_memory=data_config.pin_memory and
                      torch.cuda.is_available(), drop_last=drop_last, generator=generator,
                      worker_init_fn=worker_init_fn)


class DatasetSource:
    """Global batches from annotation files for the trainers: step -> list of :class:`Sample` (all replicas).

    The batch of a step is a pure function of the step index, so the batches of the next steps are prepared ahead
    on ``data.num_workers`` threads (image decoding, resizing and patch extraction release the GIL for most of
    their time) while the GPU runs the current step; ``num_workers: 0`` prepares every batch when it is asked for.
    The reference gets the same overlap from ``DataLoader`` worker processes (python/ray/trainer.py:92-104).
    """

    PREFETCH_STEPS = 2

    def __init__(self, config: dict, model_cfg, mesh, processor=None):
        self.cfg = DataConfig.from_flat(config)
        if processor is None:
            processor = default_processor(config.get("model_name"), model_cfg)
        self.dataset = LazySupervisedDataset(processor, self.cfg, modality="all", seed=int(config.get("seed", 42)),
                                             spatial_merge_size=model_cfg.vision.spatial_merge_size,
                                             image_token_id=model_cfg.image_token_id,
                                             vision_start_token_id=model_cfg.vision_start_token_id)
        self.global_batch = int(config["batch_size"]) * max(mesh.tdp, 1)
        self.dtype = torch.bfloat16 if torch.cuda.is_available() else torch.float32
        self._pool = None
        self._futures: dict[tuple[int, int], object] = {}
        workers = int(self.cfg.num_workers or 0)
        if workers > 0:
            from concurrent.futures import ThreadPoolExecutor
            self._pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="mmt-data")

    def _sample(self, step: int, j: int) -> Sample:
        idx = (step * self.global_batch + j) % len(self.dataset)
        it = self.dataset[idx]
        px = it.get("pixel_values")
        grid = it.get("image_grid_thw")
        return Sample(it["input_ids"].reshape(-1), it["labels"].reshape(-1),
                      None if px is None else px.to(self.dtype),
                      [] if grid is None else [tuple(int(x) for x in g) for g in grid.tolist()], idx)

    def global_batch_at(self, step: int) -> list[Sample]:
        if self._pool is None:
            return [self._sample(step, j) for j in range(self.global_batch)]
        for s in range(step, step + 1 + self.PREFETCH_STEPS):
            for j in range(self.global_batch):
                if (s, j) not in self._futures:
                    self._futures[(s, j)] = self._pool.submit(self._sample, s, j)
        out = [self._futures.pop((step, j)).result() for j in range(self.global_batch)]
        for key in [k for k in self._futures if k[0] < step]:          # steps that were skipped (resume, evaluation)
            self._futures.pop(key).cancel()
        return out
