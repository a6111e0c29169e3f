"""Batch collators (reference: python/data/collator.py:11-156).

* :class:`DataCollatorForSupervisedDataset` pads a batch to [B, S_max].
* :class:`FlattenedDataCollatorForSupervisedDataset` packs the batch into ONE sequence: ``input_ids`` and
  ``labels`` concatenated along the token axis, ``position_ids`` along their last axis, and
  ``attention_mask`` = cumulative sequence lengths (int32) for varlen attention.
* :class:`VisionDataCollator` concatenates ``pixel_values`` and ``image_grid_thw``.
Video clips ride along the same way (``pixel_values_videos`` / ``video_grid_thw``, python/data/collator.py:51-71).
All carry ``sample_index`` so that the vision and text halves can check that they see the same samples.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .preprocessing import IGNORE_INDEX


def pad_and_cat(position_ids: list[torch.Tensor]) -> torch.Tensor:
    """[3, 1, S_i] tensors -> [3, B, S_max], padded with 1 (any valid position id)."""
    s_max = max(p.shape[2] for p in position_ids)
    out = [torch.nn.functional.pad(p, (0, s_max - p.shape[2]), value=1) for p in position_ids]
    return torch.cat(out, dim=1)


def _images(instances):
    px = [i["pixel_values"] for i in instances if i.get("pixel_values") is not None]
    grids = [i["image_grid_thw"] for i in instances if i.get("image_grid_thw") is not None]
    return (torch.cat(px, 0) if px else None), (torch.cat(grids, 0) if grids else None)


def _videos(instances):
    px = [i["pixel_values_videos"] for i in instances if i.get("pixel_values_videos") is not None]
    grids = [i["video_grid_thw"] for i in instances if i.get("video_grid_thw") is not None]
    return (torch.cat(px, 0) if px else None), (torch.cat(grids, 0) if grids else None)


def _sample_index(instances):
    return torch.cat([torch.as_tensor(i["sample_index"]).reshape(-1) for i in instances], dim=0)


@dataclass
class DataCollatorForSupervisedDataset:
    pad_token_id: int = 0
    model_max_length: int = 8192

    def __call__(self, instances):
        ids = [i["input_ids"].reshape(-1) for i in instances]
        labels = [i["labels"].reshape(-1) for i in instances]
        L = self.model_max_length
        input_ids = torch.nn.utils.rnn.pad_sequence(ids, batch_first=True, padding_value=self.pad_token_id)[:, :L]
        lab = torch.nn.utils.rnn.pad_sequence(labels, batch_first=True, padding_value=IGNORE_INDEX)[:, :L]
        pos = pad_and_cat([i["position_ids"] for i in instances])[:, :, :L]
        lens = torch.tensor([min(len(x), L) for x in ids])
        mask = torch.arange(input_ids.shape[1])[None, :] < lens[:, None]
        px, grid = _images(instances)
        vx, vgrid = _videos(instances)
        return {"input_ids": input_ids, "labels": lab, "attention_mask": mask, "position_ids": pos,
                "pixel_values": px, "image_grid_thw": grid, "pixel_values_videos": vx, "video_grid_thw": vgrid,
                "sample_index": _sample_index(instances)}


@dataclass
class FlattenedDataCollatorForSupervisedDataset(DataCollatorForSupervisedDataset):
    def __call__(self, instances):
        ids = [i["input_ids"].reshape(1, -1) for i in instances]
        labels = [i["labels"].reshape(1, -1) for i in instances]
        lens = [0] + [x.shape[1] for x in ids]
        cu = torch.tensor(lens, dtype=torch.int32).cumsum(0).to(torch.int32)
        px, grid = _images(instances)
        vx, vgrid = _videos(instances)
        return {"input_ids": torch.cat(ids, 1), "labels": torch.cat(labels, 1),
                "position_ids": torch.cat([i["position_ids"] for i in instances], dim=2), "attention_mask": cu,
                "pixel_values": px, "image_grid_thw": grid, "pixel_values_videos": vx, "video_grid_thw": vgrid,
                "sample_index": _sample_index(instances)}


@dataclass
class VisionDataCollator:
    def __call__(self, instances):
        px, grid = _images(instances)
        vx, vgrid = _videos(instances)
        return {"pixel_values": px, "image_grid_thw": grid, "pixel_values_videos": vx, "video_grid_thw": vgrid,
                "sample_index": _sample_index(instances)}
