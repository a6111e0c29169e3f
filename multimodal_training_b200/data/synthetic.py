"""Synthetic multimodal batches: N(0,1) pixels, uniform-random token ids, image placeholders.

Shapes follow the benchmark configurations: one square image per sample (patches in the
processor's merge-block order, [n_patches, 3*2*14*14]) spliced into the middle of a run of random
text ids; labels are the ids with image positions set to -100.  Samples are generated on the host
(optionally in pinned memory) from ``seed + global sample index`` so every rank can materialise
any sample of the global batch without communication.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.model_configs import VLConfig

IGNORE_INDEX = -100


@dataclass
class Sample:
    input_ids: torch.Tensor          # [S] long
    labels: torch.Tensor             # [S] long, -100 at image positions
    pixel_values: torch.Tensor | None  # [n_patches, patch_dim]
    grid_thw: list[tuple[int, int, int]]
    sample_index: int


def synthetic_sample(cfg: VLConfig, index: int, *, image_size: int, text_tokens: int, seed: int = 0,
                     dtype=torch.float32, with_pixels: bool = True, pin: bool = False) -> Sample:
    v = cfg.vision
    g = torch.Generator().manual_seed(seed * 7919 + index)
    side = image_size // v.patch_size
    side -= side % v.spatial_merge_size
    n_patches = side * side
    n_merged = n_patches // v.merge_unit
    hi = min(cfg.image_token_id, cfg.text.vocab_size)
    special = {cfg.image_token_id, cfg.video_token_id, cfg.vision_start_token_id, cfg.vision_end_token_id}
    hi = min([hi] + [s for s in special if s > 1])
    ids = torch.randint(1, hi, (text_tokens,), generator=g)
    first = text_tokens // 2
    input_ids = torch.cat([ids[:first], torch.full((n_merged,), cfg.image_token_id, dtype=torch.long), ids[first:]])
    labels = input_ids.clone()
    labels[first:first + n_merged] = IGNORE_INDEX
    pixels = None
    if n_patches == 0:          # text-only sample
        return Sample(input_ids, labels, None, [], index)
    if with_pixels:
        pixels = torch.randn(n_patches, v.patch_dim, generator=g).to(dtype)
        if pin and torch.cuda.is_available():
            pixels = pixels.pin_memory()
    return Sample(input_ids, labels, pixels, [(1, side, side)], index)


def synthetic_global_batch(cfg: VLConfig, step: int, global_batch: int, *, image_sizes=None, text_token_choices=None,
                           **kw) -> list[Sample]:
    """``global_batch`` samples of step ``step``.  With ``image_sizes`` / ``text_token_choices`` (lists) the samples
    cycle through those image sides and text lengths, so that consecutive samples and steps differ in shape the way
    batches of a real data set do (ragged sequence-parallel splits, heap regions that have to grow)."""
    out = []
    for i in range(global_batch):
        index = step * global_batch + i
        k = dict(kw)
        if image_sizes:
            k["image_size"] = int(image_sizes[index % len(image_sizes)])
        if text_token_choices:
            k["text_tokens"] = int(text_token_choices[(index // max(len(image_sizes or [1]), 1) + index)
                                                      % len(text_token_choices)])
        out.append(synthetic_sample(cfg, index, **k))
    return out
