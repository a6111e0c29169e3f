"""Model architecture configs, embedded in the package.

The reference fetches ``config.json`` from the Hugging Face hub through
``from_pretrained`` (python/ray/vision.py:668, python/ray/text.py:1147); a
training box without network cannot, so the published Qwen2.5-VL shapes live
here.  Field names follow the reference's config classes
(python/models/qwen2_5_vl/configuration_qwen2_5_vl.py:32-339).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


@dataclass
class VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    out_hidden_size: int = 3584
    patch_size: int = 14
    temporal_patch_size: int = 2
    in_channels: int = 3
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: list[int] = field(default_factory=lambda: [7, 15, 23, 31])
    rms_norm_eps: float = 1e-6
    hidden_act: str = "silu"
    sequence_parallel: bool = False
    initializer_range: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def merge_unit(self) -> int:
        return self.spatial_merge_size * self.spatial_merge_size

    @property
    def padded_intermediate_size(self) -> int:
        """MLP width rounded up so that activation rows start on 16-byte boundaries (TMA)."""
        return (self.intermediate_size + 7) // 8 * 8


@dataclass
class TextConfig:
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    mrope_section: list[int] = field(default_factory=lambda: [16, 24, 24])
    tie_word_embeddings: bool = False
    initializer_range: float = 0.02
    max_position_embeddings: int = 128000

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
class VLConfig:
    name: str = "qwen2_5_vl_7b"
    model_type: str = "qwen2_5_vl"
    vision: VisionConfig = field(default_factory=VisionConfig)
    text: TextConfig = field(default_factory=TextConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision_end_token_id: int = 151653
    pad_token_id: int = 151643

    def to_dict(self) -> dict[str, Any]:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "VLConfig":
        d = dict(d)
        v = d.pop("vision", d.pop("vision_config", {})) or {}
        t = d.pop("text", d.pop("text_config", {})) or {}
        vf = {f.name for f in dataclasses.fields(VisionConfig)}
        tf = {f.name for f in dataclasses.fields(TextConfig)}
        cf = {f.name for f in dataclasses.fields(cls)}
        # HF config.json keeps rope_scaling.mrope_section and puts text fields at the top level
        rs = t.get("rope_scaling") or d.get("rope_scaling")
        if isinstance(rs, dict) and "mrope_section" in rs:
            t.setdefault("mrope_section", rs["mrope_section"])
        for k in list(d):
            if k in tf and k not in cf:
                t.setdefault(k, d[k])
        return cls(vision=VisionConfig(**{k: x for k, x in v.items() if k in vf}),
                   text=TextConfig(**{k: x for k, x in t.items() if k in tf}),
                   **{k: x for k, x in d.items() if k in cf and k not in ("vision", "text")})


def _vl(name: str, vision: dict, text: dict, **kw) -> VLConfig:
    return VLConfig(name=name, vision=VisionConfig(**vision), text=TextConfig(**text), **kw)


def _registry() -> dict[str, VLConfig]:
    vis = dict(depth=32, hidden_size=1280, num_heads=16, patch_size=14, spatial_merge_size=2, window_size=112,
               fullatt_block_indexes=[7, 15, 23, 31])
    reg = {
        # tiny model of the CPU parity configuration (fp32, gloo)
        "tiny": _vl(
            "tiny",
            dict(depth=4, hidden_size=128, num_heads=4, intermediate_size=512, out_hidden_size=256, patch_size=14,
                 spatial_merge_size=2, window_size=112, fullatt_block_indexes=[3]),
            dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
                 num_key_value_heads=2, mrope_section=[8, 12, 12], tie_word_embeddings=False),
            image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003,
            pad_token_id=0),
        # the tiny model with the input embedding reused as the output projection (as in the 3B model)
        "tiny_tied": _vl(
            "tiny_tied",
            dict(depth=4, hidden_size=128, num_heads=4, intermediate_size=512, out_hidden_size=256, patch_size=14,
                 spatial_merge_size=2, window_size=112, fullatt_block_indexes=[3]),
            dict(vocab_size=1024, hidden_size=256, intermediate_size=688, num_hidden_layers=4, num_attention_heads=4,
                 num_key_value_heads=2, mrope_section=[8, 12, 12], tie_word_embeddings=True),
            image_token_id=1000, video_token_id=1001, vision_start_token_id=1002, vision_end_token_id=1003,
            pad_token_id=0),
        # a bf16-friendly small model for single-GPU smoke runs (head_dim 80 vision / 128 text like the real ones)
        "smoke": _vl(
            "smoke",
            dict(depth=4, hidden_size=320, num_heads=4, intermediate_size=856, out_hidden_size=512, patch_size=14,
                 spatial_merge_size=2, window_size=112, fullatt_block_indexes=[1, 3]),
            dict(vocab_size=4096, hidden_size=512, intermediate_size=1408, num_hidden_layers=2, num_attention_heads=4,
                 num_key_value_heads=2, mrope_section=[16, 24, 24], tie_word_embeddings=False),
            image_token_id=4000, video_token_id=4001, vision_start_token_id=4002, vision_end_token_id=4003,
            pad_token_id=0),
        "qwen2_5_vl_3b": _vl(
            "qwen2_5_vl_3b", dict(vis, intermediate_size=3420, out_hidden_size=2048),
            dict(vocab_size=151936, hidden_size=2048, intermediate_size=11008, num_hidden_layers=36,
                 num_attention_heads=16, num_key_value_heads=2, tie_word_embeddings=True)),
        "qwen2_5_vl_7b": _vl(
            "qwen2_5_vl_7b", dict(vis, intermediate_size=3420, out_hidden_size=3584),
            dict(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
                 num_attention_heads=28, num_key_value_heads=4)),
        "qwen2_5_vl_32b": _vl(
            "qwen2_5_vl_32b", dict(vis, intermediate_size=3456, out_hidden_size=5120),
            dict(vocab_size=152064, hidden_size=5120, intermediate_size=27648, num_hidden_layers=64,
                 num_attention_heads=40, num_key_value_heads=8)),
        "qwen2_5_vl_72b": _vl(
            "qwen2_5_vl_72b", dict(vis, intermediate_size=3456, out_hidden_size=8192),
            dict(vocab_size=152064, hidden_size=8192, intermediate_size=29568, num_hidden_layers=80,
                 num_attention_heads=64, num_key_value_heads=8)),
    }
    return reg


_ALIASES = {
    "qwen/qwen2.5-vl-3b-instruct": "qwen2_5_vl_3b",
    "qwen/qwen2.5-vl-7b-instruct": "qwen2_5_vl_7b",
    "qwen/qwen2.5-vl-32b-instruct": "qwen2_5_vl_32b",
    "qwen/qwen2.5-vl-72b-instruct": "qwen2_5_vl_72b",
}


def available_models() -> list[str]:
    return sorted(_registry())


def get_model_config(name_or_path: str) -> VLConfig:
    """Resolve a config by embedded name, HF repo id, or a directory/file holding ``config.json``."""
    key = name_or_path.strip()
    reg = _registry()
    low = key.lower()
    if low in reg:
        return reg[low]
    if low in _ALIASES:
        return reg[_ALIASES[low]]
    p = Path(key)
    if p.is_dir():
        p = p / "config.json"
    if p.is_file() and p.suffix == ".json":
        cfg = VLConfig.from_dict(json.loads(p.read_text()))
        cfg.name = key
        return cfg
    raise KeyError(f"unknown model '{name_or_path}'; embedded configs: {available_models()}")
