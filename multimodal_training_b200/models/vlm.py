"""The whole vision-language model in one process: encoder + decoder + splice, logits, loss and greedy decoding.

The trainers never use this class (they run the two halves as separate ranks); it exists for what the
reference keeps its HF-style wrappers for (``Qwen2_5_VLModel`` / ``Qwen2_5_VLForConditionalGeneration``,
python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:1531-2328): evaluating or sampling from a merged checkpoint,
and as a single-process oracle of the disaggregated pipeline in the tests.

* ``forward(input_ids, pixel_values, image_grid_thw)`` packs the batch into one token stream, encodes all
  images, writes the merged vision tokens over the image placeholders (the reference's ``masked_scatter`` at
  modeling_qwen2_5_vl.py:1858-1872), builds the 3-axis M-RoPE ids and runs the decoder.
* ``loss`` is the shifted causal cross-entropy with ``-100`` ignored (mean over valid tokens).
* ``generate`` is greedy decoding that recomputes the prefix each step (no KV cache): enough for evaluation
  of short answers and for tests, not a serving path.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config.model_configs import VLConfig, get_model_config
from ..data.rope_utils import get_rope_index_for_images
from ..ops.attention import SeqInfo
from ..parallel.sp import build_vision_plan
from .text import TextDecoder, mrope_cos_sin
from .vision import VisionEncoder


class Qwen2_5_VLModel(nn.Module):
    def __init__(self, config: VLConfig | str, dtype=torch.float32, device="cpu", seed: int = 0,
                 activation_checkpointing: bool = False):
        super().__init__()
        self.config = get_model_config(config) if isinstance(config, str) else config
        self.visual = VisionEncoder(self.config.vision, dtype=dtype, device=device, seed=seed,
                                    activation_checkpointing=activation_checkpointing)
        self.language_model = TextDecoder(self.config.text, dtype=dtype, device=device, seed=seed + 1,
                                          activation_checkpointing=activation_checkpointing)

    # ------------------------------------------------------------------ pieces
    def encode_images(self, pixel_values: torch.Tensor, image_grid_thw) -> torch.Tensor:
        """[N_patches, patch_dim] patches of all images (row-major per image) -> merged tokens
        [N_patches / merge^2, text_hidden] in the images' own raster order."""
        v = self.config.vision
        grids = [tuple(int(x) for x in g) for g in image_grid_thw]
        plan = build_vision_plan(grids, sp=1, rank=0, spatial_merge_size=v.spatial_merge_size,
                                 window_size=v.window_size, patch_size=v.patch_size, head_dim=v.head_dim)
        dev = pixel_values.device
        local = pixel_values.index_select(0, plan.local_patch_index.to(dev))
        merged = self.visual(local, plan)                     # window order
        out = torch.empty_like(merged)
        return out.index_copy(0, plan.local_merged_ids.to(dev), merged)

    def get_rope_index(self, input_ids: torch.Tensor, image_grid_thw, attention_mask=None, video_grid_thw=None,
                       second_per_grid_ts=None):
        """3-axis M-RoPE ids for images and videos (modeling_qwen2_5_vl.py:1561-1741 in the reference)."""
        if video_grid_thw is None or len(video_grid_thw) == 0:
            return get_rope_index_for_images(self.config.vision.spatial_merge_size, input_ids.cpu(), image_grid_thw,
                                             None if attention_mask is None else attention_mask.cpu(),
                                             image_token_id=self.config.image_token_id,
                                             vision_start_token_id=self.config.vision_start_token_id)
        from ..data.rope_utils import get_rope_index
        return get_rope_index(self.config.vision.spatial_merge_size, input_ids.cpu(), image_grid_thw, video_grid_thw,
                              second_per_grid_ts, None if attention_mask is None else attention_mask.cpu(),
                              image_token_id=self.config.image_token_id, video_token_id=self.config.video_token_id,
                              vision_start_token_id=self.config.vision_start_token_id)

    def _pack(self, input_ids: torch.Tensor, attention_mask):
        """[B, S] (right padded) -> packed ids [T], cu_seqlens, and the per-sample keep masks."""
        if input_ids.dim() == 1:
            input_ids = input_ids.unsqueeze(0)
        if attention_mask is None:
            attention_mask = torch.ones_like(input_ids)
        keep = attention_mask.bool()
        lens = keep.sum(1).tolist()
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + int(n))
        return input_ids[keep], cu, keep

    def hidden_states(self, input_ids, pixel_values=None, image_grid_thw=None, attention_mask=None,
                      pixel_values_videos=None, video_grid_thw=None, second_per_grid_ts=None):
        """Packed final hidden states [T, H] (before the last norm), cu_seqlens and the keep mask."""
        cfg = self.config
        ids, cu, keep = self._pack(input_ids, attention_mask)
        dev = self.language_model.embed_tokens.device
        x = self.language_model.embed(ids.to(dev))
        if pixel_values is not None and len(image_grid_thw):
            vis = self.encode_images(pixel_values.to(dev), image_grid_thw).to(x.dtype)
            rows = (ids == cfg.image_token_id).nonzero().flatten().to(dev)
            if rows.numel() != vis.shape[0]:
                raise ValueError(f"{rows.numel()} image placeholder tokens but {vis.shape[0]} merged vision tokens")
            x = x.index_copy(0, rows, vis)
        if pixel_values_videos is not None and video_grid_thw is not None and len(video_grid_thw):
            vid = self.encode_images(pixel_values_videos.to(dev), video_grid_thw).to(x.dtype)
            rows = (ids == cfg.video_token_id).nonzero().flatten().to(dev)
            if rows.numel() != vid.shape[0]:
                raise ValueError(f"{rows.numel()} video placeholder tokens but {vid.shape[0]} merged video tokens")
            x = x.index_copy(0, rows, vid)
        pos, _ = self.get_rope_index(input_ids if input_ids.dim() == 2 else input_ids.unsqueeze(0),
                                     image_grid_thw if image_grid_thw is not None else [], attention_mask,
                                     video_grid_thw, second_per_grid_ts)
        pos = pos[:, keep.cpu()]                                    # [3, T]
        cos, sin = mrope_cos_sin(pos, cfg.text.head_dim, cfg.text.rope_theta, cfg.text.mrope_section)
        h = self.language_model(x, cos.to(dev), sin.to(dev), SeqInfo.from_list(cu, dev))
        return h, cu, keep

    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, attention_mask=None, **video_kw):
        """Logits of every kept token, packed: [T, vocab].  ``video_kw``: ``pixel_values_videos``, ``video_grid_thw``,
        ``second_per_grid_ts`` as the processor returns them."""
        h, _, _ = self.hidden_states(input_ids, pixel_values, image_grid_thw, attention_mask, **video_kw)
        return self.language_model.logits(h)


class Qwen2_5_VLForConditionalGeneration(nn.Module):
    def __init__(self, config: VLConfig | str, **kw):
        super().__init__()
        self.model = Qwen2_5_VLModel(config, **kw)
        self.config = self.model.config

    def forward(self, input_ids, pixel_values=None, image_grid_thw=None, attention_mask=None, labels=None,
                **video_kw):
        """Returns ``{"logits": [T, V]}`` and, with labels [B, S], ``"loss"`` (next-token CE, -100 ignored)."""
        h, cu, keep = self.model.hidden_states(input_ids, pixel_values, image_grid_thw, attention_mask, **video_kw)
        out = {"logits": self.model.language_model.logits(h)}
        if labels is not None:
            if labels.dim() == 1:
                labels = labels.unsqueeze(0)
            shifted = torch.full_like(labels, -100)
            shifted[:, :-1] = labels[:, 1:]
            # the last kept token of every sample has nothing to predict
            lens = keep.sum(1)
            shifted[torch.arange(labels.shape[0]), (lens - 1).clamp(min=0)] = -100
            out["loss"] = self.model.language_model.loss(h, shifted[keep].to(h.device))
        return out

    @torch.no_grad()
    def generate(self, input_ids, pixel_values=None, image_grid_thw=None, max_new_tokens: int = 16,
                 eos_token_id: int | None = None) -> torch.Tensor:
        """Greedy continuation of ONE sample; returns the full id sequence [S + new]."""
        ids = input_ids.flatten().clone()
        for _ in range(max_new_tokens):
            logits = self.model(ids.unsqueeze(0), pixel_values, image_grid_thw)
            nxt = int(logits[-1].float().argmax())
            ids = torch.cat([ids, torch.tensor([nxt], dtype=ids.dtype, device=ids.device)])
            if eos_token_id is not None and nxt == eos_token_id:
                break
        return ids

    def load_merged_state_dict(self, state: dict) -> None:
        """Keys of a merged checkpoint (``visual.*`` / ``language_model.*`` / ``lm_head.*``, as written by
        ``cli/merge_checkpoint.py`` and by HF)."""
        vis = {k.split("visual.", 1)[1]: v for k, v in state.items() if "visual." in k}
        txt = {}
        for k, v in state.items():
            if "visual." in k:
                continue
            k2 = k.split("language_model.", 1)[1] if "language_model." in k else k
            txt[k2[len("model."):] if k2.startswith("model.") else k2] = v
        self.model.visual.load_reference_state_dict(vis)
        self.model.language_model.load_reference_state_dict(txt)
