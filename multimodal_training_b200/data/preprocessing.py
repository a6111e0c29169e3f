"""LLaVA-style conversations -> Qwen chat messages -> model inputs
(reference: python/data/preprocessing.py:20-163).

A sample is ``{"image": path | [paths], "conversations": [{"from": "human"|"gpt", "value": text}, ...]}``;
``<image>`` / ``<video>`` placeholders in the text consume the sample's media in order.  Labels are
``IGNORE_INDEX`` everywhere except the assistant answers (tokens after ``<|im_start|>assistant\\n`` up to
and including ``<|im_end|>``).  Token ids are taken from the tokenizer / config, not hard-coded.
"""
from __future__ import annotations

import math
import re

import torch

IGNORE_INDEX = -100
IMAGE_TOKEN_INDEX = 151655
VIDEO_TOKEN_INDEX = 151656
ASSISTANT_TOKEN_ID = 77091
IM_END_TOKEN_ID = 151645


def build_messages(conversations: list[dict], images: list, videos: list | None = None) -> list[dict]:
    """Chat messages with typed content parts; placeholders take media from the pools in order."""
    roles = {"human": "user", "gpt": "assistant", "user": "user", "assistant": "assistant", "system": "system"}
    img_pool, vid_pool = list(images or []), list(videos or [])
    out = []
    for turn in conversations:
        role = roles.get(turn["from"], turn["from"])
        parts = []
        for piece in re.split(r"(<image>|<video>)", turn["value"]):
            if piece == "<image>":
                if not img_pool:
                    raise ValueError("more <image> placeholders than images")
                parts.append({"type": "image", "image": img_pool.pop(0)})
            elif piece == "<video>":
                if not vid_pool:
                    raise ValueError("more <video> placeholders than videos")
                parts.append({"type": "video", "video": vid_pool.pop(0)})
            elif piece.strip():
                parts.append({"type": "text", "text": piece.strip() if role == "user" else piece})
        out.append({"role": role, "content": parts})
    return out


def fixed_size_resize(image, max_pixels: int, patch_multiple: int = 28):
    """Bilinear resize to a square of side ~sqrt(max_pixels), rounded to the patch-merge multiple."""
    side = int(math.sqrt(max_pixels)) // patch_multiple * patch_multiple
    side = max(side, patch_multiple)
    try:
        from PIL import Image
        return image.resize((side, side), Image.BILINEAR)
    except Exception:
        return image


def mask_labels(input_ids: torch.Tensor, assistant_id: int = ASSISTANT_TOKEN_ID,
                im_end_id: int = IM_END_TOKEN_ID) -> torch.Tensor:
    """Labels = ids inside assistant answers, IGNORE_INDEX elsewhere."""
    ids = input_ids.reshape(-1).tolist()
    labels = [IGNORE_INDEX] * len(ids)
    i = 0
    while i < len(ids):
        if ids[i] == assistant_id:
            j = i + 2          # skip "assistant" and the newline after it
            while j < len(ids):
                labels[j] = ids[j]
                if ids[j] == im_end_id:
                    break
                j += 1
            i = j
        i += 1
    return torch.tensor(labels, dtype=torch.long).reshape(input_ids.shape)


def chat_token_ids(processor) -> tuple[int, int]:
    """(id of the ``assistant`` role token, id of ``<|im_end|>``) of the processor's tokenizer; Qwen's ids when the
    tokenizer cannot say."""
    tok = getattr(processor, "tokenizer", None)
    assistant, im_end = ASSISTANT_TOKEN_ID, IM_END_TOKEN_ID
    if tok is None:
        return assistant, im_end
    if hasattr(tok, "assistant_token_id"):                       # in-tree byte tokenizer
        return int(tok.assistant_token_id), int(tok.special.get("<|im_end|>", im_end))
    try:                                                          # Hugging Face tokenizer
        ids = tok.encode("assistant", add_special_tokens=False)
        if len(ids) == 1:
            assistant = int(ids[0])
        e = tok.convert_tokens_to_ids("<|im_end|>")
        if isinstance(e, int) and e >= 0:
            im_end = e
    except Exception:
        pass
    return assistant, im_end


def preprocess_qwen_visual(sources: list[dict], processor, *, data_path: str = "", max_pixels: int | None = None,
                           min_pixels: int | None = None, force_fixed_size: bool = False) -> dict:
    """One sample -> ``{"input_ids" [1,S], "labels" [1,S], "pixel_values", "image_grid_thw"}``."""
    import os
    sample = sources[0] if isinstance(sources, (list, tuple)) else sources
    paths = sample.get("image") or []
    paths = [paths] if isinstance(paths, str) else list(paths)
    images = []
    for p in paths:
        full = os.path.join(data_path, p) if data_path else p
        try:
            from PIL import Image
            img = Image.open(full).convert("RGB")
        except ImportError:
            img = full
        if force_fixed_size and max_pixels:
            img = fixed_size_resize(img, max_pixels)
        images.append(img)
    messages = build_messages(sample["conversations"], images)
    kwargs = {}
    if max_pixels:
        kwargs["max_pixels"] = max_pixels
    if min_pixels:
        kwargs["min_pixels"] = min_pixels
    enc = processor.apply_chat_template(messages, tokenize=True, return_dict=True, return_tensors="pt", **kwargs)
    input_ids = enc["input_ids"]
    if not isinstance(input_ids, torch.Tensor):
        input_ids = torch.tensor(input_ids)
    input_ids = input_ids.reshape(1, -1)
    assistant_id, im_end_id = chat_token_ids(processor)
    out = {"input_ids": input_ids, "labels": mask_labels(input_ids, assistant_id, im_end_id)}
    for k in ("pixel_values", "image_grid_thw"):
        if k in enc and enc[k] is not None:
            out[k] = enc[k] if isinstance(enc[k], torch.Tensor) else torch.tensor(enc[k])
    return out
