"""In-tree Qwen2.5-VL processor: image -> patches, placeholder expansion, chat template.

The reference ships a copy of HF's ``Qwen2_5_VLProcessor`` (python/models/qwen2_5_vl/processing_qwen2_5_vl.py:67-284)
and loads the image processor and tokenizer through ``AutoProcessor`` (python/ray/trainer.py:46-50), which needs
the model repository on disk or the network.  This module restates the parts the data pipeline depends on, so a
run needs nothing but a tokenizer:

* :func:`smart_resize` -- height and width rounded to multiples of ``patch * merge`` (28) inside
  ``[min_pixels, max_pixels]``, aspect ratio kept;
* :class:`Qwen2_5_VLImageProcessor` -- bicubic resize, scale to [0,1], normalise, cut into
  ``[N, 3 * 2 * 14 * 14]`` patch rows in the order the vision encoder expects (2x2 merge blocks contiguous,
  the single frame repeated to fill the temporal patch), plus ``image_grid_thw``;
* videos: a clip (frames array or list of frames) becomes ``ceil(F / 2)`` temporal patches of the same patch
  layout, ``video_grid_thw`` and ``second_per_grid_ts``; ``<|video_pad|>`` expands like ``<|image_pad|>``;
* :class:`Qwen2_5_VLProcessor` -- replaces every ``<|image_pad|>`` by one placeholder per merged vision token
  (``grid.prod() // merge**2``, processing_qwen2_5_vl.py:178-186), tokenises, and renders Qwen's chat template
  (``apply_chat_template``) for LLaVA-style messages;
* :class:`ByteTokenizer` -- a dependency-free byte-level tokenizer with the special tokens at their Qwen ids,
  for offline tests and synthetic runs.  Real training passes the model's own tokenizer instead.
"""
from __future__ import annotations

import math

import numpy as np
import torch

IMAGE_MEAN = (0.48145466, 0.4578275, 0.40821073)
IMAGE_STD = (0.26862954, 0.26130258, 0.27577711)
IMAGE_PAD, VISION_START, VISION_END = "<|image_pad|>", "<|vision_start|>", "<|vision_end|>"
VIDEO_PAD = "<|video_pad|>"
IM_START, IM_END = "<|im_start|>", "<|im_end|>"


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 1280) -> tuple[int, int]:
    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError(f"aspect ratio of a {height}x{width} image is above 200")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def _to_chw_float(image) -> torch.Tensor:
    """PIL image, HWC uint8 array or CHW float tensor -> CHW float32 in [0, 1]."""
    if isinstance(image, torch.Tensor):
        t = image.float()
        if t.dim() == 3 and t.shape[0] not in (1, 3) and t.shape[-1] in (1, 3):
            t = t.permute(2, 0, 1)
        return t / 255.0 if t.max() > 1.5 else t
    arr = np.asarray(image)
    if arr.ndim == 2:
        arr = np.stack([arr] * 3, axis=-1)
    t = torch.from_numpy(np.array(arr[..., :3])).permute(2, 0, 1).float()        # a writable copy
    return t / 255.0 if arr.dtype == np.uint8 or t.max() > 1.5 else t


class Qwen2_5_VLImageProcessor:
    def __init__(self, patch_size: int = 14, temporal_patch_size: int = 2, merge_size: int = 2,
                 min_pixels: int = 56 * 56, max_pixels: int = 14 * 14 * 4 * 1280, image_mean=IMAGE_MEAN,
                 image_std=IMAGE_STD):
        self.patch_size, self.temporal_patch_size, self.merge_size = patch_size, temporal_patch_size, merge_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.mean = torch.tensor(image_mean).view(3, 1, 1)
        self.std = torch.tensor(image_std).view(3, 1, 1)

    def preprocess_one(self, image, min_pixels=None, max_pixels=None):
        x = _to_chw_float(image)
        if x.shape[0] == 1:
            x = x.expand(3, -1, -1)
        H, W = x.shape[1:]
        f = self.patch_size * self.merge_size
        h, w = smart_resize(H, W, f, min_pixels or self.min_pixels, max_pixels or self.max_pixels)
        if (h, w) != (H, W):
            x = torch.nn.functional.interpolate(x[None], size=(h, w), mode="bicubic", align_corners=False,
                                                antialias=True)[0].clamp(0, 1)
        x = (x - self.mean) / self.std
        P, T, m = self.patch_size, self.temporal_patch_size, self.merge_size
        gh, gw = h // P, w // P
        frames = x[None].expand(T, -1, -1, -1)                    # one image fills the temporal patch
        # [T, C, gh/m, m, P, gw/m, m, P] -> [gh/m, gw/m, m, m, C, T, P, P]: merge blocks contiguous
        t = frames.reshape(T, 3, gh // m, m, P, gw // m, m, P).permute(2, 5, 3, 6, 1, 0, 4, 7)
        return t.reshape(gh * gw, 3 * T * P * P).contiguous(), (1, gh, gw)

    def preprocess_video(self, frames, min_pixels=None, max_pixels=None):
        """A clip as [F, H, W, 3] array / tensor or a list of frames -> patch rows [t * gh * gw, 3 * T * P * P] with
        ``t = ceil(F / T)`` temporal patches (the last frame is repeated to fill the last one) and its grid."""
        if isinstance(frames, (str, bytes)):
            # no video decoder ships with this package: clips arrive as decoded frames
            raise NotImplementedError(f"video '{frames}': pass the decoded frames ([F, H, W, 3] array or a list of "
                                      "frames); decoding container files is left to the caller")
        if isinstance(frames, (torch.Tensor, np.ndarray)) and getattr(frames, "ndim", 0) == 4:
            frames = [frames[i] for i in range(frames.shape[0])]
        xs = [_to_chw_float(f) for f in frames]
        if not xs:
            raise ValueError("a video needs at least one frame")
        H, W = xs[0].shape[1:]
        f = self.patch_size * self.merge_size
        h, w = smart_resize(H, W, f, min_pixels or self.min_pixels, max_pixels or self.max_pixels)
        x = torch.stack([v.expand(3, -1, -1) if v.shape[0] == 1 else v for v in xs])       # [F, 3, H, W]
        if (h, w) != (H, W):
            x = torch.nn.functional.interpolate(x, size=(h, w), mode="bicubic", align_corners=False,
                                                antialias=True).clamp(0, 1)
        x = (x - self.mean) / self.std
        P, T, m = self.patch_size, self.temporal_patch_size, self.merge_size
        if x.shape[0] % T:
            x = torch.cat([x, x[-1:].expand(T - x.shape[0] % T, -1, -1, -1)])
        t, gh, gw = x.shape[0] // T, h // P, w // P
        # [t, T, C, gh/m, m, P, gw/m, m, P] -> [t, gh/m, gw/m, m, m, C, T, P, P]
        r = x.reshape(t, T, 3, gh // m, m, P, gw // m, m, P).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
        return r.reshape(t * gh * gw, 3 * T * P * P).contiguous(), (t, gh, gw)

    def videos(self, videos, fps: float = 2.0, min_pixels=None, max_pixels=None):
        rows, grids = [], []
        for v in videos:
            r, g = self.preprocess_video(v, min_pixels, max_pixels)
            rows.append(r)
            grids.append(g)
        return {"pixel_values_videos": torch.cat(rows),
                "video_grid_thw": torch.tensor(grids, dtype=torch.long).reshape(-1, 3),
                "second_per_grid_ts": [self.temporal_patch_size / float(fps)] * len(grids)}

    def __call__(self, images, min_pixels=None, max_pixels=None, **_):
        images = images if isinstance(images, (list, tuple)) else [images]
        rows, grids = [], []
        for im in images:
            r, g = self.preprocess_one(im, min_pixels, max_pixels)
            rows.append(r)
            grids.append(g)
        return {"pixel_values": torch.cat(rows) if rows else torch.zeros(0, 3 * self.temporal_patch_size *
                                                                          self.patch_size ** 2),
                "image_grid_thw": torch.tensor(grids, dtype=torch.long).reshape(-1, 3)}


class ByteTokenizer:
    """UTF-8 bytes as ids 0..255 plus the special tokens of the chat template at their Qwen2.5 ids."""

    SPECIAL = {IM_START: 151644, IM_END: 151645, VISION_START: 151652, VISION_END: 151653, IMAGE_PAD: 151655,
               "<|video_pad|>": 151656, "<|endoftext|>": 151643}
    ROLE_IDS = {"assistant": 77091}       # single id the label mask looks for after <|im_start|>

    def __init__(self, special: dict[str, int] | None = None):
        self.special = dict(self.SPECIAL if special is None else special)
        self.inv = {v: k for k, v in self.special.items()}
        self.pad_token_id = self.special.get("<|endoftext|>", 0)
        self.eos_token_id = self.special.get(IM_END, 0)

    @classmethod
    def for_config(cls, model_cfg) -> "ByteTokenizer":
        """Special tokens at the ids of ``model_cfg``.  Configurations with Qwen's vocabulary keep Qwen's ids; small
        test configurations get the chat-control tokens right above the byte range."""
        vocab = getattr(getattr(model_cfg, "text", None), "vocab_size", 0)
        if model_cfg is None or vocab > max(cls.SPECIAL.values()):
            return cls()
        special = {IMAGE_PAD: model_cfg.image_token_id, VISION_START: model_cfg.vision_start_token_id,
                   VISION_END: model_cfg.vision_end_token_id, "<|video_pad|>": model_cfg.video_token_id,
                   IM_START: 256, IM_END: 257, "<|endoftext|>": 259}
        if len(set(special.values())) != len(special) or max(special.values()) >= vocab:
            raise ValueError(f"special token ids {special} do not fit a vocabulary of {vocab}")
        tok = cls(special)
        tok.ROLE_IDS = {"assistant": 258}
        tok.pad_token_id = getattr(model_cfg, "pad_token_id", 0) or 0
        return tok

    @property
    def assistant_token_id(self) -> int:
        return self.ROLE_IDS["assistant"]

    def encode(self, text: str) -> list[int]:
        ids: list[int] = []
        i = 0
        keys = sorted(self.special, key=len, reverse=True)
        while i < len(text):
            for k in keys:
                if text.startswith(k, i):
                    ids.append(self.special[k])
                    i += len(k)
                    # a role name right after <|im_start|> is one token, as in the real vocabulary
                    if k == IM_START:
                        for role, rid in self.ROLE_IDS.items():
                            if text.startswith(role, i):
                                ids.append(rid)
                                i += len(role)
                    break
            else:
                ids.extend(text[i].encode("utf-8"))
                i += 1
        return ids

    def decode(self, ids) -> str:
        out, buf = [], bytearray()
        role = {v: k for k, v in self.ROLE_IDS.items()}
        for t in (int(x) for x in ids):
            if t < 256:
                buf.append(t)
                continue
            out.append(buf.decode("utf-8", errors="replace"))
            buf = bytearray()
            out.append(self.inv.get(t, role.get(t, "")))
        out.append(buf.decode("utf-8", errors="replace"))
        return "".join(out)

    def __call__(self, text, **_):
        texts = [text] if isinstance(text, str) else list(text)
        return {"input_ids": [self.encode(t) for t in texts]}


class Qwen2_5_VLProcessor:
    def __init__(self, image_processor: Qwen2_5_VLImageProcessor | None = None, tokenizer=None):
        self.image_processor = image_processor or Qwen2_5_VLImageProcessor()
        self.tokenizer = tokenizer or ByteTokenizer()

    # ------------------------------------------------------------------ chat template
    def render(self, messages: list[dict], add_generation_prompt: bool = False) -> tuple[str, list]:
        """Qwen chat format; returns the text (one ``<|image_pad|>`` per image, one ``<|video_pad|>`` per video), the
        images in order and, as ``self.last_videos``, the videos in order."""
        parts, images = [], []
        self.last_videos = []
        if not messages or messages[0].get("role") != "system":
            parts.append(f"{IM_START}system\nYou are a helpful assistant.{IM_END}\n")
        for msg in messages:
            content = msg["content"]
            body = []
            if isinstance(content, str):
                body.append(content)
            else:
                for item in content:
                    if item.get("type") == "image":
                        images.append(item.get("image"))
                        body.append(f"{VISION_START}{IMAGE_PAD}{VISION_END}")
                    elif item.get("type") == "text":
                        body.append(item["text"])
                    elif item.get("type") == "video":
                        self.last_videos.append(item.get("video"))
                        body.append(f"{VISION_START}{VIDEO_PAD}{VISION_END}")
            parts.append(f"{IM_START}{msg['role']}\n{''.join(body)}{IM_END}\n")
        if add_generation_prompt:
            parts.append(f"{IM_START}assistant\n")
        return "".join(parts), images

    def apply_chat_template(self, messages, tokenize: bool = True, return_dict: bool = True, return_tensors=None,
                            add_generation_prompt: bool = False, **image_kw):
        text, images = self.render(messages, add_generation_prompt)
        if not tokenize:
            return text
        return self(text=[text], images=images or None, videos=self.last_videos or None,
                    return_tensors=return_tensors, **image_kw)

    # ------------------------------------------------------------------ text + images -> model inputs
    def __call__(self, text=None, images=None, videos=None, return_tensors=None, fps: float = 2.0, **image_kw):
        texts = [text] if isinstance(text, str) else list(text or [])
        out = {}
        grids, vgrids = [], []
        if images is not None and len(images):
            img = self.image_processor(images, **image_kw)
            out.update(img)
            grids = img["image_grid_thw"].tolist()
        if videos is not None and len(videos):
            vid = self.image_processor.videos(videos, fps=fps, **image_kw)
            out.update(vid)
            vgrids = vid["video_grid_thw"].tolist()
        unit = self.image_processor.merge_size ** 2
        k = kv = 0
        expanded = []
        for t in texts:
            while IMAGE_PAD in t:
                if k >= len(grids):
                    raise ValueError("more <|image_pad|> placeholders than images")
                n = int(np.prod(grids[k])) // unit
                t = t.replace(IMAGE_PAD, "<|placeholder|>" * n, 1)
                k += 1
            t = t.replace("<|placeholder|>", IMAGE_PAD)
            while VIDEO_PAD in t:
                if kv >= len(vgrids):
                    raise ValueError("more <|video_pad|> placeholders than videos")
                n = int(np.prod(vgrids[kv])) // unit
                t = t.replace(VIDEO_PAD, "<|placeholder|>" * n, 1)
                kv += 1
            expanded.append(t.replace("<|placeholder|>", VIDEO_PAD))
        if k != len(grids):
            raise ValueError(f"{len(grids)} images but {k} <|image_pad|> placeholders")
        if kv != len(vgrids):
            raise ValueError(f"{len(vgrids)} videos but {kv} <|video_pad|> placeholders")
        enc = self.tokenizer(expanded)
        ids = enc["input_ids"]
        if return_tensors == "pt":
            width = max((len(x) for x in ids), default=0)
            pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
            mask = [[1] * len(x) + [0] * (width - len(x)) for x in ids]
            ids = [list(x) + [pad] * (width - len(x)) for x in ids]
            out["input_ids"] = torch.tensor(ids, dtype=torch.long)
            out["attention_mask"] = torch.tensor(mask, dtype=torch.long)
        else:
            out["input_ids"] = ids
        return out
