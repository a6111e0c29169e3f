"""3-axis (temporal, height, width) position ids for M-RoPE, built on the data side.

Text runs count 0,1,2,... on all three axes; an image run keeps the temporal axis fixed per frame
and walks the merged (h, w) grid, offset by the length of the text before it; the text after an
image continues from the largest id used so far plus one.  Same rule as the reference's
``get_rope_index_for_images`` (python/data/rope_utils.py:6-124); the token ids come from the model
config instead of being hard-coded.
"""
from __future__ import annotations

import torch


def get_rope_index_for_images(spatial_merge_size: int, input_ids: torch.Tensor, image_grid_thw, attention_mask=None,
                              image_token_id: int = 151655, vision_start_token_id: int = 151652):
    """``input_ids`` [B, S] -> ``(position_ids [3, B, S], mrope_position_deltas [B, 1])``.

    ``image_grid_thw`` lists the (t, h, w) patch grids of all images of the batch in order of appearance.
    """
    if input_ids.dim() == 1:
        input_ids = input_ids.unsqueeze(0)
    B, S = input_ids.shape
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    position_ids = torch.ones(3, B, S, dtype=torch.long)
    deltas = []
    grids = [tuple(int(x) for x in g) for g in (image_grid_thw if image_grid_thw is not None else [])]
    img_i = 0
    for b in range(B):
        keep = attention_mask[b] == 1
        ids = input_ids[b][keep].tolist()
        n_img = sum(1 for i, tok in enumerate(ids[:-1]) if tok == vision_start_token_id and ids[i + 1] == image_token_id)
        if n_img == 0 and image_token_id in ids:
            # placeholders without a start marker (synthetic data): one run per contiguous block
            n_img = sum(1 for i, tok in enumerate(ids) if tok == image_token_id and (i == 0 or ids[i - 1] != tok))
        chunks = []
        st = 0
        for _ in range(n_img):
            ed = ids.index(image_token_id, st)
            t, h, w = grids[img_i]
            img_i += 1
            gh, gw = h // spatial_merge_size, w // spatial_merge_size
            text_len = ed - st
            st_idx = int(chunks[-1].max()) + 1 if chunks else 0
            chunks.append(torch.arange(text_len).view(1, -1).expand(3, -1) + st_idx)
            t_index = torch.arange(t).view(-1, 1).expand(-1, gh * gw).flatten()
            h_index = torch.arange(gh).view(1, -1, 1).expand(t, -1, gw).flatten()
            w_index = torch.arange(gw).view(1, 1, -1).expand(t, gh, -1).flatten()
            chunks.append(torch.stack([t_index, h_index, w_index]) + text_len + st_idx)
            st = ed + t * gh * gw
        if st < len(ids):
            st_idx = int(chunks[-1].max()) + 1 if chunks else 0
            chunks.append(torch.arange(len(ids) - st).view(1, -1).expand(3, -1) + st_idx)
        pos = torch.cat(chunks, dim=1) if chunks else torch.zeros(3, 0, dtype=torch.long)
        position_ids[:, b, keep] = pos
        deltas.append(int(pos.max()) + 1 - len(ids) if pos.numel() else 0)
    return position_ids, torch.tensor(deltas).unsqueeze(1)


def get_rope_index(spatial_merge_size: int, input_ids: torch.Tensor, image_grid_thw=None, video_grid_thw=None,
                   second_per_grid_ts=None, attention_mask=None, image_token_id: int = 151655,
                   video_token_id: int = 151656, vision_start_token_id: int = 151652, tokens_per_second: float = 2.0):
    """3-axis position ids for sequences with images AND videos (the model-side rule of the reference,
    python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:1561-1741).

    Media are taken in order of appearance: the token after ``<|vision_start|>`` says whether the next run is an image
    or a video.  A video's temporal index advances by ``second_per_grid_ts[k] * tokens_per_second`` per temporal patch
    (time-aligned M-RoPE); an image is a video with one temporal patch.  Returns ``(position_ids [3, B, S],
    mrope_position_deltas [B, 1])``.
    """
    if input_ids.dim() == 1:
        input_ids = input_ids.unsqueeze(0)
    B, S = input_ids.shape
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    images = [tuple(int(x) for x in g) for g in (image_grid_thw if image_grid_thw is not None else [])]
    videos = [tuple(int(x) for x in g) for g in (video_grid_thw if video_grid_thw is not None else [])]
    secs = [float(x) for x in (second_per_grid_ts if second_per_grid_ts is not None else [])]
    position_ids = torch.ones(3, B, S, dtype=torch.long)
    deltas = []
    ii = vi = 0
    m = spatial_merge_size
    for b in range(B):
        keep = attention_mask[b] == 1
        ids = input_ids[b][keep].tolist()
        chunks = []
        st = 0
        while True:
            # next media run: first image / video placeholder at or after st
            nxt = [(ids.index(tok, st), kind) for tok, kind in ((image_token_id, "image"), (video_token_id, "video"))
                   if tok in ids[st:]]
            if not nxt:
                break
            ed, kind = min(nxt)
            if kind == "image":
                t, h, w = images[ii]
                ii += 1
                step = 0.0
            else:
                t, h, w = videos[vi]
                step = (secs[vi] if vi < len(secs) else 1.0) * tokens_per_second
                vi += 1
            gh, gw = h // m, w // m
            text_len = ed - st
            st_idx = int(chunks[-1].max()) + 1 if chunks else 0
            chunks.append(torch.arange(text_len).view(1, -1).expand(3, -1) + st_idx)
            t_index = (torch.arange(t).view(-1, 1).expand(-1, gh * gw) * step).long().flatten() if kind == "video" \
                else torch.arange(t).view(-1, 1).expand(-1, gh * gw).flatten()
            h_index = torch.arange(gh).view(1, -1, 1).expand(t, -1, gw).flatten()
            w_index = torch.arange(gw).view(1, 1, -1).expand(t, gh, -1).flatten()
            chunks.append(torch.stack([t_index, h_index, w_index]) + text_len + st_idx)
            st = ed + t * gh * gw
        if st < len(ids):
            st_idx = int(chunks[-1].max()) + 1 if chunks else 0
            chunks.append(torch.arange(len(ids) - st).view(1, -1).expand(3, -1) + st_idx)
        pos = torch.cat(chunks, dim=1) if chunks else torch.zeros(3, 0, dtype=torch.long)
        position_ids[:, b, keep] = pos
        deltas.append(int(pos.max()) + 1 - len(ids) if pos.numel() else 0)
    return position_ids, torch.tensor(deltas).unsqueeze(1)
