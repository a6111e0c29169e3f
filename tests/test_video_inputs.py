"""Video inputs of the single-process wrappers: the in-tree processor cuts a clip into temporal patches, the M-RoPE
index advances the temporal axis per temporal patch, and the vision encoder attends inside one temporal patch at a
time (the model-side rules of the reference, python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:944-952,1561-1741)."""
import numpy as np
import torch

from multimodal_training_b200.config.model_configs import get_model_config
from multimodal_training_b200.data.processor import ByteTokenizer, Qwen2_5_VLImageProcessor, Qwen2_5_VLProcessor
from multimodal_training_b200.data.rope_utils import get_rope_index, get_rope_index_for_images
from multimodal_training_b200.models.vlm import Qwen2_5_VLForConditionalGeneration


def _processor(cfg):
    return Qwen2_5_VLProcessor(Qwen2_5_VLImageProcessor(min_pixels=28 * 28, max_pixels=112 * 112),
                               ByteTokenizer.for_config(cfg))


def test_clip_becomes_temporal_patches_and_placeholders():
    cfg = get_model_config("tiny")
    proc = _processor(cfg)
    rng = np.random.default_rng(0)
    clip = rng.integers(0, 255, size=(5, 56, 84, 3), dtype=np.uint8)          # 5 frames -> 3 temporal patches
    msgs = [{"role": "user", "content": [{"type": "video", "video": clip}, {"type": "text", "text": "what moves?"}]}]
    enc = proc.apply_chat_template(msgs, return_tensors="pt")
    assert enc["video_grid_thw"].tolist() == [[3, 4, 6]]
    assert enc["pixel_values_videos"].shape == (3 * 4 * 6, 3 * 2 * 14 * 14)
    assert enc["second_per_grid_ts"] == [1.0]
    assert int((enc["input_ids"] == cfg.video_token_id).sum()) == 3 * 4 * 6 // 4
    # the last frame is repeated to fill the last temporal patch: its two frame slots hold the same pixels
    last = enc["pixel_values_videos"][2 * 24:].reshape(24, 3, 2, 14, 14)
    assert torch.equal(last[:, :, 0], last[:, :, 1])


def test_rope_index_counts_time_per_temporal_patch():
    # text(3) <vs> video(t=2, 2x2 merged) text(2): 4 merged tokens per temporal patch, 2 s per patch at 2 tokens/s
    VS, VID, IMG = 1002, 1001, 1000
    ids = torch.tensor([[5, 6, 7, VS] + [VID] * 8 + [9, 10]])
    pos, delta = get_rope_index(2, ids, [], [(2, 4, 4)], [2.0], image_token_id=IMG, video_token_id=VID,
                                vision_start_token_id=VS, tokens_per_second=2.0)
    t, h, w = pos[0, 0].tolist(), pos[1, 0].tolist(), pos[2, 0].tolist()
    assert t[:4] == h[:4] == w[:4] == [0, 1, 2, 3]
    assert t[4:12] == [4] * 4 + [8] * 4                     # second temporal patch: 2 s * 2 tokens/s further
    assert h[4:12] == [4, 4, 5, 5] * 2 and w[4:12] == [4, 5, 4, 5] * 2
    assert t[12:] == h[12:] == w[12:] == [9, 10]            # text continues after the largest id used
    assert delta.tolist() == [[11 - 14]]
    # an image is a clip with one temporal patch: both builders agree
    ids_img = torch.tensor([[5, VS] + [IMG] * 4 + [9]])
    a, _ = get_rope_index(2, ids_img, [(1, 4, 4)], [], [], image_token_id=IMG, video_token_id=VID,
                          vision_start_token_id=VS)
    b, _ = get_rope_index_for_images(2, ids_img, [(1, 4, 4)], image_token_id=IMG, vision_start_token_id=VS)
    assert torch.equal(a, b)


def test_video_attention_stays_inside_a_temporal_patch_and_the_wrapper_trains_on_it():
    cfg = get_model_config("tiny")
    torch.manual_seed(0)
    model = Qwen2_5_VLForConditionalGeneration(cfg)
    proc = _processor(cfg)
    clip = np.random.default_rng(1).integers(0, 255, size=(4, 56, 56, 3), dtype=np.uint8)
    enc = proc.apply_chat_template(
        [{"role": "user", "content": [{"type": "video", "video": clip}, {"type": "text", "text": "describe"}]},
         {"role": "assistant", "content": [{"type": "text", "text": "two patches"}]}], return_tensors="pt")
    vid, grid = enc["pixel_values_videos"], enc["video_grid_thw"].tolist()
    assert grid == [[2, 4, 4]]
    # the clip's tokens equal those of its temporal patches encoded as two separate stills
    whole = model.model.encode_images(vid, grid)
    parts = torch.cat([model.model.encode_images(vid[:16], [(1, 4, 4)]), model.model.encode_images(vid[16:], [(1, 4, 4)])])
    assert torch.allclose(whole, parts, atol=1e-5)
    out = model(enc["input_ids"], labels=enc["input_ids"].clone(), pixel_values_videos=vid, video_grid_thw=grid,
                second_per_grid_ts=enc["second_per_grid_ts"])
    assert torch.isfinite(out["loss"])
    out["loss"].backward()
    assert model.model.visual.patch_embed_w.grad.abs().sum() > 0


def test_collators_carry_video_clips():
    """The collators concatenate clips and their grids like images (python/data/collator.py:51-71)."""
    import torch
    from multimodal_training_b200.data.collator import (DataCollatorForSupervisedDataset,
                                                        FlattenedDataCollatorForSupervisedDataset, VisionDataCollator)

    def inst(i, with_video):
        d = {"input_ids": torch.arange(4 + i)[None], "labels": torch.arange(4 + i)[None],
             "position_ids": torch.zeros(3, 1, 4 + i, dtype=torch.long), "sample_index": torch.tensor([i])}
        if with_video:
            d["pixel_values_videos"] = torch.full((8, 6), float(i))
            d["video_grid_thw"] = torch.tensor([[2, 2, 2]])
        return d
    batch = [inst(0, True), inst(1, False), inst(2, True)]
    for coll in (DataCollatorForSupervisedDataset(), FlattenedDataCollatorForSupervisedDataset(), VisionDataCollator()):
        out = coll(batch)
        assert out["pixel_values_videos"].shape == (16, 6) and out["video_grid_thw"].tolist() == [[2, 2, 2], [2, 2, 2]]
        assert out["pixel_values"] is None and out["image_grid_thw"] is None
    assert VisionDataCollator()([inst(1, False)])["pixel_values_videos"] is None
