"""In-tree Qwen2.5-VL processor (data/processor.py): resize rule, patch layout, placeholder expansion, chat template."""
import numpy as np
import pytest
import torch

from multimodal_training_b200.data.processor import (ByteTokenizer, Qwen2_5_VLImageProcessor, Qwen2_5_VLProcessor,
                                                     smart_resize)


def test_smart_resize_rounds_to_28_and_respects_pixel_bounds():
    assert smart_resize(896, 896) == (896, 896)
    assert smart_resize(900, 1000) == (896, 1008)
    h, w = smart_resize(4000, 3000, max_pixels=802816)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 802816 and abs(h / w - 4 / 3) < 0.05
    h, w = smart_resize(20, 30, min_pixels=56 * 56)
    assert h * w >= 56 * 56
    with pytest.raises(ValueError):
        smart_resize(10, 5000)


def test_patch_rows_are_merge_block_major_and_normalised():
    ip = Qwen2_5_VLImageProcessor()
    img = (np.random.RandomState(0).rand(56, 84, 3) * 255).astype(np.uint8)
    out = ip([img])
    assert out["image_grid_thw"].tolist() == [[1, 4, 6]]
    pv = out["pixel_values"]
    assert pv.shape == (24, 3 * 2 * 14 * 14)
    x = (torch.from_numpy(img).permute(2, 0, 1).float() / 255.0 - ip.mean) / ip.std
    # row 0..3 = the 2x2 merge block at the top-left: patches (0,0), (0,1), (1,0), (1,1)
    for row, (py, px) in enumerate([(0, 0), (0, 1), (1, 0), (1, 1)]):
        patch = x[:, py * 14:(py + 1) * 14, px * 14:(px + 1) * 14]
        got = pv[row].view(3, 2, 14, 14)
        assert torch.allclose(got[:, 0], patch, atol=1e-6) and torch.allclose(got[:, 1], patch, atol=1e-6)
    # row 4 starts the next block to the right: patch (0, 2)
    assert torch.allclose(pv[4].view(3, 2, 14, 14)[:, 0], x[:, 0:14, 28:42], atol=1e-6)


def test_placeholders_expand_to_merged_token_count_and_counts_must_match():
    proc = Qwen2_5_VLProcessor()
    img = np.zeros((112, 112, 3), dtype=np.uint8)
    enc = proc(text=["a<|vision_start|><|image_pad|><|vision_end|>b"], images=[img], return_tensors="pt")
    ids = enc["input_ids"][0]
    assert int((ids == ByteTokenizer.SPECIAL["<|image_pad|>"]).sum()) == (112 // 14) ** 2 // 4
    with pytest.raises(ValueError):
        proc(text=["no placeholder"], images=[img])
    with pytest.raises(ValueError):
        proc(text=["<|image_pad|><|image_pad|>"], images=[img])


def test_llava_sample_through_chat_template_masks_everything_but_the_answer():
    proc = Qwen2_5_VLProcessor()
    img = (np.random.RandomState(1).rand(64, 64, 3) * 255).astype(np.uint8)
    sample = {"conversations": [{"from": "human", "value": "<image>\nWhat is this?"},
                                {"from": "gpt", "value": "A test."}]}
    import multimodal_training_b200.data.preprocessing as pp
    msgs = pp.build_messages(sample["conversations"], [img])
    enc = proc.apply_chat_template(msgs, tokenize=True, return_dict=True, return_tensors="pt")
    ids = enc["input_ids"]
    labels = pp.mask_labels(ids)
    tok = proc.tokenizer
    kept = labels[0][labels[0] != -100].tolist()
    assert tok.decode(kept).startswith("\nA test.") or tok.decode(kept).startswith("A test.")
    assert int((labels[0] != -100).sum()) < ids.shape[1] // 2
    assert enc["pixel_values"].shape[0] == int(enc["image_grid_thw"].prod())


def test_an_undecoded_video_file_is_refused_not_dropped():
    """Clips are accepted as decoded frames (tests/test_video_inputs.py); a path to a container file is refused with
    a message instead of being dropped from the prompt."""
    import pytest
    from multimodal_training_b200.data.processor import Qwen2_5_VLProcessor
    with pytest.raises(NotImplementedError, match="decoded frames"):
        Qwen2_5_VLProcessor().apply_chat_template([{"role": "user", "content": [{"type": "video", "video": "clip.mp4"},
                                                                                {"type": "text", "text": "What happens?"}]}])
