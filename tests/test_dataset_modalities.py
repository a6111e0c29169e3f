"""Dataset / collators / preprocessing / M-RoPE ids with a dummy processor and annotation files in a temp dir
(modelled on the reference's tests/test_dataset_modalities.py; no Hugging Face download)."""
import json

import pytest
import torch

from multimodal_training_b200.data import (DataCollatorForSupervisedDataset, DataConfig,
                                           FlattenedDataCollatorForSupervisedDataset, VisionDataCollator,
                                           get_rope_index_for_images)
from multimodal_training_b200.data.dataset import (LazySupervisedDataset, build_dataloader, get_dataset_configs,
                                                   parse_sampling_rate)
from multimodal_training_b200.data.preprocessing import IGNORE_INDEX, build_messages, mask_labels

pytestmark = pytest.mark.cpu_only
IMG, START, ASSIST, END = 151655, 151652, 77091, 151645


class DummyProcessor:
    """Tokenises by hashing words; every image becomes vision_start + 4 placeholders (a 4x4 patch grid)."""

    class tokenizer:
        pad_token_id = 0

    def apply_chat_template(self, messages, tokenize=True, return_dict=True, return_tensors="pt", **kw):
        ids, n_img = [], 0
        for m in messages:
            ids += [100, ASSIST if m["role"] == "assistant" else 872, 198]
            for part in m["content"]:
                if part["type"] == "image":
                    ids += [START] + [IMG] * 4 + [151653]
                    n_img += 1
                else:
                    ids += [1000 + (hash(w) % 5000) for w in part["text"].split()]
            ids += [END, 198]
        out = {"input_ids": torch.tensor([ids])}
        if n_img:
            out["pixel_values"] = torch.randn(16 * n_img, 1176)
            out["image_grid_thw"] = torch.tensor([[1, 4, 4]] * n_img)
        return out


@pytest.fixture()
def data_cfg(tmp_path, monkeypatch):
    monkeypatch.setattr("multimodal_training_b200.data.preprocessing.fixed_size_resize", lambda img, mp, pm=28: img)
    ann = [{"image": f"img_{i}.jpg", "conversations": [{"from": "human", "value": f"<image>\nwhat is {i} ?"},
                                                       {"from": "gpt", "value": f"answer number {i}"}]}
           for i in range(10)]
    p = tmp_path / "ann.jsonl"
    p.write_text("\n".join(json.dumps(a) for a in ann))
    monkeypatch.setattr("PIL.Image.open", lambda path: type("I", (), {"convert": lambda self, m: str(path)})())
    return DataConfig(datasets=["toy%50", "toy"], data_registry={"toy": {"annotation_path": str(p),
                                                                        "data_path": str(tmp_path)}},
                      num_workers=0, pin_memory=False, max_pixels=3136, min_pixels=784)


def test_sampling_rate_and_registry():
    assert parse_sampling_rate("coco%25") == ("coco", 0.25) and parse_sampling_rate("coco") == ("coco", 1.0)
    with pytest.raises(KeyError):
        get_dataset_configs(["nope"], {})


def test_messages_and_label_mask():
    msgs = build_messages([{"from": "human", "value": "<image>\ndescribe"}, {"from": "gpt", "value": "a cat"}], ["x"])
    assert msgs[0]["content"][0] == {"type": "image", "image": "x"} and msgs[1]["role"] == "assistant"
    with pytest.raises(ValueError):
        build_messages([{"from": "human", "value": "<image><image>"}], ["only one"])
    ids = torch.tensor([[5, 872, 198, 9, END, 198, 5, ASSIST, 198, 41, 42, END, 198]])
    lab = mask_labels(ids)
    assert lab.tolist() == [[IGNORE_INDEX] * 9 + [41, 42, END, IGNORE_INDEX]]


def test_modalities_share_order_and_drop_the_right_keys(data_cfg):
    proc = DummyProcessor()
    sets = {m: LazySupervisedDataset(proc, data_cfg, modality=m, seed=7) for m in ("all", "image", "text")}
    assert len(sets["all"]) == 15                                     # 50% of 10 + 10
    for i in (0, 3, 14):
        a, im, tx = sets["all"][i], sets["image"][i], sets["text"][i]
        assert a["sample_index"].item() == im["sample_index"].item() == tx["sample_index"].item() == i
        assert "input_ids" not in im and "pixel_values" in im and "pixel_values" not in tx
        assert torch.equal(a["input_ids"], tx["input_ids"]) and a["position_ids"].shape[0] == 3
        assert (a["labels"][a["input_ids"] == IMG] == IGNORE_INDEX).all()
    other = LazySupervisedDataset(proc, data_cfg, modality="all", seed=8)
    assert [s["image"] for s in other.samples] != [s["image"] for s in sets["all"].samples]


def test_collators(data_cfg):
    proc = DummyProcessor()
    ds = LazySupervisedDataset(proc, data_cfg, seed=1)
    items = [ds[0], ds[1], ds[2]]
    flat = FlattenedDataCollatorForSupervisedDataset(pad_token_id=0)(items)
    lens = [i["input_ids"].shape[1] for i in items]
    assert flat["input_ids"].shape == (1, sum(lens)) and flat["position_ids"].shape == (3, 1, sum(lens))
    assert flat["attention_mask"].dtype == torch.int32 and flat["attention_mask"].tolist() == [
        0, lens[0], lens[0] + lens[1], sum(lens)]
    assert flat["pixel_values"].shape == (48, 1176) and flat["sample_index"].tolist() == [0, 1, 2]
    padded = DataCollatorForSupervisedDataset(pad_token_id=0)(items)
    assert padded["input_ids"].shape == (3, max(lens)) and padded["attention_mask"].sum().item() == sum(lens)
    vis = VisionDataCollator()([{k: v for k, v in i.items() if k in ("pixel_values", "image_grid_thw",
                                                                     "sample_index")} for i in items])
    assert vis["image_grid_thw"].shape == (3, 3)
    dl = build_dataloader(proc, data_cfg, batch_size=2, seed=1)
    batch = next(iter(dl))
    assert batch["input_ids"].shape[0] == 1 and batch["sample_index"].tolist() == [0, 1]


def test_mrope_index_for_text_image_text():
    ids = torch.tensor([[11, 12, START, IMG, IMG, IMG, IMG, 13, 14]])
    pos, delta = get_rope_index_for_images(2, ids, [(1, 4, 4)])
    assert pos.shape == (3, 1, 9)
    assert pos[:, 0, :3].tolist() == [[0, 1, 2]] * 3                   # text counts on all axes
    assert pos[0, 0, 3:7].tolist() == [3, 3, 3, 3]                     # one frame
    assert pos[1, 0, 3:7].tolist() == [3, 3, 4, 4] and pos[2, 0, 3:7].tolist() == [3, 4, 3, 4]
    assert pos[:, 0, 7:].tolist() == [[5, 6]] * 3                      # continues after the largest id
    assert delta.item() == 7 - 9


def test_broken_samples_fall_back_to_neighbours(data_cfg, monkeypatch):
    ds = LazySupervisedDataset(DummyProcessor(), data_cfg, seed=1)
    orig = ds._get_item
    monkeypatch.setattr(ds, "_get_item", lambda i: (_ for _ in ()).throw(IOError("bad")) if i == 4 else orig(i))
    assert ds[4]["sample_index"].item() == 5
    monkeypatch.setattr(ds, "_get_item", lambda i: (_ for _ in ()).throw(IOError("bad")))
    with pytest.raises(RuntimeError):
        ds[4]
