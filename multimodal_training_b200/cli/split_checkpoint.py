"""Split a full Qwen2.5-VL checkpoint into the vision and text halves that the trainers load.

    python -m multimodal_training_b200.cli.split_checkpoint --model-name <dir-or-state-dict> --output-dir out

Writes ``vision_model.pt`` and ``text_model.pt`` (``{"model": state_dict, "config": ...}``), ``config.json`` and
``split_metadata.json``: the layout consumed through ``pretrained_checkpoint_dir`` (reference:
scripts/split_checkpoint.py:28-185).  Key routing: ``model.visual.*`` / ``visual.*`` -> vision (prefix removed);
``model.language_model.*`` / ``language_model.*`` / ``model.*`` -> text; ``lm_head.*`` stays with the text half.
The source is a local directory with ``pytorch_model.bin`` / ``*.safetensors`` / ``model.pt`` or a single
state-dict file; nothing is downloaded.
"""
from __future__ import annotations

import argparse
import glob
import json
import logging
import os

import torch

from ..config.model_configs import get_model_config

log = logging.getLogger("mmt_b200.split")


def route_key(key: str) -> tuple[str, str]:
    """``(half, new_key)`` with half in {"vision", "text"}."""
    for pre in ("model.visual.", "visual."):
        if key.startswith(pre):
            return "vision", key[len(pre):]
    for pre in ("model.language_model.", "language_model."):
        if key.startswith(pre):
            return "text", key[len(pre):]
    if key.startswith("lm_head."):
        return "text", key
    if key.startswith("model."):
        return "text", key[len("model."):]
    return "text", key


def split_state_dict(sd: dict) -> tuple[dict, dict]:
    vision, text = {}, {}
    for k, v in sd.items():
        half, nk = route_key(k)
        (vision if half == "vision" else text)[nk] = v
    return vision, text


def load_full_state_dict(src: str) -> dict:
    if os.path.isfile(src):
        obj = torch.load(src, map_location="cpu", weights_only=False)
        return obj.get("model", obj) if isinstance(obj, dict) and "model" in obj and isinstance(obj["model"], dict) \
            else obj
    sd = {}
    st = sorted(glob.glob(os.path.join(src, "*.safetensors")))
    if st:
        from safetensors.torch import load_file
        for f in st:
            sd.update(load_file(f))
        return sd
    for name in ("pytorch_model.bin", "model.pt"):
        p = os.path.join(src, name)
        if os.path.exists(p):
            return torch.load(p, map_location="cpu", weights_only=False)
    raise FileNotFoundError(f"no weights found under {src}")


def split_checkpoint(model_name: str, output_dir: str) -> str:
    sd = load_full_state_dict(model_name)
    vision, text = split_state_dict(sd)
    try:
        cfg = get_model_config(model_name).to_dict()
    except KeyError:
        cfg = {"name": model_name}
    os.makedirs(output_dir, exist_ok=True)
    torch.save({"model": vision, "config": cfg.get("vision", {})}, os.path.join(output_dir, "vision_model.pt"))
    torch.save({"model": text, "config": cfg.get("text", {})}, os.path.join(output_dir, "text_model.pt"))
    with open(os.path.join(output_dir, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    with open(os.path.join(output_dir, "split_metadata.json"), "w") as f:
        json.dump({"source": model_name, "vision_tensors": len(vision), "text_tensors": len(text)}, f, indent=2)
    log.info("vision: %d tensors, text: %d tensors -> %s", len(vision), len(text), output_dir)
    return output_dir


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model-name", required=True)
    ap.add_argument("--output-dir", required=True)
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO)
    split_checkpoint(a.model_name, a.output_dir)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
