"""Generate the configs and the runner script of the throughput sweep.

    python experiments/generate_configs.py --output-dir experiments/generated [--synthetic]

The sweep is the reference's (experiments/generate_configs.py:24-68,205-231 there): two models
(7B with parallel size 4, 32B with parallel size 8) x six image sizes (1k ... 64k vision patches) x
vision parallelism {sequence, tensor} x batch size {1, 2, 4, 8}.  Every YAML follows
``configs/sample.yaml``; ``manifest.txt`` lists them; ``run_sweep.sh`` runs each config, greps the
``Training completed! ... (avg X s/step)`` line and continues past failures.
"""
from __future__ import annotations

import argparse
import os
from pathlib import Path

import yaml

MODELS = {"7b": {"name": "Qwen/Qwen2.5-VL-7B-Instruct", "parallel_size": 4},
          "32b": {"name": "Qwen/Qwen2.5-VL-32B-Instruct", "parallel_size": 8}}
# label -> image side in pixels (patches = (side/14)^2; sides keep the number of windows a multiple of 8)
TOKEN_SIZES = {"1k_tokens": 448, "4k_tokens": 896, "9k_tokens": 1344, "16k_tokens": 1792, "25k_tokens": 2240,
               "64k_tokens": 3584}
VISION_PARALLELISM = ("sequence", "tensor")
BATCH_SIZES = (1, 2, 4, 8)
NUM_ITERATIONS, WARMUP_STEPS = 20, 10


def make_config(model: str, size: str, vision_par: str, batch_size: int, data: dict, synthetic: bool) -> dict:
    side = TOKEN_SIZES[size]
    max_pixels = side * side
    m = MODELS[model]
    cfg = {
        "debug": False,
        "vision": {"model_type": "qwen2_5_vl", "model_name": m["name"], "parallelism": vision_par,
                   "dtype": "bfloat16", "attention_backend": "sm100", "activation_checkpointing": True,
                   "autocast": True, "zero_stage": 1},
        "text": {"model_type": "qwen2_5_vl", "model_name": m["name"], "parallelism": "tensor", "dtype": "bfloat16",
                 "attention_backend": "sm100", "activation_checkpointing": True, "autocast": True, "zero_stage": 1},
        "training": {"batch_size": batch_size, "learning_rate": 5e-5, "num_epochs": 1,
                     "num_iterations": NUM_ITERATIONS, "warmup_steps": WARMUP_STEPS, "warmup_ratio": 0.03,
                     "lr_scheduler_type": "cosine", "weight_decay": 0.01, "gradient_accumulation_steps": 1,
                     "seed": 42, "parallel_size": m["parallel_size"], "dp_size": 1, "collocate": True,
                     "clip_grad_norm": False, "max_grad_norm": 1.0, "no_checkpoint": True,
                     "checkpoint_dir": "/tmp/checkpoints", "log_interval": 1},
        "data": dict(data, min_pixels=max_pixels, max_pixels=max_pixels, force_fixed_size=True, num_workers=4,
                     pin_memory=True, data_flatten=True),
        "deepspeed": {"reduce_bucket_size": 100000000 if max_pixels > 2_000_000 else 500000000},
    }
    if synthetic:
        cfg["data"]["synthetic"] = {"image_size": side, "text_tokens": 512}
    return cfg


RUNNER = """#!/usr/bin/env bash
# Runs every config of manifest.txt; one line per config in results.txt.
set -u
cd "$(dirname "$0")"
HERE="$PWD"
REPO="${MMT_REPO:-__REPO__}"      # where the package lives (override with MMT_REPO)
: > results.txt
while read -r name; do
  [ -z "$name" ] && continue
  log="logs/${name}.log"
  mkdir -p logs
  echo "=== $name"
  if (cd "$REPO" && __LAUNCH__ --config-path "$HERE/configs" --config-name "$name") > "$log" 2>&1; then
    line=$(grep -E "Training completed!.*avg [0-9.]+s/step" "$log" | tail -1)
    avg=$(echo "$line" | sed -E 's/.*avg ([0-9.]+)s\\/step.*/\\1/')
    echo "$name OK Average iteration time: ${avg}s" | tee -a results.txt
  else
    if grep -qi "out of memory" "$log"; then echo "$name OOM" | tee -a results.txt; else echo "$name FAILED" | tee -a results.txt; fi
  fi
done < manifest.txt
"""


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--output-dir", default=str(Path(__file__).parent / "generated"))
    ap.add_argument("--mscoco-data-path", default="/path/to/mscoco2017")
    ap.add_argument("--laion-data-path", default="/path/to/laion_pop")
    ap.add_argument("--synthetic", action="store_true", help="random data, no dataset files needed")
    ap.add_argument("--launcher", default="actors", choices=["actors", "torchrun"],
                    help="actors: the driver spawns one host process per GPU itself; torchrun: one rank per GPU "
                         "launched by torch.distributed.run (multimodal_training_b200.train_spmd)")
    a = ap.parse_args(argv)
    out = Path(a.output_dir)
    (out / "configs").mkdir(parents=True, exist_ok=True)
    data = {"datasets": ["laion_pop_train"],
            "data_registry": {
                "mscoco2017_train_captions": {"annotation_path": f"{a.mscoco_data_path}/annotations/coco2017_train.json",
                                              "data_path": a.mscoco_data_path},
                "laion_pop_train": {"annotation_path": f"{a.laion_data_path}/laion_pop_train.jsonl",
                                    "data_path": f"{a.laion_data_path}/images"}}}
    names = []
    for model in MODELS:
        for size in TOKEN_SIZES:
            for vp in VISION_PARALLELISM:
                for bs in BATCH_SIZES:
                    name = f"{model}_{size}_{vp}_bs{bs}"
                    with open(out / "configs" / f"{name}.yaml", "w") as f:
                        yaml.safe_dump(make_config(model, size, vp, bs, data, a.synthetic), f, sort_keys=False)
                    names.append(name)
    (out / "manifest.txt").write_text("\n".join(names) + "\n")
    runner = out / "run_sweep.sh"
    if a.launcher == "torchrun":
        # one rank per GPU of the config's own layout (parallel_size x dp_size)
        launch = ("python -m torch.distributed.run --nnodes=1 --nproc-per-node \"$(python -c \"import yaml; "
                  "t = yaml.safe_load(open('$HERE/configs/$name.yaml'))['training']; "
                  "print(t['parallel_size'] * t.get('dp_size', 1))\")\" --master-addr 127.0.0.1 "
                  "-m multimodal_training_b200.train_spmd")
    else:
        launch = "python -m multimodal_training_b200.train"
    repo = str(Path(__file__).resolve().parent.parent)
    runner.write_text(RUNNER.replace("__LAUNCH__", launch).replace("__REPO__", repo))
    os.chmod(runner, 0o755)
    print(f"wrote {len(names)} configs to {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
