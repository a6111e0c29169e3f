"""Stand-alone tensor-parallel text training without the actor runtime
(reference: python/text_autotp_example.py:22-181).

    torchrun --standalone --local-addr 127.0.0.1 --nproc-per-node 2 -m multimodal_training_b200.examples.text_tp_example

Every rank builds a :class:`TextTrainer` shard of a small decoder, feeds it synthetic token batches
(no images) and runs a few AdamW steps; works on CPU (gloo, fp32) and on GPUs (nccl, bf16).
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist


def main(argv=None) -> list[float]:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="tiny")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--batch-size", type=int, default=2)
    a = ap.parse_args(argv)
    from ..config.loader import load_config, trainer_configs
    from ..trainers.text import TextTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    gpu = torch.cuda.is_available()
    cfg = load_config(None, [f"vision.model_name={a.model}", f"text.model_name={a.model}", "vision.parallelism=none",
                             "text.parallelism=" + ("tensor" if world > 1 else "none"),
                             f"training.parallel_size={world}", f"training.batch_size={a.batch_size}",
                             "text.dtype=" + ("bfloat16" if gpu else "float32"),
                             "vision.dtype=" + ("bfloat16" if gpu else "float32"),
                             "+data.synthetic.image_size=0", f"+data.synthetic.text_tokens={a.tokens}",
                             "training.warmup_ratio=0", "training.warmup_steps=0", "training.learning_rate=1e-3",
                             "training.lr_scheduler_type=constant"])
    _, tcfg = trainer_configs(cfg)
    tcfg["mesh_sp"] = 1
    trainer = TextTrainer(tcfg, int(os.environ.get("RANK", "0")))
    trainer.build_model()
    trainer.initialize_trainer()
    losses = []
    for step in range(a.steps):
        trainer.zero_grad()
        out = trainer.forward_step(None, step)
        trainer.backward_step()
        trainer.optimizer_step()
        losses.append(float(out["loss"]))
        if trainer.rank == 0:
            print(f"step {step}: loss {losses[-1]:.4f}")
    if dist.is_initialized():
        dist.barrier()
    return losses


if __name__ == "__main__":
    main()
