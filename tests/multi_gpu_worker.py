"""Worker of tests/test_gpu_multi.py (run under torch.distributed.run, one rank per GPU):
trains the small bf16 model for a few steps with the fused peer-memory collectives, again with the NCCL
collectives, and once more with a tensor-parallel vision encoder, each from the same initial weights, and prints
the loss series as JSON on rank 0."""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def run(fused: bool, steps: int, vision: str = "sequence", ragged: bool = False, tp_block: bool = True,
        ckpt: str = "true", ul_block: bool = False):
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine
    from multimodal_training_b200.ops import native as nv
    from multimodal_training_b200.trainers.trainer import process_state, reset_process_state

    world = dist.get_world_size()
    cfg = load_config(None, [
        "vision.model_name=smoke", "text.model_name=smoke", f"vision.parallelism={vision}", "text.parallelism=tensor",
        f"training.parallel_size={world}", f"text.tensor_parallel_size={min(world, 2)}", "training.batch_size=2",
        "training.learning_rate=1e-3", "training.warmup_ratio=0", "training.warmup_steps=0",
        "training.lr_scheduler_type=constant", "+data.synthetic.image_size=448", "+data.synthetic.text_tokens=256",
        f"+data.synthetic.global_batch={2 * (world // min(world, 2))}", "+data.synthetic.repeat=1",
        f"training.fused_comm={'true' if fused else 'false'}", f"+training.tp_block={'true' if tp_block else 'false'}",
        f"vision.activation_checkpointing={ckpt}", f"text.activation_checkpointing={ckpt}"]
        # images of three sizes and texts of three lengths, new ones every step: ragged sequence-parallel splits
        # (81 and 225 merged tokens do not divide by 2) and heap regions that have to grow after the first step
        + (["+data.synthetic.image_sizes=252,448,420", "+data.synthetic.text_token_choices=96,256,40",
            "+data.synthetic.repeat=0"] if ragged else []))
    reset_process_state()
    os.environ["MMT_ULYSSES_BLOCK"] = "1" if ul_block else "0"
    eng = HybridEngine.from_config(cfg)
    assert (process_state().fused is not None) == fused
    losses = []
    for s in range(steps):
        losses.append(eng.mean_loss(eng.train_step(s if ragged else 0)))
        nv.raise_on_device_error()        # fail at the first step whose exchanges gave up, not after crawling through all
    if fused and ragged:
        heap = process_state().fused.ctx.heap
        assert heap.regions.version == heap.verified_version     # every layout change was compared across ranks
    nv.raise_on_device_error()
    return losses


def main():
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    fused = run(True, 4)
    lib = run(False, 4)
    vtp = run(False, 4, vision="tensor")          # tensor-parallel vision encoder (all-reduce per block)
    per_op = run(True, 4, tp_block=False)         # fused exchanges through the per-op autograd graph
    keep = run(True, 4, ckpt="false")             # one-node layers that keep their activations
    ul = run(True, 4, ul_block=True)                # full-attention layers as one node, exchanges inside the GEMMs
    ul_keep = run(True, 4, ul_block=True, ckpt="false")
    rag_ul = run(True, 6, ragged=True, ul_block=True)
    rag_fused = run(True, 6, ragged=True)
    rag_lib = run(False, 6, ragged=True)
    if dist.get_rank() == 0:
        print("RESULT " + json.dumps({"fused": fused, "lib": lib, "vision_tp": vtp, "fused_per_op": per_op, "fused_keep": keep, "ulysses_block": ul, "ulysses_block_keep": ul_keep, "ragged_ulysses_block": rag_ul,
                                      "ragged_fused": rag_fused,
                                      "ragged_lib": rag_lib}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
