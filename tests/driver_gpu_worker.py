"""Worker of tests/test_gpu_drivers.py: trains the small bf16 model for ten steps on the GPUs of this box through one
of the three entry points and prints the losses (and the wall-clock step time the drivers report) as JSON.

    python driver_gpu_worker.py actor WORLD [key=value ...]   one driver process, ActorGroup with built-in hosts
    torchrun ... driver_gpu_worker.py spmd [key=value ...]     one rank per GPU (train_spmd.main)
    torchrun ... driver_gpu_worker.py engine [key=value ...]   one rank per GPU, HybridEngine.train_step called directly

``key=value`` arguments override the small default configuration (model, sizes, number of steps).
"""
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

STEPS = 10


def config(world: int, extra=()):
    from multimodal_training_b200.config.loader import load_config
    return load_config(None, [
        "vision.model_name=smoke", "text.model_name=smoke", "vision.parallelism=sequence",
        "text.parallelism=tensor", f"training.parallel_size={world}", "training.batch_size=2",
        f"training.num_iterations={STEPS}", "training.num_epochs=1", "training.warmup_steps=2",
        "training.learning_rate=1e-3", "training.warmup_ratio=0", "training.lr_scheduler_type=constant",
        "training.runtime=builtin", "training.clip_grad_norm=true", "training.no_checkpoint=true",
        "+data.synthetic.image_size=448", "+data.synthetic.text_tokens=256", "+data.synthetic.global_batch=2",
        "+data.synthetic.repeat=1", *extra])


def main():
    mode = sys.argv[1]
    if mode == "actor":
        from multimodal_training_b200 import train
        res = train.main(config(int(sys.argv[2]), sys.argv[3:]))
        print("RESULT " + json.dumps({"losses": res["losses"], "avg_step_s": res.get("avg_step_s")}))
        return
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    world = dist.get_world_size()
    if mode == "spmd":
        from multimodal_training_b200 import train_spmd
        res = train_spmd.main(config(world, sys.argv[2:]))
        out = {"losses": res["losses"], "avg_step_s": res.get("avg_step_s")}
    else:
        from multimodal_training_b200.engine import HybridEngine
        cfg = config(world, sys.argv[2:])
        eng = HybridEngine.from_config(cfg)
        out = {"losses": [eng.mean_loss(eng.train_step(0)) for _ in range(int(cfg["training"]["num_iterations"]))]}
    if dist.get_rank() == 0:
        print("RESULT " + json.dumps(out))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
