"""Run a function as N gloo ranks (child processes on CPU) and collect what each returns."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, out_dir):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "CUDA_VISIBLE_DEVICES": ""})
    torch.set_num_threads(1)
    try:
        import torch.distributed as dist
        dist.init_process_group("gloo", rank=rank, world_size=world)
        res = fn(rank, world, *args)
        torch.save({"ok": True, "result": res}, os.path.join(out_dir, f"rank_{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
    except BaseException:
        torch.save({"ok": False, "error": traceback.format_exc()}, os.path.join(out_dir, f"rank_{rank}.pt"))
        raise


def run_ranks(fn, world: int, tmp_path, *args, timeout: float = 240.0):
    """``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the list of results (raises on failure)."""
    port = free_port()
    out_dir = str(tmp_path)
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, out_dir)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.terminate()
    results = []
    for r in range(world):
        path = os.path.join(out_dir, f"rank_{r}.pt")
        if not os.path.exists(path):
            raise RuntimeError(f"rank {r} produced no result (timed out: {bool(alive)})")
        d = torch.load(path, weights_only=False)
        if not d["ok"]:
            raise RuntimeError(f"rank {r} failed:\n{d['error']}")
        results.append(d["result"])
    return results
