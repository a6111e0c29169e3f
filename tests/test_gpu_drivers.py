"""The public entry points on GPUs (skipped with fewer than 2): the actor driver (``train.main``: one driver process,
ActorGroup with built-in host processes, one per GPU) and the torchrun-style driver (``train_spmd.main``) train the
small bf16 model for ten steps and give the losses of ``HybridEngine.train_step`` called directly."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = os.path.join(HERE, "driver_gpu_worker.py")


def _run(cmd):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def _torchrun(mode, port):
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
            "127.0.0.1", "--master-port", str(port), WORKER, mode]


@pytest.mark.timeout(420)
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_actor_and_spmd_drivers_train_like_the_engine_on_two_gpus():
    engine = _run(_torchrun("engine", 29541))
    spmd = _run(_torchrun("spmd", 29542))
    actor = _run([sys.executable, WORKER, "actor", "2"])
    assert len(engine["losses"]) == 10 and engine["losses"][-1] < engine["losses"][0]
    for name, res in (("spmd", spmd), ("actor", actor)):
        assert len(res["losses"]) == 10, (name, res)
        for a, b in zip(res["losses"], engine["losses"]):
            assert abs(a - b) < 2e-2 * abs(b), (name, res["losses"], engine["losses"])


@pytest.mark.timeout(420)
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_non_collocated_placement_on_two_gpus():
    """``training.collocate: false`` with one actor per half: the vision encoder on GPU 0, the text decoder on GPU 1,
    rows and gradients handed over by value; the losses are those of the collocated run on one GPU."""
    base = ["+data.synthetic.global_batch=2"]
    together = _run([sys.executable, WORKER, "actor", "1"] + base)
    apart = _run([sys.executable, WORKER, "actor", "1", "training.collocate=false"] + base)
    assert len(apart["losses"]) == 10 and apart["losses"][-1] < apart["losses"][0]
    for a, b in zip(apart["losses"], together["losses"]):
        assert abs(a - b) < 2e-2 * abs(b), (apart["losses"], together["losses"])
