"""Multi-GPU checks (skipped on a single-GPU box): the fused peer-memory collectives train like the NCCL path, and so
does the tensor-parallel layout of the vision encoder."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.timeout(420)
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_collectives_match_nccl_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "multi_gpu_worker.py")]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=400)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("RESULT ")][-1]
    res = json.loads(line[len("RESULT "):])
    assert res["fused"][-1] < res["fused"][0]
    for a, b in zip(res["fused"], res["lib"]):
        assert abs(a - b) < 3e-2 * abs(b), res
    for a, b in zip(res["vision_tp"], res["lib"]):
        assert abs(a - b) < 3e-2 * abs(b), res
    # the one-node tensor-parallel layers (default) against the per-op graph on the same fused exchanges, with
    # recomputation and with kept activations
    for key in ("fused_per_op", "fused_keep", "ulysses_block", "ulysses_block_keep"):
        for a, b in zip(res[key], res["fused"]):
            assert abs(a - b) < 2e-2 * abs(b), (key, res)
    # six steps on images of three sizes and texts of three lengths (new shapes every step): the peer-memory paths,
    # whose heap regions are sized per step and grow, give the NCCL path's losses
    assert len(res["ragged_fused"]) == 6
    for a, b in zip(res["ragged_fused"], res["ragged_lib"]):
        assert abs(a - b) < 3e-2 * abs(b), res
    for a, b in zip(res["ragged_ulysses_block"], res["ragged_lib"]):
        assert abs(a - b) < 3e-2 * abs(b), res
