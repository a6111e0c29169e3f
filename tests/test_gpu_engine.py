"""Whole training steps of the small bf16 model on one GPU through the native kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(global_batch: int, accum: int, steps: int, ckpt: str):
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine
    from multimodal_training_b200.ops import native as nv
    from multimodal_training_b200.trainers.trainer import reset_process_state

    cfg = load_config(None, [
        "vision.model_name=smoke", "text.model_name=smoke", "vision.parallelism=none", "text.parallelism=none",
        f"training.batch_size={global_batch}", f"+data.synthetic.global_batch={global_batch}",
        f"training.gradient_accumulation_steps={accum}", "training.learning_rate=1e-3", "training.warmup_ratio=0",
        "training.warmup_steps=0", "training.lr_scheduler_type=constant", "training.clip_grad_norm=true",
        f"vision.activation_checkpointing={ckpt}", f"text.activation_checkpointing={ckpt}",
        "+data.synthetic.image_size=448", "+data.synthetic.text_tokens=256",
        f"+data.synthetic.repeat={accum}"])      # the same two samples in every optimizer step
    reset_process_state()
    eng = HybridEngine.from_config(cfg)
    losses = [float(eng.train_step(s)) for s in range(steps)]
    nv.raise_on_device_error()
    return losses, float(eng.last_grad_norm)


@pytest.mark.parametrize("ckpt", ["true", "false"])
def test_gradient_accumulation_matches_the_larger_batch(ckpt):
    """Micro-batches accumulate in the bf16 flat gradient through the kernels' accumulate flag: two micro-batches of
    one sample train like one batch of the same two samples, up to bf16 rounding of the accumulated gradient."""
    big, norm_big = _run(2, 1, 4, ckpt)
    acc, norm_acc = _run(1, 2, 4, ckpt)
    assert all(b == b for b in big + acc)
    assert big[-1] < big[0] and acc[-1] < acc[0]
    for a, b in zip(big, acc):
        assert abs(a - b) < 3e-2 * abs(a), (big, acc)
    assert abs(norm_big - norm_acc) < 5e-2 * norm_big, (norm_big, norm_acc)


def test_checkpointing_settings_agree():
    """Recomputing activations, keeping them, and the automatic choice give the same losses (same kernels, same
    order of operations inside a block)."""
    ref, _ = _run(2, 1, 3, "true")
    for mode in ("false", "auto"):
        got, _ = _run(2, 1, 3, mode)
        for a, b in zip(ref, got):
            assert abs(a - b) < 1e-3 * abs(a), (mode, ref, got)


def test_tensor_transfer_over_cuda_ipc(tmp_path):
    """runtime/tensor_transfer.py, "ipc" transport: a second process on the same GPU maps the producer's memory from
    the request (CUDA IPC handle + interprocess event), reads it and writes into it."""
    import os
    import pickle
    import subprocess
    import sys
    from multimodal_training_b200.runtime.tensor_transfer import prepare_tensor_for_transfer
    from multimodal_training_b200.runtime.utils import get_physical_gpu_id
    t = torch.arange(1 << 16, device="cuda", dtype=torch.float32).reshape(256, 256)
    want = float(t.double().sum())
    req = prepare_tensor_for_transfer(t, receiver_gpu_ids=[get_physical_gpu_id()], same_process=False)
    assert req.transport == "ipc"
    path = tmp_path / "req.pkl"
    pickle.dump(req.to_dict(), open(path, "wb"))
    here = os.path.dirname(os.path.abspath(__file__))
    out = subprocess.run([sys.executable, os.path.join(here, "ipc_receiver.py"), str(path), os.path.dirname(here)],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    got = float([ln for ln in out.stdout.splitlines() if ln.startswith("SUM ")][-1][4:])
    assert got == want
    torch.cuda.synchronize()
    assert float(t.double().sum()) == 2 * want            # the receiver's in-place update landed in this tensor
