"""Hybrid-parallel training equals single-process training (tiny VLM, fp32, CPU/gloo).

Vision sequence parallel (ragged, window aligned, Ulysses exchange in the full-attention layer) +
ZeRO-1, text tensor parallel with sequence-parallel activations, vocab-parallel embedding and
cross-entropy, the vision->text row handoff and real data-parallel sharding are compared against one
process on the same global batch: losses of 3 AdamW steps and the FULL gradient of every parameter
at step 0 (the reference's own parity tests compare two LayerNorm vectors and print,
tests/test_vision_sp.py:350-417, tests/test_text_autotp.py in the reference).
"""
import pytest
import torch

from dist_utils import run_ranks

OV = ["vision.model_name=tiny", "text.model_name=tiny", "vision.dtype=float32", "text.dtype=float32",
      "training.learning_rate=1e-4", "training.warmup_ratio=0", "training.warmup_steps=0",
      "training.lr_scheduler_type=constant", "training.weight_decay=0.01", "+training.device=cpu",
      "+data.synthetic.image_size=224", "+data.synthetic.text_tokens=64", "+data.synthetic.global_batch=2",
      "vision.activation_checkpointing=true", "text.activation_checkpointing=true"]


def _grads_reference_layout(model):
    saved = [(p, p.data) for p in model.parameters()]
    try:
        for p, _ in saved:
            p.data = p.grad if p.grad is not None else torch.zeros_like(p.data)
        return {k: v.clone() for k, v in model.reference_state_dict().items()}
    finally:
        for p, d in saved:
            p.data = d


def _worker(rank, world, sp, tp, steps, model="tiny"):
    import torch.distributed as dist
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine

    ov = [o.replace("model_name=tiny", f"model_name={model}") for o in OV] + ["vision.parallelism=" + ("sequence" if sp > 1 else "none"),
               "text.parallelism=" + ("tensor" if tp > 1 else "none"), f"text.tensor_parallel_size={tp}",
               f"training.parallel_size={world}", f"training.batch_size={2 // (world // tp)}"]
    cfg = load_config(None, ov)
    # mesh factors: sp ranks share images, tp ranks share a text replica
    eng = HybridEngine.from_config(cfg) if (sp == world or world == 1) else None
    if eng is None:
        from multimodal_training_b200.config.loader import trainer_configs
        v, t = trainer_configs(cfg)
        v["mesh_sp"] = t["mesh_sp"] = sp
        eng = HybridEngine(v, t)
    m = eng.mesh
    # ---- step-0 gradients
    eng.vision.zero_grad()
    eng.text.zero_grad()
    vo = eng.vision.forward_step(0)
    to = eng.text.forward_step(vo, 0)
    g = eng.text.backward_step()
    eng.vision.backward_step(g)
    # vision: sum over all ranks (they split tokens or samples); the data-parallel mean is the divisor
    fg = eng.vision.optimizer.flat_grad
    if world > 1:
        dist.all_reduce(fg)
    fg /= eng.vision.optimizer.grad_divisor
    vgrads = _grads_reference_layout(eng.vision.model)
    # text: partial sums of sequence-parallel params over tp, then mean over data-parallel replicas
    to_ = eng.text.optimizer
    to_._finish_grads()
    if m.tp > 1 and to_.partial_end > to_.partial_start:
        dist.all_reduce(to_.flat_grad[to_.partial_start:to_.partial_end], group=m.tp_group)
    if m.tdp > 1:
        dist.all_reduce(to_.flat_grad, group=m.tdp_group)
        to_.flat_grad /= m.tdp
    tgrads = _grads_reference_layout(eng.text.model)
    loss0 = eng.mean_loss(to["loss"])
    # ---- three optimisation steps from the same start
    losses = []
    for s in range(steps):
        losses.append(eng.mean_loss(eng.train_step(s)))
    return {"loss0": loss0, "losses": losses, "vgrads": vgrads, "tgrads": tgrads, "tp_rank": m.tp_rank,
            "tdp_rank": m.tdp_rank}


def _merge_text(results, tp):
    from multimodal_training_b200.cli.merge_checkpoint import merge_state_dicts
    shards = [r["tgrads"] for r in results if r["tdp_rank"] == 0]
    shards.sort(key=lambda _: 0)
    by_rank = sorted([r for r in results if r["tdp_rank"] == 0], key=lambda r: r["tp_rank"])
    return merge_state_dicts([r["tgrads"] for r in by_rank]) if tp > 1 else by_rank[0]["tgrads"]


def _compare(single, multi, tp):
    assert abs(single["loss0"] - multi[0]["loss0"]) < 2e-5 * abs(single["loss0"])
    for a, b in zip(single["losses"], multi[0]["losses"]):
        assert abs(a - b) < 5e-5 * abs(a), (single["losses"], multi[0]["losses"])
    worst = 0.0
    for k, ref in single["vgrads"].items():
        got = multi[0]["vgrads"][k]
        err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-12)
        worst = max(worst, err)
        assert err < 2e-4, ("vision", k, err)
    merged = _merge_text(multi, tp)
    for k, ref in single["tgrads"].items():
        got = merged[k]
        assert got.shape == ref.shape, (k, got.shape, ref.shape)
        err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-12)
        worst = max(worst, err)
        assert err < 2e-4, ("text", k, err)
    return worst


@pytest.fixture(scope="module")
def single(tmp_path_factory):
    return run_ranks(_worker, 1, tmp_path_factory.mktemp("single"), 1, 1, 3)[0]


@pytest.mark.integration
def test_sp2_tp2_matches_single_process(single, tmp_path):
    multi = run_ranks(_worker, 2, tmp_path, 2, 2, 3)
    _compare(single, multi, tp=2)


@pytest.mark.integration
def test_sp2_with_text_data_parallel_matches_single_process(single, tmp_path):
    # vision SP=2 over both ranks, text TP=1 x DP=2: each text replica gets one of the two samples
    multi = run_ranks(_worker, 2, tmp_path, 2, 1, 3)
    _compare(single, multi, tp=1)


@pytest.mark.integration
def test_sp4_tp2_dp2_matches_single_process(single, tmp_path):
    multi = run_ranks(_worker, 4, tmp_path, 4, 2, 3)
    _compare(single, multi, tp=2)


def _accum_worker(rank, world, global_batch, accum, steps):
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine

    ov = [o for o in OV if "global_batch" not in o] + [
        f"+data.synthetic.global_batch={global_batch}", f"training.batch_size={global_batch}",
        f"training.gradient_accumulation_steps={accum}", "vision.parallelism=none", "text.parallelism=none",
        "training.parallel_size=1", "training.clip_grad_norm=true", "training.max_grad_norm=0.5"]
    eng = HybridEngine.from_config(load_config(None, ov))
    losses = [float(eng.train_step(s)) for s in range(steps)]
    return {"losses": losses, "norm": float(eng.last_grad_norm),
            "vision": eng.vision.optimizer.flat_param.clone(), "text": eng.text.optimizer.flat_param.clone()}


@pytest.mark.integration
def test_gradient_accumulation_equals_the_larger_batch(tmp_path):
    """Two micro-batches of one sample per optimizer step train exactly like one batch of the same two samples
    (every synthetic sample has the same number of supervised tokens, so the mean of means is the mean)."""
    (tmp_path / "a").mkdir()
    (tmp_path / "b").mkdir()
    big = run_ranks(_accum_worker, 1, tmp_path / "a", 2, 1, 3)[0]
    acc = run_ranks(_accum_worker, 1, tmp_path / "b", 1, 2, 3)[0]
    for a, b in zip(big["losses"], acc["losses"]):
        assert abs(a - b) < 5e-5 * abs(a), (big["losses"], acc["losses"])
    assert abs(big["norm"] - acc["norm"]) < 1e-4 * big["norm"]
    for k in ("vision", "text"):
        assert torch.allclose(big[k], acc[k], rtol=0, atol=2e-6), k


def _vision_tp_worker(rank, world, steps, tp=None):
    """Vision tensor parallel over all ranks (replicated activations, all-reduce), text tensor parallel."""
    import torch.distributed as dist
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine

    tp = tp or world
    ov = OV + ["vision.parallelism=tensor", "text.parallelism=tensor", f"text.tensor_parallel_size={tp}",
               f"training.parallel_size={tp}", f"training.dp_size={world // tp}",
               f"training.batch_size={2 // (world // tp)}"]
    eng = HybridEngine.from_config(load_config(None, ov))
    assert eng.vision.tensor_parallel and eng.vision.model.tp.size == tp
    eng.vision.zero_grad()
    eng.text.zero_grad()
    vo = eng.vision.forward_step(0)
    to = eng.text.forward_step(vo, 0)
    g = eng.text.backward_step()
    eng.vision.backward_step(g)
    eng.vision.optimizer._finish_grads()
    vgrads = _grads_reference_layout(eng.vision.model)
    loss0 = eng.mean_loss(to["loss"])
    losses = [eng.mean_loss(eng.train_step(s)) for s in range(steps)]
    # clipping path: the norm counts replicated parameters once
    eng.clip, eng.max_norm = True, 1e9
    eng.train_step(steps)
    return {"loss0": loss0, "losses": losses, "vgrads": vgrads, "norm": float(eng.last_grad_norm),
            "weights": eng.vision.model.reference_state_dict(), "rank": rank, "tp_rank": eng.mesh.sp_rank}


def _single_norm_worker(rank, world, steps):
    from multimodal_training_b200.config.loader import load_config
    from multimodal_training_b200.engine import HybridEngine
    ov = OV + ["vision.parallelism=none", "text.parallelism=none", "training.parallel_size=1",
               "training.batch_size=2"]
    eng = HybridEngine.from_config(load_config(None, ov))
    for s in range(steps):
        eng.train_step(s)
    eng.clip, eng.max_norm = True, 1e9
    eng.train_step(steps)
    return {"norm": float(eng.last_grad_norm), "weights": eng.vision.model.reference_state_dict()}


@pytest.mark.integration
def test_vision_tensor_parallel_matches_single_process(single, tmp_path):
    from multimodal_training_b200.cli.merge_checkpoint import merge_state_dicts
    (tmp_path / "tp").mkdir()
    (tmp_path / "one").mkdir()
    multi = sorted(run_ranks(_vision_tp_worker, 2, tmp_path / "tp", 3), key=lambda r: r["rank"])
    assert abs(single["loss0"] - multi[0]["loss0"]) < 2e-5 * abs(single["loss0"])
    for a, b in zip(single["losses"], multi[0]["losses"]):
        assert abs(a - b) < 5e-5 * abs(a), (single["losses"], multi[0]["losses"])
    merged = merge_state_dicts([r["vgrads"] for r in multi])
    for k, ref in single["vgrads"].items():
        got = merged[k]
        assert got.shape == ref.shape, (k, got.shape, ref.shape)
        err = (got - ref).abs().max().item() / (ref.abs().max().item() + 1e-12)
        assert err < 2e-4, ("vision", k, err)
    one = run_ranks(_single_norm_worker, 1, tmp_path / "one", 3)[0]
    assert abs(one["norm"] - multi[0]["norm"]) < 1e-4 * one["norm"], (one["norm"], multi[0]["norm"])
    weights = merge_state_dicts([r["weights"] for r in multi])
    for k, ref in one["weights"].items():
        assert weights[k].shape == ref.shape, k
        # Adam's early updates are +-lr whatever the gradient's size, so elements whose gradient is rounding noise
        # may move differently; everything else must agree closely
        diff = (weights[k] - ref).abs()
        assert diff.max().item() <= 4 * 2e-4 + 1e-6, (k, diff.max().item())
        assert (diff > 1e-5).float().mean().item() < 0.02, (k, (diff > 1e-5).float().mean().item())


@pytest.mark.integration
def test_vision_tensor_parallel_with_data_parallel(single, tmp_path):
    """Vision and text tensor parallel of size 2, two data-parallel replicas with one sample each."""
    multi = run_ranks(_vision_tp_worker, 4, tmp_path, 3, 2)
    for a, b in zip(single["losses"], multi[0]["losses"]):
        assert abs(a - b) < 5e-5 * abs(a), (single["losses"], multi[0]["losses"])
    for r in multi[1:]:
        assert abs(r["norm"] - multi[0]["norm"]) < 1e-5 * multi[0]["norm"]
    # replicas hold the same weights after the steps
    for a in multi:
        for b in multi:
            if a["tp_rank"] == b["tp_rank"]:
                for k in a["weights"]:
                    assert torch.equal(a["weights"][k], b["weights"][k]), k


@pytest.mark.integration
def test_tied_embeddings_sp2_tp2_matches_single_process(tmp_path):
    """The input embedding doubles as the output projection (3B model): its gradient is the sum of both uses, on
    vocabulary shards as in one process."""
    (tmp_path / "one").mkdir()
    (tmp_path / "two").mkdir()
    one = run_ranks(_worker, 1, tmp_path / "one", 1, 1, 3, "tiny_tied")[0]
    assert "lm_head.weight" not in one["tgrads"]
    multi = run_ranks(_worker, 2, tmp_path / "two", 2, 2, 3, "tiny_tied")
    _compare(one, multi, tp=2)
