"""The library baseline (baseline/lib_arm.py: plain PyTorch modules, library collectives in the reference's
places) and this framework's models are two independent statements of the same network.  With the same weights
they must give the same loss and the same gradients: this pins the framework's vision encoder, text decoder,
M-RoPE tables, splice and cross-entropy to an implementation that shares none of its model code, and it checks the
baseline's parallel layout (Ulysses all-to-alls with padded buffers, replicated-activation tensor parallelism with
all-reduces, vocab-parallel embedding and cross-entropy, ZeRO-1) against one process."""
import os
import sys

import pytest
import torch

from dist_utils import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))


def _batch(cfg, n=2, image_size=224, text_tokens=64):
    from multimodal_training_b200.data.synthetic import synthetic_global_batch
    return synthetic_global_batch(cfg, 0, n, image_size=image_size, text_tokens=text_tokens, seed=3,
                                  dtype=torch.float32)


def _framework_loss_and_grads(cfg, vsd, tsd, samples):
    """Single-process forward/backward through this framework's own modules with the given weights."""
    from multimodal_training_b200.models.text import TextDecoder, mrope_cos_sin
    from multimodal_training_b200.models.vision import VisionEncoder
    from multimodal_training_b200.ops.attention import SeqInfo
    from multimodal_training_b200.parallel.handoff import pack_text_batch
    from multimodal_training_b200.parallel.sp import build_vision_plan

    v, t = cfg.vision, cfg.text
    vis = VisionEncoder(v, dtype=torch.float32, activation_checkpointing=False)
    txt = TextDecoder(t, dtype=torch.float32, activation_checkpointing=False)
    assert vis.load_reference_state_dict(vsd) == []
    assert txt.load_reference_state_dict(tsd) == []
    grids = [g for s in samples for g in s.grid_thw]
    plan = build_vision_plan(grids, sp=1, rank=0, spatial_merge_size=v.spatial_merge_size, window_size=v.window_size,
                             patch_size=v.patch_size, head_dim=v.head_dim)
    pixels = torch.cat([s.pixel_values for s in samples]).index_select(0, plan.local_patch_index)
    merged = vis(pixels, plan)                               # window order
    inv = torch.empty_like(plan.local_merged_ids)
    inv[plan.local_merged_ids] = torch.arange(inv.numel())
    merged = merged.index_select(0, inv)                     # original order
    tb = pack_text_batch(samples, image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id,
                         spatial_merge_size=v.spatial_merge_size, pad_multiple=8, pad_token_id=cfg.pad_token_id)
    x = txt.embed(tb.input_ids)
    rows = torch.from_numpy(__import__("numpy").concatenate(tb.image_rows))
    x = x.index_copy(0, rows, merged)
    cos, sin = mrope_cos_sin(tb.position_ids, t.head_dim, t.rope_theta, t.mrope_section)
    h = txt(x, cos, sin, SeqInfo.from_list(tb.cu_seqlens, "cpu"))
    loss = txt.loss(h, tb.shifted_labels)
    loss.backward()
    return float(loss.detach()), {"patch_embed": vis.patch_embed_w.grad.clone(), "embed": txt.embed_tokens.grad.clone(),
                         "ln_q": vis.ln_q_w.grad.clone(), "norm": txt.norm_w.grad.clone()}


def _text_full_state(cfg, seed=5):
    """Random full (unsharded) text weights under the reference's key names."""
    g = torch.Generator().manual_seed(seed)
    t = cfg.text
    H, d = t.hidden_size, t.head_dim
    r = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
    sd = {"embed_tokens.weight": r(t.vocab_size, H), "norm.weight": 1 + r(H), "lm_head.weight": r(t.vocab_size, H)}
    for i in range(t.num_hidden_layers):
        p = f"layers.{i}."
        for n, rows in (("q", t.num_attention_heads * d), ("k", t.num_key_value_heads * d),
                        ("v", t.num_key_value_heads * d)):
            sd[p + f"self_attn.{n}_proj.weight"] = r(rows, H)
            sd[p + f"self_attn.{n}_proj.bias"] = r(rows)
        sd[p + "self_attn.o_proj.weight"] = r(H, t.num_attention_heads * d)
        sd[p + "mlp.gate_proj.weight"] = r(t.intermediate_size, H)
        sd[p + "mlp.up_proj.weight"] = r(t.intermediate_size, H)
        sd[p + "mlp.down_proj.weight"] = r(H, t.intermediate_size)
        sd[p + "input_layernorm.weight"] = 1 + r(H)
        sd[p + "post_attention_layernorm.weight"] = 1 + r(H)
    return sd


def _lib_worker(rank, world, tp):
    import torch.distributed as dist

    import lib_arm
    from multimodal_training_b200.config.model_configs import get_model_config

    cfg = get_model_config("tiny")
    tr = lib_arm.LibTrainer(cfg, tp=tp, device=torch.device("cpu"), dtype=torch.float32, seed=1, lr=1e-3)
    # same weights everywhere: the vision state of rank 0's random init, one full text state sliced per rank
    vsd = {k: v.clone() for k, v in tr.vision.reference_state_dict().items()}
    g = torch.Generator().manual_seed(11)
    for k in sorted(vsd):
        if k.endswith("bias"):
            vsd[k] = torch.randn(vsd[k].shape, generator=g) * 0.05
    tr.vision.load_reference_state_dict(vsd)
    tsd = _text_full_state(cfg)
    tr.text.load_reference_state_dict(tsd)
    samples = _batch(cfg)
    loss = tr.train_step(samples)
    if world > 1:
        dist.all_reduce(loss)
        loss /= world
    # gradients after the step's reductions: vision shard of the flat gradient, gathered; text pieces as they are
    vg = tr.vopt.shard_g.clone()
    if world > 1:
        parts = [torch.empty_like(vg) for _ in range(world)]
        dist.all_gather(parts, vg)
        vg = torch.cat(parts)
    n_pe = tr.vision.patch_embed.numel()
    out = {"loss": float(loss), "patch_embed": vg[:n_pe].view_as(tr.vision.patch_embed).clone(),
           "embed": tr.text.embed.grad.clone(), "norm": tr.text.norm.grad.clone(), "rank": rank,
           "vsd": vsd if rank == 0 else None, "tsd": tsd if rank == 0 else None}
    off = 0
    for p in tr.vopt.params:
        if p is tr.vision.ln_q:
            out["ln_q"] = vg[off:off + p.numel()].clone()
        off += p.numel()
    return out


@pytest.mark.parametrize("world,tp", [(1, 1), (2, 2), (2, 1)])
def test_library_baseline_equals_the_framework_models(tmp_path, world, tp):
    from multimodal_training_b200.config.model_configs import get_model_config

    res = run_ranks(_lib_worker, world, tmp_path, tp)
    cfg = get_model_config("tiny")
    loss, grads = _framework_loss_and_grads(cfg, res[0]["vsd"], res[0]["tsd"], _batch(cfg))
    assert abs(res[0]["loss"] - loss) < 2e-5 * max(1.0, abs(loss)), (res[0]["loss"], loss)

    def close(a, b, what):
        err = (a - b).abs().max().item()
        assert err < 1e-5 + 2e-4 * b.abs().max().item(), (what, err, b.abs().max().item())

    close(res[0]["patch_embed"], grads["patch_embed"], "patch_embed grad")
    close(res[0]["ln_q"], grads["ln_q"], "merger ln_q grad")
    close(res[0]["norm"], grads["norm"], "final norm grad")
    emb = torch.cat([r["embed"] for r in sorted(res, key=lambda r: r["rank"])[:tp]], dim=0) if tp > 1 \
        else res[0]["embed"]
    if tp == 1 and world > 1:
        # two data-parallel text replicas: each holds the gradient of its own sample; their mean is the global one
        emb = (res[0]["embed"] + res[1]["embed"]) / 2
    close(emb, grads["embed"], "embedding grad")
