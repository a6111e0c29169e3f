"""The model maths pinned to statements that share no code with the package.

* Vision encoder: against the reference project's own ``Qwen2_5_VisionTransformerPretrainedModel``
  (python/models/qwen2_5_vl/modeling_qwen2_5_vl.py:809-1070), loaded from a checkout that the environment variable
  ``MMT_REFERENCE_CHECKOUT`` points at (the directory that holds ``python/``).  Skipped when the variable is unset.
* Text decoder, M-RoPE tables and the shifted cross-entropy: against the plain-PyTorch restatement below of the
  reference's decoder layer (modeling_qwen2_5_vl.py:1153-1191 rotary with sections, :1194-1286 attention with
  grouped KV heads, :1136-1150 MLP, :1341-1363 residual wiring), written from the published Qwen2.5-VL equations.
"""
import math
import os
import sys

import pytest
import torch

from multimodal_training_b200.config.model_configs import get_model_config


# ----------------------------------------------------------------------------------------------- text restatement
def _rms(x, w, eps):
    return w * (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps))


def _rot_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat((-b, a), dim=-1)


def _mrope_tables(position_ids, head_dim, theta, sections):
    """position_ids [3, T] -> cos, sin [T, head_dim]: frequency band i takes its angle from axis (t, h, w) by the
    section it falls into; the half-table is repeated for the two halves of the head."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = position_ids.float()[:, :, None] * inv[None, None, :]            # [3, T, d/2]
    pieces, start = [], 0
    for i, n in enumerate(sections):
        pieces.append(ang[i, :, start:start + n])
        start += n
    half = torch.cat(pieces, dim=-1)
    full = torch.cat((half, half), dim=-1)
    return full.cos(), full.sin()


def _decoder_restated(sd, cfg, x, position_ids, cu_seqlens, labels):
    """Embeddings-in, mean next-token loss out; packed sequences attend causally within their own segment."""
    t = cfg.text
    H, d, nq, nkv = t.hidden_size, t.head_dim, t.num_attention_heads, t.num_key_value_heads
    cos, sin = _mrope_tables(position_ids, d, t.rope_theta, t.mrope_section)
    T = x.shape[0]
    seg = torch.zeros(T, dtype=torch.long)
    for i in range(len(cu_seqlens) - 1):
        seg[cu_seqlens[i]:cu_seqlens[i + 1]] = i
    pos = torch.arange(T)
    allowed = (seg[:, None] == seg[None, :]) & (pos[None, :] <= pos[:, None])
    for i in range(t.num_hidden_layers):
        p = f"layers.{i}."
        h = _rms(x, sd[p + "input_layernorm.weight"], t.rms_norm_eps)
        q = (h @ sd[p + "self_attn.q_proj.weight"].t() + sd[p + "self_attn.q_proj.bias"]).view(T, nq, d)
        k = (h @ sd[p + "self_attn.k_proj.weight"].t() + sd[p + "self_attn.k_proj.bias"]).view(T, nkv, d)
        v = (h @ sd[p + "self_attn.v_proj.weight"].t() + sd[p + "self_attn.v_proj.bias"]).view(T, nkv, d)
        q = q * cos[:, None, :] + _rot_half(q) * sin[:, None, :]
        k = k * cos[:, None, :] + _rot_half(k) * sin[:, None, :]
        k = k.repeat_interleave(nq // nkv, dim=1)
        v = v.repeat_interleave(nq // nkv, dim=1)
        s = torch.einsum("qhd,khd->hqk", q, k) / math.sqrt(d)
        s = s.masked_fill(~allowed[None], float("-inf"))
        a = torch.einsum("hqk,khd->qhd", s.softmax(-1), v).reshape(T, nq * d)
        x = x + a @ sd[p + "self_attn.o_proj.weight"].t()
        h = _rms(x, sd[p + "post_attention_layernorm.weight"], t.rms_norm_eps)
        gate = h @ sd[p + "mlp.gate_proj.weight"].t()
        up = h @ sd[p + "mlp.up_proj.weight"].t()
        x = x + (torch.nn.functional.silu(gate) * up) @ sd[p + "mlp.down_proj.weight"].t()
    logits = _rms(x, sd["norm.weight"], t.rms_norm_eps) @ sd["lm_head.weight"].t()
    return torch.nn.functional.cross_entropy(logits.float(), labels, ignore_index=-100)


def _random_text_state(cfg, seed=5):
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


def test_text_decoder_mrope_and_loss_match_a_plain_restatement():
    from multimodal_training_b200.models.text import TextDecoder, mrope_cos_sin
    from multimodal_training_b200.ops.attention import SeqInfo

    cfg = get_model_config("tiny")
    t = cfg.text
    sd = _random_text_state(cfg)
    txt = TextDecoder(t, dtype=torch.float32, activation_checkpointing=False)
    assert txt.load_reference_state_dict(sd) == []
    g = torch.Generator().manual_seed(2)
    cu = [0, 24, 40, 72]                                         # three packed sequences
    T = cu[-1]
    x = (torch.randn(T, t.hidden_size, generator=g) * 0.5).requires_grad_(True)
    # multimodal positions: an image block in the middle of each sequence has distinct (t, h, w) indices
    position_ids = torch.zeros(3, T, dtype=torch.long)
    for a, b in zip(cu[:-1], cu[1:]):
        n = b - a
        base = torch.arange(n)
        position_ids[:, a:b] = base
        position_ids[1, a + 4:a + 12] = 4 + torch.arange(8) // 4
        position_ids[2, a + 4:a + 12] = 4 + torch.arange(8) % 4
        position_ids[0, a + 4:a + 12] = 4
    labels = torch.randint(0, t.vocab_size, (T,), generator=g)
    labels[::5] = -100
    for b in cu[1:]:
        labels[b - 1] = -100                                     # nothing to predict after a sequence's last token

    cos, sin = mrope_cos_sin(position_ids, t.head_dim, t.rope_theta, t.mrope_section)
    rc, rs = _mrope_tables(position_ids, t.head_dim, t.rope_theta, t.mrope_section)
    assert torch.allclose(cos.float().view_as(rc), rc, atol=1e-6) and torch.allclose(sin.float().view_as(rs), rs, atol=1e-6)

    h = txt(x, cos, sin, SeqInfo.from_list(cu, "cpu"))
    loss = txt.loss(h, labels)
    loss.backward()
    x2 = x.detach().clone().requires_grad_(True)
    ref = _decoder_restated(sd, cfg, x2, position_ids, cu, labels)
    ref.backward()
    assert abs(float(loss.detach()) - float(ref.detach())) < 1e-5 * max(1.0, abs(float(ref.detach())))
    assert torch.allclose(x.grad, x2.grad, atol=2e-6, rtol=1e-4)


# ----------------------------------------------------------------------------------------------- reference vision
def _reference_vision(cfg):
    root = os.environ.get("MMT_REFERENCE_CHECKOUT")
    if not root:
        pytest.skip("MMT_REFERENCE_CHECKOUT is not set")
    sys.path.insert(0, os.path.join(root, "python"))
    try:
        from models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig
        from models.qwen2_5_vl.modeling_qwen2_5_vl import Qwen2_5_VisionTransformerPretrainedModel
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"the reference's vision module does not import here: {e}")
    finally:
        sys.path.pop(0)
    v = cfg.vision
    rc = Qwen2_5_VLVisionConfig(depth=v.depth, hidden_size=v.hidden_size, intermediate_size=v.intermediate_size,
                                num_heads=v.num_heads, in_channels=v.in_channels, patch_size=v.patch_size,
                                spatial_merge_size=v.spatial_merge_size, temporal_patch_size=v.temporal_patch_size,
                                window_size=v.window_size, out_hidden_size=v.out_hidden_size,
                                fullatt_block_indexes=list(v.fullatt_block_indexes))
    rc._attn_implementation = "sdpa"
    torch.manual_seed(0)
    return Qwen2_5_VisionTransformerPretrainedModel(rc).float().eval()


def test_vision_encoder_matches_the_reference_module():
    from multimodal_training_b200.models.vision import VisionEncoder
    from multimodal_training_b200.parallel.sp import build_vision_plan

    cfg = get_model_config("tiny")
    v = cfg.vision
    ref = _reference_vision(cfg)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in ref.parameters():                                # non-trivial norms and biases
            p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    sd = {k: t.detach().clone() for k, t in ref.state_dict().items()}
    ours = VisionEncoder(v, dtype=torch.float32, activation_checkpointing=False)
    assert ours.load_reference_state_dict(sd) == []

    grids = [(1, 16, 12), (1, 8, 20)]                            # two ragged images: 192 + 160 patches
    n = sum(t * h * w for t, h, w in grids)
    pixels = torch.randn(n, v.in_channels * v.temporal_patch_size * v.patch_size ** 2, generator=g)
    p_ref = pixels.clone().requires_grad_(True)
    out_ref = ref(p_ref, grid_thw=torch.tensor(grids))
    if not torch.is_tensor(out_ref):
        out_ref = out_ref[0]

    plan = build_vision_plan(grids, sp=1, rank=0, spatial_merge_size=v.spatial_merge_size, window_size=v.window_size,
                             patch_size=v.patch_size, head_dim=v.head_dim)
    p_ours = pixels.clone().requires_grad_(True)
    merged = ours(p_ours.index_select(0, plan.local_patch_index), plan)      # window order
    inv = torch.empty_like(plan.local_merged_ids)
    inv[plan.local_merged_ids] = torch.arange(inv.numel())
    out = merged.index_select(0, inv)                                        # original order, as the reference returns
    assert out.shape == out_ref.shape
    assert float((out - out_ref).abs().max()) < 1e-5
    w = torch.randn(out.shape, generator=g)
    (out * w).sum().backward()
    (out_ref * w).sum().backward()
    assert float((p_ours.grad - p_ref.grad).abs().max()) < 1e-5 * max(1.0, float(p_ref.grad.abs().max()))
