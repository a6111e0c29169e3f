"""Single-process VLM wrappers (models/vlm.py): splice, loss, decoding and merged-checkpoint loading on CPU."""
import torch

from multimodal_training_b200.models.vlm import Qwen2_5_VLForConditionalGeneration


def _batch(cfg, grids, text_len=12, seed=0):
    torch.manual_seed(seed)
    unit = cfg.vision.spatial_merge_size ** 2
    n_patch = sum(t * h * w for t, h, w in grids)
    pix = torch.randn(n_patch, cfg.vision.patch_dim)
    ids = []
    for t, h, w in grids:
        ids += torch.randint(0, 900, (text_len,)).tolist() + [cfg.image_token_id] * (t * h * w // unit)
    ids += torch.randint(0, 900, (text_len,)).tolist()
    ids = torch.tensor([ids])
    labels = ids.clone()
    labels[ids == cfg.image_token_id] = -100
    return ids, pix, labels


def test_forward_loss_matches_manual_cross_entropy_and_backward_reaches_both_halves():
    m = Qwen2_5_VLForConditionalGeneration("tiny")
    ids, pix, labels = _batch(m.config, [(1, 16, 16)])
    out = m(ids, pix, [(1, 16, 16)], labels=labels)
    logits = out["logits"]
    assert logits.shape == (ids.numel(), m.config.text.vocab_size)
    ref = torch.nn.functional.cross_entropy(logits[:-1].float(), labels[0, 1:], ignore_index=-100)
    assert abs(float(out["loss"].detach()) - float(ref)) < 1e-4
    out["loss"].backward()
    assert m.model.visual.patch_embed_w.grad is not None and m.model.visual.patch_embed_w.grad.abs().sum() > 0
    assert m.model.language_model.embed_tokens.grad.abs().sum() > 0


def test_images_encoded_together_equal_images_encoded_alone():
    """The window permutation is undone per image: joint and separate encoding give the same merged tokens."""
    m = Qwen2_5_VLForConditionalGeneration("tiny").model
    torch.manual_seed(3)
    g1, g2 = (1, 16, 16), (1, 8, 24)
    p1 = torch.randn(16 * 16, m.config.vision.patch_dim)
    p2 = torch.randn(8 * 24, m.config.vision.patch_dim)
    with torch.no_grad():
        both = m.encode_images(torch.cat([p1, p2]), [g1, g2])
        a = m.encode_images(p1, [g1])
        b = m.encode_images(p2, [g2])
    assert torch.allclose(both, torch.cat([a, b]), atol=1e-5)


def test_greedy_generate_and_merged_checkpoint_round_trip():
    src = Qwen2_5_VLForConditionalGeneration("tiny", seed=5)
    ids, pix, _ = _batch(src.config, [(1, 16, 16)], text_len=6)
    gen = src.generate(ids[0], pix, [(1, 16, 16)], max_new_tokens=3)
    assert gen.shape[0] == ids.shape[1] + 3 and torch.equal(gen[: ids.shape[1]], ids[0])
    state = {"visual." + k: v for k, v in src.model.visual.reference_state_dict().items()}
    state.update({"language_model." + k: v for k, v in src.model.language_model.reference_state_dict().items()})
    dst = Qwen2_5_VLForConditionalGeneration("tiny", seed=99)
    dst.load_merged_state_dict(state)
    with torch.no_grad():
        assert torch.allclose(dst.model(ids, pix, [(1, 16, 16)]), src.model(ids, pix, [(1, 16, 16)]), atol=1e-5)


def test_vision_tensor_parallel_shards_round_trip():
    """Shards written by tensor-parallel vision ranks merge to the single-process state dict (MLP padding cut off),
    and a tensor-parallel rank loads its slices from full weights or its own shard."""
    from multimodal_training_b200.cli.merge_checkpoint import merge_state_dicts
    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.models.vision import VisionEncoder
    from multimodal_training_b200.parallel.tp import TPContext

    cfg = get_model_config("tiny").vision
    full = VisionEncoder(cfg, seed=3).reference_state_dict()
    ranks = [VisionEncoder(cfg, seed=3, tp=TPContext(None, 2, r)) for r in range(2)]
    merged = merge_state_dicts([m.reference_state_dict() for m in ranks])
    assert merged.keys() == full.keys()
    for k, v in full.items():
        assert torch.equal(merged[k], v), k
    other = VisionEncoder(cfg, seed=9).reference_state_dict()
    for r, m in enumerate(ranks):
        m.load_reference_state_dict(other)                                   # slices of full tensors
        shard = m.reference_state_dict()
        fresh = VisionEncoder(cfg, seed=1, tp=TPContext(None, 2, r))
        fresh.load_reference_state_dict(shard, sharded=True)                 # its own shard
        for (ka, a), (kb, b) in zip(m.state_dict().items(), fresh.state_dict().items()):
            assert ka == kb and torch.equal(a, b), ka
    merged = merge_state_dicts([m.reference_state_dict() for m in ranks])
    for k, v in other.items():
        assert torch.equal(merged[k], v), k
