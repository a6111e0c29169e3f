"""Fused lm_head + cross-entropy on CPU: plain, label-smoothed and vocab-parallel (2 gloo ranks) against explicit
formulas (the reference only checks the un-smoothed loss, tests/test_text_autotp.py:910-1034 there)."""
import pytest
import torch

from dist_utils import run_ranks
from multimodal_training_b200.ops import functional as F


def _explicit(hidden, weight, labels, a):
    """-sum_v q_v log p_v with q = 1 - a on the target and a / (V - 1) on every other id; mean over valid rows."""
    logp = torch.log_softmax(hidden.double() @ weight.double().t(), dim=-1)
    V = weight.shape[0]
    valid = labels >= 0
    t = labels.clamp(min=0)
    q = torch.full_like(logp, a / (V - 1))
    q.scatter_(1, t[:, None], 1.0 - a)
    return (-(q * logp).sum(-1) * valid).sum() / valid.sum()


@pytest.mark.parametrize("a", [0.0, 0.1])
def test_label_smoothing_matches_the_explicit_target_distribution(a):
    torch.manual_seed(0)
    h = torch.randn(37, 16, requires_grad=True)
    w = torch.randn(50, 16, requires_grad=True)
    labels = torch.randint(0, 50, (37,))
    labels[::5] = -100
    loss = F.lm_head_cross_entropy(h, w, labels, label_smoothing=a)
    ref = _explicit(h, w, labels, a)
    assert abs(float(loss) - float(ref)) < 1e-5
    gh, gw = torch.autograd.grad(loss, (h, w))
    rh, rw = torch.autograd.grad(ref, (h, w))
    assert torch.allclose(gh, rh.float(), atol=1e-5) and torch.allclose(gw, rw.float(), atol=1e-5)
    with pytest.raises(ValueError):
        F.lm_head_cross_entropy(h, w, labels, label_smoothing=1.0)


def _vp_worker(rank, world, a):
    import torch.distributed as dist
    torch.manual_seed(1)
    h = torch.randn(29, 12, requires_grad=True)
    w_full = torch.randn(40, 12)
    labels = torch.randint(0, 40, (29,))
    labels[3] = -100
    per = 40 // world
    w = w_full[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    from multimodal_training_b200.parallel.comm import copy_to_group
    loss = F.lm_head_cross_entropy(copy_to_group(h, dist.group.WORLD), w, labels, vocab_lo=rank * per,
                                   group=dist.group.WORLD, label_smoothing=a)
    loss.backward()
    ref = _explicit(h.detach().requires_grad_(True), w_full.requires_grad_(True), labels, a)
    return float(loss), float(ref), h.grad.clone(), w.grad.clone()


@pytest.mark.parametrize("a", [0.0, 0.2])
def test_vocab_parallel_label_smoothing_uses_the_whole_vocabulary(tmp_path, a):
    res = run_ranks(_vp_worker, 2, tmp_path, a)
    torch.manual_seed(1)
    h = torch.randn(29, 12, requires_grad=True)
    w_full = torch.randn(40, 12, requires_grad=True)
    labels = torch.randint(0, 40, (29,))
    labels[3] = -100
    ref = _explicit(h, w_full, labels, a)
    rh, rw = torch.autograd.grad(ref, (h, w_full))
    for r, (loss, _, gh, gw) in enumerate(res):
        assert abs(loss - float(ref)) < 1e-5
        assert torch.allclose(gh, rh.float(), atol=1e-5)
        assert torch.allclose(gw, rw.float()[r * 20:(r + 1) * 20], atol=1e-5)
