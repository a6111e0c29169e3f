"""``training.optimizer_master_weights: false``: AdamW directly on bf16 parameters with bf16 moments and no fp32 master
copy -- the optimizer the reference runs (torch.optim.AdamW on a bf16 model, python/ray/trainer.py:503-572)."""
import torch

from multimodal_training_b200.parallel.zero import ZeroAdamW


def _params(seed=0):
    g = torch.Generator().manual_seed(seed)
    w = torch.nn.Parameter((torch.randn(64, 48, generator=g) * 0.1).to(torch.bfloat16))
    b = torch.nn.Parameter((torch.randn(48, generator=g) * 0.1).to(torch.bfloat16))
    return [("layer.weight", w), ("layer.bias", b)]


def test_matches_torch_adamw_on_bf16_parameters():
    ours = _params()
    ref = [(n, torch.nn.Parameter(p.detach().clone())) for n, p in _params()]
    opt = ZeroAdamW(ours, lr=1e-2, weight_decay=0.1, master_weights=False)
    assert opt.master is None and opt.exp_avg.dtype == torch.bfloat16
    topt = torch.optim.AdamW([{"params": [ref[0][1]], "weight_decay": 0.1}, {"params": [ref[1][1]], "weight_decay": 0.0}],
                             lr=1e-2, fused=True)
    g = torch.Generator().manual_seed(1)
    for _ in range(4):
        opt.zero_grad()
        for (_, p), (_, q) in zip(ours, ref):
            gr = (torch.randn(p.shape, generator=g) * 0.05).to(torch.bfloat16)
            p.grad.copy_(gr)
            q.grad = gr.clone()
        opt.step()
        topt.step()
    for (_, p), (_, q) in zip(ours, ref):
        diff = (p.detach().float() - q.detach().float()).abs()
        ulp = q.detach().float().abs() * 2.0 ** -6 + 1e-12        # at least one bf16 step at that magnitude
        assert bool((diff <= ulp).all())                          # same update, at most one rounding step apart
        assert float((diff == 0).float().mean()) > 0.9


def test_master_weights_keep_updates_that_bf16_rounds_away():
    """Why the default keeps an fp32 master copy: an update far below one bf16 step of the weight is lost without it
    and accumulates with it."""
    def run(master):
        p = torch.nn.Parameter(torch.ones(128, dtype=torch.bfloat16))
        opt = ZeroAdamW([("w", p)], lr=1e-4, weight_decay=0.0, master_weights=master)
        for _ in range(40):
            opt.zero_grad()
            p.grad.fill_(1.0)
            opt.step()
        return p, opt
    p_bf16, _ = run(False)
    p_master, opt = run(True)
    assert float(p_bf16.detach().float().mean()) == 1.0           # 1 - 1e-4 rounds back to 1 every step
    assert abs(float(opt.master[:128].mean()) - (1.0 - 40e-4)) < 1e-5   # the master copy moved by 40 steps
    assert float(p_master.detach().float().mean()) < 1.0


def test_state_dict_round_trip_and_mismatch():
    import pytest
    a = ZeroAdamW(_params(), lr=1e-2, master_weights=False)
    for p in a.params:
        p.grad.fill_(0.01)
    a.step()
    sd = a.state_dict()
    assert sd["master"] is None and sd["exp_avg"].dtype == torch.bfloat16
    b = ZeroAdamW(_params(), lr=1e-2, master_weights=False)
    b.load_state_dict(sd)
    assert torch.equal(b.exp_avg, a.exp_avg) and b.step_count == 1
    with pytest.raises(ValueError, match="optimizer_master_weights"):
        ZeroAdamW(_params(), lr=1e-2, master_weights=True).load_state_dict(sd)
