"""tcgen05 flash attention (forward and backward) against a plain PyTorch fp32 attention."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run(cu, n_q, n_kv, dim, causal, seed=0):
    from multimodal_training_b200.ops import functional as F
    from multimodal_training_b200.ops import native as nv
    from multimodal_training_b200.ops.attention import SeqInfo
    torch.manual_seed(seed)
    T = cu[-1]
    W = (n_q + 2 * n_kv) * dim
    qkv = torch.randn(T, W, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    info = SeqInfo.from_list(cu, DEV)
    out = F.attention(qkv, n_q, n_kv, dim, info, causal=causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    assert nv.get_error()[0] == 0, nv.get_error()
    ref_in = qkv.detach().float().requires_grad_()
    q = ref_in[:, : n_q * dim].reshape(T, n_q, dim)
    k = ref_in[:, n_q * dim:(n_q + n_kv) * dim].reshape(T, n_kv, dim)
    v = ref_in[:, (n_q + n_kv) * dim:].reshape(T, n_kv, dim)
    ref = F.attention_reference(q, k, v, cu, causal, 1.0 / math.sqrt(dim)).reshape(T, n_q * dim)
    ref.backward(dout.float())

    def rel(a, b):
        return ((a.float() - b).abs().max() / (b.abs().max() + 1e-9)).item()

    e_out = rel(out, ref)
    nq, nk = n_q * dim, n_kv * dim
    e_dq = rel(qkv.grad[:, :nq], ref_in.grad[:, :nq])
    e_dk = rel(qkv.grad[:, nq:nq + nk], ref_in.grad[:, nq:nq + nk])
    e_dv = rel(qkv.grad[:, nq + nk:], ref_in.grad[:, nq + nk:])
    return e_out, e_dq, e_dk, e_dv


@pytest.mark.parametrize("cu", [[0, 64, 128, 192, 256], [0, 64, 100, 164, 228, 260, 324], [0, 256], [0, 1024],
                                [0, 300, 1324]])
def test_vision_noncausal_d80(cu):
    errs = _run(cu, 4, 4, 80, False)
    assert max(errs) < 2.5e-2, errs


@pytest.mark.parametrize("cu", [[0, 128], [0, 200, 456], [0, 1000, 1096, 2120], [0, 77, 90, 91, 600]])
@pytest.mark.parametrize("heads", [(4, 4), (8, 2), (7, 1)])
def test_text_causal_gqa_d128(cu, heads):
    errs = _run(cu, heads[0], heads[1], 128, True)
    assert max(errs) < 2.5e-2, errs


def test_two_runs_bit_equal():
    """The kernels use no atomics: repeated runs must give identical bits."""
    from multimodal_training_b200.ops import functional as F
    from multimodal_training_b200.ops.attention import SeqInfo
    torch.manual_seed(1)
    cu = [0, 500, 900]
    qkv = torch.randn(900, 6 * 128, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    info = SeqInfo.from_list(cu, DEV)
    outs, grads = [], []
    for _ in range(2):
        qkv.grad = None
        o = F.attention(qkv, 4, 1, 128, info, causal=True)
        o.backward(torch.ones_like(o))
        outs.append(o.detach().clone())
        grads.append(qkv.grad.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(grads[0], grads[1])
