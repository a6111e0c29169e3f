"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _F():
    from multimodal_training_b200.ops import functional as F
    from multimodal_training_b200.ops import native as nv
    assert nv.available(), "libmmt_b200.so must be built: the GPU path has no fallback"
    nv.lib()
    return F, nv


def rel_err(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (304, 1288, 1176), (2048, 3584, 3584), (77, 3840, 1280),
                                   (4096, 1280, 3424)])
@pytest.mark.parametrize("layout", ["kk", "k_mn", "mn_mn"])
def test_gemm_layouts(M, N, K, layout):
    F, nv = _F()
    torch.manual_seed(0)
    a_mn = layout == "mn_mn"
    if a_mn:
        M = (M + 7) // 8 * 8     # an MN-major A has leading dimension M: multiple of 8 elements (16 bytes)
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    ref = A.float() @ B.float().t()
    b_mn = layout != "kk"
    out = F.gemm(A.t().contiguous() if a_mn else A, B.t().contiguous() if b_mn else B, a_mn=a_mn, b_mn=b_mn)
    assert rel_err(out, ref) < 8e-3
    assert nv.get_error()[0] == 0


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (304, 520, 328), (1000, 1176, 1176), (2048, 3584, 3584),
                                   (4096, 1288, 1280)])
@pytest.mark.parametrize("layout", ["kk", "k_mn", "mn_mn"])
@pytest.mark.parametrize("mt,bn", [(3, 256), (2, 192), (2, 256), (1, 192)])
def test_gemm_tile_variants(M, N, K, layout, mt, bn):
    """Every tile variant forced by hand -- the 2-CTA kernel (mt 3: two interleaved 128-wide accumulators per tile),
    256-row tiles at width 192 and 256, 128-row tiles at width 192 -- in all three operand layouts, with tails in M,
    N and K, bias and residual in the epilogue, against an fp32 PyTorch product."""
    F, nv = _F()
    lib = nv.lib()
    torch.manual_seed(M + N + K)
    a_mn = layout == "mn_mn"
    if a_mn:
        M = (M + 7) // 8 * 8
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ref = A.float() @ B.float().t()
    b_mn = layout != "kk"
    try:
        lib.mmt_gemm_force_mt(mt)
        lib.mmt_gemm_force_bn(bn)
        Aa, Bb = (A.t().contiguous() if a_mn else A), (B.t().contiguous() if b_mn else B)
        out = F.gemm(Aa, Bb, a_mn=a_mn, b_mn=b_mn)
        out2 = F.gemm(Aa, Bb, a_mn=a_mn, b_mn=b_mn, bias=bias, residual=res)
    finally:
        lib.mmt_gemm_force_mt(0)
        lib.mmt_gemm_force_bn(0)
    assert rel_err(out, ref) < 8e-3
    assert rel_err(out2, ref + bias.float() + res.float()) < 8e-3
    assert nv.get_error()[0] == 0


def test_gemm_epilogue_bias_residual_accumulate_f32():
    F, nv = _F()
    torch.manual_seed(1)
    M, N, K = 520, 1280, 1024
    A = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    B = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ref = A.float() @ B.float().t() + bias.float() + res.float()
    out = F.gemm(A, B, bias=bias, residual=res)
    assert rel_err(out, ref) < 8e-3
    acc = torch.ones(M, N, device=DEV, dtype=torch.float32)
    F.gemm(A, B, out=acc, accumulate=True, out_f32=True)
    assert rel_err(acc, A.float() @ B.float().t() + 1.0) < 2e-3
    g = F.gemm(A, B, act=1)
    assert rel_err(g, torch.nn.functional.gelu(A.float() @ B.float().t())) < 8e-3


def test_linear_autograd_matches_reference():
    F, nv = _F()
    torch.manual_seed(2)
    T, K, N = 640, 512, 768
    x = torch.randn(T, K, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    b = torch.randn(N, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, N, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.linear(x, w, b, r)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf, bf, rf = (t.detach().float().requires_grad_() for t in (x, w, b, r))
    yr = torch.nn.functional.linear(xf, wf, bf) + rf
    yr.backward(dy.float())
    assert rel_err(y, yr) < 8e-3
    assert rel_err(x.grad, xf.grad) < 8e-3
    assert rel_err(w.grad, wf.grad) < 8e-3
    assert rel_err(b.grad, bf.grad) < 8e-3
    assert rel_err(r.grad, rf.grad) < 1e-6


@pytest.mark.parametrize("rows,cols", [(1001, 1280), (333, 3584), (65, 5120), (37, 8192), (17, 256)])
def test_rmsnorm(rows, cols):
    F, nv = _F()
    torch.manual_seed(3)
    x = torch.randn(rows, cols, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = F.rmsnorm(x, w, 1e-6)
    dy = torch.randn_like(y)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2
    assert rel_err(x.grad, xf.grad) < 1e-2
    assert rel_err(w.grad, wf.grad) < 1e-2


@pytest.mark.parametrize("heads,dim,extra", [(32, 80, 1280), (8, 128, 512)])
def test_rope(heads, dim, extra):
    F, nv = _F()
    torch.manual_seed(4)
    T = 300
    x = torch.randn(T, heads * dim + extra, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ang = torch.rand(T, dim // 2, device=DEV) * 6.28
    ang = torch.cat([ang, ang], -1)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    y = F.rope(x, cos, sin, heads, dim)
    dy = torch.randn_like(y)
    y.backward(dy)
    xc = x.detach().cpu().float().requires_grad_()
    yr = F.rope(xc, cos.cpu(), sin.cpu(), heads, dim)
    yr.backward(dy.cpu().float())
    assert rel_err(y.cpu(), yr) < 1e-2
    assert rel_err(x.grad.cpu(), xc.grad) < 1e-2


def test_swiglu_gelu():
    F, nv = _F()
    torch.manual_seed(5)
    gu = torch.randn(500, 2 * 3424, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = F.swiglu(gu)
    dy = torch.randn_like(y)
    y.backward(dy)
    gf = gu.detach().float().requires_grad_()
    g, u = gf.chunk(2, -1)
    yr = torch.nn.functional.silu(g) * u
    yr.backward(dy.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(gu.grad, gf.grad) < 1e-2
    x = torch.randn(300, 5120, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    z = F.gelu(x)
    z.backward(dy[:300, :5120].contiguous() if dy.shape[1] >= 5120 else torch.ones_like(z))
    xf = x.detach().float().requires_grad_()
    zr = torch.nn.functional.gelu(xf)
    zr.backward(torch.ones_like(zr) if dy.shape[1] < 5120 else dy[:300, :5120].float())
    assert rel_err(z, zr) < 1e-2 and rel_err(x.grad, xf.grad) < 1e-2


def test_gather_scatter_embedding():
    F, nv = _F()
    torch.manual_seed(6)
    table = torch.randn(1000, 512, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 2000, (777,), device=DEV)
    out = F.embedding(ids, table, vocab_lo=500)
    ref = torch.zeros(777, 512, device=DEV)
    ok = (ids >= 500) & (ids < 1500)
    ref[ok] = table.detach().float()[ids[ok] - 500]
    assert torch.equal(out.float(), ref)
    dy = torch.randn_like(out)
    out.backward(dy)
    gref = torch.zeros(1000, 512, device=DEV)
    gref.index_add_(0, ids[ok] - 500, dy.float()[ok])
    assert rel_err(table.grad, gref) < 2e-2
    perm = torch.randperm(777, device=DEV)
    src = torch.randn(777, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = F.gather_rows(src, perm)
    assert torch.equal(g, src.detach()[perm])
    g.backward(torch.ones_like(g))
    assert torch.equal(src.grad, torch.ones_like(src))


@pytest.mark.parametrize("T,V,H", [(300, 4096, 512), (1000, 38016, 256)])
def test_lm_head_cross_entropy(T, V, H):
    F, nv = _F()
    torch.manual_seed(7)
    h = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, H, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::7] = -100
    loss = F.lm_head_cross_entropy(h, w, labels, chunk_rows=256)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = torch.nn.functional.cross_entropy(hf @ wf.t(), labels, ignore_index=-100)
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2 * abs(lr.item())
    assert rel_err(h.grad, hf.grad) < 3e-2
    assert rel_err(w.grad, wf.grad) < 3e-2


def test_lm_head_cross_entropy_with_label_smoothing():
    """The smoothed loss and its gradients against an fp32 evaluation of -sum_v q_v log p_v (q = 1 - a on the target,
    a / (V - 1) on every other id)."""
    F, nv = _F()
    torch.manual_seed(9)
    T, V, H, a = 300, 4096, 256, 0.1
    h = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(V, H, device=DEV, dtype=torch.bfloat16) * 0.05).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    labels[::5] = -100
    loss = F.lm_head_cross_entropy(h, w, labels, chunk_rows=128, label_smoothing=a)
    loss.backward()
    hf, wf = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    logp = torch.log_softmax(hf @ wf.t(), dim=-1)
    q = torch.full_like(logp, a / (V - 1))
    q.scatter_(1, labels.clamp(min=0)[:, None], 1.0 - a)
    valid = labels >= 0
    lr = (-(q * logp).sum(-1) * valid).sum() / valid.sum()
    lr.backward()
    assert abs(loss.item() - lr.item()) < 2e-2 * abs(lr.item())
    assert rel_err(h.grad, hf.grad) < 3e-2
    assert rel_err(w.grad, wf.grad) < 3e-2


def test_adamw_and_sumsq():
    F, nv = _F()
    torch.manual_seed(8)
    n = 8 * 12345
    p = torch.randn(n, device=DEV, dtype=torch.bfloat16)
    g = torch.randn(n, device=DEV, dtype=torch.bfloat16) * 0.1
    master = p.float().clone()
    m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    pc, gc = p.cpu().float(), g.cpu()
    mc, vc, wc = torch.zeros(n), torch.zeros(n), pc.clone()
    pcb = p.cpu().clone()
    scale = torch.tensor([0.5], device=DEV)
    for step in (1, 2, 3):
        F.adamw_step(p, g, master, m, v, n_decay=n // 2, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1,
                     step=step, grad_scale=scale)
        F.adamw_step(pcb, gc, wc, mc, vc, n_decay=n // 2, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1,
                     step=step, grad_scale=torch.tensor([0.5]))
    assert rel_err(master.cpu(), wc) < 1e-5
    # the kernel's fp32 arithmetic (fast division / square root) may differ from the CPU's in the last bits, which can
    # flip the bf16 rounding of a few parameters by one unit in the last place, never more
    got, want = p.cpu().float(), wc.to(torch.bfloat16).float()
    assert (got != want).float().mean().item() < 1e-3
    assert ((got - want).abs() <= want.abs() * 2.0 ** -7 + 1e-30).all()
    out = torch.zeros(1, device=DEV)
    F.sum_squares(g, out)
    assert abs(out.item() - g.float().pow(2).sum().item()) < 1e-3 * out.item()


def test_adamw_without_master_weights():
    """AdamW directly on bf16 parameters with bf16 moments (the reference's optimizer precision): the kernel against
    the CPU path of the same function and against torch's fused AdamW on a bf16 tensor."""
    F, nv = _F()
    torch.manual_seed(9)
    n = 8 * 4321
    p0 = torch.randn(n, dtype=torch.bfloat16) * 0.2
    p, pc = p0.to(DEV), p0.clone()
    m, v = torch.zeros(n, device=DEV, dtype=torch.bfloat16), torch.zeros(n, device=DEV, dtype=torch.bfloat16)
    mc, vc = torch.zeros(n, dtype=torch.bfloat16), torch.zeros(n, dtype=torch.bfloat16)
    q = torch.nn.Parameter(p0.to(DEV).clone())
    topt = torch.optim.AdamW([q], lr=1e-2, weight_decay=0.1, fused=True)
    for step in (1, 2, 3):
        g = (torch.randn(n) * 0.1).to(torch.bfloat16)
        F.adamw_step(p, g.to(DEV), None, m, v, n_decay=n, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1,
                     step=step)
        F.adamw_step(pc, g, None, mc, vc, n_decay=n, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.1,
                     step=step)
        q.grad = g.to(DEV)
        topt.step()
    for want in (pc.float(), q.detach().cpu().float()):
        got = p.cpu().float()
        assert (got != want).float().mean().item() < 2e-2            # rounding flips of single elements only
        # one bf16 step at the magnitude of the operands (weights up to ~0.5, updates of ~lr = 1e-2)
        assert ((got - want).abs() <= want.abs() * 2.0 ** -6 + 2e-4).all()
    assert rel_err(m.cpu().float(), mc.float()) < 1e-2 and rel_err(v.cpu().float(), vc.float()) < 1e-2


def test_native_library_is_loaded():
    import ctypes
    F, nv = _F()
    assert isinstance(nv.lib(), ctypes.CDLL)
    assert nv.lib().mmt_version().decode().startswith("mmt_b200")


@pytest.mark.parametrize("recompute", [True, False, "keep_all"])
@pytest.mark.parametrize("kind", ["vision", "text"])
def test_local_block_matches_per_op_graph(kind, recompute):
    """The one-node transformer block (hand-written backward) against the same block built from the per-op
    autograd functions: same kernels, so outputs and every gradient agree to rounding."""
    import math
    F, nv = _F()
    from multimodal_training_b200.ops import blocks
    from multimodal_training_b200.ops.attention import SeqInfo
    torch.manual_seed(11)
    if kind == "vision":
        n_q, n_kv, d, C, inter, causal, cu = 4, 4, 80, 320, 512, False, [0, 64, 128, 192, 300]
        has_bias = (True, True, True, True)
    else:
        n_q, n_kv, d, C, inter, causal, cu = 4, 2, 128, 512, 768, True, [0, 200, 456]
        has_bias = (True, False, False, False)
    T = cu[-1]
    W = (n_q + 2 * n_kv) * d

    def P(*shape, scale=0.05):
        return (torch.randn(*shape, device=DEV, dtype=torch.bfloat16) * scale).requires_grad_()

    def make():
        torch.manual_seed(12)
        return dict(ln1=P(C, scale=1.0), qkv_w=P(W, C), qkv_b=P(W) if has_bias[0] else None, o_w=P(C, n_q * d),
                    o_b=P(C) if has_bias[1] else None, ln2=P(C, scale=1.0), gu_w=P(2 * inter, C),
                    gu_b=P(2 * inter) if has_bias[2] else None, dn_w=P(C, inter), dn_b=P(C) if has_bias[3] else None)

    x0 = torch.randn(T, C, device=DEV, dtype=torch.bfloat16)
    dy = torch.randn(T, C, device=DEV, dtype=torch.bfloat16)
    cos = torch.rand(T, d, device=DEV, dtype=torch.float32)
    sin = torch.rand(T, d, device=DEV, dtype=torch.float32)
    seq = SeqInfo.from_list(cu, DEV)
    rope_heads = n_q + n_kv

    def per_op(x, p):
        h = F.rmsnorm(x, p["ln1"], 1e-6)
        qkv = F.rope(F.linear(h, p["qkv_w"], p["qkv_b"]), cos, sin, rope_heads, d)
        a = F.attention(qkv, n_q, n_kv, d, seq, causal=causal)
        x1 = F.linear(a, p["o_w"], p["o_b"], x)
        h2 = F.rmsnorm(x1, p["ln2"], 1e-6)
        m = F.swiglu(F.linear(h2, p["gu_w"], p["gu_b"]))
        return F.linear(m, p["dn_w"], p["dn_b"], x1)

    pa, pb = make(), make()
    xa = x0.clone().requires_grad_()
    ya = per_op(xa, pa)
    ya.backward(dy)
    xb = x0.clone().requires_grad_()
    spec = blocks.BlockSpec(n_q=n_q, n_kv=n_kv, head_dim=d, rope_heads=rope_heads, causal=causal, eps=1e-6,
                            scale=1.0 / math.sqrt(d))
    yb = blocks.local_block(xb, spec, cos, sin, seq, (pb["ln1"], pb["qkv_w"], pb["qkv_b"], pb["o_w"], pb["o_b"],
                                                      pb["ln2"], pb["gu_w"], pb["gu_b"], pb["dn_w"], pb["dn_b"]),
                           recompute=recompute is True, keep_elementwise=recompute == "keep_all")
    yb.backward(dy)
    assert nv.get_error()[0] == 0
    assert rel_err(yb, ya.float()) < 1e-3
    assert rel_err(xb.grad, xa.grad.float()) < 1e-2
    for k in pa:
        if pa[k] is not None:
            assert rel_err(pb[k].grad, pa[k].grad.float()) < 1e-2, k


@pytest.mark.parametrize("M,N,K", [(2048, 3584, 3584), (2048, 3584, 9472), (4096, 1280, 3424), (1000, 1176, 4096),
                                   (300, 520, 2048)])
@pytest.mark.parametrize("mt", [1, 2])
def test_gemm_stream_k_matches_whole_tiles(M, N, K, mt):
    """Tiles of a partial last wave are cut along K across all CTAs (fp32 partial sums, fixed order): same result
    as whole tiles up to fp32 summation order, on both tile heights, with bias and residual in the epilogue."""
    F, nv = _F()
    L = nv.lib()
    torch.manual_seed(3)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    ref = a.float() @ b.float().t() + bias.float() + res.float()
    L.mmt_gemm_force_mt(mt)
    try:
        L.mmt_gemm_set_stream_k(0)
        whole = F.gemm(a, b, bias=bias, residual=res)
        L.mmt_gemm_set_stream_k(1)
        cut1 = F.gemm(a, b, bias=bias, residual=res)
        cut2 = F.gemm(a, b, bias=bias, residual=res)
    finally:
        L.mmt_gemm_force_mt(0)
        L.mmt_gemm_set_stream_k(0)
    assert nv.get_error()[0] == 0, nv.get_error()
    assert rel_err(cut1, ref) < 1e-2 and rel_err(whole, ref) < 1e-2
    assert rel_err(cut1, whole.float()) < 1e-2      # one bf16 ulp of the largest outputs
    assert torch.equal(cut1, cut2)          # fixed summation order: bit-reproducible
