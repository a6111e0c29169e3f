"""Peer-memory kernels on ONE GPU: the ranks of a tensor-parallel group are emulated as separate
buffers of the same device, producers run to completion before any consumer is launched (so no kernel
ever waits on a kernel that has not been launched), and results are compared with plain PyTorch.
The multi-GPU behaviour of the same kernels is covered by ``tests/test_gpu_multi.py``."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _mods():
    from multimodal_training_b200.ops import functional as F
    from multimodal_training_b200.ops import native as nv
    from multimodal_training_b200.parallel import fused
    nv.lib()
    return F, nv, fused


def rel(a, b):
    return ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-9)).item()


def _peerset(fused, bases, flags, my_index):
    ps = fused.PeerSetC()
    ps.n = len(bases)
    for i, (b, f) in enumerate(zip(bases, flags)):
        ps.base[i] = b.data_ptr()
        ps.flag[i] = f.data_ptr() + 4 * my_index
    return ps


def test_allgather_gemm_with_fused_rmsnorm():
    F, nv, fused = _mods()
    torch.manual_seed(0)
    tp, rows, K, N = 2, 256, 512, 384
    x = [torch.randn(rows, K, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    nw = (1 + 0.1 * torch.randn(K, device=DEV)).to(torch.bfloat16)
    w = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05 for _ in range(tp)]
    gather = [torch.zeros(tp * rows, K, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    flags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(tp)]
    counters = [torch.zeros(1, device=DEV, dtype=torch.int32) for _ in range(tp)]
    rstd = [torch.empty(rows, device=DEV, dtype=torch.float32) for _ in range(tp)]
    for r in range(tp):      # producers
        ps = _peerset(fused, gather, flags, r)
        nv.call("mmt_rmsnorm_push", x[r].data_ptr(), nw.data_ptr(), rstd[r].data_ptr(), ctypes.byref(ps),
                counters[r].data_ptr(), 1, r * rows, rows, K, 1e-6, nv.stream())
    torch.cuda.synchronize()
    xf = torch.cat(x).float()
    href = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    for r in range(tp):      # consumers
        assert flags[r][:tp].tolist() == [1] * tp
        c = fused.GemmCommC()
        c.ag_flags, c.ag_epoch, c.ag_rows, c.ag_self, c.rs_rows = flags[r].data_ptr(), 1, rows, r, 0
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        y = F.gemm(gather[r], w[r])
        assert rel(gather[r], href) < 1e-2
        assert rel(y, href @ w[r].float().t()) < 1e-2
    assert nv.get_error()[0] == 0


@pytest.mark.parametrize("direct", [False, True])
@pytest.mark.parametrize("tp,rows,K,N", [(2, 512, 512, 384), (4, 1024, 1280, 640), (2, 2048, 3584, 1152),
                                          (2, 2048, 3584, 9472), (2, 4096, 512, 5376), (4, 2048, 256, 5120)])
def test_allgather_inside_the_gemm(tp, rows, K, N, direct):
    """The all-gather fused INTO the consuming GEMM: the CTAs that compute the first column tile of this rank's own
    rows forward every A tile they load to the peers' gather buffers (bulk stores from shared memory) and raise one
    flag per row block; the TMA producer waits per (source rank, row block) before reading a peer's rows.  Ranks are
    emulated on one GPU one after the other: the rows and flags a rank waits for are put in place by the host before
    its launch (no launch ever waits for another), and what it forwards lands in separate buffers that are checked
    afterwards.  ``direct``: own rows are read from the shard itself and also stored to the rank's own gather buffer."""
    F, nv, fused = _mods()
    torch.manual_seed(rows + K)
    counter = torch.zeros(64, device=DEV, dtype=torch.int32)
    h = torch.randn(tp * rows, K, device=DEV, dtype=torch.bfloat16)
    w = [torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05 for _ in range(tp)]
    land = [torch.full((tp * rows, K), float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    landflags = [torch.zeros(8 * 64, device=DEV, dtype=torch.int32) for _ in range(tp)]
    for r in range(tp):
        gathered = h.clone()
        flags = torch.ones(8 * 64, device=DEV, dtype=torch.int32)          # every peer's blocks have "arrived"
        c = fused.GemmCommC()
        c.ag_flags, c.ag_epoch, c.ag_rows, c.ag_self, c.rs_rows = flags.data_ptr(), 1, rows, r, 0
        peers = [q for q in range(tp) if q != r]
        for i, q in enumerate(peers):
            c.fwd_dst[i] = land[q].data_ptr()
            c.fwd_flag[i] = landflags[q].data_ptr()
        c.fwd_peers = len(peers)
        c.fwd_counter = counter.data_ptr()
        shard = h[r * rows:(r + 1) * rows].clone()
        if direct:
            gathered[r * rows:(r + 1) * rows] = float("nan")               # filled by the kernel itself
            c.fwd_src, c.fwd_src_ld = shard.data_ptr(), K
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        y = F.gemm(gathered, w[r])
        torch.cuda.synchronize()
        assert rel(y, h.float() @ w[r].float().t()) < 1e-2
        assert torch.equal(gathered, h) and int(counter.abs().sum()) == 0
    for q in range(tp):
        got = landflags[q].view(8, 64)
        for r in range(tp):
            mine = land[q][r * rows:(r + 1) * rows]
            if r == q:
                assert bool(torch.isnan(mine).all()) and int(got[r].sum()) == 0      # nobody forwards to itself
                continue
            assert torch.equal(mine, h[r * rows:(r + 1) * rows])                    # bit-exact copies of the rows
            n = int(got[r].sum())
            assert n in (rows // 128, rows // 256) and bool((got[r, :n] == 1).all())  # one flag per tile-high block
        assert int(got[tp:].sum()) == 0
    assert nv.get_error()[0] == 0


def _piecewise_rows(n_rows, total, pieces, gen):
    """``n_rows`` destination rows inside [0, total) made of ``pieces`` runs of consecutive rows (how a rank's rows of
    several images sit in the image-major order)."""
    cuts = sorted(torch.randperm(n_rows - 1, generator=gen)[:pieces - 1].add(1).tolist()) if pieces > 1 else []
    lens = [b - a for a, b in zip([0] + cuts, cuts + [n_rows])]
    gaps = total - n_rows
    starts, pos = [], 0
    for i, ln in enumerate(lens):
        pos += int(torch.randint(0, gaps // len(lens) + 1, (1,), generator=gen))
        starts.append(pos)
        pos += ln
    return torch.cat([torch.arange(s0, s0 + ln) for s0, ln in zip(starts, lens)]).to(torch.int32)


@pytest.mark.parametrize("sp,C,rows,pieces", [(2, 1280, 1024, 1), (4, 1280, 1000, 3), (8, 1280, 777, 4), (2, 128, 300, 2)])
def test_qkv_gemm_scatters_heads_to_their_owners(sp, C, rows, pieces):
    """Ulysses sequence -> heads exchange as the epilogue of the QKV projection: column block r of q, k and v goes to
    rank r's [T_all, 3 * W] buffer at the row's position in the image-major order.  Slabs with one owner and 32
    consecutive destination rows leave as bulk stores, the rest (ragged pieces, W = 160) as 16-byte stores.  Ranks are
    emulated one after the other on one GPU."""
    F, nv, fused = _mods()
    gen = torch.Generator().manual_seed(sp * 1000 + rows)
    W, K = C // sp, 256
    t_all = rows * sp + 64
    w = (torch.randn(3 * C, K, generator=gen) * 0.05).to(DEV, torch.bfloat16)
    b = (torch.randn(3 * C, generator=gen) * 0.1).to(DEV, torch.bfloat16)
    dst = [torch.full((t_all, 3 * W), float("nan"), device=DEV, dtype=torch.bfloat16) for _ in range(sp)]
    flags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(sp)]
    counter = torch.zeros(1, device=DEV, dtype=torch.int32)
    want = [torch.full((t_all, 3 * W), float("nan")) for _ in range(sp)]
    band = t_all // sp
    for r in range(sp):
        h = (torch.randn(rows, K, generator=gen)).to(DEV, torch.bfloat16)
        row_map = (_piecewise_rows(rows, band, pieces, gen) + r * band).to(DEV)
        c = fused.GemmCommC()
        c.rs_rows, c.rs_self, c.rs_ranks, c.rs_epoch = 0, r, sp, 1
        c.rs_counter = counter.data_ptr()
        for i in range(sp):
            c.rs_base[i] = dst[i].data_ptr()
            c.rs_flag[i] = flags[i].data_ptr() + 4 * r
        c.sc_row, c.sc_part, c.sc_w, c.sc_ld, c.sc_rows_dst = row_map.data_ptr(), C, W, 3 * W, t_all
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(h, w, bias=b, out=torch.empty(8, 3 * C, device=DEV, dtype=torch.bfloat16))
        torch.cuda.synchronize()
        ref = (h.float() @ w.float().t() + b.float()).cpu().view(rows, 3, sp, W)
        for g in range(sp):
            want[g][row_map.cpu().long()] = ref[:, :, g, :].reshape(rows, 3 * W)
    for g in range(sp):
        got = dst[g].cpu().float()
        assert torch.equal(torch.isnan(got), torch.isnan(want[g]))               # exactly the rows that were sent
        ok = ~torch.isnan(want[g])
        assert rel(got[ok], want[g][ok]) < 1e-2
        assert flags[g][:sp].tolist() == [1] * sp and int(counter.item()) == 0
    assert nv.get_error()[0] == 0


@pytest.mark.parametrize("sp,C,self_rank", [(2, 1280, 1), (4, 1280, 2), (8, 1280, 5), (2, 256, 0)])
def test_out_projection_reads_k_slices_behind_flags(sp, C, self_rank):
    """Ulysses heads -> sequence exchange in front of the output projection: columns [s * W, (s + 1) * W) of A come
    from rank s; the GEMM walks its k-blocks starting with its own slice and waits per source (flags are set by the
    host here).  The result is the plain GEMM's."""
    F, nv, fused = _mods()
    torch.manual_seed(sp + C)
    rows, N = 900, 320
    a = torch.randn(rows, C, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, C, device=DEV, dtype=torch.bfloat16) * 0.05
    res = torch.randn(rows, N, device=DEV, dtype=torch.bfloat16)
    flags = torch.full((8,), 3, device=DEV, dtype=torch.int32)
    c = fused.GemmCommC()
    c.kf_flags, c.kf_epoch, c.kf_w, c.kf_self, c.kf_ranks = flags.data_ptr(), 3, C // sp, self_rank, sp
    c.rs_rows = 0
    nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
    y = F.gemm(a, w, residual=res)
    assert rel(y, a.float() @ w.float().t() + res.float()) < 1e-2
    assert nv.get_error()[0] == 0


def test_gemm_reduce_scatter_with_residual():
    F, nv, fused = _mods()
    torch.manual_seed(1)
    tp, T, Kl, N = 2, 512, 256, 640
    rows = T // tp
    a = [torch.randn(T, Kl, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    w = [torch.randn(N, Kl, device=DEV, dtype=torch.bfloat16) * 0.05 for _ in range(tp)]
    res = [torch.randn(rows, N, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    staging = [torch.zeros(tp * rows, N, device=DEV, dtype=torch.bfloat16) for _ in range(tp)]
    flags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(tp)]
    counters = [torch.zeros(1, device=DEV, dtype=torch.int32) for _ in range(tp)]
    for r in range(tp):      # producers: GEMM epilogues store partial tiles into the owners' staging slots
        c = fused.GemmCommC()
        c.ag_flags = None
        c.rs_rows, c.rs_self, c.rs_ranks, c.rs_epoch = rows, r, tp, 1
        c.rs_counter = counters[r].data_ptr()
        for i in range(tp):
            c.rs_base[i] = staging[i].data_ptr()
            c.rs_flag[i] = flags[i].data_ptr() + 4 * r
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(a[r], w[r], out=staging[r][:T])
    torch.cuda.synchronize()
    full = sum(a[r].float() @ w[r].float().t() for r in range(tp))
    for r in range(tp):      # owners
        out = torch.empty(rows, N, device=DEV, dtype=torch.bfloat16)
        nv.call("mmt_rs_reduce", staging[r].data_ptr(), flags[r].data_ptr(), 1, tp, r, res[r].data_ptr(),
                out.data_ptr(), rows, N, nv.stream())
        assert rel(out, full[r * rows:(r + 1) * rows] + res[r].float()) < 1.5e-2
    assert nv.get_error()[0] == 0


def test_route_rows_and_wait():
    F, nv, fused = _mods()
    torch.manual_seed(2)
    world, H = 3, 256
    src = [torch.randn(40 + 8 * r, H, device=DEV, dtype=torch.bfloat16) for r in range(world)]
    region = [torch.zeros(200, H, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(world)]
    counters = [torch.zeros(1, device=DEV, dtype=torch.int32) for _ in range(world)]
    expect = [torch.zeros(200, H, device=DEV, dtype=torch.bfloat16) for _ in range(world)]
    nxt = [0] * world
    keep = []
    for r in range(world):
        n = src[r].shape[0]
        dr = torch.randint(0, world, (n,), dtype=torch.int32)
        drow = torch.empty(n, dtype=torch.int64)
        for i in range(n):
            d = int(dr[i])
            drow[i] = nxt[d]
            expect[d][nxt[d]] = src[r][i]
            nxt[d] += 1
        ps = _peerset(fused, region, flags, r)
        dr_d, drow_d = dr.to(DEV), drow.to(DEV)      # keep the device copies alive across the launch
        keep.append((dr_d, drow_d))
        nv.call("mmt_route_rows", src[r].data_ptr(), dr_d.data_ptr(), drow_d.data_ptr(), ctypes.byref(ps),
                counters[r].data_ptr(), 1, n, H, H, H, 200, nv.stream())
    torch.cuda.synchronize()
    for r in range(world):
        nv.call("mmt_wait_flags", flags[r].data_ptr(), world, -1, 1, nv.stream())
        assert torch.equal(region[r], expect[r])
    assert nv.get_error()[0] == 0
    # a destination row outside the region is skipped and reported, never stored
    ps = _peerset(fused, region, flags, 0)
    bad_rank = torch.zeros(8, device=DEV, dtype=torch.int32)
    bad_row = torch.full((8,), 10 ** 9, device=DEV, dtype=torch.int64)
    nv.call("mmt_route_rows", src[0].data_ptr(), bad_rank.data_ptr(), bad_row.data_ptr(), ctypes.byref(ps),
            counters[0].data_ptr(), 2, 8, H, H, H, 200, nv.stream())
    torch.cuda.synchronize()
    code, where = nv.get_error()[:2]
    assert (code, where) == (3, 920)
    nv.lib().mmt_clear_error()
    assert torch.equal(region[0], expect[0])


def test_zero1_adamw_matches_reduce_then_adamw():
    F, nv, fused = _mods()
    torch.manual_seed(3)
    ranks, n = 2, 8 * 4096
    total = ranks * n
    grads = [torch.randn(total, device=DEV, dtype=torch.bfloat16) * 0.1 for _ in range(ranks)]
    p0 = torch.randn(total, device=DEV, dtype=torch.bfloat16)
    params = [p0.clone() for _ in range(ranks)]
    gflags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(ranks)]
    pflags = [torch.zeros(8, device=DEV, dtype=torch.int32) for _ in range(ranks)]
    counters = [torch.zeros(1, device=DEV, dtype=torch.int32) for _ in range(ranks)]
    for r in range(ranks):           # "backward complete" published by everyone first
        ps = _peerset(fused, grads, gflags, r)
        nv.call("mmt_publish", ctypes.byref(ps), 1, nv.stream())
    torch.cuda.synchronize()
    gsum = sum(g.float() for g in grads)
    ref_p = p0.clone()
    for r in range(ranks):
        lo = r * n
        master = p0[lo:lo + n].float().clone()
        m, v = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        zp = fused.ZeroPeersC()
        zp.n = ranks
        for i in range(ranks):
            zp.grad[i], zp.param[i] = grads[i].data_ptr(), params[i].data_ptr()
            zp.param_flag[i] = pflags[i].data_ptr() + 4 * r
        nv.call("mmt_zero1_adamw", ctypes.byref(zp), gflags[r].data_ptr(), 1, r, counters[r].data_ptr(), 1,
                master.data_ptr(), m.data_ptr(), v.data_ptr(), lo, n, n // 2, 1e-2, 0.9, 0.999, 1e-8, 0.1, 1, None,
                None, nv.stream())
        # reference: reduced gradient (bf16 inputs, fp32 sum) then the plain fused AdamW kernel
        rm = p0[lo:lo + n].float().clone()
        rmm, rv = torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
        rp = p0[lo:lo + n].clone()
        gs = gsum[lo:lo + n]
        rmm.mul_(0.9).add_(gs, alpha=0.1)
        rv.mul_(0.999).addcmul_(gs, gs, value=0.001)
        upd = (rmm / 0.1) / ((rv / 0.001).sqrt() + 1e-8)
        wd = torch.zeros(n, device=DEV)
        wd[: n // 2] = 0.1
        rm -= 1e-2 * (upd + wd * rm)
        ref_p[lo:lo + n] = rm.to(torch.bfloat16)
        assert rel(master, rm) < 1e-5
    torch.cuda.synchronize()
    for r in range(ranks):
        assert pflags[r][:ranks].tolist() == [1] * ranks
        assert rel(params[r], ref_p) < 1e-2
    assert nv.get_error()[0] == 0


def test_bounded_wait_reports_instead_of_hanging():
    """A flag that nothing sets: the kernel gives up at its deadline, records where, and the context stays usable."""
    F, nv, fused = _mods()
    flags = torch.zeros(8, device=DEV, dtype=torch.int32)
    nv.lib().mmt_clear_error()
    nv.call("mmt_wait_flags", flags.data_ptr(), 2, -1, 5, nv.stream())
    code, where, _, aux = nv.get_error()
    assert code == 2 and where == 910 and aux == 5
    nv.lib().mmt_clear_error()
    x = torch.ones(16, device=DEV)
    assert float(x.sum()) == 16.0
    with pytest.raises(RuntimeError):
        flags.zero_()
        nv.call("mmt_wait_flags", flags.data_ptr(), 1, -1, 1, nv.stream())
        nv.raise_on_device_error()
    assert nv.get_error()[0] == 0
