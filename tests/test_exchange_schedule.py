"""Reuse of the symmetric-heap regions by the tensor-parallel layer, checked on the REAL call order.

``parallel/fused.py`` reuses one heap region per exchange role for every layer and never inserts a barrier: safety
rests on the order of the exchanges.  This test extracts that order from the code itself -- it runs
``ops/tp_blocks.py``'s forward and backward with a recording stand-in for ``FusedComm`` and stubs for the compute
kernels -- and replays the resulting per-rank programs on a simulated group in which ranks advance in arbitrary
interleavings (including one rank lagging as far behind as its peers' waits allow).  Checked at every step:

* no rank writes a new epoch into a peer's region while that peer still has an unexecuted reader of the previous
  epoch (a GEMM consuming gathered rows, a weight-gradient GEMM, a reduction of staged partial sums);
* no schedule deadlocks (every wait is eventually satisfied).
"""
import random

import pytest
import torch

from multimodal_training_b200.ops import tp_blocks
from multimodal_training_b200.ops.blocks import BlockSpec


class RecorderFC:
    """Stands in for FusedComm: hands out small CPU tensors and records which region/epoch they are views of."""

    fused_ag = True                   # all-gathers run inside the consuming GEMM (one op: store to all, then read)

    def __init__(self):
        self.ops = []                 # the program: ("push", role, epoch) / ("read", region, epoch, waits) / ...
        self.epochs = {}
        self.region_of = {}           # id(tensor) -> (region name, epoch)
        self.keepalive = []

    def _epoch(self, region):
        self.epochs[region] = self.epochs.get(region, 0) + 1
        return self.epochs[region]

    def push_gather(self, x_shard, norm_w, eps, role):
        region = "ag_" + role
        e = self._epoch(region)
        self.ops.append(("write_all", region, e))                  # my rows into every peer's region, then flags
        g = torch.zeros(4, x_shard.shape[1])
        self.region_of[id(g)] = (region, e)
        self.keepalive.append(g)
        return g, (torch.ones(x_shard.shape[0]) if norm_w is not None else None), 0, e

    def ag_gemm(self, x_shard, norm_w, eps, w, *, role, bias=None, b_mn=False):
        g, rstd, _, e = self.push_gather(x_shard, norm_w, eps, role)
        y = self.gemm_gathered(g, 0, e, x_shard.shape[0], w, b_mn=b_mn, bias=bias)
        return y, g, rstd

    def gemm_gathered(self, gathered, flags, epoch, rows, w, *, b_mn=False, bias=None):
        region, e = self.region_of[id(gathered)]
        assert e == epoch
        self.ops.append(("read", region, e, True))                 # waits for every peer's flag of this epoch
        n = w.shape[1] if b_mn else w.shape[0]
        return torch.zeros(gathered.shape[0], n)

    def gemm_reduce_scatter(self, a, w, *, b_mn, residual, role):
        region = "rs_" + role
        e = self._epoch(region)
        self.note_reads(a, w)
        self.ops.append(("write_all", region, e))                  # partial tiles into every owner's staging slot
        self.ops.append(("read", region, e, True))                 # rs_reduce: waits for all flags, sums the slots
        n = w.shape[1] if b_mn else w.shape[0]
        return torch.zeros(max(a.shape[0] // 2, 1), n)

    def note_reads(self, *tensors):
        for t in tensors:
            hit = self.region_of.get(id(t))
            if hit is not None:
                self.ops.append(("read", hit[0], hit[1], False))   # a plain read of a heap view (no wait)


class FakeCtx:
    def save_for_backward(self, *t):
        self.saved_tensors = t


def _program(layers: int, recompute: bool, monkeypatch):
    """Run tp_blocks forward over ``layers`` layers and backward in reverse; return the recorded op list."""
    fc = RecorderFC()
    H, rows = 8, 2
    z = lambda *s: torch.zeros(*s)  # noqa: E731
    monkeypatch.setattr(tp_blocks, "_rope_", lambda *a, **k: None)
    monkeypatch.setattr(tp_blocks, "_attn_fwd", lambda qkv, s, seq: (z(qkv.shape[0], H), z(1, qkv.shape[0])))
    monkeypatch.setattr(tp_blocks, "_attn_bwd", lambda qkv, a, da, lse, s, seq: z(*qkv.shape))
    monkeypatch.setattr(tp_blocks, "_swiglu_fwd", lambda gu: z(gu.shape[0], gu.shape[1] // 2))
    monkeypatch.setattr(tp_blocks, "_swiglu_bwd", lambda dm, gu: z(*gu.shape))
    monkeypatch.setattr(tp_blocks, "_rmsnorm_bwd", lambda dy, x, w, rstd, extra: z(*x.shape))
    monkeypatch.setattr(tp_blocks, "_grad_into", lambda p, compute: compute(z(*p.shape), False))

    def fake_gemm(a, b, **kw):
        fc.note_reads(a, b)
        return kw.get("out", z(1, 1))
    monkeypatch.setattr(tp_blocks.F, "gemm", fake_gemm)
    monkeypatch.setattr(tp_blocks.F, "colsum", lambda x, **kw: None)
    spec = BlockSpec(n_q=1, n_kv=1, head_dim=H, rope_heads=2, causal=True, eps=1e-6, scale=1.0)
    P = (z(H), z(3 * H, H), z(3 * H), z(H, H), z(H), z(4 * H, H), z(H, 2 * H))
    ctxs = []
    x = z(rows, H)
    for _ in range(layers):
        ctx = FakeCtx()
        x = tp_blocks._TPBlockFn.forward(ctx, x, spec, z(1), z(1), None, recompute, fc, *P)
        ctxs.append(ctx)
    dy = z(rows, H)
    for ctx in reversed(ctxs):
        dy = tp_blocks._TPBlockFn.backward(ctx, dy)[0]
    return fc.ops


def _replay(program, n_ranks: int, rng: random.Random, laggard=None):
    """Every rank runs ``program``; an op runs when its waits are satisfied; ranks are picked at random (the laggard
    only when nobody else can move).  Returns the number of executed ops; raises AssertionError on a hazard."""
    pc = [0] * n_ranks
    written = {}                      # (dst rank, region) -> {src rank: highest epoch written}
    # for every rank: indices of its reader ops per (region, epoch)
    readers = {}
    for i, op in enumerate(program):
        if op[0] == "read":
            readers.setdefault((op[1], op[2]), []).append(i)

    def runnable(r):
        if pc[r] >= len(program):
            return False
        op = program[pc[r]]
        if op[0] == "read" and op[3]:
            return all(written.get((r, op[1]), {}).get(s, 0) >= op[2] for s in range(n_ranks))
        return True

    done = 0
    while any(p < len(program) for p in pc):
        cand = [r for r in range(n_ranks) if runnable(r)]
        assert cand, f"deadlock at {pc}: {[program[p] if p < len(program) else None for p in pc]}"
        others = [r for r in cand if r != laggard]
        r = rng.choice(others) if others else cand[0]
        op = program[pc[r]]
        if op[0] == "write_all":
            _, region, e = op
            for dst in range(n_ranks):
                # the previous epoch of this region on `dst` must have no reader left to run
                for i in readers.get((region, e - 1), []):
                    assert pc[dst] > i, (f"rank {r} writes epoch {e} of {region} into rank {dst}, whose reader of "
                                         f"epoch {e - 1} (op {i}: {program[i]}) has not run yet (rank {dst} is at op "
                                         f"{pc[dst]})")
                written.setdefault((dst, region), {})[r] = e
        pc[r] += 1
        done += 1
    return done


@pytest.mark.parametrize("recompute", [True, False])
def test_region_reuse_is_safe_under_any_interleaving(monkeypatch, recompute):
    program = _program(layers=3, recompute=recompute, monkeypatch=monkeypatch)
    regions = {op[1] for op in program}
    assert {"ag_qkv", "ag_mlp", "rs_o", "rs_down", "ag_down_bwd", "rs_mlp_bwd", "ag_o_bwd", "rs_qkv_bwd"} <= regions
    if recompute:
        # heap views are read by the weight-gradient GEMMs (no private copies in this mode)
        assert any(op[0] == "read" and not op[3] and op[1] == "ag_qkv" for op in program)
    for n_ranks in (2, 4):
        for seed in range(40):
            _replay(program, n_ranks, random.Random(seed))
        for lag in range(n_ranks):
            _replay(program, n_ranks, random.Random(100 + lag), laggard=lag)


def test_the_checker_catches_an_unsafe_order(monkeypatch):
    """Moving a weight-gradient read of the gathered input behind the exchange that releases the peers is the bug the
    ordering rule prevents: the replay must flag it."""
    program = _program(layers=2, recompute=True, monkeypatch=monkeypatch)
    # find a plain read of ag_qkv in backward and move it to the end of the program
    i = max(k for k, op in enumerate(program) if op[0] == "read" and not op[3] and op[1] == "ag_qkv"
            and op[2] < max(o[2] for o in program if o[1] == "ag_qkv"))
    bad = program[:i] + program[i + 1:] + [program[i]]
    with pytest.raises(AssertionError, match="has not run yet"):
        for seed in range(60):
            _replay(bad, 2, random.Random(seed), laggard=0)


# ------------------------------------------------------------------------------------------------------------------
# The same check for the vision encoder's full-attention layers (ops/ulysses_block.py): four regions
# (ul_heads3, ul_tokens1, ul_heads1_bwd, ul_tokens3_bwd), each reused by every full-attention layer.
# ------------------------------------------------------------------------------------------------------------------
class RecorderUF:
    """Stands in for UlyssesFused: records writes into every peer's region and reads of this rank's region."""

    sp, sp_rank = 2, 0

    def __init__(self):
        self.ops, self.epochs, self.region_of, self.keepalive = [], {}, {}, []

    def _new(self, region, rows, cols):
        self.epochs[region] = self.epochs.get(region, 0) + 1
        e = self.epochs[region]
        self.ops.append(("write_all", region, e))
        t = torch.zeros(rows, cols)
        self.region_of[id(t)] = (region, e)
        self.keepalive.append(t)
        return t, e

    def _routes(self, plan, device):
        return {"t_all": 4, "t_loc_max": 2}

    def rope_tables(self, plan, device):
        return torch.zeros(1), torch.zeros(1)

    def gemm_scatter(self, a, w, bias, parts, routes, name, b_mn=False):
        self.note_reads(a, w)
        t, e = self._new(name, 4, parts * 4)
        self.ops.append(("read", name, e, True))                   # the wait behind the GEMM
        return t

    def to_tokens_nowait(self, src, W, routes, name):
        self.note_reads(src)
        t, e = self._new(name, 2, 8)
        return t, name, e

    def gemm_k_slices(self, a, w, bias, residual, flags, epoch, W):
        self.ops.append(("read", flags, epoch, True))              # waits per source inside the GEMM
        return torch.zeros(a.shape[0], 8)

    def _exchange(self, kind, src, parts, W, routes, name):
        self.note_reads(src)
        t, e = self._new(name, 2, parts * 8)
        self.ops.append(("read", name, e, True))
        return t

    def note_reads(self, *tensors):
        for t in tensors:
            base = t if id(t) in self.region_of else getattr(t, "_base", None)
            hit = self.region_of.get(id(base)) if base is not None else None
            if hit is not None:
                self.ops.append(("read", hit[0], hit[1], False))


def _ulysses_program(layers: int, recompute: bool, monkeypatch):
    from multimodal_training_b200.ops import ulysses_block as ub
    uf = RecorderUF()
    C = 8
    z = lambda *s: torch.zeros(*s)  # noqa: E731
    monkeypatch.setattr(ub, "_rope_", lambda t, *a, **k: uf.note_reads(t))
    monkeypatch.setattr(ub, "_rmsnorm_fwd", lambda x, w, eps: (z(*x.shape), z(x.shape[0])))
    monkeypatch.setattr(ub, "_rmsnorm_bwd", lambda dy, x, w, rstd, extra: z(*x.shape))
    monkeypatch.setattr(ub, "_swiglu_fwd", lambda gu: z(gu.shape[0], gu.shape[1] // 2))
    monkeypatch.setattr(ub, "_swiglu_bwd", lambda dm, gu: z(*gu.shape))
    monkeypatch.setattr(ub, "_grad_into", lambda p, compute: compute(z(*p.shape), False))

    def attn_fwd(qkv, s, seq):
        uf.note_reads(qkv)
        return z(qkv.shape[0], 4), z(1, qkv.shape[0])

    def attn_bwd(qkv, a, da, lse, s, seq):
        uf.note_reads(qkv, a, da)
        return z(*qkv.shape)

    def linear_bwd(dy, x, w, b):
        uf.note_reads(dy, x)
        return z(dy.shape[0], w.shape[1])
    monkeypatch.setattr(ub, "_attn_fwd", attn_fwd)
    monkeypatch.setattr(ub, "_attn_bwd", attn_bwd)
    monkeypatch.setattr(ub, "_linear_bwd", linear_bwd)

    def fake_gemm(a, b, **kw):
        uf.note_reads(a, b)
        n = b.shape[1] if kw.get("b_mn") else b.shape[0]
        return kw.get("out", z(a.shape[0], n))
    monkeypatch.setattr(ub.F, "gemm", fake_gemm)
    monkeypatch.setattr(ub.F, "colsum", lambda x, **kw: None)
    spec = BlockSpec(n_q=2, n_kv=2, head_dim=4, rope_heads=4, causal=False, eps=1e-6, scale=1.0)
    spec_h = BlockSpec(n_q=1, n_kv=1, head_dim=4, rope_heads=2, causal=False, eps=1e-6, scale=1.0)
    P = (z(C), z(3 * C, C), z(3 * C), z(C, C), z(C), z(C), z(4 * C, C), z(4 * C), z(C, 2 * C), z(C))
    ctxs, x = [], z(2, C)
    for _ in range(layers):
        ctx = FakeCtx()
        x = ub._UlyssesBlockFn.forward(ctx, x, spec, spec_h, None, None, recompute, uf, *P)
        ctxs.append(ctx)
    dy = z(2, C)
    for ctx in reversed(ctxs):
        dy = ub._UlyssesBlockFn.backward(ctx, dy)[0]
    return uf.ops


@pytest.mark.parametrize("recompute", [True, False])
def test_ulysses_layer_region_reuse_is_safe_under_any_interleaving(monkeypatch, recompute):
    program = _ulysses_program(layers=3, recompute=recompute, monkeypatch=monkeypatch)
    regions = {op[1] for op in program}
    assert {"ul_heads3", "ul_tokens1", "ul_heads1_bwd", "ul_tokens3_bwd"} <= regions
    if recompute:
        # backward reads the heap views that its own recomputation produced (no private copies in this mode)
        assert any(op[0] == "read" and not op[3] and op[1] == "ul_heads3" for op in program)
        assert any(op[0] == "read" and not op[3] and op[1] == "ul_tokens1" for op in program)
    for n_ranks in (2, 4):
        for seed in range(40):
            _replay(program, n_ranks, random.Random(seed))
        for lag in range(n_ranks):
            _replay(program, n_ranks, random.Random(200 + lag), laggard=lag)
