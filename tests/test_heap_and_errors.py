"""Host-side rules of the symmetric heap (regions that grow, move and stay aligned across ranks) and of the device
error word on the training path; no GPU needed."""

import ctypes

import pytest
import torch

from multimodal_training_b200.parallel.symm import RegionAllocator


def test_regions_grow_move_and_reuse_freed_blocks():
    a = RegionAllocator(1 << 20)
    x0 = a.alloc("x", 1000)
    y0 = a.alloc("y", 5000)
    assert x0 == 0 and y0 % 1024 == 0 and y0 >= 1000
    assert a.alloc("x", 800) == x0                      # a smaller batch keeps the region where it is
    v = a.version
    assert a.alloc("x", 1000) == x0 and a.version == v   # nothing changed: no new layout to verify
    x1 = a.alloc("x", 3000)                             # a longer batch: the region moves
    assert x1 != x0 and x1 >= y0 + 5000 and a.version > v
    z = a.alloc("z", 900)                               # the freed block of x is reused
    assert z == x0
    with pytest.raises(MemoryError):
        a.alloc("huge", 2 << 20)


def test_ranks_that_issue_the_same_requests_get_the_same_layout():
    # ragged batches: every rank asks for the step's world-wide maxima, so their tables are identical however the
    # step sizes rise and fall; a rank that sized a region from its own token count would drift
    sizes = [(4096, 300), (8192, 280), (2048, 512), (8192, 512), (16384, 100)]
    ranks = [RegionAllocator(1 << 26) for _ in range(4)]
    for shard, merged in sizes:
        for a in ranks:
            for name, n in (("ag_qkv", shard * 64), ("rs_o", shard * 64), ("handoff_in", shard * 16),
                            ("handoff_grad", merged * 16)):
                a.alloc(name, n)
        assert len({a.digest() for a in ranks}) == 1
    drifting, good = RegionAllocator(1 << 26), RegionAllocator(1 << 26)
    differs = []
    for (shard, merged), own in zip(sizes, [299, 280, 511, 512, 99]):     # sized from its OWN merged-token count
        for a, m in ((drifting, own), (good, merged)):
            for name, n in (("ag_qkv", shard * 64), ("rs_o", shard * 64), ("handoff_in", shard * 16),
                            ("handoff_grad", m * 16)):
                a.alloc(name, n)
        differs.append(drifting.digest() != good.digest())
    assert any(differs)                                  # which verify_layout would report on a real job


def test_region_plan_is_identical_on_every_rank_of_a_ragged_step():
    """Step contexts of all ranks of a job with images of different sizes: the plan of exchange buffers that each
    rank derives (``FusedComm.region_plan``) must be the same list, also where a rank's own share is smaller."""
    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.data.synthetic import synthetic_sample
    from multimodal_training_b200.parallel.fused import FusedComm
    from multimodal_training_b200.parallel.mesh import Mesh
    from multimodal_training_b200.trainers.context import build_step_context

    cfg = get_model_config("tiny")
    samples = [synthetic_sample(cfg, i, image_size=s, text_tokens=t, seed=0)
               for i, (s, t) in enumerate([(224, 37), (336, 64), (448, 20), (280, 51)])]
    plans, merged = [], []
    for rank in range(4):
        mesh = Mesh(world=4, rank=rank, sp=2, tp=2)
        ctx = build_step_context(0, samples, cfg, mesh)
        fc = FusedComm.__new__(FusedComm)
        fc.mesh, fc.text_hidden, fc.vision_hidden, fc.ulysses = mesh, cfg.text.hidden_size, cfg.vision.hidden_size, True
        plans.append(fc.region_plan(ctx.sizes))
        merged.append(ctx.vision_plan.local_merged_ids.numel())
        assert ctx.sizes.merged_rows >= merged[-1] and ctx.sizes.shard_rows >= ctx.handoff.shard_rows
    assert len(set(merged)) > 1                         # the ranks really hold different numbers of merged tokens
    assert all(p == plans[0] for p in plans[1:])
    names = [n for n, _ in plans[0]]
    assert "handoff_grad" in names and "ul_heads3" in names and "rs_down" in names


def test_a_set_error_word_aborts_the_loop_when_the_loss_is_read():
    from multimodal_training_b200.engine import DeviceStepError, LossHandle

    ok = LossHandle(torch.tensor([1.5]), None, torch.zeros(4, dtype=torch.int32))
    assert ok.value() == 1.5
    bad = LossHandle(torch.tensor([1.5]), None, torch.tensor([2, 910, 0, 7], dtype=torch.int32))
    with pytest.raises(DeviceStepError, match="peer's flag"):
        bad.value()
    losses = []
    with pytest.raises(DeviceStepError):
        for h in (ok, bad, ok):                          # the loop stops at the failed step
            losses.append(h.value())
    assert losses == [1.5]


def test_a_failed_checkpoint_load_puts_the_old_weights_back(tmp_path):
    from multimodal_training_b200.trainers.trainer import Trainer

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.Parameter(torch.ones(3))
            self.b = torch.nn.Parameter(torch.ones(3))

    tr = Trainer.__new__(Trainer)
    tr.config, tr.rank, tr.kind, tr.optimizer, tr.global_step = {"device": "cpu"}, 0, "text", None, 0
    tr.model = Tiny()

    def load(sd, sharded):                               # loads the first tensor, then finds the shard broken
        with torch.no_grad():
            tr.model.a.copy_(sd["a"])
        raise KeyError("b")

    tr._load_model_state = load
    path = tmp_path / "epoch_0" / "text"
    path.mkdir(parents=True)
    torch.save({"model": {"a": torch.full((3,), 7.0)}}, path / "rank_0.pt")
    assert tr.load_checkpoint(str(tmp_path), 0) is False
    assert torch.equal(tr.model.a.detach(), torch.ones(3)) and torch.equal(tr.model.b.detach(), torch.ones(3))


def test_region_allocator_invariants_under_random_request_streams():
    """Property check (hypothesis): whatever the stream of (name, size) requests, live regions never overlap, stay
    inside the heap and aligned, a request that fits returns the same offset again, and two allocators fed the same
    stream (two ranks) end with the same table and digest."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    from multimodal_training_b200.parallel.symm import RegionAllocator

    names = st.sampled_from(["ag_qkv", "ag_mlp", "rs_o", "rs_down", "handoff_in", "ul_heads3", "ul_tokens1"])
    sizes = st.integers(min_value=1, max_value=1 << 20)

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.tuples(names, sizes), min_size=1, max_size=60))
    def check(stream):
        a, b = RegionAllocator(1 << 26), RegionAllocator(1 << 26)
        for name, size in stream:
            off = a.alloc(name, size)
            assert b.alloc(name, size) == off and off % 1024 == 0
            assert a.alloc(name, size) == off                        # asking again does not move it
            live = sorted(a.table(), key=lambda kv: kv[1][0])
            for (_, (o1, s1)), (_, (o2, _)) in zip(live, live[1:]):
                assert o1 + s1 <= o2                                 # no overlap
            assert all(o + s <= 1 << 26 for _, (o, s) in live)
            assert dict(a.table())[name][1] >= size
        assert a.digest() == b.digest() and a.table() == b.table()

    check()


def test_ctypes_mirror_of_the_gemm_roles_matches_the_library():
    """``parallel.fused.GemmCommC`` is a hand-written mirror of a C struct; the library reports its own layout."""
    from multimodal_training_b200.ops import native as nv
    from multimodal_training_b200.parallel import fused
    if not nv.available():
        pytest.skip("the kernel library is not built")
    fused.check_gemm_comm_layout()
    saved = fused.GemmCommC._fields_
    try:
        class Shifted(ctypes.Structure):                      # the same fields with one int inserted: must be noticed
            _fields_ = [("extra", ctypes.c_int)] + list(saved)
        fused.GemmCommC, real = Shifted, fused.GemmCommC
        with pytest.raises(RuntimeError, match="does not match"):
            fused.check_gemm_comm_layout()
    finally:
        fused.GemmCommC = real
