"""Ragged sequence-parallel utilities: window order, window-aligned cuts, pack/pad round trips, local rope,
exchange permutations (modelled on the reference's tests/test_sequence_parallel_ragged.py, with asserts)."""
import numpy as np
import pytest
import torch

from multimodal_training_b200.parallel.sp import (RaggedSequenceMeta, build_local_rope, build_vision_plan,
                                                  compute_geometry, pad_pack_to_batch, rebuild_local_cu_seqlens,
                                                  split_pack_by_sp, token_cut_positions, unpad_batch_to_pack,
                                                  window_cut_positions, window_index)

pytestmark = pytest.mark.cpu_only


def test_window_index_16x16_has_four_full_windows_and_no_empty_ones():
    idx, cu = window_index([(1, 16, 16)], 2, 112, 14)
    assert cu == [0, 64, 128, 192, 256]
    assert sorted(idx.tolist()) == list(range(64))
    assert idx[:4].tolist() == [0, 1, 2, 3] and idx[4:8].tolist() == [8, 9, 10, 11]


def test_window_index_ragged_grid_keeps_partial_windows():
    idx, cu = window_index([(1, 20, 12)], 2, 112, 14)      # merged grid 10 x 6 -> windows 4x4, 4x2, ... , 2x2
    lens = np.diff(cu)
    assert lens.sum() == 20 * 12 and (lens > 0).all()
    assert sorted(idx.tolist()) == list(range(60))


def test_token_cuts_give_remainder_to_low_ranks():
    assert token_cut_positions(10, 4) == [0, 3, 6, 8, 10]
    assert token_cut_positions(8, 4) == [0, 2, 4, 6, 8]


def test_window_cuts_fall_on_boundaries_and_leave_no_rank_empty():
    b = [0, 64, 128, 192, 256, 320]
    cuts = window_cut_positions(b, 4)
    assert cuts[0] == 0 and cuts[-1] == 320 and all(c in b for c in cuts)
    assert all(y > x for x, y in zip(cuts, cuts[1:]))
    assert window_cut_positions([0, 64, 128, 192, 256], 2) == [0, 128, 256]


def test_split_even_uneven_and_windowed():
    pack = torch.arange(30).float().unsqueeze(1)
    cu = [0, 10, 30]
    parts = [split_pack_by_sp(pack, cu, 3, r) for r in range(3)]
    assert [p[1].local_lengths for p in parts] == [[4, 7], [3, 7], [3, 6]]
    back = []
    for s in range(2):
        for r in range(3):
            lo = parts[r][1].local_offsets[s]
            back.append(parts[r][0][lo:lo + parts[r][1].local_lengths[s]])
    assert torch.equal(torch.cat(back), pack)
    wl, wm = split_pack_by_sp(torch.arange(256).float().unsqueeze(1), [0, 256], 2, 1, [0, 64, 128, 192, 256])
    assert wm.local_lengths == [128] and wm.local_starts == [128] and wl[0, 0] == 128


def test_pad_unpad_round_trip_and_cu_seqlens():
    pack = torch.randn(9, 3)
    lengths = [4, 0, 5]
    batch, mask = pad_pack_to_batch(pack, lengths)
    assert batch.shape == (3, 5, 3) and mask.sum() == 9 and not mask[1].any()
    assert torch.equal(unpad_batch_to_pack(batch, lengths), pack)
    cu = rebuild_local_cu_seqlens(lengths)
    assert cu.dtype == torch.int32 and cu.tolist() == [0, 4, 4, 9]


def test_build_local_rope_slices_every_sample():
    cos, sin = torch.arange(20).float().unsqueeze(1), -torch.arange(20).float().unsqueeze(1)
    meta = RaggedSequenceMeta([3, 4], [8, 12], [5, 0], 2, 1)
    c, s = build_local_rope(cos, sin, [0, 8, 20], meta)
    assert c.flatten().tolist() == [5, 6, 7, 8, 9, 10, 11] and torch.equal(s, -c)


@pytest.mark.parametrize("grids,sp", [([(1, 16, 16), (1, 32, 24)], 2), ([(1, 64, 64)] * 2, 4), ([(1, 32, 32)], 1)])
def test_plan_partitions_tokens_and_exchange_is_a_permutation(grids, sp):
    geom = compute_geometry(grids, sp=sp)
    plans = [build_vision_plan(None, sp=sp, rank=r, head_dim=32, geom=geom) for r in range(sp)]
    total = sum(t * h * w for t, h, w in grids)
    all_patches = torch.cat([p.local_patch_index for p in plans])
    assert sorted(all_patches.tolist()) == list(range(total))
    merged = torch.cat([p.local_merged_ids for p in plans])
    assert sorted(merged.tolist()) == list(range(total // 4))
    for p in plans:
        assert p.win_cu[0] == 0 and p.win_cu[-1] == p.local_tokens
        assert all(b > a for a, b in zip(p.win_cu, p.win_cu[1:]))
        assert p.local_tokens % 4 == 0 and p.local_cos.shape == (p.local_tokens, 32)
        if sp > 1:
            assert sorted(p.to_image_major.tolist()) == list(range(total))
            assert torch.equal(p.to_image_major[p.to_rank_major], torch.arange(total))
    if sp > 1:
        # rows in exchange order are (rank, image); after the permutation every image is contiguous
        owner_image = torch.cat([torch.cat([torch.full((n,), b) for b, (_, n) in enumerate(p.per_image_local)])
                                 for p in plans])
        im = owner_image[plans[0].to_image_major]
        assert (im[1:] >= im[:-1]).all()


def test_rank_without_tokens_is_an_error():
    with pytest.raises(ValueError):
        build_vision_plan([(1, 8, 8)], sp=8, rank=0, head_dim=32)


def test_image_major_order_is_the_window_order_of_all_patches():
    """A head owner rotates rows that arrive un-rotated from all ranks, using tables built from the positions of ALL
    patches in window order (VisionPlan.all_pos).  That is only right if the image-major order of the gathered
    sequence IS the window order: every rank's local tables must be rows of the global tables at the rank's
    image-major positions."""
    import numpy as np
    from multimodal_training_b200.parallel.sp import build_vision_plan, rope_table
    grids = [(1, 18, 26), (1, 8, 12), (2, 10, 6)]
    for sp in (2, 4):
        plans = [build_vision_plan(grids, sp=sp, rank=r, spatial_merge_size=2, window_size=112, patch_size=14,
                                   head_dim=16) for r in range(sp)]
        cos_all, sin_all = rope_table(plans[0].all_pos, 16)
        off = np.concatenate([[0], np.cumsum(plans[0].rank_tokens)])
        inv = plans[0].to_rank_major.numpy()
        for r, p in enumerate(plans):
            dst = torch.from_numpy(inv[off[r]:off[r + 1]])
            assert torch.equal(cos_all[dst], p.local_cos) and torch.equal(sin_all[dst], p.local_sin)


def test_plan_invariants_for_random_image_sets():
    """Property check (hypothesis) over random batches of ragged images and sequence-parallel sizes: the ranks' local
    patches partition all patches; every rank's cut falls on a window boundary and on a merge-unit boundary; the
    exchange maps are inverse permutations; per-image sequence boundaries add up; the Ulysses routes of all ranks
    tile the gathered sequence exactly once."""
    import numpy as np
    from hypothesis import assume, given, settings
    from hypothesis import strategies as st

    from multimodal_training_b200.parallel.sp import build_vision_plan

    side = st.integers(min_value=2, max_value=20).map(lambda v: 2 * v)          # even grids (2 x 2 merge)
    grid = st.tuples(st.sampled_from([1, 1, 1, 2]), side, side)

    @settings(max_examples=60, deadline=None)
    @given(st.lists(grid, min_size=1, max_size=4), st.sampled_from([1, 2, 4]))
    def check(grids, sp):
        total = sum(t * h * w for t, h, w in grids)
        try:
            plans = [build_vision_plan(grids, sp=sp, rank=r, spatial_merge_size=2, window_size=112, patch_size=14,
                                       head_dim=16) for r in range(sp)]
        except ValueError:
            assume(False)                       # a split that would leave a rank without tokens is refused
        assert plans[0].n_patches == total and sum(plans[0].rank_tokens) == total
        seen = np.concatenate([p.local_patch_index.numpy() for p in plans])
        assert sorted(seen.tolist()) == list(range(total))                       # a partition of all patches
        for r, p in enumerate(plans):
            assert p.local_tokens == p.rank_tokens[r] == int(p.local_patch_index.numel())
            assert p.local_tokens % 4 == 0 and p.local_merged_ids.numel() == p.local_tokens // 4
            assert p.win_cu[0] == 0 and p.win_cu[-1] == p.local_tokens and all(b > a for a, b in zip(p.win_cu, p.win_cu[1:]))
            assert p.full_cu[-1] == total
        if sp > 1:
            fwd, inv = plans[0].to_image_major.numpy(), plans[0].to_rank_major.numpy()
            assert sorted(fwd.tolist()) == list(range(total)) and (inv[fwd] == np.arange(total)).all()
            off = np.concatenate([[0], np.cumsum(plans[0].rank_tokens)])
            rows = np.concatenate([inv[off[r]:off[r + 1]] for r in range(sp)])
            assert sorted(rows.tolist()) == list(range(total))                   # destination rows: each exactly once
        merged = np.concatenate([p.local_merged_ids.numpy() for p in plans])
        assert sorted(merged.tolist()) == list(range(total // 4))

    check()


@pytest.mark.parametrize("world,sp,tp", [(2, 2, 2), (4, 2, 2), (4, 4, 2), (8, 8, 4)])
def test_handoff_routes_are_consistent_across_the_world(world, sp, tp):
    """The handoff plans of all ranks, built independently from the same batch: what rank a says it sends to rank b
    is what b expects from a; every merged vision token has exactly one destination row; every image-placeholder row
    of every text shard receives exactly one token; the peer-memory routes (dest_rank, dest_row) agree with the
    all-to-all routes."""
    import numpy as np
    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.data.synthetic import synthetic_global_batch
    from multimodal_training_b200.parallel.mesh import Mesh
    from multimodal_training_b200.trainers.context import build_step_context

    cfg = get_model_config("tiny")
    vdp = world // sp
    B = 2 * max(vdp, world // tp)
    samples = synthetic_global_batch(cfg, 0, B, image_size=224, text_tokens=48, seed=9, dtype=torch.float32,
                                     image_sizes=[224, 252, 336], text_token_choices=[48, 80, 33])
    ctxs = [build_step_context(0, samples, cfg, Mesh(world=world, rank=r, sp=sp, tp=tp)) for r in range(world)]
    plans = [c.handoff for c in ctxs]
    assert all(p is not None for p in plans)
    for a in range(world):
        for b in range(world):
            assert plans[a].send_counts[b] == plans[b].recv_counts[a], (a, b)
    n_merged = sum(int(t * h * w) // 4 for s in samples for (t, h, w) in s.grid_thw)
    assert sum(sum(p.send_counts) for p in plans) == n_merged
    taken = set()
    for r, p in enumerate(plans):
        rows = p.recv_rows.numpy()
        assert len(set(rows.tolist())) == len(rows) and (rows < p.shard_rows).all()      # one token per row
        taken |= {(r, int(x)) for x in rows}
        # peer-memory routes: the same pairs, grouped by destination
        dest = p.dest_rank.numpy()
        assert np.bincount(dest, minlength=world).tolist() == p.send_counts
    pairs = set()
    for p in plans:
        pairs |= set(zip(p.dest_rank.numpy().tolist(), p.dest_row.numpy().tolist()))
    assert pairs == taken and len(pairs) == n_merged
    # the rows that receive a token are exactly the image placeholders of the text shards
    for r, c in enumerate(ctxs):
        tb, m = c.text_batch, Mesh(world=world, rank=r, sp=sp, tp=tp)
        shard = plans[r].shard_rows
        ph = np.concatenate(tb.image_rows) if tb.image_rows else np.zeros(0, np.int64)
        mine = ph[(ph // shard) == m.tp_rank] % shard
        assert sorted(mine.tolist()) == sorted(plans[r].recv_rows.numpy().tolist())
