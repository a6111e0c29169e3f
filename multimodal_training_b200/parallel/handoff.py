"""Vision -> text embedding handoff.

Every merged vision token has exactly one home: the row of its image placeholder in the packed
text sequence of the data-parallel replica that owns the sample, on the tensor-parallel rank that
owns that row (activations are token shards).  The plan below is computed on the host from
``input_ids`` and ``grid_thw``; the exchange itself is one all-to-all of rows (library path) or a
peer-memory store kernel (``parallel/fused.py``).  The gradient returns along the same routes in
backward, so each token's gradient is delivered exactly once.

Replaces the reference's CUDA-IPC / Ray object-store transfer of the replicated vision output, its
two clones and the ``masked_scatter`` splice (python/ray/tensor_transfer.py:35-96,
python/ray/text.py:868-920,1010-1019).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..data.rope_utils import get_rope_index_for_images
from ..ops import functional as F
from . import comm
from .mesh import Mesh
from .sp import Geometry

IGNORE_INDEX = -100


@dataclass
class TextBatch:
    """One text replica's packed batch (identical on all of its TP ranks)."""

    input_ids: torch.Tensor        # [T] long, padded
    shifted_labels: torch.Tensor   # [T] long: label of the NEXT token, -100 = ignore
    position_ids: torch.Tensor     # [3, T]
    cu_seqlens: list[int]          # sample boundaries (padding is a sequence of its own)
    image_rows: list[np.ndarray]   # per image of this replica: packed rows of its placeholders, in order
    n_real: int
    sample_index: list[int]


def pack_text_batch(samples, *, image_token_id: int, vision_start_token_id: int, spatial_merge_size: int,
                    pad_multiple: int = 8, pad_token_id: int = 0) -> TextBatch:
    """Flatten samples into one sequence (the reference's FlattenedDataCollator, python/data/collator.py:80-104)
    and derive shifted labels, M-RoPE ids and placeholder rows."""
    ids, labs, pos, cu, rows, sidx = [], [], [], [0], [], []
    for s in samples:
        n = s.input_ids.numel()
        lab = torch.full((n,), IGNORE_INDEX, dtype=torch.long)
        lab[:-1] = s.labels[1:]
        p, _ = get_rope_index_for_images(spatial_merge_size, s.input_ids.unsqueeze(0), s.grid_thw,
                                         image_token_id=image_token_id, vision_start_token_id=vision_start_token_id)
        where = (s.input_ids == image_token_id).nonzero().flatten().numpy()
        off = 0
        for (t, h, w) in s.grid_thw:
            m = t * h * w // (spatial_merge_size ** 2)
            if off + m > len(where):
                raise ValueError(f"sample {s.sample_index}: {len(where)} image placeholders but the images need more")
            rows.append(where[off:off + m] + cu[-1])
            off += m
        if off != len(where):
            raise ValueError(f"sample {s.sample_index}: {len(where)} image placeholders for {off} merged tokens")
        ids.append(s.input_ids)
        labs.append(lab)
        pos.append(p[:, 0])
        cu.append(cu[-1] + n)
        sidx.append(s.sample_index)
    n_real = cu[-1]
    pad = (-n_real) % pad_multiple
    if pad:
        ids.append(torch.full((pad,), pad_token_id, dtype=torch.long))
        labs.append(torch.full((pad,), IGNORE_INDEX, dtype=torch.long))
        pos.append(torch.arange(pad).view(1, -1).expand(3, -1))
        cu.append(n_real + pad)
    return TextBatch(torch.cat(ids), torch.cat(labs), torch.cat(pos, dim=1), cu, rows, n_real, sidx)


@dataclass
class HandoffPlan:
    send_perm: torch.Tensor        # [M_loc] local merged tokens in destination order
    send_counts: list[int]         # per world rank
    recv_counts: list[int]         # per world rank
    recv_rows: torch.Tensor        # [sum(recv_counts)] row in this rank's token shard
    shard_rows: int                # rows of the text token shard on this rank
    # direct routes for the peer-memory path (no sorting by destination needed)
    dest_rank: torch.Tensor | None = None       # [M_loc] int32 world rank that owns the text row
    dest_row: torch.Tensor | None = None        # [M_loc] int64 row inside that rank's token shard
    recv_src_rank: torch.Tensor | None = None   # [R] int32 world rank that produced each received row
    recv_src_index: torch.Tensor | None = None  # [R] int64 index of the row in the producer's local merged tokens


def build_handoff_plan(mesh: Mesh, geoms: list[Geometry], images_per_vreplica: list[list[int]],
                       text_batches_rows: list[list[np.ndarray]], text_lengths: list[int],
                       image_owner: dict[int, tuple[int, int]]) -> HandoffPlan:
    """Routes of all merged tokens between world ranks.

    ``geoms[v]``: geometry of vision replica v.  ``images_per_vreplica[v]``: global image ids in the order
    the replica packs them.  ``text_batches_rows[d][k]``: packed rows of the k-th image of text replica d;
    ``image_owner[g] = (d, k)`` locates global image g on the text side.  ``text_lengths[d]``: padded T.
    """
    world, sp, tp = mesh.world, mesh.sp, mesh.tp
    me = mesh.rank
    send_dest, send_row, my_drow = None, None, None
    recv_lists = [[] for _ in range(world)]
    recv_src_idx = [[] for _ in range(world)]
    send_counts = [0] * world
    for v, geom in enumerate(geoms):
        if geom is None:
            continue
        merged_start = [s // geom.unit for s in geom.img_start]
        for s in range(sp):
            ws = v * sp + s
            mids = geom.merged_ids_of_rank(s)
            if len(mids) == 0:
                continue
            img_local = np.searchsorted(np.asarray(merged_start), mids, side="right") - 1
            j = mids - np.asarray(merged_start)[img_local]
            dest = np.empty(len(mids), np.int64)
            drow = np.empty(len(mids), np.int64)
            for il in np.unique(img_local):
                g = images_per_vreplica[v][il]
                d, k = image_owner[g]
                rows = text_batches_rows[d][k]
                sel = img_local == il
                r = rows[j[sel]]
                shard = text_lengths[d] // tp
                dest[sel] = d * tp + r // shard
                drow[sel] = r % shard
            order = np.argsort(dest, kind="stable")
            if ws == me:
                send_dest, send_row, my_drow = dest, order, drow
                cnt = np.bincount(dest, minlength=world)
                send_counts = [int(c) for c in cnt]
            mine = dest[order] == me
            if mine.any():
                recv_lists[ws] = drow[order][mine]
                recv_src_idx[ws] = order[mine]
    recv_counts = [len(x) for x in recv_lists]
    recv_rows = np.concatenate([np.asarray(x, np.int64) for x in recv_lists]) if sum(recv_counts) else np.zeros(0,
                                                                                                                 np.int64)
    send_perm = send_row if send_row is not None else np.zeros(0, np.int64)
    src_rank = np.concatenate([np.full(len(x), w, np.int32) for w, x in enumerate(recv_lists)]) if sum(
        recv_counts) else np.zeros(0, np.int32)
    src_idx = np.concatenate([np.asarray(x, np.int64) for x in recv_src_idx]) if sum(recv_counts) else np.zeros(
        0, np.int64)
    return HandoffPlan(torch.from_numpy(np.ascontiguousarray(send_perm)), send_counts, recv_counts,
                       torch.from_numpy(recv_rows), text_lengths[mesh.tdp_rank] // tp,
                       dest_rank=torch.from_numpy((np.zeros(0) if send_dest is None else send_dest).astype(np.int32)),
                       dest_row=torch.from_numpy((np.zeros(0) if my_drow is None else my_drow).astype(np.int64)),
                       recv_src_rank=torch.from_numpy(src_rank), recv_src_index=torch.from_numpy(src_idx))


class _Splice(torch.autograd.Function):
    """out = base with rows[i] replaced by vis[i]; the replaced rows of base get no gradient."""

    @staticmethod
    def forward(ctx, base, vis, rows):
        out = base.clone()
        if rows.numel():
            if base.is_cuda:
                F.scatter_rows_raw(vis.contiguous(), rows, out)
            else:
                out.index_copy_(0, rows, vis)
        ctx.save_for_backward(rows)
        return out

    @staticmethod
    def backward(ctx, dout):
        (rows,) = ctx.saved_tensors
        dbase = dout.clone()
        if rows.numel():
            dvis = F.gather_rows_raw(dout.contiguous(), rows) if dout.is_cuda else dout.index_select(0, rows)
            dbase.index_fill_(0, rows, 0)
        else:
            dvis = dout.new_zeros((0, dout.shape[1]))
        return dbase, dvis, None


def splice_rows(base: torch.Tensor, vis: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
    return _Splice.apply(base, vis, rows)


def exchange_vision_rows(merged_local: torch.Tensor, plan: HandoffPlan, mesh: Mesh) -> torch.Tensor:
    """Library path: sort local merged tokens by destination and all-to-all them over the world group."""
    perm = plan.send_perm.to(merged_local.device)
    ordered = F.gather_rows(merged_local, perm)
    return comm.all_to_all_rows(ordered, plan.send_counts, plan.recv_counts, mesh.world_group)
