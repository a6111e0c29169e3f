"""Host-side plan for ragged sequence parallelism in the vision encoder.

Everything the encoder needs to know about a batch of images is derived here from
``grid_thw`` alone, once per batch and without touching the GPU: window order, window
boundaries, 2-D rotary position ids, the window-aligned split of every image over the
sequence-parallel (SP) ranks, the row exchange of the four full-attention layers and the
destination row of every merged token in the text sequence.  The reference computes the
same facts with ~15 host syncs inside the forward pass
(modeling_qwen2_5_vl.py:841-909,957-1064; sequence_parallel_utils.py:105-459).

Conventions.  Patches arrive in the processor's merge-block order: 4 consecutive patches
(2x2) form one merged token.  "Window order" permutes merged tokens so that every
attention window is contiguous; all per-rank tensors are in window order.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass, field

import numpy as np
import torch


# --------------------------------------------------------------------------------------
# Window order and rotary position ids
# --------------------------------------------------------------------------------------
def window_index(grid_thw, spatial_merge_size: int, window_size: int, patch_size: int):
    """Window order of merged tokens and the window boundaries in PATCH units.

    Returns ``(index, cu_window_seqlens)``: ``index[j]`` is the merged-token id (in the original
    order over all images) that sits at position j in window order; ``cu_window_seqlens`` is an
    increasing list starting at 0 with no empty windows.
    """
    m = spatial_merge_size
    win = window_size // m // patch_size
    unit = m * m
    index_parts = []
    cu = [0]
    base = 0
    for (t, h, w) in grid_thw:
        gh, gw = h // m, w // m
        ids = np.arange(t * gh * gw, dtype=np.int64).reshape(t, gh, gw)
        nwh, nww = -(-gh // win), -(-gw // win)
        padded = np.full((t, nwh * win, nww * win), -1, dtype=np.int64)
        padded[:, :gh, :gw] = ids
        padded = padded.reshape(t, nwh, win, nww, win).transpose(0, 1, 3, 2, 4).reshape(t, nwh * nww, win * win)
        counts = (padded >= 0).sum(-1).reshape(-1)
        flat = padded.reshape(-1)
        index_parts.append(flat[flat >= 0] + base)
        for c in counts:
            if c > 0:
                cu.append(cu[-1] + int(c) * unit)
        base += t * gh * gw
    return np.concatenate(index_parts), cu


def rot_pos_ids(grid_thw, spatial_merge_size: int) -> np.ndarray:
    """(h, w) position of every patch in merge-block order, [n_patches, 2]."""
    m = spatial_merge_size
    out = []
    for (t, h, w) in grid_thw:
        hp = np.repeat(np.arange(h)[:, None], w, axis=1)
        wp = np.repeat(np.arange(w)[None, :], h, axis=0)
        hp = hp.reshape(h // m, m, w // m, m).transpose(0, 2, 1, 3).reshape(-1)
        wp = wp.reshape(h // m, m, w // m, m).transpose(0, 2, 1, 3).reshape(-1)
        out.append(np.tile(np.stack([hp, wp], axis=-1), (t, 1)))
    return np.concatenate(out, axis=0)


def rope_table(pos_hw: np.ndarray, head_dim: int, theta: float = 10000.0):
    """cos/sin [n, head_dim] fp32 for 2-D rotary embedding: half of the rotary dims follow h, half w."""
    dim = head_dim // 2
    inv_freq = 1.0 / (theta ** (np.arange(0, dim, 2, dtype=np.float64) / dim))
    fh = pos_hw[:, 0:1].astype(np.float64) * inv_freq[None, :]
    fw = pos_hw[:, 1:2].astype(np.float64) * inv_freq[None, :]
    f = np.concatenate([fh, fw], axis=-1)
    emb = np.concatenate([f, f], axis=-1)
    return torch.from_numpy(np.cos(emb).astype(np.float32)), torch.from_numpy(np.sin(emb).astype(np.float32))


# --------------------------------------------------------------------------------------
# Window-aligned split
# --------------------------------------------------------------------------------------
def token_cut_positions(length: int, sp: int) -> list[int]:
    """Even split with the remainder going to the low ranks."""
    base, rem = divmod(length, sp)
    cuts = [0]
    for r in range(sp):
        cuts.append(cuts[-1] + base + (1 if r < rem else 0))
    return cuts


def window_cut_positions(boundaries: list[int], sp: int) -> list[int]:
    """Cut one image's window-ordered sequence into ``sp`` pieces on window boundaries.

    ``boundaries`` are the image's window boundaries relative to its start (first 0, last = length).
    Cut k is the first boundary >= floor(length * k / sp), kept monotone and clamped so that enough
    boundaries remain for the ranks that follow.
    """
    length = boundaries[-1]
    nb = len(boundaries)
    cuts = [0]
    prev = 0
    for k in range(1, sp):
        target = (length * k) // sp
        i = bisect.bisect_left(boundaries, target)
        if nb - 1 >= sp:   # enough windows: every rank gets at least one
            i = min(max(i, prev + 1), nb - 1 - (sp - k))
        else:
            i = min(max(i, prev), nb - 1)
        cuts.append(boundaries[i])
        prev = i
    cuts.append(length)
    return cuts


@dataclass
class VisionPlan:
    """Per-rank view of one batch of images."""

    sp: int
    rank: int
    grid_thw: list[tuple[int, int, int]]
    n_patches: int                      # all images, all ranks
    local_patch_index: torch.Tensor     # [T_loc] rows of the global patch array, in local window order
    local_cos: torch.Tensor             # [T_loc, head_dim] fp32
    local_sin: torch.Tensor
    win_cu: list[int]                   # local window boundaries (patch units)
    rank_tokens: list[int]              # T of every rank
    # full attention: rows after the exchange are ordered (rank, image); attention wants (image, rank)
    full_cu: list[int]                  # per-image boundaries in the gathered sequence
    to_image_major: torch.Tensor | None  # [T_all] gather index: image-major row -> exchange-order row
    to_rank_major: torch.Tensor | None   # inverse
    # merged tokens of this rank: global merged id (original order) of every local merged token
    local_merged_ids: torch.Tensor      # [T_loc / unit]
    local_merged_image: torch.Tensor    # [T_loc / unit] image id
    per_image_local: list[tuple[int, int]] = field(default_factory=list)  # (start, length) of image b in local pack
    # (h, w) position of EVERY patch in window order (= the image-major order of the gathered sequence) and the
    # rotary width: what a head owner needs to rotate rows that arrived un-rotated (shared with the geometry, no copy)
    all_pos: "np.ndarray | None" = None
    head_dim: int = 0

    @property
    def local_tokens(self) -> int:
        return self.rank_tokens[self.rank]


@dataclass
class Geometry:
    """Rank-independent facts of one batch of images (shared by the plans of all SP ranks)."""

    grid_thw: list
    unit: int
    widx: np.ndarray                   # window order of merged tokens
    cu_arr: np.ndarray                 # window boundaries, patch units
    img_start: list[int]               # patch offset of every image
    patch_in_window_order: np.ndarray
    pos: np.ndarray                    # (h, w) of every patch in window order
    slices: list                       # slices[r][b] = (lo, hi) in window-order patch coordinates
    n_patches: int

    def merged_ids_of_rank(self, r: int) -> np.ndarray:
        """Global merged-token ids (original order) held by SP rank r, in its local order."""
        parts = [self.widx[lo // self.unit: hi // self.unit] for lo, hi in self.slices[r]]
        return np.concatenate(parts) if parts else np.zeros(0, np.int64)


# Geometry and plans depend only on the image grids and the split, not on the pixels; batches of a fixed
# resolution repeat them every step, so the most recent ones are kept (with the device tensors that
# ``models.vision.prepare_plan`` attaches to a plan).
_GEOM_CACHE: dict = {}
_PLAN_CACHE: dict = {}
_CACHE_LIMIT = 16


def _cache_put(cache: dict, key, value):
    if len(cache) >= _CACHE_LIMIT:
        cache.pop(next(iter(cache)))
    cache[key] = value
    return value


def compute_geometry(grid_thw, *, sp: int, spatial_merge_size: int = 2, window_size: int = 112,
                     patch_size: int = 14, window_aligned: bool = True) -> Geometry:
    grid_thw = [tuple(int(x) for x in g) for g in grid_thw]
    key = (tuple(grid_thw), sp, spatial_merge_size, window_size, patch_size, window_aligned)
    hit = _GEOM_CACHE.get(key)
    if hit is not None:
        return hit
    return _cache_put(_GEOM_CACHE, key, _compute_geometry(grid_thw, sp, spatial_merge_size, window_size, patch_size,
                                                          window_aligned))


def _compute_geometry(grid_thw, sp, spatial_merge_size, window_size, patch_size, window_aligned) -> Geometry:
    unit = spatial_merge_size ** 2
    widx, cu_win = window_index(grid_thw, spatial_merge_size, window_size, patch_size)
    n_patches = sum(t * h * w for t, h, w in grid_thw)
    # patch rows in window order: merged token j -> patches 4j..4j+3
    patch_in_window_order = (widx[:, None] * unit + np.arange(unit)[None, :]).reshape(-1)
    pos = rot_pos_ids(grid_thw, spatial_merge_size)[patch_in_window_order]
    img_start = [0]
    for (t, h, w) in grid_thw:
        img_start.append(img_start[-1] + t * h * w)
    cu_arr = np.asarray(cu_win)
    slices = [[None] * len(grid_thw) for _ in range(sp)]
    for b in range(len(grid_thw)):
        s, e = img_start[b], img_start[b + 1]
        i0, i1 = np.searchsorted(cu_arr, s), np.searchsorted(cu_arr, e)
        bounds = [int(x) - s for x in cu_arr[i0:i1 + 1]]
        if window_aligned:
            cuts = window_cut_positions(bounds, sp)
        else:
            cuts = [c // unit * unit for c in token_cut_positions(e - s, sp)]
            cuts[-1] = e - s
        for r in range(sp):
            slices[r][b] = (s + cuts[r], s + cuts[r + 1])
    return Geometry(grid_thw, unit, widx, cu_arr, img_start, patch_in_window_order, pos, slices, n_patches)


def build_vision_plan(grid_thw, *, sp: int, rank: int, spatial_merge_size: int = 2, window_size: int = 112,
                      patch_size: int = 14, head_dim: int = 80, window_aligned: bool = True,
                      geom: Geometry | None = None) -> VisionPlan:
    if geom is None:
        geom = compute_geometry(grid_thw, sp=sp, spatial_merge_size=spatial_merge_size, window_size=window_size,
                                patch_size=patch_size, window_aligned=window_aligned)
    key = (id(geom), sp, rank, head_dim)
    hit = _PLAN_CACHE.get(key)
    if hit is not None and hit[0] is geom:
        return hit[1]
    plan = _build_vision_plan(geom, sp, rank, head_dim)
    _cache_put(_PLAN_CACHE, key, (geom, plan))
    return plan


def _build_vision_plan(geom: Geometry, sp: int, rank: int, head_dim: int) -> VisionPlan:
    grid_thw, unit, widx, cu_arr = geom.grid_thw, geom.unit, geom.widx, geom.cu_arr
    img_start, patch_in_window_order, pos, slices = geom.img_start, geom.patch_in_window_order, geom.pos, geom.slices
    n_patches = geom.n_patches

    rank_tokens = [sum(hi - lo for lo, hi in slices[r]) for r in range(sp)]
    if min(rank_tokens) == 0 and sp > 1:
        raise ValueError(f"sequence-parallel split leaves a rank without tokens: {rank_tokens}; "
                         "use larger images or a smaller sequence_parallel_size")

    # local pack of this rank
    loc = np.concatenate([np.arange(lo, hi) for lo, hi in slices[rank]]) if rank_tokens[rank] else np.zeros(0, int)
    per_image_local = []
    off = 0
    for lo, hi in slices[rank]:
        per_image_local.append((off, hi - lo))
        off += hi - lo
    # local window boundaries
    win_cu = [0]
    for lo, hi in slices[rank]:
        if hi == lo:
            continue
        i0, i1 = np.searchsorted(cu_arr, lo), np.searchsorted(cu_arr, hi)
        inner = [int(x) for x in cu_arr[i0:i1 + 1]]
        if inner[0] != lo:
            inner = [lo] + inner
        if inner[-1] != hi:
            inner = inner + [hi]
        base = win_cu[-1] - lo
        for x in inner[1:]:
            win_cu.append(base + x)
    cos, sin = rope_table(pos[loc], head_dim)

    # exchange order for full attention: rows arrive as (rank s, image b); attention needs (image b, rank s)
    to_img = to_rank = None
    # one attention sequence per temporal patch of every image / video (a still image has one): window order keeps
    # the patches of a temporal patch contiguous (modeling_qwen2_5_vl.py:944-952 builds cu_seqlens the same way)
    full_cu = [0]
    for (t, h, w) in grid_thw:
        for _ in range(t):
            full_cu.append(full_cu[-1] + h * w)
    if sp > 1:
        rank_off = [0]
        for r in range(sp):
            rank_off.append(rank_off[-1] + rank_tokens[r])
        src = []
        for b in range(len(grid_thw)):
            for s in range(sp):
                lo, hi = slices[s][b]
                inner = sum(h2 - l2 for l2, h2 in slices[s][:b])
                src.append(np.arange(rank_off[s] + inner, rank_off[s] + inner + (hi - lo)))
        to_img_np = np.concatenate(src)
        inv = np.empty_like(to_img_np)
        inv[to_img_np] = np.arange(len(to_img_np))
        to_img = torch.from_numpy(to_img_np)
        to_rank = torch.from_numpy(inv)

    # merged tokens (window order) owned by this rank
    assert all(lo % unit == 0 and hi % unit == 0 for lo, hi in slices[rank])
    merged_pos = loc.reshape(-1, unit)[:, 0] // unit if len(loc) else np.zeros(0, int)
    merged_ids = widx[merged_pos]
    merged_starts = np.asarray([s // unit for s in img_start])
    merged_image = np.searchsorted(merged_starts, merged_ids, side="right") - 1

    return VisionPlan(
        sp=sp, rank=rank, grid_thw=grid_thw, n_patches=n_patches,
        local_patch_index=torch.from_numpy(patch_in_window_order[loc]),
        local_cos=cos, local_sin=sin, win_cu=win_cu, rank_tokens=rank_tokens, full_cu=full_cu,
        to_image_major=to_img, to_rank_major=to_rank,
        local_merged_ids=torch.from_numpy(merged_ids), local_merged_image=torch.from_numpy(merged_image),
        all_pos=pos, head_dim=head_dim,
        per_image_local=per_image_local)


# --------------------------------------------------------------------------------------
# Ragged pack helpers with the reference's names (sequence_parallel_utils.py:167-427)
# --------------------------------------------------------------------------------------
@dataclass
class RaggedSequenceMeta:
    """Where every sample's slice sits in a rank-local pack."""

    local_lengths: list[int]
    global_lengths: list[int]
    local_starts: list[int]            # start of the local slice inside the sample
    sp_size: int
    sp_rank: int

    @property
    def local_offsets(self) -> list[int]:
        out = [0]
        for n in self.local_lengths:
            out.append(out[-1] + n)
        return out


def split_pack_by_sp(pack: torch.Tensor, cu_seqlens, sp_size: int, sp_rank: int, cu_window_seqlens=None):
    """Slice a packed [T, ...] tensor per sample for one SP rank; returns ``(local_pack, meta)``."""
    cu = [int(x) for x in cu_seqlens]
    wins = None if cu_window_seqlens is None else sorted(set(int(x) for x in cu_window_seqlens))
    parts, l_len, g_len, l_start = [], [], [], []
    for s, e in zip(cu[:-1], cu[1:]):
        n = e - s
        if wins is None:
            cuts = token_cut_positions(n, sp_size)
        else:
            b = [x - s for x in wins if s <= x <= e]
            if not b or b[0] != 0:
                b = [0] + b
            if b[-1] != n:
                b = b + [n]
            cuts = window_cut_positions(b, sp_size)
        lo, hi = cuts[sp_rank], cuts[sp_rank + 1]
        parts.append(pack[s + lo:s + hi])
        l_len.append(hi - lo)
        g_len.append(n)
        l_start.append(lo)
    local = torch.cat(parts, dim=0) if parts else pack[:0]
    return local, RaggedSequenceMeta(l_len, g_len, l_start, sp_size, sp_rank)


def pad_pack_to_batch(pack: torch.Tensor, lengths: list[int], pad_len: int | None = None):
    """[sum(lengths), ...] -> [B, pad_len, ...] plus a [B, pad_len] validity mask."""
    pad_len = max(lengths, default=0) if pad_len is None else pad_len
    out = pack.new_zeros((len(lengths), pad_len) + tuple(pack.shape[1:]))
    mask = torch.zeros(len(lengths), pad_len, dtype=torch.bool, device=pack.device)
    off = 0
    for i, n in enumerate(lengths):
        out[i, :n] = pack[off:off + n]
        mask[i, :n] = True
        off += n
    return out, mask


def unpad_batch_to_pack(batch: torch.Tensor, lengths: list[int]) -> torch.Tensor:
    return torch.cat([batch[i, :n] for i, n in enumerate(lengths)], dim=0) if lengths else batch.reshape(
        (0,) + tuple(batch.shape[2:]))


def rebuild_local_cu_seqlens(lengths: list[int], device=None) -> torch.Tensor:
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + int(n))
    return torch.tensor(cu, dtype=torch.int32, device=device)


def build_local_rope(cos: torch.Tensor, sin: torch.Tensor, cu_seqlens, meta: RaggedSequenceMeta):
    """Slice global [T, d] rotary tables to one rank's local pack."""
    cu = [int(x) for x in cu_seqlens]
    idx = torch.cat([torch.arange(s + st, s + st + n) for s, st, n in zip(cu[:-1], meta.local_starts,
                                                                       meta.local_lengths)])
    idx = idx.to(cos.device)
    return cos.index_select(0, idx), sin.index_select(0, idx)


def compute_max_length_across_ranks(local_len: int, group=None) -> int:
    import torch.distributed as dist

    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return int(local_len)
    t = torch.tensor([local_len], dtype=torch.int64)
    if dist.get_backend(group) == "nccl":
        t = t.cuda()
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return int(t.item())
