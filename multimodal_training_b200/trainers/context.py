"""Per-step host context shared by the vision and text trainers of one process.

The global batch of a step is known to every rank (deterministic synthetic data, or dataloaders
with a common seed as in the reference, python/ray/trainer.py:69-104).  From it each rank derives,
without communication: which images its vision replica encodes and how they are split over the
sequence-parallel ranks, which samples its text replica packs, and the routes of the merged vision
tokens between the two (``parallel/handoff.py``).  Unlike the reference, data-parallel replicas get
DIFFERENT samples: replica d of R takes samples [d*B/R, (d+1)*B/R) of the global batch.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config.model_configs import VLConfig
from ..parallel.handoff import HandoffPlan, TextBatch, build_handoff_plan, pack_text_batch
from ..parallel.mesh import Mesh
from ..parallel.sp import Geometry, VisionPlan, build_vision_plan, compute_geometry


@dataclass(frozen=True)
class StepSizes:
    """Largest extents of this step over ALL ranks of the job: the same numbers on every rank (each rank knows
    every replica's geometry), which is what makes the regions of the symmetric heap line up across ranks."""

    shard_rows: int = 0          # rows of a text token shard (packed, padded tokens of a replica / tp)
    merged_rows: int = 0         # merged vision tokens held by one vision rank
    vision_tokens_all: int = 0   # patches of all images of one vision replica
    vision_tokens_rank: int = 0  # patches held by one vision rank
    has_images: bool = False


@dataclass
class StepContext:
    step: int
    samples: list                       # global batch (list of data.synthetic.Sample-like objects)
    vision_samples: list[int]           # indices (into samples) encoded by this rank's vision replica
    vision_plan: VisionPlan | None
    text_batch: TextBatch | None
    handoff: HandoffPlan | None
    n_vision_patches_global: int
    n_text_tokens_global: int
    sizes: StepSizes = StepSizes()


def _slice(n: int, parts: int, i: int) -> range:
    if n % parts:
        raise ValueError(f"global batch of {n} samples is not divisible by {parts} data-parallel replicas")
    per = n // parts
    return range(i * per, (i + 1) * per)


def build_step_context(step: int, samples: list, cfg: VLConfig, mesh: Mesh, *, pad_multiple: int | None = None,
                       window_aligned: bool = True) -> StepContext:
    v = cfg.vision
    B = len(samples)
    # ---------------- vision side: geometry of every replica (needed for routing), plan of mine
    geoms: list[Geometry] = []
    images_per_vreplica: list[list[int]] = []
    image_ids: dict[tuple[int, int], int] = {}
    gid = 0
    for si, s in enumerate(samples):
        for k in range(len(s.grid_thw)):
            image_ids[(si, k)] = gid
            gid += 1
    for r in range(mesh.vdp):
        grids, ids = [], []
        for si in _slice(B, mesh.vdp, r):
            for k, g in enumerate(samples[si].grid_thw):
                grids.append(g)
                ids.append(image_ids[(si, k)])
        images_per_vreplica.append(ids)
        geoms.append(compute_geometry(grids, sp=mesh.sp, spatial_merge_size=v.spatial_merge_size,
                                      window_size=v.window_size, patch_size=v.patch_size,
                                      window_aligned=window_aligned) if grids else None)
    my_geom = geoms[mesh.vdp_rank]
    vplan = None
    if my_geom is not None:
        vplan = build_vision_plan(None, sp=mesh.sp, rank=mesh.sp_rank, head_dim=v.head_dim, geom=my_geom)

    # ---------------- text side: every replica's packed batch (rows of the placeholders are needed for routing)
    pad = pad_multiple or max(8, mesh.tp * 8)
    text_rows, text_len, image_owner = [], [], {}
    my_tb = None
    for d in range(mesh.tdp):
        sl = [samples[i] for i in _slice(B, mesh.tdp, d)]
        tb = pack_text_batch(sl, image_token_id=cfg.image_token_id, vision_start_token_id=cfg.vision_start_token_id,
                             spatial_merge_size=v.spatial_merge_size, pad_multiple=pad, pad_token_id=cfg.pad_token_id)
        text_rows.append(tb.image_rows)
        text_len.append(tb.input_ids.numel())
        k = 0
        for si in _slice(B, mesh.tdp, d):
            for kk in range(len(samples[si].grid_thw)):
                image_owner[image_ids[(si, kk)]] = (d, k)
                k += 1
        if d == mesh.tdp_rank:
            my_tb = tb
    handoff = build_handoff_plan(mesh, [g for g in geoms], images_per_vreplica, text_rows, text_len, image_owner) \
        if gid > 0 else None
    n_patches = sum(t * h * w for s in samples for (t, h, w) in s.grid_thw)
    n_text = sum(s.input_ids.numel() for s in samples)
    live = [g for g in geoms if g is not None]
    sizes = StepSizes(
        shard_rows=max(text_len) // mesh.tp if text_len else 0,
        merged_rows=max((sum(hi - lo for lo, hi in g.slices[r]) // g.unit for g in live for r in range(mesh.sp)),
                        default=0),
        vision_tokens_all=max((g.n_patches for g in live), default=0),
        vision_tokens_rank=max((sum(hi - lo for lo, hi in g.slices[r]) for g in live for r in range(mesh.sp)),
                               default=0),
        has_images=gid > 0)
    for d, n in enumerate(text_len):
        if n % mesh.tp:
            raise ValueError(f"text replica {d} packs {n} tokens, which the tensor-parallel size {mesh.tp} does not "
                             "divide; set data.pad_multiple to a multiple of it")
    return StepContext(step, samples, list(_slice(B, mesh.vdp, mesh.vdp_rank)), vplan, my_tb, handoff, n_patches,
                       n_text, sizes)


def local_pixels(ctx: StepContext, out: torch.Tensor | None = None, plan: VisionPlan | None = None) -> torch.Tensor:
    """Host gather of this rank's patches (local window order) from the samples' pixel arrays."""
    plan = plan or ctx.vision_plan
    pix = [ctx.samples[i].pixel_values for i in ctx.vision_samples if ctx.samples[i].pixel_values is not None]
    allpix = pix[0] if len(pix) == 1 else torch.cat(pix, dim=0)
    if out is not None:
        return torch.index_select(allpix, 0, plan.local_patch_index, out=out)
    return allpix.index_select(0, plan.local_patch_index)


class StagingRing:
    """Host buffers for host->device copies that are enqueued, not awaited.

    The host runs ahead of the GPU (the loss is read a step late), so a single pinned buffer would be overwritten
    with the next step's pixels before the copy of this step has executed.  The ring hands out ``slots`` buffers in
    turn; a buffer is reused only after the event recorded behind its last copy has completed, which normally
    happened long ago.  On CPU (``pin=False``) the buffers are plain tensors and nothing is waited for.
    """

    def __init__(self, slots: int = 3, pin: bool = True):
        self.slots = [[None, None] for _ in range(slots)]      # [buffer, event of the last copy out of it]
        self.pin = pin
        self._next = 0
        self._current = None

    def acquire(self, rows: int, cols: int, dtype) -> torch.Tensor:
        slot = self.slots[self._next % len(self.slots)]
        self._next += 1
        buf, event = slot
        if event is not None:
            event.synchronize()
            slot[1] = None
        if buf is None or buf.shape[0] < rows or buf.shape[1] != cols or buf.dtype != dtype:
            buf = torch.empty(rows, cols, dtype=dtype)
            if self.pin:
                buf = buf.pin_memory()
            slot[0] = buf
        self._current = slot
        return buf[:rows]

    def copied(self) -> None:
        """Call right after enqueueing the copy out of the buffer that ``acquire`` returned last."""
        if self.pin and self._current is not None:
            event = torch.cuda.Event()
            event.record()
            self._current[1] = event
