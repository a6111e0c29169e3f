"""Fused compute+collective paths over peer memory (NVLink / NVSwitch), host side.

The kernels live in ``csrc/fused.cu`` and ``csrc/gemm.cu``; this module owns the symmetric heap, the
epoch counters of every flag slot and the autograd functions that replace the NCCL versions of

* tensor-parallel ``all-gather -> GEMM`` (``ag_gemm``: the GEMM forwards the shared-memory stages of its own rows
  to the peers while it computes on them and waits per (source rank, row block) before it reads a peer's rows;
  ``push_gather`` + ``gemm_gathered``: the earlier form with a push kernel in front of the GEMM, still used for
  shards that do not split into 256-row blocks) and ``GEMM -> reduce-scatter`` (the GEMM epilogue stores partial
  tiles into the owner's staging slot; the owner sums them with the residual) -- forward and backward of the
  attention and MLP projections of the text decoder (one autograd node per layer: ``ops/tp_blocks.py``);
* the vision encoder's Ulysses exchanges inside the QKV and output projections (``fused_ulysses.py``,
  ``ops/ulysses_block.py``);
* the vision -> text handoff (merged tokens stored straight into the text ranks' rows) and its gradient;
* ZeRO-1: gradient reduce-scatter + AdamW + parameter all-gather as one kernel (``FusedZero``).

Buffer reuse needs no extra barriers: every region has one role, two uses of a role are separated by
at least one other exchange that every rank can only finish after all peers have started it, flags
count epochs upward, and the backward pass computes weight gradients (which read gathered inputs)
before it pushes anything that lets a peer run ahead (``tests/test_exchange_schedule.py`` replays the layers' real
exchange order under arbitrary rank skew).  Every wait is bounded on the device; the host checks the error word
where it synchronises anyway (``LossHandle.value``, ``Trainer.check_device_errors``).
"""
from __future__ import annotations

import ctypes
import logging
import os

import torch

from ..ops import functional as F
from ..ops import native as nv
from .symm import SymmetricHeap

log = logging.getLogger("mmt_b200")

MAX_PEERS = 8
N_SLOTS = 64
AG_ROLES = 8          # exchange roles that may use the in-GEMM all-gather (each owns one block of chunk flags)
AG_CHUNKS = 64        # chunk flags per source rank (csrc/gemm.cu: kAgChunks)


class PeerSetC(ctypes.Structure):
    _fields_ = [("base", ctypes.c_uint64 * 8), ("flag", ctypes.c_uint64 * 8), ("n", ctypes.c_int)]


class GemmCommC(ctypes.Structure):
    _fields_ = [("ag_flags", ctypes.c_void_p), ("ag_epoch", ctypes.c_int), ("ag_rows", ctypes.c_int),
                ("ag_self", ctypes.c_int), ("fwd_dst", ctypes.c_uint64 * 8), ("fwd_flag", ctypes.c_uint64 * 8),
                ("fwd_peers", ctypes.c_int), ("fwd_src", ctypes.c_void_p), ("fwd_src_ld", ctypes.c_int),
                ("fwd_counter", ctypes.c_void_p),
                ("rs_base", ctypes.c_uint64 * 8), ("rs_flag", ctypes.c_void_p * 8),
                ("rs_counter", ctypes.c_void_p), ("rs_rows", ctypes.c_int), ("rs_self", ctypes.c_int),
                ("rs_ranks", ctypes.c_int), ("rs_epoch", ctypes.c_int),
                # column scatter of the output (Ulysses sequence -> heads in the QKV epilogue)
                ("sc_row", ctypes.c_void_p), ("sc_part", ctypes.c_int), ("sc_w", ctypes.c_int),
                ("sc_ld", ctypes.c_int), ("sc_rows_dst", ctypes.c_int),
                # K-slice consumer (Ulysses heads -> sequence in front of the output projection)
                ("kf_flags", ctypes.c_void_p), ("kf_epoch", ctypes.c_int), ("kf_w", ctypes.c_int),
                ("kf_self", ctypes.c_int), ("kf_ranks", ctypes.c_int)]


def check_gemm_comm_layout() -> None:
    """Compare the ctypes mirror of the GEMM's collective-role struct with the layout the library was compiled with."""
    fields = ["ag_flags", "ag_self", "fwd_dst", "fwd_flag", "fwd_peers", "fwd_src", "fwd_src_ld", "fwd_counter",
              "rs_base", "rs_flag", "rs_counter", "rs_rows", "rs_epoch", "sc_row", "sc_rows_dst", "kf_flags", "kf_ranks"]
    mine = [ctypes.sizeof(GemmCommC)] + [getattr(GemmCommC, f).offset for f in fields]
    buf = (ctypes.c_int * 32)()
    fn = nv.lib().mmt_gemm_comm_layout
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    n = fn(buf, 32)
    theirs = list(buf[:n])
    if theirs != mine:
        raise RuntimeError(f"GemmCommC does not match the library's MmtGemmComm: {mine} vs {theirs}; rebuild the "
                           "library (python -m multimodal_training_b200.csrc.build) or fix the binding")


class ZeroPeersC(ctypes.Structure):
    _fields_ = [("grad", ctypes.c_uint64 * 8), ("param", ctypes.c_uint64 * 8), ("param_flag", ctypes.c_uint64 * 8),
                ("n", ctypes.c_int)]


_P, _I, _L, _Fl = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
nv.declare("mmt_gemm_set_comm", None, [ctypes.POINTER(GemmCommC)])
nv.declare("mmt_rmsnorm_push", _I, [_P, _P, _P, ctypes.POINTER(PeerSetC), _P, _I, _L, _L, _I, _Fl, _P])
nv.declare("mmt_rs_reduce", _I, [_P, _P, _I, _I, _I, _P, _P, _L, _I, _P])
nv.declare("mmt_route_rows", _I, [_P, _P, _P, ctypes.POINTER(PeerSetC), _P, _I, _L, _I, _L, _L, _L, _P])
nv.declare("mmt_wait_flags", _I, [_P, _I, _I, _I, _P])
nv.declare("mmt_publish", _I, [ctypes.POINTER(PeerSetC), _I, _P])
nv.declare("mmt_zero1_adamw", _I, [ctypes.POINTER(ZeroPeersC), _P, _I, _I, _P, _I, _P, _P, _P, _L, _L, _L, _Fl, _Fl,
                                   _Fl, _Fl, _Fl, _I, _P, _P, _P])


class HeapContext:
    """A symmetric heap plus flag slots: [N_SLOTS, 8] int32 flags and [N_SLOTS] int32 CTA counters per rank."""

    def __init__(self, group, nbytes: int, device):
        self.heap = SymmetricHeap(group, nbytes + 2 * N_SLOTS * 64 + AG_ROLES * MAX_PEERS * AG_CHUNKS * 4 + 4096, device)
        self.size, self.rank = self.heap.size, self.heap.rank
        self.flags_off = self.heap.alloc("__flags", N_SLOTS * MAX_PEERS * 4)
        self.counters_off = self.heap.alloc("__counters", N_SLOTS * 4)
        # chunk flags of the all-gathers fused into GEMMs: [role][source rank][chunk] int32, zero at start
        self.agflags_off = self.heap.alloc("__agflags", AG_ROLES * MAX_PEERS * AG_CHUNKS * 4)
        self._slots: dict[str, int] = {}
        self._epochs: dict[int, int] = {}

    def slot(self, name: str) -> int:
        if name not in self._slots:
            if len(self._slots) >= N_SLOTS:
                raise RuntimeError("out of flag slots")
            self._slots[name] = len(self._slots)
        return self._slots[name]

    def next_epoch(self, slot: int) -> int:
        self._epochs[slot] = self._epochs.get(slot, 0) + 1
        return self._epochs[slot]

    def flag_addr(self, rank: int, slot: int, index: int) -> int:
        return self.heap.ptrs[rank] + self.flags_off + (slot * MAX_PEERS + index) * 4

    def local_flags(self, slot: int) -> int:
        return self.flag_addr(self.rank, slot, 0)

    def counter_addr(self, slot: int) -> int:
        return self.heap.local_ptr + self.counters_off + slot * 4

    def peerset(self, region_off: int, ranks: list[int], slot: int, my_index: int) -> PeerSetC:
        """Destinations = ``ranks`` (heap ranks); this rank signs flag word ``my_index`` of ``slot`` on each."""
        ps = PeerSetC()
        ps.n = len(ranks)
        for i, r in enumerate(ranks):
            ps.base[i] = self.heap.ptrs[r] + region_off
            ps.flag[i] = self.flag_addr(r, slot, my_index)
        return ps


class FusedComm:
    """Activation-side fused exchanges of one process (tensor parallel + handoff)."""

    def __init__(self, mesh, device, heap_bytes: int, checkpointed: bool = True, text_hidden: int = 0,
                 vision_hidden: int = 0):
        self.mesh = mesh
        self.device = device
        self.text_hidden, self.vision_hidden = int(text_hidden), int(vision_hidden)
        self.ulysses = False             # set by the vision trainer when the Ulysses exchange runs over the heap
        self._sizes = None
        # True: all-gather inside the consuming GEMM (ag_gemm); False: a push kernel in front of it (push_gather)
        self.fused_ag = os.environ.get("MMT_FUSED_AG", "1") == "1"
        self._ag_roles: dict[str, int] = {}
        self._views: dict = {}           # (region, shape, dtype) -> (offset, tensor view of this rank's buffer)
        self._ag_counter = None          # [AG_ROLES, AG_CHUNKS] int32: shares of a row block that have been forwarded
        check_gemm_comm_layout()
        self.ctx = HeapContext(mesh.world_group, heap_bytes, device)
        # results that live in reusable heap regions may be handed out as views only while BOTH halves recompute
        # their activations in backward; otherwise they are cloned (see set_checkpointed)
        self._ckpt = {"vision": bool(checkpointed), "text": bool(checkpointed)}
        base = mesh.tdp_rank * mesh.tp
        self.tp_ranks = [base + i for i in range(mesh.tp)]      # world (= heap) ranks of my TP group
        self.world_ranks = list(range(mesh.world))

    @property
    def checkpointed(self) -> bool:
        return all(self._ckpt.values())

    def set_checkpointed(self, half: str, on: bool) -> None:
        """Per-step decision of one half of the model ("vision" / "text") on activation recomputation."""
        self._ckpt[half] = bool(on)

    # ------------------------------------------------------------------ region capacities
    def region_plan(self, sizes) -> list[tuple[str, int]]:
        """(name, bytes) of every exchange buffer for a step whose largest extents over all ranks are ``sizes``
        (``trainers.context.StepSizes``).  Row counts are rounded up to quarter-octave buckets so that data sets
        whose batches vary in length settle after a few steps instead of growing a region every step."""
        from ..utils.checkpointing import bucket_tokens
        m, H, C = self.mesh, self.text_hidden, self.vision_hidden
        plan: list[tuple[str, int]] = []
        shard = bucket_tokens(max(int(sizes.shard_rows), 1))
        if m.tp > 1 and H:
            for role in ("qkv", "mlp", "o_bwd", "down_bwd"):
                plan.append(("ag_" + role, shard * m.tp * H * 2))
            for role in ("o", "down", "qkv_bwd", "mlp_bwd"):
                plan.append(("rs_" + role, shard * m.tp * H * 2))
        if sizes.has_images and H:
            plan.append(("handoff_in", shard * H * 2))
            plan.append(("handoff_grad", bucket_tokens(max(int(sizes.merged_rows), 1)) * H * 2))
        if self.ulysses and m.sp > 1 and C and sizes.has_images:
            t_all = bucket_tokens(max(int(sizes.vision_tokens_all), 1))
            t_loc = bucket_tokens(max(int(sizes.vision_tokens_rank), 1))
            W = C // m.sp
            plan += [("ul_heads3", t_all * 3 * W * 2), ("ul_tokens1", t_loc * C * 2),
                     ("ul_tokens3_bwd", t_loc * 3 * C * 2), ("ul_heads1_bwd", t_all * W * 2)]
        return plan

    def begin_step(self, sizes) -> None:
        """Reserve (or grow) every exchange buffer for this step, on every rank, in one fixed order and with sizes
        that are the same on all ranks -- whether or not this rank will use a given buffer in this step.  That is
        what keeps a region at the same offset in every rank's heap when batches are ragged: replicas with fewer
        tokens, or without images, still reserve what the largest replica needs."""
        if sizes == self._sizes:
            return
        self._sizes = sizes
        for name, nbytes in self.region_plan(sizes):
            self.ctx.heap.alloc(name, nbytes)

    def end_step(self) -> None:
        """Collective, main thread: after a step that reserved or moved regions, all ranks compare their tables."""
        heap = self.ctx.heap
        if heap.regions.version != heap.verified_version:
            heap.verify_layout()

    def reset_after_error(self) -> None:
        """A kernel that gave up on a wait may have left a completion counter half way (the CTA that would have
        published and reset it never came): zero this rank's counters so that a later step does not publish early.
        Called (after a device synchronisation) when the error word was found set; the step is invalid anyway."""
        if self._ag_counter is not None:
            self._ag_counter.zero_()
        self.ctx.heap.tensor(self.ctx.counters_off, (N_SLOTS,), torch.int32).zero_()

    def capacity_rows(self, what: str, rows: int) -> int:
        """Rows to reserve for a buffer of kind ``what`` that needs ``rows`` now: the step's world-wide maximum."""
        s = self._sizes
        if s is None:
            return rows
        return max(rows, {"shard": s.shard_rows, "merged": s.merged_rows}.get(what, 0))

    # ------------------------------------------------------------------ tensor parallel
    def _region(self, name: str, shape, dtype=torch.bfloat16) -> tuple[int, torch.Tensor]:
        n = 1
        for s in shape:
            n *= int(s)
        off = self.ctx.heap.alloc(name, n * 2)
        # wrapping a raw device pointer in a tensor costs tens of microseconds of host time, and a step asks for the
        # same few regions hundreds of times: keep the view while the region stays where it is
        key = (name, tuple(int(s) for s in shape), dtype)
        hit = self._views.get(key)
        if hit is not None and hit[0] == off:
            return off, hit[1]
        view = self.ctx.heap.tensor(off, shape, dtype)
        if len(self._views) > 256:
            self._views.clear()
        self._views[key] = (off, view)
        return off, view

    def push_gather(self, x_shard: torch.Tensor, norm_w, eps: float, role: str):
        """(RMSNorm of) a [T/tp, K] shard into every TP peer's [T, K] gather buffer.
        Returns ``(gathered_view, rstd, flags_ptr, epoch)``."""
        m = self.mesh
        rows, cols = x_shard.shape
        off, gathered = self._region("ag_" + role, (rows * m.tp, cols))
        slot = self.ctx.slot("ag_" + role)
        epoch = self.ctx.next_epoch(slot)
        rstd = torch.empty(rows, device=x_shard.device, dtype=torch.float32) if norm_w is not None else None
        ps = self.ctx.peerset(off, self.tp_ranks, slot, m.tp_rank)
        nv.call("mmt_rmsnorm_push", x_shard.data_ptr(), nv.ptr(norm_w), nv.ptr(rstd), ctypes.byref(ps),
                self.ctx.counter_addr(slot), epoch, m.tp_rank * rows, rows, cols, float(eps), nv.stream())
        return gathered, rstd, self.ctx.local_flags(slot), epoch

    def ag_gemm(self, x_shard: torch.Tensor, norm_w, eps: float, w, *, role: str, bias=None, b_mn: bool = False):
        """(RMSNorm of) a [T/tp, K] shard all-gathered INSIDE the GEMM that consumes it: ``gather(h) @ w^T + bias``.

        The GEMM starts on this rank's own rows; the CTAs that compute the first few column tiles of those rows
        forward the A tiles they load -- from shared memory, as bulk stores over NVLink -- to the same place of every
        peer's gather buffer and raise a flag per row block; the GEMM's TMA producer waits per (source rank, row
        block) before it reads a peer's rows.  The rows cross the link while the tensor cores work and are read from
        HBM once.  With a norm, a small kernel first leaves the normalised rows in this rank's own gather buffer;
        without one the GEMM reads them from ``x_shard`` directly and fills its own buffer on the way.  Falls back to
        the push kernel in front of the GEMM when the shard does not split into whole 256-row blocks.
        Returns ``(y, gathered, rstd)``."""
        m = self.mesh
        x_shard = x_shard.contiguous()
        rows, cols = x_shard.shape
        if rows % 256 or rows > 128 * AG_CHUNKS or m.tp > MAX_PEERS:
            gathered, rstd, flags, epoch = self.push_gather(x_shard, norm_w, eps, role)
            return self.gemm_gathered(gathered, flags, epoch, rows, w, b_mn=b_mn, bias=bias), gathered, rstd
        off, gathered = self._region("ag_" + role, (rows * m.tp, cols))
        ridx = self._ag_roles.setdefault(role, len(self._ag_roles))
        if ridx >= AG_ROLES:
            raise RuntimeError("too many all-gather roles")
        slot = self.ctx.slot("agc_" + role)
        epoch = self.ctx.next_epoch(slot)
        rstd = torch.empty(rows, device=x_shard.device, dtype=torch.float32) if norm_w is not None else None
        if norm_w is not None:
            # normalised own rows -> own buffer (the flag this raises is not read by anyone)
            me = self.ctx.peerset(off, [self.tp_ranks[m.tp_rank]], slot, m.tp_rank)
            nv.call("mmt_rmsnorm_push", x_shard.data_ptr(), nv.ptr(norm_w), nv.ptr(rstd), ctypes.byref(me),
                    self.ctx.counter_addr(slot), epoch, m.tp_rank * rows, rows, cols, float(eps), nv.stream())
        if self._ag_counter is None:
            self._ag_counter = torch.zeros(AG_ROLES * AG_CHUNKS, dtype=torch.int32, device=x_shard.device)
        block = self.ctx.agflags_off + ridx * MAX_PEERS * AG_CHUNKS * 4
        c = GemmCommC()
        c.ag_flags = self.ctx.heap.local_ptr + block
        c.ag_epoch, c.ag_rows, c.ag_self = epoch, rows, m.tp_rank
        peers = [r for i, r in enumerate(self.tp_ranks) if i != m.tp_rank]
        for i, r in enumerate(peers):
            c.fwd_dst[i] = self.ctx.heap.ptrs[r] + off
            c.fwd_flag[i] = self.ctx.heap.ptrs[r] + block
        c.fwd_peers = len(peers)
        if norm_w is None:
            c.fwd_src, c.fwd_src_ld = x_shard.data_ptr(), cols
        c.fwd_counter = self._ag_counter.data_ptr() + ridx * AG_CHUNKS * 4
        c.rs_rows = 0
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        y = F.gemm(gathered, w, b_mn=b_mn, bias=bias)
        return y, gathered, rstd

    def gemm_gathered(self, gathered, flags_ptr, epoch, rows_per_rank, w, *, b_mn=False, bias=None):
        c = GemmCommC()
        c.ag_flags, c.ag_epoch, c.ag_rows, c.ag_self = flags_ptr, epoch, rows_per_rank, self.mesh.tp_rank
        c.rs_rows = 0
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        return F.gemm(gathered, w, b_mn=b_mn, bias=bias)

    def gemm_reduce_scatter(self, a, w, *, b_mn: bool, residual, role: str) -> torch.Tensor:
        """``sum over TP ranks of (a @ w^T)`` scattered by token rows (+ residual): [T, K/tp] -> [T/tp, N]."""
        m = self.mesh
        T = a.shape[0]
        N = w.shape[1] if b_mn else w.shape[0]
        if T % m.tp:
            raise ValueError(f"GEMM -> reduce-scatter over {m.tp} ranks needs a token count that {m.tp} divides, "
                             f"got {T} (the row owner would be out of range)")
        rows = T // m.tp
        off, staging = self._region("rs_" + role, (m.tp * rows, N))
        slot = self.ctx.slot("rs_" + role)
        epoch = self.ctx.next_epoch(slot)
        c = GemmCommC()
        c.ag_flags = None
        c.rs_rows, c.rs_self, c.rs_ranks, c.rs_epoch = rows, m.tp_rank, m.tp, epoch
        c.rs_counter = self.ctx.counter_addr(slot)
        for i, r in enumerate(self.tp_ranks):
            c.rs_base[i] = self.ctx.heap.ptrs[r] + off
            c.rs_flag[i] = self.ctx.flag_addr(r, slot, m.tp_rank)
        nv.lib().mmt_gemm_set_comm(ctypes.byref(c))
        F.gemm(a, w, b_mn=b_mn, out=staging[:T])
        out = torch.empty(rows, N, device=a.device, dtype=a.dtype)
        nv.call("mmt_rs_reduce", staging.data_ptr(), self.ctx.local_flags(slot), epoch, m.tp, m.tp_rank,
                nv.ptr(residual), out.data_ptr(), rows, N, nv.stream())
        return out

    def ag_linear(self, x_shard, w, b, norm_w=None, eps: float = 1e-6, role: str = "qkv"):
        return _FusedColLinearFn.apply(x_shard, norm_w, w, b, self, role, eps)

    def linear_rs(self, a, w, residual_shard, role: str = "o"):
        return _FusedRowLinearFn.apply(a, w, residual_shard, self, role)

    # ------------------------------------------------------------------ vision -> text handoff
    def handoff(self, leaf: torch.Tensor, x_shard: torch.Tensor, plan) -> torch.Tensor:
        return _FusedHandoffFn.apply(leaf, x_shard, plan, self)

    def route(self, src, dest_rank, dest_row, region: str, region_rows: int, cols: int):
        """Store src rows to (world rank, row) destinations of ``region`` and wait for everybody's rows."""
        if dest_rank.dtype != torch.int32 or dest_row.dtype != torch.int64:
            raise TypeError("route: dest_rank must be int32 and dest_row int64")
        off, local = self._region(region, (region_rows, cols))
        slot = self.ctx.slot(region)
        epoch = self.ctx.next_epoch(slot)
        ps = self.ctx.peerset(off, self.world_ranks, slot, self.mesh.rank)
        nv.call("mmt_route_rows", src.data_ptr(), dest_rank.data_ptr(), dest_row.data_ptr(), ctypes.byref(ps),
                self.ctx.counter_addr(slot), epoch, src.shape[0], cols, src.stride(0) if src.shape[0] else cols, cols,
                region_rows, nv.stream())
        nv.call("mmt_wait_flags", self.ctx.local_flags(slot), self.mesh.world, -1, epoch, nv.stream())
        return local

    def close(self) -> None:
        self.ctx.heap.close()


def _dev_plan(plan, device):
    if getattr(plan, "_dev", None) is None:
        plan._dev = {k: getattr(plan, k).to(device, non_blocking=True)
                     for k in ("dest_rank", "dest_row", "recv_src_rank", "recv_src_index", "recv_rows")}
    return plan._dev


class _FusedColLinearFn(torch.autograd.Function):
    """[T/tp, K] token shard -> (RMSNorm) -> all-gather fused into ``x @ w^T + b`` -> [T, N/tp]."""

    @staticmethod
    def forward(ctx, x_shard, norm_w, w, b, fc: FusedComm, role, eps):
        x_shard = x_shard.contiguous()
        rows = x_shard.shape[0]
        if fc.fused_ag:
            y, gathered, rstd = fc.ag_gemm(x_shard, norm_w, eps, w, role=role, bias=b)
        else:
            gathered, rstd, flags, epoch = fc.push_gather(x_shard, norm_w, eps, role)
            y = fc.gemm_gathered(gathered, flags, epoch, rows, w, bias=b)
        if not fc.checkpointed:
            gathered = gathered.clone()
        ctx.save_for_backward(x_shard, norm_w, rstd, w, gathered)
        ctx.misc = (fc, role, b, eps)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_shard, norm_w, rstd, w, gathered = ctx.saved_tensors
        fc, role, b, eps = ctx.misc
        dy = dy.contiguous()
        # weight gradients first: they read the gathered input, which a peer may overwrite as soon as
        # this rank's partial input-gradients are published below
        dw = F._write_param_grad(w, lambda out, acc: F.gemm(dy, gathered, a_mn=True, b_mn=True, out=out,
                                                           accumulate=acc))
        db = None
        if b is not None:
            db = F._write_param_grad(b, lambda out, acc: F.colsum(dy, out=out, accumulate=acc))
        dh = fc.gemm_reduce_scatter(dy, w, b_mn=True, residual=None, role=role + "_bwd")
        dnw = None
        if norm_w is not None:
            rows, cols = x_shard.shape
            dx = torch.empty_like(x_shard)
            parts = nv.lib().mmt_rmsnorm_bwd_parts(rows)
            scratch = F._scratch_f32(parts * cols, x_shard.device, "rmsnorm")

            def run(out, acc):
                nv.call("mmt_rmsnorm_bwd", dh.data_ptr(), x_shard.data_ptr(), norm_w.data_ptr(), rstd.data_ptr(),
                        dx.data_ptr(), out.data_ptr(), scratch.data_ptr(), rows, cols, int(acc), nv.stream())

            dnw = F._write_param_grad(norm_w, run)
        else:
            dx = dh
        return dx, dnw, dw, db, None, None, None


class _FusedRowLinearFn(torch.autograd.Function):
    """[T, K/tp] -> ``a @ w^T`` with the reduce-scatter in the GEMM epilogue -> [T/tp, N] (+ residual)."""

    @staticmethod
    def forward(ctx, a, w, residual, fc: FusedComm, role):
        a = a.contiguous()
        out = fc.gemm_reduce_scatter(a, w, b_mn=False, residual=residual, role=role)
        ctx.save_for_backward(a, w)
        ctx.misc = (fc, role, residual is not None)
        return out

    @staticmethod
    def backward(ctx, dy_shard):
        a, w = ctx.saved_tensors
        fc, role, has_res = ctx.misc
        dy_shard = dy_shard.contiguous()
        rows = dy_shard.shape[0]
        if fc.fused_ag:
            da, gathered, _ = fc.ag_gemm(dy_shard, None, 0.0, w, role=role + "_bwd", b_mn=True)
        else:
            gathered, _, flags, epoch = fc.push_gather(dy_shard, None, 0.0, role + "_bwd")
            da = fc.gemm_gathered(gathered, flags, epoch, rows, w, b_mn=True)
        dw = F._write_param_grad(w, lambda out, acc: F.gemm(gathered, a, a_mn=True, b_mn=True, out=out,
                                                           accumulate=acc))
        return da, dw, (dy_shard if has_res else None), None, None


class _FusedHandoffFn(torch.autograd.Function):
    """Merged vision tokens stored straight into the owning text ranks' rows; gradient returns the same way."""

    @staticmethod
    def forward(ctx, leaf, x_shard, plan, fc: FusedComm):
        dev = x_shard.device
        d = _dev_plan(plan, dev)
        H = x_shard.shape[1]
        region = fc.route(leaf.contiguous(), d["dest_rank"], d["dest_row"], "handoff_in",
                          fc.capacity_rows("shard", x_shard.shape[0]), H)
        out = x_shard.clone()
        rows = d["recv_rows"]
        if rows.numel():
            F.scatter_rows_raw(F.gather_rows_raw(region, rows), rows, out)
        ctx.plan, ctx.fc, ctx.n_local = plan, fc, leaf.shape[0]
        return out

    @staticmethod
    def backward(ctx, dout):
        plan, fc = ctx.plan, ctx.fc
        dout = dout.contiguous()
        d = _dev_plan(plan, dout.device)
        rows = d["recv_rows"]
        H = dout.shape[1]
        g = F.gather_rows_raw(dout, rows) if rows.numel() else dout.new_zeros((0, H))
        # the region is sized by the LARGEST rank's merged-token count (ragged splits give the ranks different
        # counts): a region has to have the same size on every rank, and rows of a larger peer must pass the
        # destination bound of a smaller one
        region = fc.route(g, d["recv_src_rank"], d["recv_src_index"], "handoff_grad",
                          fc.capacity_rows("merged", max(ctx.n_local, 1)), H)
        dleaf = region[:ctx.n_local].clone()
        dx = dout.clone()
        if rows.numel():
            dx.index_fill_(0, rows, 0)
        return dleaf, dx, None, None


class FusedZero:
    """ZeRO-1 step as one kernel over a heap that holds the flat parameters and gradients of a ZeRO group."""

    def __init__(self, group, total_elems: int, device):
        self.ctx = HeapContext(group, total_elems * 2 * 2 + 4096, device)
        self.param_off = self.ctx.heap.alloc("flat_param", total_elems * 2)
        self.grad_off = self.ctx.heap.alloc("flat_grad", total_elems * 2)
        self.flat_param = self.ctx.heap.tensor(self.param_off, (total_elems,), torch.bfloat16)
        self.flat_grad = self.ctx.heap.tensor(self.grad_off, (total_elems,), torch.bfloat16)
        self.grad_slot = self.ctx.slot("grad_ready")
        self.param_slot = self.ctx.slot("param_ready")
        self.ranks = list(range(self.ctx.size))

    def step(self, master, m, v, lo: int, n: int, n_decay_local: int, lr, b1, b2, eps, wd, step: int, gscale,
             normsq) -> None:
        c = self.ctx
        ge = c.next_epoch(self.grad_slot)
        pe = c.next_epoch(self.param_slot)
        ps = c.peerset(0, self.ranks, self.grad_slot, c.rank)
        nv.call("mmt_publish", ctypes.byref(ps), ge, nv.stream())
        zp = ZeroPeersC()
        zp.n = c.size
        for i, r in enumerate(self.ranks):
            zp.grad[i] = c.heap.ptrs[r] + self.grad_off
            zp.param[i] = c.heap.ptrs[r] + self.param_off
            zp.param_flag[i] = c.flag_addr(r, self.param_slot, c.rank)
        nv.call("mmt_zero1_adamw", ctypes.byref(zp), c.local_flags(self.grad_slot), ge, c.rank,
                c.counter_addr(self.param_slot), pe, master.data_ptr(), m.data_ptr(), v.data_ptr(), lo, n,
                n_decay_local, lr, b1, b2, eps, wd, step, nv.ptr(gscale), nv.ptr(normsq), nv.stream())
        nv.call("mmt_wait_flags", c.local_flags(self.param_slot), c.size, -1, pe, nv.stream())


def try_create(mesh, config):
    """Returns ``(heap_context, FusedComm)`` or ``(None, None)`` when peer memory cannot be set up."""
    try:
        dev = torch.device("cuda", torch.cuda.current_device())
        lib = nv.lib()
        for peer in range(torch.cuda.device_count()):
            if peer != dev.index and not lib.mmt_can_access_peer(dev.index, peer):
                log.warning("GPU %d cannot access GPU %d: fused collectives are off", dev.index, peer)
                return None, None
        if mesh.world > MAX_PEERS:
            return None, None
        heap_mb = int(config.get("symm_heap_mb", 8192))
        from ..config.model_configs import get_model_config
        mc = get_model_config(config.get("model_name", "qwen2_5_vl_7b"))
        fc = FusedComm(mesh, dev, heap_mb << 20, checkpointed=config.get("activation_checkpointing", True) is True,
                       text_hidden=mc.text.hidden_size, vision_hidden=mc.vision.hidden_size)
        return fc.ctx, fc
    except Exception as e:  # the NCCL path still works; say why the fused one does not
        log.warning("fused collectives unavailable: %s", e)
        return None, None
