"""Symmetric heap over CUDA IPC: the memory that the fused compute+collective kernels address.

Every rank allocates one buffer of the same size; the IPC handles travel through
``torch.distributed`` (host control plane) and each rank maps all peers' buffers.  Regions are carved
with a bump allocator (plus a free list for regions that had to grow) that every rank calls in the same
order with the same sizes, so a region has the same offset on all ranks and a peer's copy is
``peer_base + offset``; ``verify_layout`` checks exactly that across the ranks.  Flags are int32 words inside the heap that
count epochs upward and are never reset.

Counterpart in the reference: this replaces the reference's per-tensor IPC handle + event transfer
(python/ray/tensor_transfer.py:35-96) and is the substrate of ``parallel/fused.py``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native as nv

nv.declare("mmt_symm_alloc", ctypes.c_int, [ctypes.c_size_t, ctypes.POINTER(ctypes.c_void_p)])
nv.declare("mmt_symm_free", ctypes.c_int, [ctypes.c_void_p])
nv.declare("mmt_symm_export", ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p])
nv.declare("mmt_symm_import", ctypes.c_int, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)])
nv.declare("mmt_symm_unimport", ctypes.c_int, [ctypes.c_void_p])
nv.declare("mmt_can_access_peer", ctypes.c_int, [ctypes.c_int, ctypes.c_int])

_DT = {torch.bfloat16: ("<u2", 2), torch.float32: ("<f4", 4), torch.int32: ("<i4", 4), torch.int64: ("<i8", 8),
       torch.uint8: ("|u1", 1)}


class _RawCuda:
    """Adapter exposing a raw device pointer through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                         "strides": None}


def tensor_from_ptr(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    nbytes = n * _DT[dtype][1]
    raw = torch.as_tensor(_RawCuda(ptr, max(nbytes, 1)), device=device)
    return raw[:nbytes].view(dtype).view(*shape)


class RegionAllocator:
    """Named regions of a symmetric buffer: a bump allocator plus a free list for regions that had to grow.

    Pure host-side bookkeeping (no CUDA), so the policy can be tested anywhere.  Every rank must issue the same
    calls in the same order with the same sizes; ``digest`` lets the ranks check that they did."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self._off = 0
        self._regions: dict[str, tuple[int, int]] = {}
        self._free: list[tuple[int, int]] = []
        self.version = 0                 # bumped by every reservation or move

    def alloc(self, name: str, nbytes: int, align: int = 1024) -> int:
        """Reserve a region (same calls, in the same order and with the same sizes, on every rank); returns its byte
        offset.  Asking again for a name returns the same offset while the request fits; a larger request MOVES the
        region to a new block (its old block goes to a free list that later requests reuse), so callers never keep
        an offset across calls.  Contents are not carried over: regions hold one exchange at a time."""
        nbytes = int(nbytes)
        if name in self._regions:
            off, size = self._regions[name]
            if size >= nbytes:
                return off
            self._free.append((off, size))
            del self._regions[name]
        self.version += 1
        # first fit among freed blocks, else bump
        for i, (foff, fsize) in enumerate(self._free):
            if fsize >= nbytes:
                del self._free[i]
                self._regions[name] = (foff, fsize)
                return foff
        off = (self._off + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: {off + nbytes} > {self.nbytes} bytes (region {name}); "
                              "raise training.symm_heap_mb")
        self._off = off + nbytes
        self._regions[name] = (off, nbytes)
        return off

    def digest(self) -> str:
        """Hash of (name, offset, size) of every region: equal on all ranks or peer addresses are wrong."""
        import hashlib
        h = hashlib.sha256()
        for name in sorted(self._regions):
            off, size = self._regions[name]
            h.update(f"{name}:{off}:{size};".encode())
        return h.hexdigest()

    def table(self) -> list:
        return sorted(self._regions.items())

    def used(self) -> int:
        return self._off


class SymmetricHeap:
    def __init__(self, group, nbytes: int, device: torch.device):
        self.group = group
        self.size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.nbytes = int(nbytes)
        lib = nv.lib()
        p = ctypes.c_void_p()
        nv.check(lib.mmt_symm_alloc(self.nbytes, ctypes.byref(p)), "mmt_symm_alloc")
        self.local_ptr = p.value
        buf = ctypes.create_string_buffer(64)
        nv.check(lib.mmt_symm_export(self.local_ptr, buf), "mmt_symm_export")
        handles = [None] * self.size
        dist.all_gather_object(handles, bytes(buf.raw), group=group)
        self.ptrs = []
        self._imported = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local_ptr)
                continue
            q = ctypes.c_void_p()
            nv.check(lib.mmt_symm_import(h, ctypes.byref(q)), f"mmt_symm_import(rank {r})")
            self.ptrs.append(q.value)
            self._imported.append(q.value)
        self.ptr_table = torch.tensor(self.ptrs, dtype=torch.int64, device=device)
        self.regions = RegionAllocator(self.nbytes)
        self.verified_version = 0        # allocator version that verify_layout last confirmed on all ranks
        dist.barrier(group=group)

    def alloc(self, name: str, nbytes: int, align: int = 1024) -> int:
        """Reserve (or grow) a region; see :meth:`RegionAllocator.alloc`."""
        return self.regions.alloc(name, nbytes, align)

    def verify_layout(self) -> None:
        """Collective: raise unless every rank of the heap's group has the same region table."""
        digests = [None] * self.size
        dist.all_gather_object(digests, (self.regions.digest(), self.regions.table()), group=self.group)
        mine = digests[self.rank][0]
        for r, (d, table) in enumerate(digests):
            if d != mine:
                diff = [(k, v, dict(digests[self.rank][1]).get(k)) for k, v in table
                        if dict(digests[self.rank][1]).get(k) != v]
                raise RuntimeError(f"symmetric heap layout differs between rank {self.rank} and rank {r}: {diff[:4]}; "
                                   "a peer address would point at the wrong buffer")
        self.verified_version = self.regions.version

    def tensor(self, offset: int, shape, dtype: torch.dtype, rank: int | None = None) -> torch.Tensor:
        """View of a region in this rank's buffer (or, for debugging only, in a peer's mapping)."""
        base = self.local_ptr if rank is None else self.ptrs[rank]
        return tensor_from_ptr(base + offset, shape, dtype, self.device)

    def close(self) -> None:
        lib = nv.lib()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier(group=self.group)
        for q in self._imported:
            lib.mmt_symm_unimport(q)
        self._imported = []
        if self.local_ptr:
            lib.mmt_symm_free(self.local_ptr)
            self.local_ptr = 0
