"""Process mesh of the collocated hybrid-parallel job.

One process per GPU hosts a vision rank and a text rank.  The same ``world`` ranks are
factored twice: vision = ``sp`` (sequence parallel, fastest) x ``vdp`` (data parallel),
text = ``tp`` (tensor parallel, fastest) x ``tdp`` (data parallel).  The reference builds two
unrelated worlds, one per ActorGroup (python/ray/actor_group.py:103-138), and moves tensors
between them through Ray; sharing one world lets the handoff be a collective or a peer store.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch.distributed as dist


@dataclass
class Mesh:
    world: int = 1
    rank: int = 0
    sp: int = 1
    tp: int = 1
    world_group: object = None
    sp_group: object = None        # vision ranks sharing the same images
    vdp_group: object = None       # vision ranks with the same sp rank across replicas
    vision_zero_group: object = None  # all vision ranks holding the same parameters (= world)
    tp_group: object = None
    tdp_group: object = None       # text ranks with the same tp rank across replicas (ZeRO / grad reduce)

    @property
    def vdp(self) -> int:
        return self.world // self.sp

    @property
    def tdp(self) -> int:
        return self.world // self.tp

    @property
    def sp_rank(self) -> int:
        return self.rank % self.sp

    @property
    def vdp_rank(self) -> int:
        return self.rank // self.sp

    @property
    def tp_rank(self) -> int:
        return self.rank % self.tp

    @property
    def tdp_rank(self) -> int:
        return self.rank // self.tp


def build_mesh(sp: int, tp: int) -> Mesh:
    """Create every sub-group (all ranks must call this in the same order)."""
    if not dist.is_initialized():
        if sp != 1 or tp != 1:
            raise RuntimeError("torch.distributed is not initialised but sp/tp > 1 was requested")
        return Mesh()
    world, rank = dist.get_world_size(), dist.get_rank()
    if world % sp or world % tp:
        raise ValueError(f"world size {world} is not divisible by sp={sp} / tp={tp}")
    m = Mesh(world=world, rank=rank, sp=sp, tp=tp, world_group=dist.group.WORLD)

    def make(groups):
        mine = None
        for ranks in groups:
            g = dist.new_group(ranks) if len(ranks) < world else dist.group.WORLD
            if rank in ranks:
                mine = g
        return mine

    m.sp_group = make([list(range(i * sp, (i + 1) * sp)) for i in range(world // sp)])
    m.vdp_group = make([list(range(i, world, sp)) for i in range(sp)])
    m.tp_group = make([list(range(i * tp, (i + 1) * tp)) for i in range(world // tp)])
    m.tdp_group = make([list(range(i, world, tp)) for i in range(tp)])
    m.vision_zero_group = dist.group.WORLD
    return m
