"""ZeRO-1-style sharding of a parameter list over the GPUs of one node.

No counterpart in the reference (it has no distributed code).  Tensors are independent units of the
optimizer step (every reduction is per tensor), so whole tensors are assigned to ranks: greedy
largest-first onto the lightest rank.  Each rank's tensors sit back to back (128-element aligned) in one
flat weight buffer of ``world * shard_len`` elements whose rank-r slice holds rank r's tensors, so the
updated weights are exchanged with ONE in-place all-gather and no packing - or, with ``symmetric=True``,
with no collective at all: the buffer is allocated as symmetric memory, every rank maps the others'
copies, and the step kernels store each updated weight into all copies as they go (plain peer stores
over NVLink), so the exchange overlaps the step tile by tile and only a barrier follows.  Optimizer
state exists only on the owner.  ``tensor_id`` stays the global list position, so the stochastic-rounding stream - and
with it every weight - is the same for any number of ranks.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

ALIGN = 128  # elements; keeps every tensor 16-byte aligned and 4-bit blocks whole


@dataclass
class Partition:
    world: int
    owner: list[int]            # owner[i] = rank of tensor i
    offset: list[int]           # element offset of tensor i inside its owner's shard
    shard_len: int              # elements per rank (equal, padded)
    load: list[int]             # elements per rank before padding

    def owned(self, rank: int) -> list[int]:
        return [i for i, r in enumerate(self.owner) if r == rank]


def partition(shapes, world: int) -> Partition:
    sizes = [math.prod(s) for s in shapes]
    order = sorted(range(len(sizes)), key=lambda i: (-sizes[i], i))
    load = [0] * world
    owner = [0] * len(sizes)
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += sizes[i]
    offset = [0] * len(sizes)
    cursor = [0] * world
    for i in range(len(sizes)):  # list order inside a shard
        r = owner[i]
        offset[i] = cursor[r]
        cursor[r] += (sizes[i] + ALIGN - 1) // ALIGN * ALIGN
    shard_len = max(cursor) if cursor else 0
    shard_len = (shard_len + ALIGN - 1) // ALIGN * ALIGN
    return Partition(world, owner, offset, shard_len, load)


class ShardedWeights:
    """The flat weight buffer of one rank and views of every tensor in it.

    ``views[i]`` is tensor i's weights on this rank (owned or gathered); ``all_gather()`` publishes the
    owned slice to every rank.
    """

    def __init__(self, shapes, world: int, rank: int, dtype, device, symmetric: bool = False, group=None):
        import torch
        self.part = partition(shapes, world)
        self.rank, self.world, self.group = rank, world, group
        n = world * self.part.shard_len
        self.peer_deltas: list[int] = []
        if symmetric and world > 1:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            self.flat = symm_mem.empty(n, dtype=dtype, device=device)
            self.flat.zero_()
            hdl = symm_mem.rendezvous(self.flat, group=group if group is not None else dist.group.WORLD)
            self._hdl = hdl  # keeps the peer mappings alive
            base = self.flat.data_ptr()
            self.peer_deltas = [int(ptr) - base for r, ptr in enumerate(hdl.buffer_ptrs) if r != rank]
            self._tick = torch.zeros(1, dtype=torch.float32, device=device)
        else:
            self.flat = torch.zeros(n, dtype=dtype, device=device)
        self.views = []
        for i, s in enumerate(shapes):
            start = self.part.owner[i] * self.part.shard_len + self.part.offset[i]
            self.views.append(self.flat[start:start + math.prod(s)].view(s))
        self.shard = self.flat[rank * self.part.shard_len:(rank + 1) * self.part.shard_len]

    def attach(self, optimizer) -> None:
        """Have ``optimizer``'s step kernels store the weights they write into every rank's copy."""
        if self.peer_deltas:
            optimizer.set_weight_mirrors(self.flat.data_ptr(), self.flat.numel() * self.flat.element_size(),
                                         self.peer_deltas)

    def publish(self):
        """After ``optimizer.step()``: make this step's weights of every rank usable on every rank.
        Mirrored buffers need only a barrier in stream order (a one-element all-reduce: no rank passes
        it before every rank's step kernels have finished, peer stores included); otherwise all-gather."""
        if self.world == 1:
            return None
        if self.peer_deltas:
            import torch.distributed as dist
            return dist.all_reduce(self._tick, group=self.group)
        return self.all_gather(group=self.group)

    def all_gather(self, group=None, async_op: bool = False):
        import torch.distributed as dist
        if self.world == 1:
            return None
        return dist.all_gather_into_tensor(self.flat, self.shard, group=group, async_op=async_op)
