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


class ShardedGrads:
    """Gradients of the whole list in the weights' layout, and their reduce-scatter into this rank's
    shard: the front half of the sharded step.  ``views[i]`` is where backward leaves tensor i's local
    gradient; after ``reduce_scatter()`` ``owned[k]`` holds the reduced gradient of the k-th owned
    tensor, inside the collective's own output buffer, which is what the step kernels read (the
    gradient pointers never change, so the plan's pointer column is uploaded once)."""

    def __init__(self, weights: ShardedWeights, shapes, dtype=None):
        import torch
        sw = self.weights = weights
        dtype = dtype or sw.flat.dtype
        self.flat = torch.zeros(sw.world * sw.part.shard_len, dtype=dtype, device=sw.flat.device)
        self.shard = (self.flat if sw.world == 1 else
                      torch.zeros(sw.part.shard_len, dtype=dtype, device=sw.flat.device))
        self.views, self.owned = [], []
        for i, s in enumerate(shapes):
            n = math.prod(s)
            start = sw.part.owner[i] * sw.part.shard_len + sw.part.offset[i]
            self.views.append(self.flat[start:start + n].view(s))
            if sw.part.owner[i] == sw.rank:
                self.owned.append(self.shard[sw.part.offset[i]:sw.part.offset[i] + n].view(s))

    def reduce_scatter(self, average: bool = True, async_op: bool = False):
        import torch.distributed as dist
        sw = self.weights
        if sw.world == 1:
            return None
        if dist.get_backend(sw.group) == "gloo":
            # gloo (CPU tests of the host flow) has no reduce-scatter: all-reduce, keep this rank's slice
            dist.all_reduce(self.flat, group=sw.group)
            self.shard.copy_(self.flat[sw.rank * sw.part.shard_len:(sw.rank + 1) * sw.part.shard_len])
            if average:
                self.shard.div_(sw.world)
            return None
        op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
        return dist.reduce_scatter_tensor(self.shard, self.flat, op=op, group=sw.group, async_op=async_op)


# ---- checkpoints of a sharded optimizer in the single-process layout ----

def _global_ids(optimizer) -> list[int]:
    """Global list position of every parameter, in the optimizer's packed (param_groups) order."""
    ids = []
    for g in optimizer.param_groups:
        for p in g["params"]:
            if not hasattr(p, "kaon_tensor_id"):
                raise ValueError("sharded checkpoints need p.kaon_tensor_id (the global list position) on every parameter")
            ids.append(int(p.kaon_tensor_id))
    return ids


def gather_state_dict(optimizer, group=None, dst: int = 0):
    """Every rank's optimizer state merged into ONE ``state_dict`` with the layout a single-process
    optimizer over the whole list would save (state keyed by global list position; tensors on the CPU).
    Returned on rank ``dst``, ``None`` elsewhere.  Collective: every rank calls it."""
    import torch
    import torch.distributed as dist
    sd = optimizer.state_dict()
    ids = _global_ids(optimizer)
    to_cpu = lambda v: v.detach().cpu() if torch.is_tensor(v) else v  # noqa: E731
    state = {ids[k]: {key: to_cpu(v) for key, v in st.items()} for k, st in sd["state"].items()}
    groups, k = [], 0
    for g in sd["param_groups"]:
        n = len(g["params"])
        groups.append({**g, "params": ids[k:k + n]})
        k += n
    payload = {"state": state, "param_groups": groups}
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        parts = [payload]
    else:
        parts = [None] * world if dist.get_rank(group) == dst else None
        dist.gather_object(payload, parts, dst=dst, group=group)
        if parts is None:
            return None
    merged_state, merged_groups = {}, [dict(g, params=[]) for g in parts[0]["param_groups"]]
    for part in parts:
        merged_state.update(part["state"])
        for gi, g in enumerate(part["param_groups"]):
            merged_groups[gi]["params"].extend(g["params"])
    for g in merged_groups:
        g["params"] = sorted(g["params"])
    out = {k: v for k, v in sd.items() if k not in ("state", "param_groups")}
    out["state"] = dict(sorted(merged_state.items()))
    out["param_groups"] = merged_groups
    return out


def scatter_state_dict(optimizer, full_state_dict) -> None:
    """Load this rank's part of a single-process (or gathered) ``state_dict`` into a sharded optimizer.
    Every rank passes the same full dict (e.g. each reads the checkpoint file)."""
    ids = _global_ids(optimizer)
    local_state = {k: full_state_dict["state"][gid] for k, gid in enumerate(ids) if gid in full_state_dict["state"]}
    groups, k = [], 0
    if len(full_state_dict["param_groups"]) != len(optimizer.param_groups):
        raise ValueError("checkpoint and optimizer have different numbers of parameter groups")
    for g_full, g in zip(full_state_dict["param_groups"], optimizer.param_groups):
        n = len(g["params"])
        missing = set(ids[k:k + n]) - set(g_full["params"])
        if missing:
            raise ValueError(f"checkpoint group lacks tensors {sorted(missing)[:5]} of this rank's group")
        groups.append({**g_full, "params": list(range(k, k + n))})
        k += n
    local = {key: v for key, v in full_state_dict.items() if key not in ("state", "param_groups")}
    local["state"] = local_state
    local["param_groups"] = groups
    optimizer.load_state_dict(local)
