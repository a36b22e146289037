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
    """Gradients of the whole list and their reduce-scatter into this rank's shard: the front half of the
    sharded step.  ``views[i]`` is where backward leaves tensor i's local gradient; after the reduce-scatter
    ``owned[k]`` holds the reduced gradient of the k-th owned tensor, inside the collective's own output
    buffer, which is what the step kernels read (the gradient pointers never change, so the plan's pointer
    column is uploaded once).

    ``waves > 1`` cuts every rank's tensors (in list order) into that many consecutive waves of about equal
    size and lays the buffers out wave by wave (wave w: ``[rank 0's part | rank 1's part | ...]``, parts
    padded to the longest), so that each wave is ONE contiguous reduce-scatter.  ``wave_of[i]`` names tensor
    i's wave; ``reduce_scatter_waves()`` issues them back to back and returns their handles, so a step
    that waits per wave (one parameter group per wave) runs wave w while wave w+1 is still on the wire."""

    def __init__(self, weights: ShardedWeights, shapes, dtype=None, waves: int = 1):
        import torch
        sw = self.weights = weights
        dtype = dtype or sw.flat.dtype
        world, W = sw.world, max(1, int(waves))
        sizes = [math.prod(s) for s in shapes]
        pad = lambda n: (n + ALIGN - 1) // ALIGN * ALIGN  # noqa: E731
        # waves per rank: consecutive owned tensors, cut where the running size passes w/W of the rank's load
        self.wave_of = [0] * len(shapes)
        wave_len = [0] * W                      # longest part of each wave over the ranks
        off_in_wave = [0] * len(shapes)
        for r in range(world):
            owned = sw.part.owned(r)
            total = sum(pad(sizes[i]) for i in owned)
            run, cur = 0, [0] * W
            for i in owned:
                w = min(W - 1, run * W // total) if total else 0
                self.wave_of[i] = w
                off_in_wave[i] = cur[w]
                cur[w] += pad(sizes[i])
                run += pad(sizes[i])
            wave_len = [max(a, b) for a, b in zip(wave_len, cur)]
        self.waves = W
        self.wave_len = wave_len
        wave_base = [0] * (W + 1)               # offset of each wave inside a shard
        for w in range(W):
            wave_base[w + 1] = wave_base[w] + wave_len[w]
        self._wave_base = wave_base
        shard_len = wave_base[W]
        self.flat = torch.zeros(world * shard_len, dtype=dtype, device=sw.flat.device)
        self.shard = (self.flat if world == 1 else torch.zeros(shard_len, dtype=dtype, device=sw.flat.device))
        self.views, self.owned = [], []
        for i, s in enumerate(shapes):
            n, w, r = sizes[i], self.wave_of[i], sw.part.owner[i]
            start = world * wave_base[w] + r * wave_len[w] + off_in_wave[i]
            self.views.append(self.flat[start:start + n].view(s))
            if r == sw.rank:
                o = (start if world == 1 else wave_base[w] + off_in_wave[i])
                self.owned.append(self.shard[o:o + n].view(s))

    def _wave_buffers(self, w: int):
        world, b, n = self.weights.world, self._wave_base[w], self.wave_len[w]
        return self.shard[b:b + n], self.flat[world * b:world * (b + n)]

    def reduce_scatter_wave(self, w: int, average: bool = True, async_op: bool = False):
        import torch.distributed as dist
        sw = self.weights
        if sw.world == 1 or self.wave_len[w] == 0:
            return None
        out, inp = self._wave_buffers(w)
        if dist.get_backend(sw.group) == "gloo":
            # gloo (CPU tests of the host flow) has no reduce-scatter: all-reduce, keep this rank's part
            dist.all_reduce(inp, group=sw.group)
            n = self.wave_len[w]
            out.copy_(inp[sw.rank * n:(sw.rank + 1) * n])
            if average:
                out.div_(sw.world)
            return None
        op = dist.ReduceOp.AVG if average else dist.ReduceOp.SUM
        return dist.reduce_scatter_tensor(out, inp, op=op, group=sw.group, async_op=async_op)

    def reduce_scatter(self, average: bool = True, async_op: bool = False):
        """All waves, in order; with one wave (the default) this is a single collective."""
        last = None
        for w in range(self.waves):
            last = self.reduce_scatter_wave(w, average=average, async_op=async_op)
        return last

    def reduce_scatter_waves(self, average: bool = True):
        """Issue every wave's collective asynchronously; ``handles[w].wait()`` orders the current stream after
        wave w (``None`` for an empty wave or a single rank)."""
        return [self.reduce_scatter_wave(w, average=average, async_op=True) for w in range(self.waves)]


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
