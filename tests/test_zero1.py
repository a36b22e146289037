"""ZeRO-1 partitioner and the flat-buffer weight exchange, on CPU with gloo (world_size 2)."""
import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kaon_b200 import workloads as W
from kaon_b200.zero1 import ALIGN, ShardedWeights, partition


def test_partition_is_balanced_aligned_and_complete():
    shapes = W.unet_2p6b()
    for world in (1, 2, 4, 8):
        part = partition(shapes, world)
        assert sorted(sum((part.owned(r) for r in range(world)), [])) == list(range(len(shapes)))
        assert sum(part.load) == W.numel(shapes)
        assert max(part.load) - min(part.load) <= max(math.prod(s) for s in shapes)
        assert max(part.load) / (W.numel(shapes) / world) < 1.01
        assert part.shard_len % ALIGN == 0
        for r in range(world):
            end = 0
            for i in part.owned(r):
                assert part.offset[i] % ALIGN == 0 and part.offset[i] >= end
                end = part.offset[i] + math.prod(shapes[i])
            assert end <= part.shard_len


def test_partition_is_deterministic_and_keeps_list_order_inside_a_shard():
    shapes = [(7, 5), (300,), (64, 64), (3,), (128, 2)]
    a, b = partition(shapes, 2), partition(shapes, 2)
    assert a == b
    for r in range(2):
        offs = [a.offset[i] for i in a.owned(r)]
        assert offs == sorted(offs)


def _worker(rank, world, port, shapes):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sw = ShardedWeights(shapes, world, rank, torch.float32, torch.device("cpu"))
        # each rank writes a recognisable value into the tensors it owns ("the step")
        for i in sw.part.owned(rank):
            sw.views[i].fill_(float(i + 1))
        sw.all_gather()
        for i, s in enumerate(shapes):
            assert torch.all(sw.views[i] == float(i + 1)), (rank, i)
            assert sw.views[i].shape == torch.Size(s)
        # second exchange after another "step" on the owner only
        for i in sw.part.owned(rank):
            sw.views[i].mul_(2.0)
        sw.all_gather()
        for i in range(len(shapes)):
            assert torch.all(sw.views[i] == 2.0 * (i + 1)), (rank, i)
    finally:
        dist.destroy_process_group()


def test_all_gather_publishes_owned_tensors_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    shapes = [(7, 5), (300,), (64, 64), (3,), (128, 2), (33, 9)]
    mp.spawn(_worker, args=(2, port, shapes), nprocs=2, join=True)
