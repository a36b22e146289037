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


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _grads_worker(rank, world, port, shapes):
    from kaon_b200.zero1 import ShardedGrads
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sw = ShardedWeights(shapes, world, rank, torch.float32, torch.device("cpu"))
        sg = ShardedGrads(sw, shapes)
        for i, v in enumerate(sg.views):           # "backward": rank r contributes (r+1) * (i+1)
            v.fill_(float((rank + 1) * (i + 1)))
        sg.reduce_scatter(average=True)
        mean_factor = sum(r + 1 for r in range(world)) / world
        owned = sw.part.owned(rank)
        assert len(sg.owned) == len(owned)
        for g, i in zip(sg.owned, owned):
            assert g.shape == torch.Size(shapes[i])
            assert torch.all(g == mean_factor * (i + 1)), (rank, i)
        ptrs = [g.data_ptr() for g in sg.owned]
        sg.reduce_scatter(average=False)           # the output buffer is reused: pointers stay put
        assert ptrs == [g.data_ptr() for g in sg.owned]
    finally:
        dist.destroy_process_group()


def test_reduce_scatter_feeds_owned_gradients_gloo_world2():
    shapes = [(7, 5), (300,), (64, 64), (3,), (128, 2), (33, 9)]
    mp.spawn(_grads_worker, args=(2, _free_port(), shapes), nprocs=2, join=True)


def _waves_worker(rank, world, port, shapes, waves):
    from kaon_b200.zero1 import ShardedGrads
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sw = ShardedWeights(shapes, world, rank, torch.float32, torch.device("cpu"))
        sg = ShardedGrads(sw, shapes, waves=waves)
        assert sg.waves == waves and len(sg.wave_of) == len(shapes) and set(sg.wave_of) <= set(range(waves))
        # every rank's owned tensors are cut into consecutive waves
        for r in range(world):
            ws = [sg.wave_of[i] for i in sw.part.owned(r)]
            assert ws == sorted(ws), (r, ws)
        # no two gradient views overlap
        spans = sorted((v.data_ptr(), v.data_ptr() + v.numel() * 4) for v in sg.views)
        assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
        for i, v in enumerate(sg.views):
            v.fill_(float((rank + 1) * (i + 1)))
        mean_factor = sum(r + 1 for r in range(world)) / world
        owned = sw.part.owned(rank)
        done = set()
        for w in range(waves):                     # wave by wave: only that wave's tensors are reduced
            sg.reduce_scatter_wave(w, average=True)
            done.add(w)
            for g, i in zip(sg.owned, owned):
                if sg.wave_of[i] in done:
                    assert torch.all(g == mean_factor * (i + 1)), (rank, w, i)
                else:
                    assert torch.all(g == 0.0), (rank, w, i)
    finally:
        dist.destroy_process_group()


def test_reduce_scatter_in_waves_gloo_world2():
    shapes = [(7, 5), (300,), (64, 64), (3,), (128, 2), (33, 9), (40, 40), (17,), (256, 8), (5, 5, 3, 3)]
    mp.spawn(_waves_worker, args=(2, _free_port(), shapes, 3), nprocs=2, join=True)


def _fake_state(i, shape):
    """What a quantised-momentum optimizer keeps for tensor i (values recognisable by i)."""
    n = math.prod(shape)
    return {"m": torch.full(((n + 1) // 2,), i % 251, dtype=torch.uint8),
            "m_scale": torch.full(((n + 127) // 128,), float(i + 1)), "m_numel": n, "m_block": min(128, n)}


def _ckpt_worker(rank, world, port, shapes, out):
    import kaon_b200
    from kaon_b200.zero1 import gather_state_dict, scatter_state_dict
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        part = partition(shapes, world)
        # two param groups: >=2-D tensors, 1-D tensors; global id = position in the flattened group order
        order = [i for i, s in enumerate(shapes) if len(s) >= 2] + [i for i, s in enumerate(shapes) if len(s) < 2]
        gid_of = {i: k for k, i in enumerate(order)}
        def build():
            groups = [[], []]
            for i in order:
                if part.owner[i] != rank:
                    continue
                p = torch.nn.Parameter(torch.zeros(shapes[i]))
                p.kaon_tensor_id = gid_of[i]
                groups[0 if len(shapes[i]) >= 2 else 1].append(p)
            return kaon_b200.Lion([{"params": groups[0], "lr": 3e-4}, {"params": groups[1], "weight_decay": 0.5}],
                                  momentum_dtype="4bit")
        opt = build()
        for g in opt.param_groups:
            for p in g["params"]:
                i = order[p.kaon_tensor_id]
                opt.state[p].update(_fake_state(i, shapes[i]))
        opt._t, opt.sr_seed = 7, 123
        full = gather_state_dict(opt, dst=0)
        if rank == 0:
            assert sorted(full["state"]) == list(range(len(shapes)))
            for gid, st in full["state"].items():
                want = _fake_state(order[gid], shapes[order[gid]])
                assert st.keys() == want.keys()
                assert torch.equal(st["m"], want["m"]) and torch.equal(st["m_scale"], want["m_scale"])
            n2d = sum(1 for s in shapes if len(s) >= 2)
            assert full["param_groups"][0]["params"] == list(range(n2d))
            assert full["param_groups"][1]["params"] == list(range(n2d, len(shapes)))
            assert full["param_groups"][0]["lr"] == 3e-4 and full["param_groups"][1]["weight_decay"] == 0.5
            assert full["_kaon_b200"] == {"step": 7, "sr_seed": 123}
            torch.save(full, out)
        dist.barrier()
        full = torch.load(out)
        fresh = build()
        scatter_state_dict(fresh, full)
        assert fresh._t == 7 and fresh.sr_seed == 123
        for g in fresh.param_groups:
            for p in g["params"]:
                i = order[p.kaon_tensor_id]
                want = _fake_state(i, shapes[i])
                st = fresh.state[p]
                assert torch.equal(st["m"], want["m"]) and torch.equal(st["m_scale"], want["m_scale"]), (rank, i)
                assert st["m_numel"] == want["m_numel"]
        assert fresh.param_groups[0]["lr"] == 3e-4
    finally:
        dist.destroy_process_group()


def test_sharded_checkpoint_gathers_to_the_single_process_layout_gloo_world2(tmp_path):
    shapes = [(7, 5), (300,), (64, 64), (3,), (128, 2), (33, 9), (40,)]
    mp.spawn(_ckpt_worker, args=(2, _free_port(), shapes, str(tmp_path / "full.pt")), nprocs=2, join=True)
