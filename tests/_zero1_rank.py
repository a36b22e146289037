"""One rank of the sharded-step test: gradients reduce-scattered into the owner's shard, ZeRO-1 step over
symmetric memory with the publish fused into the step kernels, optimizer state gathered into the
single-process checkpoint layout.  Saves every tensor's final weights as this rank sees them, and (rank 0)
the gathered state_dict."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "k-optimizers_b200"))
import kaon_b200  # noqa: E402
from kaon_b200.zero1 import ShardedGrads, ShardedWeights, gather_state_dict  # noqa: E402

SHAPES = [(640, 256), (64, 32, 3, 3), (1280,), (512, 640), (333, 77), (3, 4096), (4000, 1), (7,), (256, 1024)]


# rows that are multiples of 16 elements: the streaming stages and the separate COUNT / APPLY launches
SHAPES_STREAM = [(640, 256), (64, 32, 4, 4), (1280,), (512, 640), (336, 80), (3, 4096), (4000, 16), (7,), (256, 1024)]


def main():
    global SHAPES
    opt_name, out = sys.argv[1], sys.argv[2]
    waves = 1
    if opt_name.endswith("-stream"):
        opt_name, SHAPES = opt_name[:-len("-stream")], SHAPES_STREAM
    if opt_name.endswith("-waves"):   # the gradient reduce-scatter in three waves, one parameter group per wave
        opt_name, waves = opt_name[:-len("-waves")], 3
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    sw = ShardedWeights(SHAPES, world, rank, torch.bfloat16, dev, symmetric=True)
    gen = torch.Generator().manual_seed(5)
    for v, s in zip(sw.views, SHAPES):  # every rank starts from the same full weights
        v.copy_((torch.randn(s, generator=gen) * 0.02).bfloat16())
    owned = sw.part.owned(rank)
    params = []
    for i in owned:
        p = torch.nn.Parameter(sw.views[i])
        p.kaon_tensor_id = i
        params.append(p)
    kw = dict(lr=2e-4, momentum_dtype="4bit") if opt_name == "Lion" else dict(lr=1e-4, momentum_dtype="int8")
    if opt_name == "KProdigy":   # the one optimizer with a scalar over all tensors: its sums are all-reduced
        kw = dict(momentum_dtype="4bit", second_moment="factored", growth_rate=3.0)
    sg = ShardedGrads(sw, SHAPES, waves=waves)
    by_wave = {}
    for p, i in zip(params, owned):
        by_wave.setdefault(sg.wave_of[i], []).append(p)
    group_wave = sorted(by_wave)
    opt = getattr(kaon_b200, opt_name)([{"params": by_wave[w]} for w in group_wave] if waves > 1 else params, **kw)
    if opt_name == "KProdigy" and world > 1:
        opt.set_shard_group(True)
    opt.sr_seed = 3
    sw.attach(opt)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    for p, g in zip(params, sg.owned):
        p.grad = g                                   # the reduce-scatter's output buffer, for good
    base = [torch.randn(s, generator=gen) * 1e-3 for s in SHAPES]   # a steady direction: KProdigy's d has something to find
    for step in range(8 if opt_name == "KProdigy" else 4):
        grads = [((b if opt_name == "KProdigy" else 0.0) + torch.randn(s, generator=gen) * (3e-4 if opt_name == "KProdigy" else 1e-3)).bfloat16()
                 for b, s in zip(base, SHAPES)]
        for v, g in zip(sg.views, grads):            # "backward": every rank holds the same local gradient,
            v.copy_(g)                               # so the average is exact in bf16
        if waves > 1:
            works = sg.reduce_scatter_waves(average=True)
            opt.before_group = lambda gi, works=works: works[group_wave[gi]].wait() if works[group_wave[gi]] is not None else None
        else:
            sg.reduce_scatter(average=True)
        opt.step()
        sw.publish()
    torch.cuda.synchronize()
    opt.check_device_status()
    torch.save([v.detach().cpu() for v in sw.views], f"{out}.w{world}.r{rank}.pt")
    full = gather_state_dict(opt, dst=0)
    if rank == 0:
        torch.save(full, f"{out}.w{world}.state.pt")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
