#!/usr/bin/env python
"""Benchmark of the fused optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one optimizer step over the whole synthetic parameter list (weights N(0,0.02), grads
N(0,1e-3), bf16).  Default workload: Lion, 4-bit momentum, betas (0.95,0.98), lr 2e-4, cautious, on the
2.6 B-parameter UNet-shaped list.  With N > 1 the list is sharded ZeRO-1-style (each rank steps the
tensors it owns, then one all-gather of the updated bf16 weights); total work is fixed (strong scaling).
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "k-optimizers_b200"))

WORKLOADS = {
    # optimizer, constructor kwargs, shape list, algorithmic bytes per parameter, options
    # Lion-4bit (BASELINE config 2): g 2 + p 2+2 + m 0.5+0.5 + scales 2*4/128
    # traffic_bpp: DRAM bytes per parameter of one step from an ncu capture of the *_sample workload
    # (dram__bytes_read.sum + dram__bytes_write.sum over the step's kernels / 40 967 680 parameters)
    "lion4bit_unet2p6b": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True),
                          "unet_2p6b", 7.0625, {"traffic_bpp": 5.95}),
    "lion4bit_sample": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True),
                        "unet_sample", 7.0625, {"traffic_bpp": 5.95}),
    # the same without gradient centralization (no row means: the step is purely elementwise + 4-bit blocks)
    "lion4bit_nogc_unet2p6b": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True,
                                            gradient_centralization=False), "unet_2p6b", 7.0625, {}),
    # Adakaon-int8 (config 3): g 2 + p 2+2 + m 1+1 + row scales, row/col stats, 1-D v; 1 % of grads x100
    "adakaon_int8_unet2p6b": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8"),
                              "unet_2p6b", 8.015, {"outlier": True, "traffic_bpp": 12.0}),
    "adakaon_int8_sample": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8"),
                            "unet_sample", 8.015, {"outlier": True, "traffic_bpp": 12.0}),
    # Nekaon-4bit (config 4): as Lion-4bit + stats; climb and removal ride on the same weight access
    "nekaon4bit_unet2p6b": ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999)), "unet_2p6b", 7.073, {"cosine": (1e-4, 1e-5, 50)}),
    # AdaMuon-int8 (config 5): 11.3 B-parameter DiT list; the non-NS passes move 8.006 B/param, the
    # Newton-Schulz GEMMs are 3.24e14 flop per step
    "adamuon_int8_dit11b": ("AdaMuon", dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8"),
                            "dit_11b", 8.006, {"one_grad_set": True}),
    "adamuon_int8_ditblock": ("AdaMuon", dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8"),
                              "dit_block", 8.006, {}),
    "nekaon4bit_sample": ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999)), "unet_sample", 7.073, {"cosine": (1e-4, 1e-5, 50)}),
}
KERNEL_NAME = {"AdaMuon": "ns_gemm_kernel", "Lion": "lion_kernel<bf16,4bit>", "Adakaon": "adakaon_kernel<bf16,int8>", "Nekaon": "adakaon_kernel<bf16,4bit>"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(workload: str, steps: int = 2):
    """The CPU oracle (OpenMP C port of the reference's step) on a bounded sample of the workload."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np
    import kaon_oracle as ko
    from kaon_b200 import workloads as W
    opt_name, kw, _, _, _ = WORKLOADS[workload]
    shapes = W.unet_sample()
    n = W.numel(shapes)
    rng = np.random.default_rng(0)
    ps = [ko.f32_to_bf16_bits(rng.standard_normal(int(np.prod(s)), dtype=np.float32) * 0.02) for s in shapes]
    gs = [ko.f32_to_bf16_bits(rng.standard_normal(int(np.prod(s)), dtype=np.float32) * 1e-3) for s in shapes]
    cls = {"Lion": ko.OracleLion, "Adakaon": ko.OracleAdakaon, "Nekaon": ko.OracleNekaon, "AdaMuon": ko.OracleAdaMuon}[opt_name]
    opt = cls(ps, shapes, **kw)
    opt.step(gs)  # warm-up: allocates state
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        opt.step(gs)
        times.append(time.perf_counter() - t0)
    times.sort()
    dt = times[len(times) // 2]
    cores = int(os.environ.get("OMP_NUM_THREADS", os.cpu_count() or 1))
    return {"value": n / dt, "unit": "params/s", "cores": cores, "kind": "port",
            "sample": f"{opt_name} on one width-1280 UNet block + one [1280,1280,3,3] conv "
                      f"({n} params), median of {steps} steps after 1 warm-up, {dt * 1e3:.0f} ms/step"}, dt, n


def run_reference(args):
    """--impl reference: the reference's CPU path for this workload, as the OpenMP C port in oracle/
    (the reference is Python and does not travel to the GPU box), all host threads, bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, dt, n = cpu_baseline(args.workload, steps=max(1, args.steps))
    line = {"impl": "reference", "metric": "optimizer_step_params_per_sec", "value": base["value"],
            "unit": "params/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": max(1, args.warmup),
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": args.workload, "sample": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    import kaon_b200
    from kaon_b200 import workloads as W
    from kaon_b200.zero1 import ShardedWeights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run); WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    opt_name, kw, shape_key, bytes_per_param, wopt = WORKLOADS[args.workload]
    shapes = W.WORKLOADS[shape_key]()
    total = W.numel(shapes)
    fused_publish = world > 1 and args.publish == "fused"
    sw = ShardedWeights(shapes, world, rank, torch.bfloat16, dev, symmetric=fused_publish)
    owned = sw.part.owned(rank)
    owned_elems = sum(sw.views[i].numel() for i in owned)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def fill_normal(dst, std, outlier=False, chunk=1 << 28):
        """dst (bf16, flat) <- N(0, std), generated in fp32 chunks so that no 4x-sized temporary exists"""
        for a in range(0, dst.numel(), chunk):
            b = min(dst.numel(), a + chunk)
            t = torch.randn(b - a, generator=gen, device=dev) * std
            if outlier:
                t = torch.where(torch.rand(b - a, generator=gen, device=dev) < 0.01, t * 100.0, t)
            dst[a:b].copy_(t)

    fill_normal(sw.shard, 0.02)
    sw.all_gather()
    # two gradient sets, alternated per step (a real loop reallocates grads: set_to_none=True)
    gsets = []
    for k in range(1 if wopt.get("one_grad_set") else 2):
        flat_g = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, device=dev)
        fill_normal(flat_g, 1e-3, outlier=bool(wopt.get("outlier")))
        gsets.append((flat_g, [flat_g[sw.part.offset[i]:sw.part.offset[i] + sw.views[i].numel()].view(shapes[i]) for i in owned]))
    params = []
    for i in owned:
        p = torch.nn.Parameter(sw.views[i], requires_grad=True)
        p.kaon_tensor_id = i  # global list position keys the SR stream: same weights for any N
        params.append(p)
    opt = getattr(kaon_b200, opt_name)(params, **kw)
    opt.sr_seed = 0
    sw.attach(opt)  # fused publish: the step kernels store the weights into every rank's copy
    sg = None
    if args.reduce_scatter and world > 1:
        from kaon_b200.zero1 import ShardedGrads
        sg = ShardedGrads(sw, shapes)              # full-list local gradients + the owner's reduced shard
        fill_normal(sg.flat, 1e-3, outlier=bool(wopt.get("outlier")))

    cos = wopt.get("cosine")

    def one_step(k, ev=None):
        gv = sg.owned if sg is not None else gsets[k % len(gsets)][1]
        if cos:
            for grp in opt.param_groups:
                grp["lr"] = cos[1] + 0.5 * (cos[0] - cos[1]) * (1.0 + math.cos(math.pi * (k % cos[2]) / cos[2]))
        for p, g in zip(params, gv):
            p.grad = g
        if sg is not None:
            sg.reduce_scatter(average=True)
        if ev:
            ev[0].record()
        opt.step()
        if ev:
            ev[1].record()
        sw.publish()
        if ev:
            ev[2].record()

    def fence():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for k in range(max(3, args.warmup)):
        one_step(k)
    fence()
    opt.check_device_status()
    launches0 = opt.stats()["kernel_launches"]
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fence()
    t_begin.record()
    for k in range(args.steps):
        one_step(k, evs[k])
    t_end.record()
    fence()
    clocks = sampler.stop() if rank == 0 else None
    opt.check_device_status()
    launches = opt.stats()["kernel_launches"] - launches0
    ms_total = t_begin.elapsed_time(t_end)
    kern_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    gather_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
    stats = torch.tensor([ms_total, kern_ms, gather_ms, float(launches)], device=dev, dtype=torch.float64)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_total, kern_ms, gather_ms = mx[0].item(), mx[1].item(), mx[2].item()
        launches = int(sm[3].item())
    ms_per_step = ms_total / args.steps

    # ---- end to end: pinned host grads in, step, (all-gather,) owned weights out, every step ----
    e2e = None
    if not args.no_e2e:
        host_g = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, pin_memory=True)
        host_w = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, pin_memory=True)
        host_g.copy_(gsets[0][0])
        torch.cuda.synchronize()
        esteps = max(1, min(args.steps, args.e2e_steps))

        # Three streams, as a training loop with a host-side gradient source would run it: the copy of
        # step k+1's gradients to the device (s_in) and the read-back of step k's weights (s_out) travel in
        # opposite directions over PCIe and overlap; the step itself waits for its gradients and for the
        # previous read-back (which reads the weights the step is about to overwrite).
        cur_s = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        nset = len(gsets)
        ev_in = [torch.cuda.Event() for _ in range(nset)]
        ev_step = [torch.cuda.Event() for _ in range(nset)]
        ev_out = torch.cuda.Event()

        def h2d(k):
            b_ = k % nset
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_step[b_])      # the step that last read this gradient buffer has finished
                gsets[b_][0].copy_(host_g, non_blocking=True)
                ev_in[b_].record(s_in)

        def e2e_run(nsteps):
            h2d(0)
            for k in range(nsteps):
                b_ = k % nset
                if k + 1 < nsteps and nset > 1:
                    h2d(k + 1)
                cur_s.wait_event(ev_in[b_])
                cur_s.wait_event(ev_out)
                for p, g in zip(params, gsets[b_][1]):
                    p.grad = g
                opt.step()
                sw.publish()
                ev_step[b_].record(cur_s)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_step[b_])
                    host_w.copy_(sw.shard, non_blocking=True)
                    ev_out.record(s_out)
                if k + 1 < nsteps and nset == 1:
                    h2d(k + 1)
            cur_s.wait_event(ev_out)

        e2e_run(1)
        fence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        e2e_run(esteps)
        b.record()
        fence()
        ems = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(ems, op=dist.ReduceOp.MAX)
        ems = ems.item() / esteps
        nbytes = sw.part.shard_len * 2 * world
        e2e = {"value": total / (ems * 1e-3), "unit": "params/s", "ms_per_step": ems, "steps": esteps,
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "pipeline": "gradients of step k+1 go up while the weights of step k come down (3 streams); "
                           "the first upload and the last download are inside the timed region"}

    ns_info = None
    if opt_name == "AdaMuon":
        # Newton-Schulz alone, per distinct matrix shape of this rank's tensors: CUDA events around the
        # GEMM chain (2 + 3*steps launches) of kaon_newton_schulz
        from kaon_b200.adamuon import zeropower_via_newtonschulz5 as ns
        steps_ns = kw.get("ns_steps", 2)
        shapes2d = sorted({(s[0], W.numel([s]) // s[0]) for i, s in enumerate(shapes) if len(s) >= 2 and i in set(owned)})
        counts = {sh: sum(1 for i in owned if len(shapes[i]) >= 2 and (shapes[i][0], W.numel([shapes[i]]) // shapes[i][0]) == sh) for sh in shapes2d}
        ns_info, tot_flop, tot_ms = {}, 0.0, 0.0
        for (R, Cc) in shapes2d:
            x = torch.randn(R, Cc, device=dev, dtype=torch.bfloat16)
            ns(x, steps_ns)
            a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            a_.record()
            for _ in range(3):
                ns(x, steps_ns)
            b_.record()
            torch.cuda.synchronize()
            ms = a_.elapsed_time(b_) / 3
            r_, k_ = min(R, Cc), max(R, Cc)
            flop = steps_ns * (4.0 * r_ * r_ * k_ + 2.0 * r_ ** 3)
            ns_info[f"{R}x{Cc}"] = {"ms": ms, "tflops": flop / (ms * 1e-3) / 1e12, "count": counts[(R, Cc)]}
            tot_flop += flop * counts[(R, Cc)]
            tot_ms += ms * counts[(R, Cc)]
        ns_info["total"] = {"flop_per_step": tot_flop, "ms_per_step": tot_ms, "tflops": tot_flop / (tot_ms * 1e-3) / 1e12}

    if rank == 0:
        peak, peak_kind = measured_peaks()
        # the dominant (only) kernel of a step: algorithmic bytes of this rank's tensors per launch
        alg_bytes = bytes_per_param * (total / world)
        achieved = alg_bytes / (kern_ms * 1e-3) / 1e9
        line = {
            "metric": "optimizer_step_params_per_sec", "value": total / (ms_per_step * 1e-3), "unit": "params/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": args.workload, "optimizer": opt_name, "params": total, "tensors": len(shapes),
                       "param_dtype": "bf16", "momentum_dtype": kw.get("momentum_dtype"),
                       "sharding": "zero1" if world > 1 else "none",
                       "publish": ("none" if world == 1 else
                                   "peer stores fused into the step kernel + barrier" if fused_publish else
                                   "nccl all_gather_into_tensor after the step"),
                       "l2": "inputs (18 GB per step) larger than L2; no flush needed"},
            "step_kernel_ms": kern_ms, "publish_ms": gather_ms,
            "gradient_reduce_scatter": "inside every step" if sg is not None else "not part of the step",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "peak_kind": f"{peak_kind} copy bandwidth",
                         "traffic": (wopt["traffic_bpp"] * total / world) if "traffic_bpp" in wopt else None,
                         "traffic_source": ("ncu capture of the 41 M-parameter sample of this workload, scaled by "
                                            "parameters (a lower bound: part of the sample stays in L2 between launches)"
                                            if "traffic_bpp" in wopt else None),
                         "bytes_per_param": bytes_per_param, "kernel": KERNEL_NAME[opt_name]},
            "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
        if fused_publish:
            # the step kernel also pushes this rank's updated weights to the other ranks: its floor is
            # the slower of the HBM pass and the NVLink egress (measured peer-copy bandwidth 770 GB/s)
            out_bytes = 2.0 * (total / world) * (world - 1)
            t_hbm, t_link = alg_bytes / (peak * 1e9), out_bytes / 770e9
            line["nvlink"] = {"egress_bytes_per_rank": out_bytes, "achieved": out_bytes / (kern_ms * 1e-3) / 1e9,
                              "peak": 770.0, "unit": "GB/s", "floor_ms": max(t_hbm, t_link) * 1e3,
                              "frac_of_floor": max(t_hbm, t_link) * 1e3 / kern_ms}
        if ns_info is not None:
            tpeak = 1678.7
            try:
                with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as fh:
                    tpeak = float(json.load(fh)["bf16_tflops"])
            except (OSError, KeyError, ValueError):
                pass
            line["hbm_passes"] = line["roofline"]
            line["roofline"] = {"bound": "tensor", "achieved": ns_info["total"]["tflops"], "peak": tpeak,
                                "unit": "TFLOP/s", "frac": ns_info["total"]["tflops"] / tpeak, "traffic": None,
                                "peak_kind": "measured cuBLAS bf16 burst", "kernel": "ns_gemm_kernel",
                                "note": "Newton-Schulz GEMM chain timed alone per shape (CUDA events); hbm_passes has the whole-step algorithmic-bytes view"}
            line["newton_schulz"] = ns_info
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"], _, _ = cpu_baseline(args.workload)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="lion4bit_unet2p6b", choices=sorted(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=6)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--reduce-scatter", action="store_true",
                    help="N>1: put the gradient reduce-scatter (NCCL, bf16 average) inside every step; the step "
                         "kernels then read the collective's output buffer")
    ap.add_argument("--publish", default="fused", choices=["fused", "allgather"],
                    help="N>1: how the owned weights reach the other ranks")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
