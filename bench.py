#!/usr/bin/env python
"""Benchmark of the fused optimizer step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A "step" is one optimizer step over the whole synthetic parameter list (weights N(0,0.02), grads
N(0,1e-3), bf16).  With no --workload the run measures the headline (Lion, 4-bit momentum, betas
(0.95,0.98), lr 2e-4, cautious, on the 2.6 B-parameter UNet-shaped list) with K timed steps, and then
the other benchmark configurations - Adakaon-int8 (K steps), Nekaon-4bit (50 steps, cosine LR) and
AdaMuon-int8 on the 11.3 B-parameter DiT list (10 steps) - whose figures go under "workloads" in the
same JSON line.  With N > 1 every list is sharded ZeRO-1-style (each rank steps the tensors it owns and
publishes the updated bf16 weights to the others); total work is fixed (strong scaling).  Each workload
is timed twice at N > 1: without any publish ("compute_only_ms") and with it ("incl_publish_ms").
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import gc
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "k-optimizers_b200"))
REF_DIR = os.path.join(ROOT, "baseline", "_ref")   # the unmodified reference package (git-ignored)

LION_KW = dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True)
ADAKAON_KW = dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8")
NEKAON_KW = dict(lr=1e-4, betas=(0.2, 0.999))
ADAMUON_KW = dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8")
# optimizer, constructor kwargs, shape list, algorithmic bytes per parameter, options.
#  Lion-4bit (BASELINE config 2): g 2 + p 2+2 + m 0.5+0.5 + scales 2*4/128 = 7.0625
#  Adakaon-int8 (config 3): g 2 + p 2+2 + m 1+1 + row scales, row/col stats, 1-D v; 1 % of grads x100
#  Nekaon-4bit (config 4): as Lion-4bit + stats; climb and removal ride on the same weight access
#  AdaMuon-int8 (config 5): the non-NS passes move 8.006 B/param; Newton-Schulz is 3.24e14 flop per step
# traffic_bpp: DRAM bytes per parameter of one step (all its launches), from the ncu launch list of the
# *_mid workload (a list of 269 M parameters with every tensor shape of the big one, 15x L2) summarised in
# profiles/lion_kernel_bf16_4bit_unet_mid.md and profiles/adakaon_kernels_bf16_unet_mid.md.
WORKLOADS = {
    "lion4bit_unet2p6b": ("Lion", LION_KW, "unet_2p6b", 7.0625, {"traffic_bpp": 7.22}),
    "lion4bit_sample": ("Lion", LION_KW, "unet_sample", 7.0625, {}),
    "lion4bit_mid": ("Lion", LION_KW, "unet_mid", 7.0625, {}),
    "lion4bit_nogc_unet2p6b": ("Lion", dict(LION_KW, gradient_centralization=False), "unet_2p6b", 7.0625, {}),
    "adakaon_int8_unet2p6b": ("Adakaon", ADAKAON_KW, "unet_2p6b", 8.015, {"outlier": True, "traffic_bpp": 13.78}),
    "adakaon_int8_sample": ("Adakaon", ADAKAON_KW, "unet_sample", 8.015, {"outlier": True}),
    "adakaon_int8_mid": ("Adakaon", ADAKAON_KW, "unet_mid", 8.015, {"outlier": True}),
    "adakaon_int8_mid_odd": ("Adakaon", ADAKAON_KW, "unet_mid_odd", 8.015, {"outlier": True}),
    "nekaon4bit_unet2p6b": ("Nekaon", NEKAON_KW, "unet_2p6b", 7.073, {"cosine": (1e-4, 1e-5, 50), "steps": 50,
                                                                       "traffic_bpp": 14.38}),
    "nekaon4bit_sample": ("Nekaon", NEKAON_KW, "unet_sample", 7.073, {"cosine": (1e-4, 1e-5, 50)}),
    "nekaon4bit_mid": ("Nekaon", NEKAON_KW, "unet_mid", 7.073, {"cosine": (1e-4, 1e-5, 50)}),
    "adamuon_int8_dit11b": ("AdaMuon", ADAMUON_KW, "dit_11b", 8.006, {"one_grad_set": True, "steps": 10}),
    "adamuon_int8_ditblock": ("AdaMuon", ADAMUON_KW, "dit_block", 8.006, {}),
    # the two optimizers beyond the benchmark configurations (not tuned; sized for a quick figure)
    #  AdaPNM-4bit: g 2 + p 2+2 + m_pos 0.5+0.5 + m_neg 0.5 + scales;  KProdigy defaults: g 2 + p 2+2 + bf16 m 2+2
    #  + fp32 v 4+4 + fp32 s 4+4 + p0 4 (slice_p = 1)
    "adapnm_4bit_mid": ("AdaPNM", dict(lr=1e-4, momentum_dtype="4bit"), "unet_mid", 7.6, {}),
    "kprodigy_default_mid": ("KProdigy", dict(), "unet_mid", 30.0, {}),
}
E2E_GROUPS = 16   # parameter groups of the end-to-end pipeline
HEADLINE = "lion4bit_unet2p6b"
RECORD = ["adakaon_int8_unet2p6b", "nekaon4bit_unet2p6b", "adamuon_int8_dit11b"]
KERNEL_NAME = {"AdaMuon": "ns_gemm_kernel", "Lion": "lion_kernel<bf16,4bit>", "Adakaon": "adakaon_kernel<bf16,int8>",
               "Nekaon": "adakaon_kernel<bf16,4bit>", "AdaPNM": "pnm_pass_kernel<bf16,4bit>",
               "KProdigy": "kp_sweep_kernel<bf16,bf16>"}


def host_cores() -> int:
    """Cores this process may run on (torch.distributed.run exports OMP_NUM_THREADS=1, which says
    nothing about the host)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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
        return self

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


# ------------------------------------------------------------------------------------- CPU arms

def _sample_desc(opt_name, n):
    return f"{opt_name} on one width-1280 UNet block + one [1280,1280,3,3] conv ({n} params)"


def cpu_port(workload: str, steps: int = 2):
    """The CPU oracle (OpenMP C restatement of the reference's step) on a bounded sample of the workload."""
    cores = host_cores()
    os.environ["OMP_NUM_THREADS"] = str(cores)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import ctypes
    import numpy as np
    import kaon_oracle as ko
    from kaon_b200 import workloads as W
    ko.lib()
    try:  # the variable is only read when the OpenMP runtime starts; another library may have started it
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(cores)
    except OSError:
        pass
    opt_name, kw, shape_key, _, _ = WORKLOADS[workload]
    shapes = W.dit_block() if shape_key.startswith("dit") else W.unet_sample()
    n = W.numel(shapes)
    rng = np.random.default_rng(0)
    ps = [ko.f32_to_bf16_bits(rng.standard_normal(int(np.prod(s)), dtype=np.float32) * 0.02) for s in shapes]
    gs = [ko.f32_to_bf16_bits(rng.standard_normal(int(np.prod(s)), dtype=np.float32) * 1e-3) for s in shapes]
    cls = {"Lion": ko.OracleLion, "Adakaon": ko.OracleAdakaon, "Nekaon": ko.OracleNekaon, "AdaMuon": ko.OracleAdaMuon}[opt_name]
    opt = cls(ps, shapes, **kw)
    if opt_name == "AdaMuon":
        # the O(n^3) CPU Newton-Schulz of 3072-wide matrices is out of reach of a bounded sample: time the
        # chain around it with the orthogonalised matrices supplied
        ov = [None if len(s) < 2 else np.zeros(int(np.prod(s)), np.float32) + 0.01 for s in shapes]
        step = lambda: opt.step(gs, ns_override=ov)  # noqa: E731
    else:
        step = lambda: opt.step(gs)  # noqa: E731
    step()  # warm-up: allocates state
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    times.sort()
    dt = times[len(times) // 2]
    sample = (f"{opt_name} chain without Newton-Schulz on one width-3072 DiT block ({n} params)"
              if opt_name == "AdaMuon" else _sample_desc(opt_name, n))
    return {"value": n / dt, "unit": "params/s", "cores": cores, "kind": "port",
            "sample": f"{sample}, median of {steps} steps after 1 warm-up, {dt * 1e3:.0f} ms/step"}, dt, n


def cpu_reference(workload: str, steps: int = 3, warmup: int = 1):
    """The reference package itself (its foreach path, CPU tensors, all host threads) on the same bounded
    sample.  Returns None when the package is not installed beside the benchmark."""
    if not os.path.isdir(os.path.join(REF_DIR, "kaon")):
        return None
    sys.path.insert(0, REF_DIR)
    import torch
    import kaon  # the reference
    from kaon_b200 import workloads as W
    cores = host_cores()
    torch.set_num_threads(cores)
    opt_name, kw, shape_key, _, wopt = WORKLOADS[workload]
    if opt_name == "AdaMuon":
        return None  # a CPU Newton-Schulz of 3072-wide matrices does not fit a bounded sample
    shapes = W.unet_sample()
    n = W.numel(shapes)
    gen = torch.Generator().manual_seed(0)
    params = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).bfloat16()) for s in shapes]
    grads = [(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes]
    opt = getattr(kaon, opt_name)(params, **kw)
    times = []
    for k in range(warmup + steps):
        for p, g in zip(params, grads):
            p.grad = g.clone()  # gradient centralization rewrites p.grad in place
        t0 = time.perf_counter()
        opt.step()
        if k >= warmup:
            times.append(time.perf_counter() - t0)
    times.sort()
    dt = times[len(times) // 2]
    return {"value": n / dt, "unit": "params/s", "cores": cores, "kind": "reference",
            "sample": f"kaon {kaon.__version__} {_sample_desc(opt_name, n)}, foreach=True, CPU tensors, "
                      f"median of {steps} steps after {warmup} warm-up, {dt * 1e3:.0f} ms/step"}, dt, n


def cpu_baseline(workload: str, steps: int = 3):
    """Reference package when present (kind "reference"), with the C port's figure beside it."""
    port, dt_p, n = cpu_port(workload, steps=max(2, steps))
    ref = cpu_reference(workload, steps=steps)
    if ref is None:
        return port, dt_p, n
    base, dt, n = ref
    base["port"] = {k: port[k] for k in ("value", "unit", "cores", "sample")}
    return base, dt, n


def run_reference(args):
    """--impl reference: the reference's CPU path for the workload on the host cores (the reference
    package itself when it sits in baseline/_ref, else the C port in oracle/), bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = args.workload or HEADLINE
    base, dt, n = cpu_baseline(workload, steps=max(1, min(args.steps, 5)))
    line = {"impl": "reference", "metric": "optimizer_step_params_per_sec", "value": base["value"],
            "unit": "params/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": max(1, args.warmup),
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload, "sample": base["sample"]},
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------- GPU bar

def run_gpu_bar(args):
    """The reference's own CUDA paths on this GPU, timed with its own method (median of per-step wall
    times with a synchronize on both sides, reference benchmarks/fused/bench_fused.py:73-89): eager foreach
    (fused=False), optionally its Triton path (fused=True, --gpu-bar-fused), and AdaMuon's cuBLAS
    Newton-Schulz chain (src/kaon/adamuon.py:97-118).  One JSON object on stdout."""
    sys.path.insert(0, REF_DIR)
    import torch
    import kaon
    from kaon.adamuon import zeropower_via_newtonschulz5 as ref_ns
    from kaon_b200 import workloads as W
    dev = torch.device("cuda", 0)
    out = {"method": "median wall ms per step, synchronize on both sides (the reference's bench_fused.step_ms)",
           "list": "unet_mid (8 width-1280 blocks + 4 [1280,1280,3,3] convs, 269 M params)"}
    shapes = W.unet_mid()
    n = W.numel(shapes)
    gen = torch.Generator(device=dev).manual_seed(0)

    def timed(fn, reps, warmup):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(reps):
            torch.cuda.synchronize()
            t0 = time.time()
            fn()
            torch.cuda.synchronize()
            ts.append((time.time() - t0) * 1e3)
        ts.sort()
        return ts[len(ts) // 2]

    cases = [("lion4bit", "Lion", LION_KW, [False]),
             ("adakaon_int8", "Adakaon", ADAKAON_KW, [False] + ([True] if args.gpu_bar_fused else [])),
             ("nekaon4bit", "Nekaon", NEKAON_KW, [False] + ([True] if args.gpu_bar_fused else []))]
    for key, cls, kw, fused_opts in cases:
        for fused in fused_opts:
            tag = f"{key}_{'triton' if fused else 'eager'}"
            try:
                params = [torch.nn.Parameter((torch.randn(s, generator=gen, device=dev) * 0.02).bfloat16()) for s in shapes]
                grads = [(torch.randn(s, generator=gen, device=dev) * 1e-3).bfloat16() for s in shapes]
                opt = getattr(kaon, cls)(params, **kw, **({"fused": True} if fused else {}))

                def one():
                    for p, g in zip(params, grads):
                        p.grad = g  # centralization rewrites it in place: timing only
                    opt.step()
                ms = timed(one, 5, 2)
                out[tag] = {"ms_per_step": ms, "params_per_s": n / (ms * 1e-3)}
                del opt, params, grads
            except Exception as e:  # noqa: BLE001 - a failing reference path is a finding, not a crash
                out[tag] = {"error": f"{type(e).__name__}: {e}"[:300]}
            gc.collect()
            torch.cuda.empty_cache()
    ns = {}
    tot_ms = tot_flop = 0.0
    for (R, Cc, count) in [(9216, 3072, 100), (3072, 3072, 100), (12288, 3072, 100), (3072, 12288, 100)]:
        x = torch.randn(R, Cc, device=dev, dtype=torch.bfloat16)
        ms = timed(lambda: ref_ns(x, 2), 5, 2)
        r_, k_ = min(R, Cc), max(R, Cc)
        flop = 2 * (4.0 * r_ * r_ * k_ + 2.0 * r_ ** 3)
        ns[f"{R}x{Cc}"] = {"ms": ms, "tflops": flop / (ms * 1e-3) / 1e12}
        tot_ms += ms * count
        tot_flop += flop * count
    ns["dit_list_total"] = {"ms_per_step": tot_ms, "tflops": tot_flop / (tot_ms * 1e-3) / 1e12}
    out["newton_schulz_cublas"] = ns
    print(json.dumps(out), flush=True)


def gpu_bar_subprocess(timeout=420):
    if not os.path.isdir(os.path.join(REF_DIR, "kaon")):
        return {"unavailable": "the reference package is not installed in baseline/_ref"}
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--gpu-bar"], capture_output=True, text=True,
                           timeout=timeout, env=env)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
        return json.loads(lines[-1]) if lines else {"error": (r.stderr or "no output")[-300:]}
    except (subprocess.TimeoutExpired, ValueError, OSError) as e:
        return {"error": f"{type(e).__name__}: {e}"[:300]}


# ------------------------------------------------------------------------------------- our arm

class Ctx:
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if args.gpus != self.world:
            raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torch.distributed.run); WORLD_SIZE={self.world}")
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.args = args

    def fence(self):
        import torch
        import torch.distributed as dist
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def reduce(self, vals, op="max"):
        import torch
        import torch.distributed as dist
        t = torch.tensor(vals, device=self.dev, dtype=torch.float64)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.SUM)
        return t.tolist()


def e2e_groups(sizes, offsets, shard_len, ngroups):
    """Cut a rank's tensors (element counts `sizes` at element `offsets` of its shard, in list order) into at
    most `ngroups` runs of consecutive tensors of about equal size.  Returns (the tensor positions of each
    run, the [lo, hi) slice of the shard each run covers); the slices tile [0, shard_len) in order, so that
    per-run copies move every byte of the shard exactly once."""
    n = len(sizes)
    ngroups = max(1, min(ngroups, n))
    total = sum(sizes)
    chunks, acc, nxt = [[]], 0, 1
    for k in range(n):
        if acc >= nxt * total / ngroups and chunks[-1]:
            chunks.append([])
            nxt += 1
        chunks[-1].append(k)
        acc += sizes[k]
    bounds = []
    for ch in chunks:
        lo = min(offsets[k] for k in ch)
        hi = max(offsets[k] + sizes[k] for k in ch)
        if bounds and lo < bounds[-1][1]:
            raise ValueError("the owned tensors are not laid out in list order")
        bounds.append((lo, hi))
    # padding between runs and at either end travels with the run before it (the first run: before it)
    bounds = [(0 if j == 0 else bounds[j][0], bounds[j + 1][0] if j + 1 < len(bounds) else shard_len)
              for j in range(len(bounds))]
    return chunks, bounds


def measure(ctx: Ctx, workload: str, steps: int, warmup: int, e2e_steps: int = 0):
    """One workload at ctx.world GPUs: device-timed steps (max over ranks), clocks, roofline."""
    import torch
    import kaon_b200
    from kaon_b200 import workloads as W
    from kaon_b200.zero1 import ShardedWeights

    args, world, rank, dev = ctx.args, ctx.world, ctx.rank, ctx.dev
    opt_name, kw, shape_key, bytes_per_param, wopt = WORKLOADS[workload]
    shapes = W.WORKLOADS[shape_key]()
    total = W.numel(shapes)
    warmup = max(3, warmup)
    fused_publish = world > 1 and args.publish == "fused"
    sw = ShardedWeights(shapes, world, rank, torch.bfloat16, dev, symmetric=fused_publish)
    owned = sw.part.owned(rank)
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
    for _ in range(1 if wopt.get("one_grad_set") else 2):
        flat_g = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, device=dev)
        fill_normal(flat_g, 1e-3, outlier=bool(wopt.get("outlier")))
        gsets.append((flat_g, [flat_g[sw.part.offset[i]:sw.part.offset[i] + sw.views[i].numel()].view(shapes[i]) for i in owned]))
    params = []
    for i in owned:
        p = torch.nn.Parameter(sw.views[i], requires_grad=True)
        p.kaon_tensor_id = i  # global list position keys the SR stream: same weights for any N
        params.append(p)
    sg = None
    group_wave = None
    if args.reduce_scatter and world > 1:
        from kaon_b200.zero1 import ShardedGrads
        # full-list local gradients + the owner's reduced shard, cut into waves: one collective and one
        # parameter group per wave, so that wave w is stepped while wave w+1 is still being reduced
        sg = ShardedGrads(sw, shapes, waves=args.waves if args.waves > 0 else (4 if world <= 2 else 1))
        fill_normal(sg.flat, 1e-3, outlier=bool(wopt.get("outlier")))
        by_wave = {}
        for p, i in zip(params, owned):
            by_wave.setdefault(sg.wave_of[i], []).append(p)
        group_wave = sorted(by_wave)
        opt = getattr(kaon_b200, opt_name)([{"params": by_wave[w]} for w in group_wave], **kw)
    else:
        opt = getattr(kaon_b200, opt_name)(params, **kw)
    opt.sr_seed = 0
    if sg is not None and sg.waves > 1 and args.comm_sms > 0:
        # the step kernels are persistent: leave the collective's CTAs somewhere to run beside them
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        getattr(opt, "inner", opt).sm_limit = max(1, sms - args.comm_sms)
    cos = wopt.get("cosine")
    state = {"k": 0}

    def one_step(ev=None, publish=True):
        k = state["k"]
        state["k"] += 1
        gv = sg.owned if sg is not None else gsets[k % len(gsets)][1]
        if cos:
            for grp in opt.param_groups:
                grp["lr"] = cos[1] + 0.5 * (cos[0] - cos[1]) * (1.0 + math.cos(math.pi * (k % cos[2]) / cos[2]))
        for p, g in zip(params, gv):
            p.grad = g
        if ev:
            ev[0].record()
        if sg is not None:
            works = sg.reduce_scatter_waves(average=True)      # asynchronous, back to back on NCCL's stream
            stepper = getattr(opt, "inner", opt)

            def wait_for_wave(gi, works=works):
                if works[group_wave[gi]] is not None:
                    works[group_wave[gi]].wait()                # orders this stream after wave gi's collective
            stepper.before_group = wait_for_wave
        opt.step()
        if ev:
            ev[1].record()
        if publish:
            sw.publish()
        if ev:
            ev[2].record()

    def timed(nsteps, publish):
        for _ in range(warmup):
            one_step(publish=publish)
        ctx.fence()
        opt.check_device_status()
        launches0 = opt.stats()["kernel_launches"]
        sampler = ClockSampler(ctx.local_rank).start() if rank == 0 else None
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(nsteps)]
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ctx.fence()
        t0.record()
        for k in range(nsteps):
            one_step(evs[k], publish=publish)
        t1.record()
        ctx.fence()
        clocks = sampler.stop() if sampler else None
        opt.check_device_status()
        launches = opt.stats()["kernel_launches"] - launches0
        kern = sum(e[0].elapsed_time(e[1]) for e in evs) / nsteps
        pub = sum(e[1].elapsed_time(e[2]) for e in evs) / nsteps
        tot_ms, kern, pub = ctx.reduce([t0.elapsed_time(t1), kern, pub])
        (launches,) = ctx.reduce([float(launches)], op="sum")
        return tot_ms / nsteps, kern, pub, int(launches), clocks

    compute_only_ms = None
    if world > 1:
        # the step without any publish (mirrors detached, no collective): the "compute only" curve
        compute_only_ms, _, _, _, _ = timed(min(steps, 10), publish=False)
        sw.attach(opt)  # fused publish: the step kernels store the weights into every rank's copy
    ms_per_step, kern_ms, pub_ms, launches, clocks = timed(steps, publish=True)
    if compute_only_ms is None:
        compute_only_ms = ms_per_step

    # ---- end to end: pinned host grads in, step, (publish,) owned weights out, every step ----
    e2e = None
    if e2e_steps > 0:
        host_g = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, pin_memory=True)
        host_w = torch.empty(sw.part.shard_len, dtype=torch.bfloat16, pin_memory=True)
        host_g.copy_(gsets[0][0])
        torch.cuda.synchronize()
        # Three streams, as a training loop with a host-side gradient source would run it, pipelined by
        # parameter group: the owned tensors are cut into E2E_GROUPS contiguous slices of the shard, one
        # parameter group each; slice j of step k+1's gradients goes up (s_in) while slice j of step k's
        # weights comes down (s_out), in opposite directions over PCIe, and group j is stepped as soon as
        # its gradients have landed and the previous read-back of its weights has finished.
        cur_s = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        nset = len(gsets)
        chunks, bounds = e2e_groups([p.numel() for p in params], [sw.part.offset[i] for i in owned],
                                    sw.part.shard_len, E2E_GROUPS)
        ngrp = len(chunks)
        chunks = [[(params[k], owned[k]) for k in ch] for ch in chunks]
        opt_e = getattr(kaon_b200, opt_name)([{"params": [p for p, _ in ch]} for ch in chunks], **kw)
        opt_e.sr_seed = 0
        if world > 1 and fused_publish:
            sw.attach(opt_e)
        stepper = getattr(opt_e, "inner", opt_e)
        ev_in = [[torch.cuda.Event() for _ in range(ngrp)] for _ in range(nset)]
        ev_step = [torch.cuda.Event() for _ in range(nset)]
        ev_grp = [torch.cuda.Event() for _ in range(ngrp)]
        ev_out = [torch.cuda.Event() for _ in range(ngrp)]
        cur_buf = {"b": 0}

        def h2d(k):
            b_ = k % nset
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_step[b_])      # the step that last read this gradient buffer has finished
                for j, (lo, hi) in enumerate(bounds):
                    gsets[b_][0][lo:hi].copy_(host_g[lo:hi], non_blocking=True)
                    ev_in[b_][j].record(s_in)

        def group_ready(j):
            cur_s.wait_event(ev_in[cur_buf["b"]][j])   # its gradients are on the device
            cur_s.wait_event(ev_out[j])                # the weights it overwrites have been read back

        def group_done(j):
            ev_grp[j].record(cur_s)
            lo, hi = bounds[j]
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_grp[j])
                host_w[lo:hi].copy_(sw.shard[lo:hi], non_blocking=True)
                ev_out[j].record(s_out)

        stepper.before_group, stepper.after_group = group_ready, group_done

        def e2e_run(nsteps):
            h2d(0)
            for k in range(nsteps):
                b_ = cur_buf["b"] = k % nset
                if k + 1 < nsteps and nset > 1:
                    h2d(k + 1)
                for p, g in zip(params, gsets[b_][1]):
                    p.grad = g
                opt_e.step()
                sw.publish()
                ev_step[b_].record(cur_s)
                if k + 1 < nsteps and nset == 1:
                    h2d(k + 1)
            for j in range(ngrp):
                cur_s.wait_event(ev_out[j])

        e2e_run(1)
        ctx.fence()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        e2e_run(e2e_steps)
        b.record()
        ctx.fence()
        (ems,) = ctx.reduce([a.elapsed_time(b)])
        ems /= e2e_steps
        nbytes = sw.part.shard_len * 2 * world
        e2e = {"value": total / (ems * 1e-3), "unit": "params/s", "ms_per_step": ems, "steps": e2e_steps,
               "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
               "pipeline": f"{ngrp} parameter groups: slice j of step k+1's gradients goes up while slice j of "
                           "step k's weights comes down (3 streams); the first upload and the last download "
                           "are inside the timed region"}
        opt_e.check_device_status()
        stepper.before_group = stepper.after_group = None
        del host_g, host_w, opt_e

    ns_info = None
    if opt_name == "AdaMuon":
        # Newton-Schulz alone, per distinct matrix shape of this rank's tensors: CUDA events around the
        # GEMM chain of kaon_newton_schulz
        from kaon_b200.adamuon import zeropower_via_newtonschulz5 as ns
        steps_ns = kw.get("ns_steps", 2)
        oset = set(owned)
        shapes2d = sorted({(s[0], W.numel([s]) // s[0]) for i, s in enumerate(shapes) if len(s) >= 2 and i in oset})
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

    res = None
    if rank == 0:
        peak, tpeak, peak_kind = measured_peaks()
        alg_bytes = bytes_per_param * (total / world)   # this rank's tensors, one step
        achieved = alg_bytes / (kern_ms * 1e-3) / 1e9
        tb = wopt.get("traffic_bpp")
        res = {
            "value": total / (ms_per_step * 1e-3), "unit": "params/s", "ms_per_step": ms_per_step,
            "step_kernel_ms": kern_ms, "publish_ms": pub_ms, "compute_only_ms": compute_only_ms,
            "incl_publish_ms": ms_per_step, "steps": steps, "warmup": warmup, "gpu_launches": launches,
            "clocks": clocks,
            "config": {"workload": workload, "optimizer": opt_name, "params": total, "tensors": len(shapes),
                       "param_dtype": "bf16", "momentum_dtype": kw.get("momentum_dtype", "4bit" if opt_name == "Nekaon" else None),
                       "sharding": "zero1" if world > 1 else "none",
                       "publish": ("none" if world == 1 else
                                   "peer stores fused into the step kernel + barrier" if fused_publish else
                                   "nccl all_gather_into_tensor after the step"),
                       "lr_schedule": "cosine 1e-4 -> 1e-5 over 50 steps" if cos else "constant",
                       "l2": f"inputs ({alg_bytes / 1e9:.1f} GB per step per GPU) larger than L2; no flush needed"},
            "gradient_reduce_scatter": (f"inside every step, {sg.waves} waves overlapped with the step" if sg is not None
                                        else "not part of the step"),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "peak_kind": f"{peak_kind} copy bandwidth",
                         "traffic": (tb * total / world) if tb else None,
                         "traffic_source": ("ncu capture of one launch of the 269 M-parameter list of the same "
                                            "shapes (profiles/), scaled by parameters" if tb else
                                            "not captured: the algorithmic bytes are the figure"),
                         "bytes_per_param": bytes_per_param, "kernel": KERNEL_NAME[opt_name]},
            "e2e": e2e,
        }
        if fused_publish:
            # the step kernel also pushes this rank's updated weights to the other ranks: its floor is the
            # slower of the HBM pass and the NVLink traffic (measured peer-copy bandwidth 770 GB/s)
            out_bytes = 2.0 * (total / world) * (world - 1)
            t_hbm, t_link = alg_bytes / (peak * 1e9), out_bytes / 770e9
            res["nvlink"] = {"ingress_bytes_per_rank": out_bytes, "achieved": out_bytes / (kern_ms * 1e-3) / 1e9,
                             "peak": 770.0, "unit": "GB/s", "floor_ms": max(t_hbm, t_link) * 1e3,
                             "frac_of_floor": max(t_hbm, t_link) * 1e3 / kern_ms}
        if ns_info is not None:
            rest_ms = max(kern_ms - ns_info["total"]["ms_per_step"], 1e-6)
            res["hbm_passes"] = dict(res["roofline"], achieved=alg_bytes / (rest_ms * 1e-3) / 1e9,
                                     frac=alg_bytes / (rest_ms * 1e-3) / 1e9 / peak, ms=rest_ms,
                                     note="everything of the step that is not a Newton-Schulz GEMM: step time minus "
                                          "the GEMM chains timed alone")
            res["hbm_passes"].pop("frac_of_nominal_8TBs", None)
            res["roofline"] = {"bound": "tensor", "achieved": ns_info["total"]["tflops"], "peak": tpeak,
                               "unit": "TFLOP/s", "frac": ns_info["total"]["tflops"] / tpeak, "traffic": None,
                               "peak_kind": f"{peak_kind} cuBLAS bf16 burst", "kernel": "ns_gemm_kernel",
                               "note": "Newton-Schulz GEMM chain of one matrix timed alone per shape (CUDA events); inside a step "
                                       "the chains of different matrices overlap on three streams: newton_schulz.whole_step_tflops "
                                       "is the same flops over the whole step time"}
            ns_info["whole_step_tflops"] = ns_info["total"]["flop_per_step"] / (kern_ms * 1e-3) / 1e12
            res["newton_schulz"] = ns_info
    return res


def measure_and_free(*a, **k):
    """measure(), then release what it held (its locals die with its frame) before the next workload."""
    import torch
    res = measure(*a, **k)
    gc.collect()
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch.distributed as dist
    ctx = Ctx(args)
    single = args.workload is not None
    head_name = args.workload or HEADLINE
    wsteps = WORKLOADS[head_name][4].get("steps") if single and args.steps_from_config else None
    head = measure_and_free(ctx, head_name, wsteps or args.steps, args.warmup,
                   e2e_steps=0 if args.no_e2e else max(1, min(args.steps, args.e2e_steps)))
    extra = {}
    if not single and not args.headline_only:
        for name in RECORD:
            steps = WORKLOADS[name][4].get("steps", args.steps)
            try:
                r = measure_and_free(ctx, name, steps, args.warmup)
            except Exception as e:  # noqa: BLE001 - the headline line must still print
                r = {"error": f"{type(e).__name__}: {e}"[:400]}
                if ctx.world > 1:
                    raise
            if ctx.rank == 0:
                extra[name] = r
    if ctx.rank == 0:
        line = {"metric": "optimizer_step_params_per_sec", "value": head["value"], "unit": "params/s",
                "n_gpus": ctx.world, "steps": head["steps"], "warmup": head["warmup"],
                "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
        for k in ("config", "step_kernel_ms", "publish_ms", "compute_only_ms", "incl_publish_ms",
                  "gradient_reduce_scatter", "roofline", "e2e", "gpu_launches", "clocks", "nvlink", "hbm_passes",
                  "newton_schulz"):
            if k in head:
                line[k] = head[k]
        line["config"]["storage_dtype"] = "bf16 weights and gradients, arithmetic in fp32"
        if extra:
            line["workloads"] = extra
            line["gpu_launches"] = head["gpu_launches"] + sum(int(r.get("gpu_launches", 0)) for r in extra.values())
            line["gpu_launches_headline"] = head["gpu_launches"]
        if ctx.world == 1 and not args.no_cpu:
            line["cpu_baseline"], _, _ = cpu_baseline(head_name)
            if extra:
                for name in RECORD:
                    if name in extra and "error" not in extra[name]:
                        extra[name]["cpu_baseline"], _, _ = cpu_baseline(name)
        if ctx.world == 1 and not single and not args.no_gpu_bar:
            line["gpu_bar"] = gpu_bar_subprocess()
        print(json.dumps(line), flush=True)
    if ctx.world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS),
                    help="measure only this workload (default: the headline, then the other configurations)")
    ap.add_argument("--headline-only", action="store_true")
    ap.add_argument("--steps-from-config", action="store_true",
                    help="with --workload: use the step count the configuration names (Nekaon 50, AdaMuon 10)")
    ap.add_argument("--e2e-steps", type=int, default=6)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-gpu-bar", action="store_true")
    ap.add_argument("--gpu-bar", action="store_true", help="time the reference's own CUDA paths (needs baseline/_ref)")
    ap.add_argument("--gpu-bar-fused", action="store_true", help="with --gpu-bar: also the reference's Triton path")
    ap.add_argument("--comm-sms", type=int, default=48,
                    help="with --reduce-scatter in waves: multiprocessors left free of the (persistent) step kernels "
                         "for the collective that runs beside them")
    ap.add_argument("--waves", type=int, default=0,
                    help="with --reduce-scatter: cut every rank's tensors into this many waves, each one collective "
                         "and one parameter group, so the step of a wave overlaps the next wave's reduce-scatter "
                         "(0: 4 waves on 2 GPUs, where the step is long enough to hide; 1 beyond, where the links are the floor)")
    ap.add_argument("--reduce-scatter", action="store_true",
                    help="N>1: put the gradient reduce-scatter (NCCL, bf16 average) inside every step; the step "
                         "kernels then read the collective's output buffer")
    ap.add_argument("--publish", default="fused", choices=["fused", "allgather"],
                    help="N>1: how the owned weights reach the other ranks")
    args = ap.parse_args()
    if args.gpu_bar:
        run_gpu_bar(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
