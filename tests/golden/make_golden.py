"""Generate the golden vectors under tests/golden/ by running the REFERENCE implementation on CPU.

Needs the reference's source tree (only this script imports it; the tests read the vectors):

    python tests/golden/make_golden.py [--ref /path/to/reference/src]

Each case is a small ``.npz``: the seeded inputs (weights, per-step grads) and, after every step, the
reference's weights and optimizer state in its own ``state_dict`` layout.  bf16 tensors are stored as
uint16 bit patterns.  The tests compare the CPU oracle (and, on a GPU, the CUDA kernels) with these.
"""
from __future__ import annotations

import argparse
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).copy()
    return t.numpy().copy()


def make_params(shapes, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter((torch.randn(s, generator=g) * 0.02).to(dtype)) for s in shapes]


def make_grads(shapes, dtype, seed, step, outlier=False, correlated=False):
    g = torch.Generator().manual_seed(seed + step)
    base = torch.Generator().manual_seed(seed + 7919)
    out = []
    for s in shapes:
        t = torch.randn(s, generator=g) * 1e-3
        if correlated:   # a steady direction under the noise, so that a distance estimate has something to find
            t = t * 0.3 + torch.randn(s, generator=base) * 1e-3
        if outlier:
            mask = torch.rand(s, generator=g) < 0.01
            t = torch.where(mask, t * 100.0, t)
        out.append(t.to(dtype))
    return out


def dump_state(out, prefix, st):
    for k, v in st.items():
        if torch.is_tensor(v):
            out[f"{prefix}_{k}"] = bits(v).reshape(-1)
        else:
            out[f"{prefix}_{k}"] = np.asarray(v)


def run_optimizer(kaon, name, kwargs, shapes, dtype, steps, seed, *, lr_sched=None, outlier=False,
                  store_inputs=True, sample=None, nekaon_eval=False, correlated=False):
    """Step the reference; returns the fixture dict."""
    torch.manual_seed(1234)  # the reference draws SR noise from the global RNG
    cls = getattr(kaon, name)
    params = make_params(shapes, dtype, seed)
    opt = cls(params, **kwargs)
    out = {"meta_shapes": np.array([str(tuple(s)) for s in shapes]),
           "meta_dtype": np.array(str(dtype)), "meta_steps": np.array(steps),
           "meta_seed": np.array(seed), "meta_outlier": np.array(outlier)}
    if store_inputs:
        for i, p in enumerate(params):
            out[f"p_in_t{i}"] = bits(p).reshape(-1)
    inner = getattr(opt, "base_optimizer", opt)
    for step in range(1, steps + 1):
        if lr_sched is not None:
            lr = lr_sched(step - 1)
            for grp in opt.param_groups:
                grp["lr"] = lr
        grads = make_grads(shapes, dtype, seed, step, outlier, correlated)
        for i, (p, g) in enumerate(zip(params, grads)):
            if store_inputs:
                out[f"g_s{step}_t{i}"] = bits(g).reshape(-1)
            p.grad = g.clone()
        opt.step()
        for key in ("d", "d_max", "d_numerator", "d_hat", "k", "step"):
            if key in opt.param_groups[0]:
                out[f"grp_s{step}_{key}"] = np.asarray(opt.param_groups[0][key], dtype=np.float64)
        for i, p in enumerate(params):
            st = inner.state[p]
            if sample is None:
                out[f"p_s{step}_t{i}"] = bits(p).reshape(-1)
                dump_state(out, f"st_s{step}_t{i}", st)
            else:
                # large case: small state in full, big tensors strided
                out[f"p_s{step}_t{i}"] = bits(p).reshape(-1)[::sample]
                for k, v in st.items():
                    if torch.is_tensor(v):
                        b = bits(v).reshape(-1)
                        out[f"st_s{step}_t{i}_{k}"] = b[::sample] if b.size > 20000 else b
                    else:
                        out[f"st_s{step}_t{i}_{k}"] = np.asarray(v)
    if nekaon_eval:
        opt.eval()
        for i, p in enumerate(params):
            out[f"p_eval_t{i}"] = bits(p).reshape(-1)
    return out


def codec_case(kaon):
    from kaon._momentum_codec import (_dequant_4bit, _quant_4bit, _quant_int8)
    g = torch.Generator().manual_seed(7)
    out = {}
    cases = {"a": (37, 53), "b": (200,), "c": (4, 3, 3, 3)}
    for key, shape in cases.items():
        x = torch.randn(shape, generator=g) * 1e-3
        if key == "a":
            x[3].zero_()          # an all-zero row -> absmax floor
            x[5, 7] = 0.25        # an outlier
        q, sc = _quant_int8(x)
        out[f"int8_{key}_in"] = x.numpy().reshape(-1)
        out[f"int8_{key}_codes"] = q.numpy().reshape(-1)
        out[f"int8_{key}_scale"] = sc.numpy().reshape(-1)
        out[f"int8_{key}_dec"] = (q.float() * sc).numpy().reshape(-1)
    for n in (1000, 77, 256, 1, 129):
        x = torch.randn(n, generator=g) * 1e-3
        if n == 1000:
            x[128:256].zero_()    # an all-zero block
        bs = min(128, n)
        packed, sc, _ = _quant_4bit(x, bs)
        out[f"q4_{n}_in"] = x.numpy()
        out[f"q4_{n}_packed"] = packed.numpy()
        out[f"q4_{n}_scale"] = sc.numpy()
        out[f"q4_{n}_dec"] = _dequant_4bit(packed, sc, n, bs).numpy()
    return out


def gc_case(kaon):
    from kaon._backend import centralize_grads_
    g = torch.Generator().manual_seed(11)
    out = {}
    for key, shape, dtype in (("bf16_2d", (24, 180), torch.bfloat16), ("bf16_conv", (6, 5, 3, 3), torch.bfloat16),
                              ("f32_2d", (24, 180), torch.float32)):
        p = torch.nn.Parameter(torch.zeros(shape, dtype=dtype))
        x = (torch.randn(shape, generator=g) * 1e-3 + 2e-4).to(dtype)
        p.grad = x.clone()
        centralize_grads_([p])
        out[f"{key}_in"] = bits(x).reshape(-1)
        out[f"{key}_out"] = bits(p.grad).reshape(-1)
    return out


def sr_case(kaon):
    from kaon._stochastic_rounding import add_stochastic_
    g = torch.Generator().manual_seed(13)
    n = 4096
    p = (torch.randn(n, generator=g) * 0.02).bfloat16()
    d = torch.randn(n, generator=g) * 1e-4
    out = {"p_in": bits(p), "delta": d.numpy()}
    for alpha in (-1.0, 1.0):
        torch.manual_seed(99)
        q = p.clone()
        add_stochastic_(q, d, alpha=alpha)
        torch.manual_seed(99)
        noise = torch.randint(0, 0x10000, (n,), dtype=torch.int32)
        out[f"noise_a{alpha:+.0f}"] = noise.numpy().astype(np.uint16)
        out[f"p_out_a{alpha:+.0f}"] = bits(q)
    return out


def ns_case(kaon):
    from kaon.adamuon import zeropower_via_newtonschulz5
    g = torch.Generator().manual_seed(17)
    out = {}
    for key, shape in (("sq", (48, 48)), ("tall", (96, 32)), ("wide", (32, 80))):
        x = torch.randn(shape, generator=g) * 1e-3
        o = zeropower_via_newtonschulz5(x, 2).float()
        out[f"{key}_in"] = x.numpy()
        out[f"{key}_out"] = o.numpy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("KAON_REFERENCE_SRC", ""),
                    help="the reference's src/ directory (holds the `kaon` package); or set KAON_REFERENCE_SRC")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    if not args.ref:
        ap.error("--ref (or KAON_REFERENCE_SRC) must name the reference's src/ directory")
    sys.path.insert(0, args.ref)
    sys.path.insert(0, HERE)
    import kaon
    torch.set_num_threads(1)

    from cases import CASES, SCHEDULES
    dt = {"bf16": torch.bfloat16, "f32": torch.float32}
    cases = {"codec": lambda: codec_case(kaon), "gc": lambda: gc_case(kaon),
             "sr": lambda: sr_case(kaon), "ns": lambda: ns_case(kaon)}
    for cname, (opt, kw, shapes, dtype, steps, seed, o) in CASES.items():
        cases[cname] = (lambda opt=opt, kw=kw, shapes=shapes, dtype=dtype, steps=steps, seed=seed, o=o:
                        run_optimizer(kaon, opt, kw, shapes, dt[dtype], steps, seed,
                                      lr_sched=SCHEDULES.get(o.get("lr_sched")),
                                      outlier=o.get("outlier", False),
                                      store_inputs=o.get("store_inputs", True),
                                      sample=o.get("sample"), nekaon_eval=o.get("nekaon_eval", False),
                                      correlated=o.get("correlated", False)))
    for name, fn in cases.items():
        if args.only and name != args.only:
            continue
        data = fn()
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **data)
        print(f"{name}: {len(data)} arrays, {os.path.getsize(path) / 1024:.1f} KiB")


if __name__ == "__main__":
    main()
