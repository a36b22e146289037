"""GPU-side drivers for the parity tests: run a golden case through the CUDA path."""
from __future__ import annotations

import numpy as np
import torch

import kaon_b200
from _golden import Fixture
from golden.cases import CASES, SCHEDULES


def to_bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16).reshape(-1).copy()
    return t.numpy().reshape(-1).copy()


def from_bits(a: np.ndarray, shape, device="cuda") -> torch.Tensor:
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).reshape(shape).to(device)
    return torch.from_numpy(a.copy()).reshape(shape).to(device)


def state_np(st: dict, key: str):
    v = st.get(key)
    if v is None:
        return None
    if torch.is_tensor(v):
        v = v.detach().cpu().contiguous()
        if v.dtype == torch.bfloat16:
            return v.view(torch.int16).numpy().view(np.uint16).reshape(-1)
        return v.numpy().reshape(-1)
    return np.asarray(v)


def run_case_gpu(name: str, seed: int = 0):
    """Yield (step, fixture, optimizer, params) after each step of the golden case on cuda:0."""
    opt_name, kw, shapes, dtype, steps, _seed, o = CASES[name]
    f = Fixture(name)
    params = [torch.nn.Parameter(from_bits(b, s)) for b, s in zip(f.params(), shapes)]
    opt = getattr(kaon_b200, opt_name)(params, **kw)
    opt.sr_seed = seed
    sched = SCHEDULES.get(o.get("lr_sched"))
    for step in range(1, steps + 1):
        if sched is not None:
            for g in opt.param_groups:
                g["lr"] = sched(step - 1)
        for p, gb, s in zip(params, f.grads(step), shapes):
            p.grad = from_bits(gb, s)
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        yield step, f, opt, params
