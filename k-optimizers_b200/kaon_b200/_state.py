"""Checkpoint load that keeps every state tensor bit for bit.

The reference snapshots the saved dtypes, lets torch's ``load_state_dict`` cast state to the
parameter dtype and casts back (src/kaon/_momentum_codec.py:417-452); with bf16 parameters that squeezes
the fp32 statistics and scales through bf16.  Here the saved tensors are copied to the parameter's
device without any cast, so resume is exact for every parameter dtype; the on-disk layout is unchanged.
"""
from __future__ import annotations

from typing import Any

import torch


def load_state_dict_exact(optimizer: torch.optim.Optimizer, state_dict: dict[str, Any]) -> None:
    saved = state_dict.get("state", {})
    torch.optim.Optimizer.load_state_dict(optimizer, state_dict)
    params = [p for group in optimizer.param_groups for p in group["params"]]
    for i, p in enumerate(params):
        src = saved.get(i, saved.get(str(i)))
        if src is None or p not in optimizer.state:
            continue
        st = optimizer.state[p]
        for key, v in src.items():
            if torch.is_tensor(v):
                st[key] = v.detach().to(device=p.device, copy=True).contiguous()
            else:
                st[key] = v


# the reference's name for the same job
load_state_dict_preserving_dtypes = load_state_dict_exact
