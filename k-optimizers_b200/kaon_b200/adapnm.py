"""AdaPNM (Adam with positive-negative momentum on the factored second moment) on the fused sm_100a step.

Same constructor, param-group keys (``step`` included), state layout (``m_pos`` / ``m_neg`` through the
shared codecs, ``row`` / ``col`` or ``v`` / ``max_v``, ``shift``) and errors as the reference class
(src/kaon/adapnm.py:275-434, 451-500); ``step()`` replaces the foreach buckets and the per-parameter step
(src/kaon/adapnm.py:599-645, 1039-1273) with CUDA launches per parameter group.  ``foreach*``, ``fused`` and
``fused_tile_cap`` are accepted and ignored.
"""
from __future__ import annotations

import ctypes as C
from collections.abc import Iterable
from typing import Any

import torch
from torch import Tensor
from torch.optim import Optimizer

from . import _lib as L
from ._autolr import DEFAULT_FUSE_REL, AutoLRMixin
from ._engine import FusedStepMixin, GroupPlan, init_momentum_state, init_shift_state
from ._state import load_state_dict_exact
from .adakaon import FOREACH_BATCH_CUTOFF, init_second_moment_state

__all__ = ["AdaPNM"]

_FOURBIT_BLOCK = 128


class AdaPNM(FusedStepMixin, AutoLRMixin, Optimizer):
    _OPT_KIND = L.OPT_ADAPNM
    _M_KEY = "m_pos"

    def __init__(
        self,
        params: Iterable[Any],
        lr: float = 1e-3,
        betas: tuple[float, float] = (0.8, 0.999),
        beta0: float = 0.5,
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        *,
        clip_threshold: float = 1.0,
        cautious: bool = True,
        gradient_centralization: bool = True,
        ams_bound: bool = False,
        momentum_dtype: str = "bfloat16",
        momentum_4bit_block: int = _FOURBIT_BLOCK,
        bf16_method: str = "stochastic_rounding",
        foreach: bool = True,
        foreach_batch_cutoff: int = FOREACH_BATCH_CUTOFF,
        foreach_stack_budget: int | None = None,
        fused: bool = False,
        fused_tile_cap: int | None = None,
        auto_lr: bool = False,
        auto_lr_scale: float = 1.0,
        auto_lr_fuse_rel: float = DEFAULT_FUSE_REL,
        auto_lr_d0: float | None = None,
    ) -> None:
        beta1, beta2 = float(betas[0]), float(betas[1])
        if not 0.0 <= beta1 < 1.0:
            raise ValueError(f"betas[0] must be in [0, 1), got {beta1}")
        if not 0.0 <= beta2 < 1.0:
            raise ValueError(f"betas[1] must be in [0, 1), got {beta2}")
        if not 0.0 <= beta0 <= 1.0:
            raise ValueError(f"beta0 must be in [0, 1], got {beta0}")
        if lr < 0.0:
            raise ValueError(f"lr must be >= 0, got {lr}")
        if eps < 0.0:
            raise ValueError(f"eps must be >= 0, got {eps}")
        if clip_threshold < 0.0:
            raise ValueError(f"clip_threshold must be >= 0, got {clip_threshold}")
        if weight_decay < 0.0:
            raise ValueError(f"weight_decay must be >= 0, got {weight_decay}")
        if momentum_dtype not in ("bfloat16", "float32", "int8", "4bit"):
            raise ValueError(f"momentum_dtype must be bfloat16/float32/int8/4bit, got {momentum_dtype!r}")
        if bf16_method not in ("stochastic_rounding", "kahan", "none"):
            raise ValueError(f"bf16_method must be stochastic_rounding/kahan/none, got {bf16_method!r}")
        if foreach_batch_cutoff < 1:
            raise ValueError(f"foreach_batch_cutoff must be >= 1, got {foreach_batch_cutoff}")
        defaults = {
            "lr": lr,
            "betas": (beta1, beta2),
            "beta0": float(beta0),
            "eps": float(eps),
            "clip_threshold": float(clip_threshold),
            "weight_decay": weight_decay,
            "cautious": cautious,
            "gradient_centralization": gradient_centralization,
            "ams_bound": ams_bound,
            "momentum_dtype": momentum_dtype,
            "momentum_4bit_block": momentum_4bit_block,
            "bf16_method": bf16_method,
            "step": 0,
        }
        super().__init__(params, defaults)
        self._foreach = foreach
        self._foreach_batch_cutoff = foreach_batch_cutoff
        self._foreach_stack_budget = foreach_stack_budget
        self._fused = bool(fused)
        self._fused_init()
        self._init_autolr(auto_lr, auto_lr_scale, auto_lr_fuse_rel, auto_lr_d0)

    @torch.no_grad()
    def _init_state(self, p: Tensor, state: dict[str, Any], group: dict[str, Any]) -> None:
        init_second_moment_state(p, state)
        if p.ndim < 2 and group["ams_bound"]:
            state["max_v"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        init_momentum_state(state, p.grad, group["momentum_dtype"], group["momentum_4bit_block"], "m_pos")
        init_momentum_state(state, p.grad, group["momentum_dtype"], group["momentum_4bit_block"], "m_neg")
        init_shift_state(p, state, group)

    def _plan_created(self, plan: GroupPlan, params: list[Tensor], states: list[dict[str, Any]]) -> None:
        n = len(params)
        neg, neg_sc, max_v = (C.c_void_p * n)(), (C.c_void_p * n)(), (C.c_void_p * n)()
        for i, (p, st) in enumerate(zip(params, states)):
            for arr, key in ((neg, "m_neg"), (neg_sc, "m_neg_scale"), (max_v, "max_v")):
                t = st.get(key)
                if t is None:
                    arr[i] = None
                    continue
                if not t.is_contiguous() or t.device != p.device:
                    raise L.KaonError(f"optimizer state '{key}' must be contiguous and on the parameter's device")
                arr[i] = t.data_ptr()
                plan._keep.append(t)
        with torch.cuda.device(plan.device):
            L.check(L.lib().kaon_adapnm_attach(plan.handle, neg, neg_sc, max_v, n))

    def _launch(self, plan: GroupPlan, group: dict[str, Any], step: int, stream: int) -> None:
        hp = L.AdaPNMHParams(
            lr=group["lr"], beta1=group["betas"][0], beta2=group["betas"][1], beta0=group["beta0"],
            eps=group["eps"], weight_decay=group["weight_decay"], clip_threshold=group["clip_threshold"],
            cautious=int(bool(group["cautious"])),
            gradient_centralization=int(bool(group["gradient_centralization"])),
            ams_bound=int(bool(group["ams_bound"])), bf16_method=L.BF16_METHOD[group["bf16_method"]],
            group_step=int(group["step"]), reserved=0)
        L.check(L.lib().kaon_adapnm_step(plan.handle, C.byref(hp), C.c_uint64(self._seed()),
                                         C.c_uint32(step), C.c_void_p(stream)))

    @torch.no_grad()
    def _step_impl(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:   # the reference counts a group's steps whether or not it has gradients
            group["step"] += 1
        self._run_groups()
        return loss

    def state_dict(self) -> dict[str, Any]:
        return self._extra_state(self._autolr_state_dict(super().state_dict()))

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self._autolr_load(self._restore_extra(state_dict), lambda sd: load_state_dict_exact(self, sd))
        self._invalidate_plans()
