"""Lion (sign momentum, one quantised buffer) on the fused sm_100a step.

Same constructor, param-group keys, state layout and errors as the reference class
(src/kaon/lion.py:152-208); ``step()`` launches one persistent CUDA kernel per parameter group instead of
the foreach buckets (src/kaon/lion.py:322-485).  ``foreach*`` knobs are accepted and ignored: they are
numerically neutral in the reference (tests/test_lion.py:190-239) and have no meaning here.
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

__all__ = ["Lion"]

_FOURBIT_BLOCK = 128
FOREACH_BATCH_CUTOFF = 2_000_000


class Lion(FusedStepMixin, AutoLRMixin, Optimizer):
    _OPT_KIND = L.OPT_LION

    def __init__(
        self,
        params: Iterable[Any],
        lr: float = 1e-4,
        betas: tuple[float, float] = (0.9, 0.99),
        weight_decay: float = 0.0,
        *,
        momentum_dtype: str = "bfloat16",
        momentum_4bit_block: int = _FOURBIT_BLOCK,
        cautious: bool = True,
        gradient_centralization: bool = True,
        bf16_method: str = "stochastic_rounding",
        foreach: bool = True,
        foreach_batch_cutoff: int = FOREACH_BATCH_CUTOFF,
        foreach_stack_budget: int | None = None,
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
        if lr < 0.0:
            raise ValueError(f"lr must be >= 0, got {lr}")
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
            "weight_decay": weight_decay,
            "momentum_dtype": momentum_dtype,
            "momentum_4bit_block": momentum_4bit_block,
            "cautious": cautious,
            "gradient_centralization": gradient_centralization,
            "bf16_method": bf16_method,
        }
        super().__init__(params, defaults)
        self._foreach = foreach
        self._foreach_batch_cutoff = foreach_batch_cutoff
        self._foreach_stack_budget = foreach_stack_budget
        self._fused_init()
        self._init_autolr(auto_lr, auto_lr_scale, auto_lr_fuse_rel, auto_lr_d0)

    @torch.no_grad()
    def _init_state(self, p: Tensor, state: dict[str, Any], group: dict[str, Any]) -> None:
        init_momentum_state(state, p.grad, group["momentum_dtype"], group["momentum_4bit_block"])
        init_shift_state(p, state, group)

    def _launch(self, plan: GroupPlan, group: dict[str, Any], step: int, stream: int) -> None:
        if group["bf16_method"] == "stochastic_rounding" and plan.params[0].dtype == torch.float16:
            raise NotImplementedError("stochastic rounding is implemented for bfloat16 parameters only")
        hp = L.LionHParams(
            lr=group["lr"], beta1=group["betas"][0], beta2=group["betas"][1],
            weight_decay=group["weight_decay"], cautious=int(bool(group["cautious"])),
            gradient_centralization=int(bool(group["gradient_centralization"])),
            bf16_method=L.BF16_METHOD[group["bf16_method"]], reserved=0)
        L.check(L.lib().kaon_lion_step(plan.handle, C.byref(hp), C.c_uint64(self._seed()),
                                       C.c_uint32(step), C.c_void_p(stream)))

    @torch.no_grad()
    def _step_impl(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        self._run_groups()
        return loss

    def state_dict(self) -> dict[str, Any]:
        return self._extra_state(self._autolr_state_dict(super().state_dict()))

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        self._autolr_load(self._restore_extra(state_dict), lambda sd: load_state_dict_exact(self, sd))
        self._invalidate_plans()
