"""KProdigy (Prodigy's parameter-free distance estimate over kaon's memory backend) on the fused sm_100a step.

Same constructor, param-group keys (``d``, ``d_max``, ``d_numerator``, ``d_hat``, ``k`` included), state
layout (``step``, ``s``, ``p0``, ``m`` through the shared codecs, ``v`` or ``row`` / ``col``, ``shift``) and
errors as the reference class (src/kaon/kprodigy.py:90-297).  A step is the reference's two passes
(src/kaon/kprodigy.py:329-404): pass 1 (the D statistics, the d-scaled momentum EMA, the second moment) and
pass 2 (the weight update) run as CUDA launches per parameter group; between them the distance estimate -
one scalar over every tensor of a scope - is updated on the host from per-tensor sums, folded in fp32 in
tensor order as the reference does.  ``foreach*`` arguments are accepted and ignored.
"""
from __future__ import annotations

import ctypes as C
import math
from collections.abc import Iterable
from typing import Any

import numpy as np
import torch
from torch import Tensor
from torch.optim import Optimizer

from . import _lib as L
from ._engine import FusedStepMixin, GroupPlan, init_momentum_state, init_shift_state
from ._state import load_state_dict_exact
from .adakaon import FOREACH_BATCH_CUTOFF

__all__ = ["KProdigy"]

_FOURBIT_BLOCK = 128


class KProdigy(FusedStepMixin, Optimizer):
    _OPT_KIND = L.OPT_KPRODIGY

    def __init__(
        self,
        params: Iterable[Any],
        lr: float = 1.0,
        betas: tuple[float, float] = (0.9, 0.999),
        beta3: float | None = None,
        eps: float = 1e-8,
        weight_decay: float = 0.0,
        *,
        decouple: bool = True,
        use_bias_correction: bool = False,
        safeguard_warmup: bool = False,
        d0: float = 1e-6,
        d_coef: float = 1.0,
        growth_rate: float = float("inf"),
        d_update_freq: int = 1,
        slice_p: int = 1,
        independent_d: bool | None = None,
        momentum_dtype: str = "bfloat16",
        momentum_4bit_block: int = _FOURBIT_BLOCK,
        second_moment: str = "full",
        eps_factored: float = 1e-30,
        cautious: bool = False,
        gradient_centralization: bool = True,
        bf16_method: str = "stochastic_rounding",
        factor_conv_as_matrix: bool = True,
        foreach: bool = True,
        foreach_batch_cutoff: int = FOREACH_BATCH_CUTOFF,
        foreach_stack_budget: int | None = None,
    ) -> None:
        beta1, beta2 = float(betas[0]), float(betas[1])
        if not d0 > 0.0:
            raise ValueError(f"d0 must be > 0, got {d0}")
        if not lr > 0.0:
            raise ValueError(f"lr must be > 0, got {lr}")
        if not eps > 0.0:
            raise ValueError(f"eps must be > 0, got {eps}")
        if not 0.0 <= beta1 < 1.0:
            raise ValueError(f"betas[0] must be in [0, 1), got {beta1}")
        if not 0.0 <= beta2 < 1.0:
            raise ValueError(f"betas[1] must be in [0, 1), got {beta2}")
        if d_update_freq < 1:
            raise ValueError(f"d_update_freq must be >= 1, got {d_update_freq}")
        if slice_p < 1:
            raise ValueError(f"slice_p must be >= 1, got {slice_p}")
        if momentum_dtype not in ("bfloat16", "float32", "int8", "4bit"):
            raise ValueError(f"momentum_dtype must be bfloat16/float32/int8/4bit, got {momentum_dtype!r}")
        if second_moment not in ("full", "factored"):
            raise ValueError(f"second_moment must be full/factored, got {second_moment!r}")
        if bf16_method not in ("stochastic_rounding", "kahan", "none"):
            raise ValueError(f"bf16_method must be stochastic_rounding/kahan/none, got {bf16_method!r}")
        if foreach_batch_cutoff < 1:
            raise ValueError(f"foreach_batch_cutoff must be >= 1, got {foreach_batch_cutoff}")
        defaults = {
            "lr": lr,
            "betas": (beta1, beta2),
            "beta3": beta3,
            "eps": eps,
            "weight_decay": weight_decay,
            "decouple": decouple,
            "use_bias_correction": use_bias_correction,
            "safeguard_warmup": safeguard_warmup,
            "d": d0,
            "d0": d0,
            "d_max": d0,
            "d_numerator": 0.0,
            "d_coef": d_coef,
            "growth_rate": growth_rate,
            "d_update_freq": d_update_freq,
            "slice_p": slice_p,
            "k": 0,
            "momentum_dtype": momentum_dtype,
            "momentum_4bit_block": momentum_4bit_block,
            "second_moment": second_moment,
            "eps_factored": eps_factored,
            "cautious": cautious,
            "gradient_centralization": gradient_centralization,
            "bf16_method": bf16_method,
            "factor_conv_as_matrix": factor_conv_as_matrix,
        }
        self.d0 = d0
        super().__init__(params, defaults)
        self._independent_d = (len(self.param_groups) > 1) if independent_d is None else independent_d
        self._foreach = foreach
        self._foreach_batch_cutoff = foreach_batch_cutoff
        self._foreach_stack_budget = foreach_stack_budget
        self._fused_init()
        self._shard_group: Any = None

    def set_shard_group(self, group: Any = True) -> None:
        """ZeRO-1: this optimizer steps only the tensors its rank owns.  The distance estimate is one scalar
        over ALL tensors, so the two sums behind it are added over the ranks of ``group`` (``True``: the default
        process group) before every update of d - one all-reduce of three floats per scope and step."""
        self._shard_group = group

    def get_d(self) -> float:
        """Current D estimate (effective learning rate) of the first group."""
        return float(self.param_groups[0].get("d", self.d0))

    def _momentum_dtype(self, group: dict[str, Any]) -> str | None:
        return group["momentum_dtype"] if group["betas"][0] > 0 else None

    @torch.no_grad()
    def _init_state(self, p: Tensor, state: dict[str, Any], group: dict[str, Any]) -> None:
        """reference src/kaon/kprodigy.py:267-295"""
        sliced = p.detach().flatten()[:: group["slice_p"]]
        state["step"] = 0
        state["s"] = torch.zeros_like(sliced, dtype=torch.float32, memory_format=torch.contiguous_format)
        if sliced.norm() > 0:
            state["p0"] = sliced.float().clone().contiguous()
        else:
            state["p0"] = torch.zeros((), device=p.device, dtype=torch.float32)
        if group["betas"][0] > 0:
            init_momentum_state(state, p.grad if p.grad is not None else p, group["momentum_dtype"],
                                group["momentum_4bit_block"])
        if group["second_moment"] == "factored" and p.ndim >= 2:
            if p.ndim > 2 and not group["factor_conv_as_matrix"]:
                raise NotImplementedError("kaon_b200.KProdigy factors convolution kernels as matrices "
                                          "(factor_conv_as_matrix=False is not built)")
            state["row"] = torch.zeros(p.shape[0], dtype=torch.float32, device=p.device)
            state["col"] = torch.zeros(math.prod(p.shape[1:]), dtype=torch.float32, device=p.device)
        else:
            state["v"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        init_shift_state(p, state, group)

    def _plan_created(self, plan: GroupPlan, params: list[Tensor], states: list[dict[str, Any]]) -> None:
        n = len(params)
        s_arr, p0_arr = (C.c_void_p * n)(), (C.c_void_p * n)()
        for i, (p, st) in enumerate(zip(params, states)):
            s, p0 = st["s"], st["p0"]
            if not s.is_contiguous() or s.device != p.device or s.dtype != torch.float32:
                raise L.KaonError("optimizer state 's' must be a contiguous fp32 tensor on the parameter's device")
            s_arr[i] = s.data_ptr()
            plan._keep.append(s)
            if p0.ndim == 0:
                p0_arr[i] = None        # the reference's zero reference point
            else:
                if not p0.is_contiguous() or p0.device != p.device or p0.numel() != s.numel():
                    raise L.KaonError("optimizer state 'p0' must be contiguous, on the parameter's device and as long as 's'")
                p0_arr[i] = p0.data_ptr()
                plan._keep.append(p0)
        plan.slice_p = int(self._plan_slice_p)
        with torch.cuda.device(plan.device):
            L.check(L.lib().kaon_kprodigy_attach(plan.handle, s_arr, p0_arr, n, C.c_int64(plan.slice_p)))
        plan.sums = (C.c_float * (2 * n))()

    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        # a scope is a set of groups that share one distance estimate (reference src/kaon/kprodigy.py:306-314)
        scopes = [[g] for g in self.param_groups] if self._independent_d else [list(self.param_groups)]
        self._t += 1
        for scope in scopes:
            self._step_scope(scope)
        return loss

    def _step_scope(self, groups: list[dict[str, Any]]) -> None:
        """reference src/kaon/kprodigy.py:329-404"""
        lead = groups[0]
        beta1, beta2 = lead["betas"]
        beta3 = lead["beta3"] if lead["beta3"] is not None else math.sqrt(beta2)
        k, d, d_max, d0 = lead["k"], lead["d"], lead["d_max"], lead["d0"]
        lr = max(g["lr"] for g in groups)
        if lead["use_bias_correction"]:
            bias_correction = ((1 - beta2 ** (k + 1)) ** 0.5) / (1 - beta1 ** (k + 1))
        else:
            bias_correction = 1.0
        dlr = d * lr * bias_correction
        should_update_d = (k % lead["d_update_freq"]) == 0
        d_over_d0 = d / d0
        d_numerator = lead["d_numerator"] * beta3
        alpha_s = (d_over_d0 * d) if lead["safeguard_warmup"] else (d_over_d0 * dlr)
        const = np.float32(d_over_d0 * dlr)
        delta_numerator, d_denom = np.float32(0.0), np.float32(0.0)
        seen = False
        launched: list[tuple[GroupPlan, dict[str, Any], int]] = []
        gindex = {id(g): i for i, g in enumerate(self.param_groups)}
        for group in groups:
            group_lr = group["lr"]
            if group_lr not in (lr, 0.0):
                raise RuntimeError(
                    "KProdigy: groups sharing one D estimate must use the same lr "
                    "(or 0 for a frozen group). Use independent_d=True for per-group lr.")
            self._plan_slice_p = group["slice_p"]
            do_d = bool(group_lr > 0.0 and should_update_d)
            factored = group["second_moment"] == "factored"
            wd = group["weight_decay"]
            if factored and wd != 0 and not group["decouple"]:
                raise NotImplementedError("kaon_b200.KProdigy: coupled weight decay (decouple=False) folds the weights "
                                          "into the gradient the factored statistics see; that combination is not built")
            for pl in self._group_plans(gindex[id(group)], group, lambda p: self.state[p]):
                with torch.cuda.device(pl.device):
                    stream = torch.cuda.current_stream(pl.device).cuda_stream
                    if not pl.set_grads(stream):
                        continue
                    seen = True
                    hp = L.KProdigyPass1(
                        beta1=beta1, beta2=beta2, beta3=beta3, d=d, alpha_s=alpha_s,
                        weight_decay_coupled=wd if (wd != 0 and not group["decouple"]) else 0.0,
                        eps_factored=group["eps_factored"], do_d=int(do_d),
                        gradient_centralization=int(bool(lead["gradient_centralization"])),
                        factored=int(factored), reserved=0)
                    L.check(L.lib().kaon_kprodigy_pass1(pl.handle, C.byref(hp), pl.sums, C.c_void_p(stream)))
                    launched.append((pl, group, stream))
                    if do_d:
                        # the reference's fp32 left fold over the tensors (src/kaon/kprodigy.py:451-455, 580-588)
                        sums = np.ctypeslib.as_array(pl.sums)
                        for i, p in enumerate(pl.params):
                            if p.grad is None:
                                continue
                            delta_numerator = np.float32(delta_numerator + np.float32(sums[2 * i] * const))
                            d_denom = np.float32(d_denom + sums[2 * i + 1])
        if self._shard_group is not None and should_update_d and lr > 0.0:
            import torch.distributed as dist
            dev = self.param_groups[0]["params"][0].device
            red = torch.tensor([float(delta_numerator), float(d_denom), 1.0 if seen else 0.0], dtype=torch.float32, device=dev)
            dist.all_reduce(red, group=None if self._shard_group is True else self._shard_group)
            vals = red.tolist()
            delta_numerator, d_denom, seen = np.float32(vals[0]), np.float32(vals[1]), vals[2] > 0.0
        if should_update_d and lr > 0.0 and seen:
            denom_val = float(d_denom)
            if denom_val > 0.0:
                global_num = d_numerator + float(delta_numerator)
                d_hat = lead["d_coef"] * global_num / denom_val
                if d == d0:
                    d = max(d, d_hat)
                d_max = max(d_max, d_hat)
                d = min(d_max, d * lead["growth_rate"])
                for group in groups:
                    group["d_numerator"] = global_num
                    group["d"] = d
                    group["d_max"] = d_max
                    group["d_hat"] = d_hat
        # pass 2 keeps the dlr of the top of the step and takes d as just updated, like the reference
        for pl, group, stream in launched:
            with torch.cuda.device(pl.device):
                for p in pl.params:
                    if p.grad is not None:
                        self.state[p]["step"] += 1
                wd = group["weight_decay"]
                hp2 = L.KProdigyPass2(
                    d=d, dlr=dlr, eps=group["eps"],
                    decay_dlr=wd * dlr if (wd != 0 and group["decouple"]) else 0.0,
                    cautious=int(bool(group["cautious"])),
                    gradient_centralization=int(bool(lead["gradient_centralization"])),
                    factored=int(group["second_moment"] == "factored"),
                    bf16_method=L.BF16_METHOD[group["bf16_method"]])
                L.check(L.lib().kaon_kprodigy_pass2(pl.handle, C.byref(hp2), C.c_uint64(self._seed()),
                                                    C.c_uint32(self._t), C.c_void_p(stream)))
        for group in groups:
            group["k"] = group["k"] + 1

    def state_dict(self) -> dict[str, Any]:
        return self._extra_state(super().state_dict())

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        load_state_dict_exact(self, self._restore_extra(state_dict))
        self._invalidate_plans()
