"""AdaMuon (orthogonalised momentum with an adaptive factored second moment) on the fused sm_100a step.

Same constructor, param-group keys, state layout and errors as the reference class
(src/kaon/adamuon.py:216-325); ``step()`` runs, per parameter group, the EMA pre-pass, the Newton-Schulz
iteration as tcgen05 GEMMs and one persistent kernel for everything after it, instead of the foreach
buckets and ``torch.bmm`` (src/kaon/adamuon.py:327-352, 393-615).  ``foreach*`` and ``compile`` are
accepted and ignored.
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
from .adakaon import init_second_moment_state

__all__ = ["AdaMuon", "zeropower_via_newtonschulz5"]

_FOURBIT_BLOCK = 128
FOREACH_BATCH_CUTOFF = 2_000_000


def zeropower_via_newtonschulz5(grad: Tensor, steps: int) -> Tensor:
    """Newton-Schulz quintic iteration on a 2-D CUDA matrix; returns the bf16 orthogonal factor
    (reference src/kaon/adamuon.py:97-118), computed by the tcgen05 GEMM chain."""
    assert grad.ndim == 2, "Newton-Schulz expects a 2-D matrix"
    if not grad.is_cuda:
        raise L.KaonError("kaon_b200 runs on CUDA tensors only")
    lib = L.lib()
    x = grad.detach().to(torch.bfloat16).contiguous()
    if x.data_ptr() == grad.data_ptr():
        x = x.clone()
    rows, cols = x.shape
    nbytes = lib.kaon_newton_schulz_workspace_bytes(C.c_int64(rows), C.c_int64(cols))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=x.device)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        L.check(lib.kaon_newton_schulz(C.c_void_p(x.data_ptr()), C.c_int64(rows), C.c_int64(cols), int(steps),
                                       C.c_void_p(out.data_ptr()), C.c_void_p(ws.data_ptr()), C.c_int64(nbytes),
                                       C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream)))
    return out


class AdaMuon(FusedStepMixin, AutoLRMixin, Optimizer):
    _OPT_KIND = L.OPT_ADAMUON

    def __init__(
        self,
        params: Iterable[Any],
        lr: float = 2e-2,
        betas: tuple[float, float] = (0.95, 0.999),
        eps: tuple[float, float] = (1e-30, 1e-3),
        weight_decay: float = 0.0,
        *,
        ns_steps: int = 2,
        clip_threshold: float = 1.0,
        momentum_dtype: str = "bfloat16",
        momentum_4bit_block: int = _FOURBIT_BLOCK,
        cautious: bool = True,
        gradient_centralization: bool = False,
        bf16_method: str = "stochastic_rounding",
        foreach: bool = True,
        foreach_batch_cutoff: int = FOREACH_BATCH_CUTOFF,
        foreach_stack_budget: int | None = None,
        compile: bool = False,  # noqa: A002 - the reference's public kwarg name
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
        if ns_steps < 1:
            raise ValueError(f"ns_steps must be >= 1, got {ns_steps}")
        if clip_threshold <= 0.0:
            raise ValueError(f"clip_threshold must be > 0, got {clip_threshold}")
        if momentum_dtype not in ("bfloat16", "float32", "int8", "4bit"):
            raise ValueError(f"momentum_dtype must be bfloat16/float32/int8/4bit, got {momentum_dtype!r}")
        if bf16_method not in ("stochastic_rounding", "kahan", "none"):
            raise ValueError(f"bf16_method must be stochastic_rounding/kahan/none, got {bf16_method!r}")
        if foreach_batch_cutoff < 1:
            raise ValueError(f"foreach_batch_cutoff must be >= 1, got {foreach_batch_cutoff}")
        defaults = {
            "lr": lr,
            "betas": (beta1, beta2),
            "eps": (float(eps[0]), float(eps[1])),
            "weight_decay": weight_decay,
            "ns_steps": ns_steps,
            "clip_threshold": clip_threshold,
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
        self._workspaces: dict[torch.device, Tensor] = {}
        self._init_autolr(auto_lr, auto_lr_scale, auto_lr_fuse_rel, auto_lr_d0)

    def _momentum_dtype(self, group: dict[str, Any]) -> str | None:
        return group["momentum_dtype"] if group["betas"][0] > 0 else None

    @torch.no_grad()
    def _init_state(self, p: Tensor, state: dict[str, Any], group: dict[str, Any]) -> None:
        init_second_moment_state(p, state)
        if group["betas"][0] > 0:
            init_momentum_state(state, p.grad, group["momentum_dtype"], group["momentum_4bit_block"])
        init_shift_state(p, state, group)

    def _workspace(self, plan: GroupPlan) -> Tensor:
        """Device scratch for the orthogonalised matrices; one buffer per device, grown on demand and
        shared by the plans of that device (they run one after another on the stream)."""
        need = int(L.lib().kaon_adamuon_workspace_bytes(plan.handle))
        ws = self._workspaces.get(plan.device)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.uint8, device=plan.device)
            self._workspaces[plan.device] = ws
        return ws

    def _launch(self, plan: GroupPlan, group: dict[str, Any], step: int, stream: int) -> None:
        hp = L.AdaMuonHParams(
            lr=group["lr"], beta1=group["betas"][0], beta2=group["betas"][1], eps1=group["eps"][0],
            weight_decay=group["weight_decay"], clip_threshold=group["clip_threshold"],
            ns_steps=int(group["ns_steps"]), cautious=int(bool(group["cautious"])),
            gradient_centralization=int(bool(group["gradient_centralization"])),
            bf16_method=L.BF16_METHOD[group["bf16_method"]])
        ws = self._workspace(plan)
        L.check(L.lib().kaon_adamuon_step(plan.handle, C.byref(hp), C.c_void_p(ws.data_ptr()),
                                          C.c_int64(ws.numel()), C.c_uint64(self._seed()), C.c_uint32(step),
                                          C.c_void_p(stream)))

    def orthogonalised(self, p: Tensor) -> Tensor | None:
        """The bf16 Newton-Schulz output the last step used for ``p`` (None for 1-D tensors)."""
        for plan in self._plans.values():
            for i, q in enumerate(plan.params):
                if q is p:
                    off = int(L.lib().kaon_adamuon_signal_offset(plan.handle, i))
                    if off < 0:
                        return None
                    ws = self._workspaces[plan.device]
                    return ws[off:off + p.numel() * 2].view(torch.bfloat16).view(p.shape[0], -1).clone()
        return None

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
