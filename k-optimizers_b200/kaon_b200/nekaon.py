"""Nekaon: Adakaon plus a k-step momentum lookahead, on the fused sm_100a step.

The reference builds it as ``MSAM(rho=-k, norm="none")`` around an inner Adakaon
(src/kaon/nekaon.py:122-185, src/kaon/msam.py:374-406): every step takes the previous climb
``e = clamp(nan_to_num(rho * m), +-|rho| * clip_threshold * lr)`` back out of the weights, runs the inner
step, and climbs again along the refreshed momentum — three separate read-modify-writes of every
weight.  Here the removal and the climb ride on the Adakaon kernel's single read and write of each
weight (``msam_*`` fields of the C-ABI hyper-parameters); ``eval()`` / ``train()`` use the stand-alone
climb kernel.  Same constructor, attributes (``k``, ``inner``, ``base_optimizer``, shared
``param_groups``), errors and ``state_dict`` layout (inner layout plus ``"msam": {}``) as the reference.
"""
from __future__ import annotations

import ctypes as C
from collections import defaultdict
from collections.abc import Iterable
from typing import Any

import torch
from torch.optim import Optimizer

from . import _lib as L
from ._autolr import DEFAULT_FUSE_REL, AutoLRMixin
from .adakaon import Adakaon

__all__ = ["Nekaon"]


class Nekaon(AutoLRMixin, Optimizer):
    def __init__(
        self,
        params: Iterable[Any],
        lr: float = 1e-3,
        k: float = 1.5,
        betas: tuple[float, float] = (0.5, 0.999),
        weight_decay: float = 0.1,
        momentum_dtype: str = "4bit",
        *,
        low_vram_above: int | None = None,
        low_vram_lr_ratio: float = 0.5,
        auto_lr: bool = False,
        auto_lr_scale: float = 1.0,
        auto_lr_fuse_rel: float = DEFAULT_FUSE_REL,
        auto_lr_d0: float | None = None,
        **adakaon_kwargs: Any,
    ) -> None:
        if k < 0.0:
            raise ValueError(f"k must be >= 0 (lookahead steps), got {k}")
        if betas[0] <= 0.0:
            raise ValueError("Nekaon requires betas[0] > 0 (the lookahead rides the momentum)")
        if low_vram_above is not None:
            if low_vram_above < 0:
                raise ValueError(f"low_vram_above must be >= 0, got {low_vram_above}")
            params = list(params)
            if params and isinstance(params[0], dict):
                raise TypeError(
                    "low_vram_above does not support param-group dicts — pass a flat "
                    "parameter iterable; Nekaon builds its own small/big groups by tensor size.")
            small = [p for p in params if p.numel() <= low_vram_above]
            big = [p for p in params if p.numel() > low_vram_above]
            if not small and not big:
                raise ValueError("Nekaon got no parameters")
            groups: list[dict[str, Any]] = []
            if small:
                groups.append({"params": small})
            if big:
                groups.append({"params": big, "lr": lr * low_vram_lr_ratio, "betas": (0.0, betas[1])})
            params = groups
        if auto_lr and low_vram_above is not None:
            raise ValueError("Nekaon(auto_lr=True) is incompatible with low_vram_above")
        self.inner = Adakaon(params, lr=lr, betas=betas, weight_decay=weight_decay,
                             momentum_dtype=momentum_dtype, **adakaon_kwargs)
        self.base_optimizer = self.inner
        self.param_groups = self.inner.param_groups
        self.rho = -float(k)
        self.norm = "none"
        self.k = float(k)
        self._train_mode = True
        self._has_e = False
        self._eclamp: dict[int, float] = {}   # per group: climb bound frozen at climb time
        self._wrap_state: dict[Any, dict[str, Any]] = defaultdict(dict)
        self._init_autolr(auto_lr, auto_lr_scale, auto_lr_fuse_rel, auto_lr_d0)

    # ---- wrapper plumbing (reference src/kaon/_wrappers.py:224-278) ----
    @property
    def state(self):  # type: ignore[override]
        return self._wrap_state

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.inner.zero_grad(set_to_none=set_to_none)

    @property
    def sr_seed(self):
        return self.inner.sr_seed

    @sr_seed.setter
    def sr_seed(self, v):
        self.inner.sr_seed = v

    def set_weight_mirrors(self, base_ptr: int, nbytes: int, byte_deltas: list[int]) -> None:
        self.inner.set_weight_mirrors(base_ptr, nbytes, byte_deltas)

    def check_device_status(self) -> None:
        self.inner.check_device_status()

    def stats(self):
        return self.inner.stats()

    # ---- the perturbation ----
    def _bound(self, group: dict[str, Any]) -> float:
        return abs(self.rho) * group.get("clip_threshold", 1.0) * group["lr"]

    def _has_momentum(self, group: dict[str, Any]) -> bool:
        return group["betas"][0] > 0

    @torch.no_grad()
    def _apply_standalone(self, sign: float, tag: int) -> None:
        """p += clamp(sign*rho*m, +-bound) on every tensor that carries a momentum, with the bound
        frozen at climb time (reference src/kaon/msam.py:169-188, 201-235)."""
        for (gi, _dev, _dt), plan in self.inner._plans.items():
            group = self.param_groups[gi]
            if not self._has_momentum(group):
                continue
            gid = id(group)
            if sign > 0 and gid not in self._eclamp:
                self._eclamp[gid] = self._bound(group)
            stream = torch.cuda.current_stream(plan.device).cuda_stream
            with torch.cuda.device(plan.device):
                L.check(L.lib().kaon_msam_apply(plan.handle, C.c_double(sign * self.rho),
                                                C.c_double(self._eclamp[gid]), C.c_uint32(tag),
                                                C.c_uint64(self.inner._seed()), C.c_uint32(self.inner._t),
                                                C.c_void_p(stream)))

    @torch.no_grad()
    def eval(self) -> None:  # noqa: A003
        if self._train_mode and self._has_e:
            self._apply_standalone(-1.0, L.TAG_EVAL)
        self._train_mode = False

    @torch.no_grad()
    def train(self) -> None:
        if not self._train_mode and self._has_e:
            self._apply_standalone(+1.0, L.TAG_TRAIN)
        self._train_mode = True

    def _all_momentum_tensors_have_grads(self) -> bool:
        for group in self.param_groups:
            if not self._has_momentum(group):
                continue
            for p in group["params"]:
                if p.grad is None and self.inner.state.get(p):
                    return False
        return True

    @torch.no_grad()
    def _step_impl(self, closure: Any = None) -> Any:
        if not self._train_mode:
            raise RuntimeError(
                "MSAM.step() called outside train mode. Call optimizer.train() before the "
                "training step (and optimizer.eval() before sampling / checkpointing).")
        inner = self.inner
        climb = self.rho != 0.0
        fused = self._all_momentum_tensors_have_grads()
        if not fused:
            # some tensor that carries a climb has no gradient this step: keep the reference's three
            # separate passes so that its climb is still swapped at the right bounds
            if self._has_e:
                inner._t += 1
                self._apply_standalone(-1.0, L.TAG_REMOVE)
                inner._t -= 1
                self._has_e = False
            self._eclamp.clear()
            inner._msam = {}
            loss = inner.step(closure)
            if climb and inner._plans:
                self._apply_standalone(+1.0, L.TAG_CLIMB)
                self._has_e = True
            return loss
        msam: dict[int, dict[str, tuple[float, float]]] = {}
        for group in self.param_groups:
            if not self._has_momentum(group):
                continue
            gid = id(group)
            entry: dict[str, tuple[float, float]] = {}
            if self._has_e and gid in self._eclamp:
                entry["remove"] = (-1.0 * self.rho, self._eclamp[gid])
            if climb:
                entry["climb"] = (+1.0 * self.rho, self._bound(group))
            msam[gid] = entry
        self._eclamp = {gid: e["climb"][1] for gid, e in msam.items() if "climb" in e}
        inner._msam = msam
        try:
            loss = inner.step(closure)
        finally:
            inner._msam = {}
        self._has_e = climb and bool(self._eclamp)
        return loss

    # ---- checkpoint (reference src/kaon/_wrappers.py:259-278, src/kaon/msam.py:409-421) ----
    def state_dict(self) -> dict[str, Any]:
        sd = self.inner.state_dict()
        sd["msam"] = {}
        return self._autolr_state_dict(sd)

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        def _load(sd: dict[str, Any]) -> None:
            sd = dict(sd)
            sd.pop("msam", None)
            self.inner.load_state_dict(sd)  # also restores the SR stream position ("_kaon_b200")
            self.param_groups = self.inner.param_groups
        self._autolr_load(state_dict, _load)
        self.base_optimizer = self.inner
        self._train_mode = True
        self._has_e = False
        self._eclamp.clear()
