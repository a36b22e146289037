"""The public ``step()`` router of the optimizer classes.

The reference routes ``step()`` through ``AutoLRMixin`` (src/kaon/_autolr.py:499-507): with
``auto_lr=False`` it is a straight call to ``_step_impl``.  The DoWG tuner itself is a host-side scalar
controller outside the fused step; asking for it raises.
"""
from __future__ import annotations

from typing import Any

import torch

DEFAULT_FUSE_REL = 20.0


class AutoLRMixin:
    def _init_autolr(self, auto_lr: bool, scale: float, fuse_rel: float, d0: float | None = None) -> None:
        if auto_lr:
            raise NotImplementedError(
                "kaon_b200: auto_lr=True (the DoWG step-size tuner) is not part of the fused step")
        self._autolr = None

    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        return self._step_impl(closure)

    def _step_impl(self, closure: Any = None) -> Any:
        raise NotImplementedError

    def get_d(self) -> float:
        return float(self.param_groups[0]["lr"])

    def is_frozen(self) -> bool:
        return False

    def _autolr_state_dict(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        return state_dict

    def _autolr_load(self, state_dict: dict[str, Any], inner_load: Any) -> None:
        copied = dict(state_dict)
        copied.pop("_autolr", None)
        inner_load(copied)
