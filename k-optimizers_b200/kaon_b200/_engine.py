"""Host side of the fused step: per-parameter-group plans over the C ABI.

A *plan* is the device-side descriptor table that replaces the reference's foreach batcher
(reference src/kaon/adakaon.py:757-838, src/kaon/lion.py:366-414, src/kaon/_backend.py:59-77): one row
per tensor (weights, momentum, scales, statistics, shape), a work list and scratch, built once and
reused every step.  Only the gradient-pointer column is refreshed per step, because
``zero_grad(set_to_none=True)`` reallocates gradients (the stale-pointer hazard the reference guards
against in src/kaon/_fused_triton.py:1229-1245).  Plans are dropped whenever optimizer state is
replaced (``load_state_dict``) or the set of stepped parameters changes.
"""
from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from . import _lib as L

_PARAM_DT = {torch.float32: L.DT_F32, torch.bfloat16: L.DT_BF16}


def fourbit_block_size(numel: int, block: int) -> int:
    """reference src/kaon/_momentum_codec.py:192-200"""
    if block <= 0:
        return numel
    return min(block, numel) if numel > 0 else 1


def init_momentum_state(state: dict[str, Any], grad: torch.Tensor, md: str, block: int, key: str = "m") -> None:
    """Allocate one first-moment buffer in the reference's layout
    (src/kaon/_momentum_codec.py:263-264, 295-301, 350-360; src/kaon/lion.py:210-241); AdaPNM keeps two,
    under the keys "m_pos" and "m_neg" (src/kaon/adapnm.py:451-480)."""
    dev = grad.device
    if md in ("bfloat16", "float32"):
        state[key] = torch.zeros_like(grad, dtype=torch.bfloat16 if md == "bfloat16" else torch.float32,
                                      memory_format=torch.contiguous_format)
    elif md == "int8":
        state[key] = torch.zeros_like(grad, dtype=torch.int8, memory_format=torch.contiguous_format)
        shape = (grad.shape[0],) + (1,) * (grad.ndim - 1) if grad.ndim >= 2 else ()
        state[f"{key}_scale"] = torch.ones(shape, dtype=torch.float32, device=dev)
    else:  # 4bit
        numel = grad.numel()
        bs = fourbit_block_size(numel, block)
        nblocks = (numel + bs - 1) // bs
        state[key] = torch.full(((numel + 1) // 2,), 0x88, dtype=torch.uint8, device=dev)
        state[f"{key}_scale"] = torch.ones(nblocks, dtype=torch.float32, device=dev)
        state[f"{key}_numel"] = numel
        state[f"{key}_block"] = bs


def init_shift_state(p: torch.Tensor, state: dict[str, Any], group: dict[str, Any]) -> None:
    """Kahan compensation buffer for low-precision weights (reference src/kaon/lion.py:240-241,
    src/kaon/adakaon.py:334-335, src/kaon/adamuon.py:315-316)."""
    if group.get("bf16_method") == "kahan" and p.dtype in (torch.bfloat16, torch.float16):
        state["shift"] = torch.zeros_like(p, memory_format=torch.contiguous_format)


class GroupPlan:
    """One C-ABI plan: the tensors of one (param group, device, dtype) bucket."""

    def __init__(self, optimizer_kind: int, params: list[torch.Tensor], states: list[dict[str, Any]],
                 tensor_ids: list[int], momentum_dtype: str | None, m_key: str = "m"):
        lib = L.lib()
        p0 = params[0]
        if not p0.is_cuda:
            raise L.KaonError("kaon_b200 steps CUDA tensors only (there is no CPU path); got a "
                              f"parameter on {p0.device}")
        if p0.dtype not in _PARAM_DT:
            raise NotImplementedError(f"kaon_b200: parameter dtype {p0.dtype} (float32 and bfloat16 are supported)")
        self.device = p0.device
        self.params = params
        self.n = len(params)
        self.param_ptrs = [p.data_ptr() for p in params]
        mk = L.M_NONE if momentum_dtype is None else L.MOMENTUM_KIND[momentum_dtype]
        descs = (L.TensorDesc * self.n)()
        self._keep = []  # state tensors the table points at
        for i, (p, st, tid) in enumerate(zip(params, states, tensor_ids)):
            if not p.is_contiguous():
                raise NotImplementedError("kaon_b200: non-contiguous parameter")
            d = descs[i]
            d.p = p.data_ptr()
            d.g = 0
            d.numel = p.numel()
            d.rows = p.shape[0] if p.ndim >= 2 else 0
            d.tensor_id = tid
            d.block = int(st.get(f"{m_key}_block", 128))
            for field, key in (("m", m_key), ("m_scale", f"{m_key}_scale")):
                t = st.get(key) if mk != L.M_NONE else None
                if t is not None:
                    if not t.is_contiguous() or t.device != p.device:
                        raise L.KaonError(f"optimizer state '{key}' must be contiguous and on the parameter's device")
                    setattr(d, field, t.data_ptr())
                    self._keep.append(t)
            sh = st.get("shift")
            if sh is not None:
                if not sh.is_contiguous() or sh.device != p.device or sh.dtype != p.dtype:
                    raise L.KaonError("optimizer state 'shift' must be contiguous, on the parameter's device and of its dtype")
                d.shift = sh.data_ptr()
                self._keep.append(sh)
            a = st.get("row") if "row" in st else st.get("v")
            b = st.get("col")
            for field, t in (("stat_a", a), ("stat_b", b)):
                if t is not None:
                    setattr(d, field, t.data_ptr())
                    self._keep.append(t)
        self.handle = C.c_void_p()
        with torch.cuda.device(self.device):
            L.check(lib.kaon_plan_create(C.byref(self.handle), optimizer_kind, _PARAM_DT[p0.dtype], mk,
                                         descs, self.n))
        self._grad_ptrs: list[int] | None = None
        self._grad_arr = (C.c_void_p * self.n)()

    def set_grads(self, stream: int) -> bool:
        """Refresh the gradient-pointer column; returns False when nothing has a gradient."""
        ptrs = []
        dt = self.params[0].dtype
        for p in self.params:
            g = p.grad
            if g is None:
                ptrs.append(0)
                continue
            if g.is_sparse:
                raise RuntimeError("kaon_b200 does not support sparse gradients")
            if g.dtype != dt or not g.is_contiguous():
                raise NotImplementedError("kaon_b200: gradients must be contiguous and of the parameter's dtype")
            ptrs.append(g.data_ptr())
        if ptrs != self._grad_ptrs:
            arr = self._grad_arr
            for i, v in enumerate(ptrs):
                arr[i] = v
            L.check(L.lib().kaon_plan_set_grads(self.handle, arr, self.n, C.c_void_p(stream)))
            self._grad_ptrs = ptrs
        return any(ptrs)

    def params_moved(self) -> bool:
        return any(p.data_ptr() != q for p, q in zip(self.params, self.param_ptrs))

    def status(self, stream: int) -> None:
        L.check(L.lib().kaon_plan_status(self.handle, C.c_void_p(stream)))

    def set_peers(self, base: int, nbytes: int, deltas: list[int]) -> None:
        """Mirror every weight store of this plan at +delta bytes (other GPUs' copies of the weight buffer)."""
        for p in self.params:
            a = p.data_ptr()
            if not (base <= a and a + p.numel() * p.element_size() <= base + nbytes):
                raise L.KaonError("weight mirrors are set, but a stepped parameter lies outside the mirrored "
                                  "weight buffer")
        arr = (C.c_int64 * max(1, len(deltas)))(*deltas)
        L.check(L.lib().kaon_plan_set_peers(self.handle, arr, len(deltas)))

    def kept_counts(self, stream: int) -> list[int]:
        out = (C.c_uint32 * self.n)()
        L.check(L.lib().kaon_plan_kept_counts(self.handle, out, self.n, C.c_void_p(stream)))
        return list(out)

    def device_bytes(self) -> int:
        return int(L.lib().kaon_plan_device_bytes(self.handle))

    def launches(self) -> int:
        return int(L.lib().kaon_plan_launch_count(self.handle))

    def destroy(self) -> None:
        if self.handle:
            L.lib().kaon_plan_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):  # plans own device memory
        try:
            self.destroy()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass


class FusedStepMixin:
    """Plan cache and step plumbing shared by the optimizer classes.

    Subclasses provide ``_OPT_KIND``, ``_init_state(p, state, group)`` and ``_launch(plan, group, step,
    stream)``.
    """

    _OPT_KIND: int
    _M_KEY = "m"   # state key of the momentum the plan's descriptors name

    def _plan_created(self, plan: GroupPlan, params: list[torch.Tensor], states: list[dict[str, Any]]) -> None:
        """Hook for optimizers whose plan needs more than the descriptor table."""

    def _fused_init(self) -> None:
        self._plans: dict[tuple, GroupPlan] = {}
        self._plan_members: dict[tuple, tuple[int, ...]] = {}
        self._group_buckets: dict[int, tuple] = {}   # per group: (params list, its length, momentum dtype, buckets)
        self._t = 0                 # completed steps; the SR stream uses the 1-based index
        self.sr_seed: int | None = None  # None -> torch.initial_seed() at the first step
        self._mirrors: tuple[int, int, list[int]] | None = None
        # called with the group index before that group's launches: lets a caller order the stream after
        # whatever produces the group's gradients (a per-wave gradient reduce-scatter)
        self.before_group = None
        # called with the group index after that group's launches are enqueued: lets a caller record an
        # event there (the group's weights are final on the stream) and start reading them back
        self.after_group = None
        # multiprocessors the step launches are sized for (None: all); see kaon_plan_set_sm_limit
        self.sm_limit: int | None = None

    def set_weight_mirrors(self, base_ptr: int, nbytes: int, byte_deltas: list[int]) -> None:
        """Fuse the ZeRO-1 publish into the step: every weight written inside
        [base_ptr, base_ptr + nbytes) is also stored at +delta for each delta (the same buffer as mapped
        from the other GPUs).  The caller orders the ranks after the step (``ShardedWeights.publish``)."""
        self._mirrors = (int(base_ptr), int(nbytes), [int(d) for d in byte_deltas]) if byte_deltas else None
        self._invalidate_plans()

    def _invalidate_plans(self) -> None:
        for pl in self._plans.values():
            pl.destroy()
        self._plans.clear()
        self._plan_members.clear()
        self._group_buckets.clear()

    def _seed(self) -> int:
        if self.sr_seed is None:
            self.sr_seed = int(torch.initial_seed()) & 0xFFFFFFFFFFFFFFFF
        return self.sr_seed

    def _tensor_ids(self) -> dict[int, int]:
        ids, i = {}, 0
        for group in self.param_groups:
            for p in group["params"]:
                # a sharded list may pin each tensor's global position so every rank draws the
                # same stochastic-rounding noise for it
                ids[id(p)] = int(getattr(p, "kaon_tensor_id", i))
                i += 1
        return ids

    def _momentum_dtype(self, group: dict[str, Any]) -> str | None:
        return group["momentum_dtype"]

    def _group_plans(self, gi: int, group: dict[str, Any], state_of) -> list[GroupPlan]:
        """Plans covering every parameter of the group that has a gradient now or had one before."""
        params = group["params"]
        fresh = active = False
        for p in params:
            g = p.grad
            if g is None:
                continue
            active = True
            if g.is_sparse:
                raise RuntimeError(f"{type(self).__name__} does not support sparse gradients")
            st = state_of(p)
            if not st:
                self._init_state(p, st, group)
                fresh = True
        if not active:
            return []
        # The buckets of the group (which tensors, in which plan) change only when a tensor gets its first
        # state, the group's list is replaced or resized, the momentum dtype changes or the plans are
        # dropped (load_state_dict, new mirrors): kept between steps, so a step of an unchanged group
        # costs one pass over the gradients.
        md = self._momentum_dtype(group)
        cached = self._group_buckets.get(gi)
        if cached is None or fresh or cached[0] is not params or cached[1] != len(params) or cached[2] != md:
            # tensors stepped now or before (a lookup must not create state for the others); an empty tensor
            # has state, as in the reference, but nothing to step and no address
            members = [p for p in params if p in self.state and state_of(p) and p.numel() > 0]
            buckets: dict[tuple, list[torch.Tensor]] = {}
            for p in members:
                buckets.setdefault((gi, p.device, p.dtype), []).append(p)
            cached = (params, len(params), md,
                      [(key, plist, tuple(id(p) for p in plist) + (md,)) for key, plist in buckets.items()])
            self._group_buckets[gi] = cached
        plans = []
        ids = None
        for key, plist, sig in cached[3]:
            pl = self._plans.get(key)
            if pl is None or fresh or self._plan_members.get(key) != sig or pl.params_moved():
                if pl is not None:
                    pl.destroy()
                if ids is None:
                    ids = self._tensor_ids()
                pl = GroupPlan(self._OPT_KIND, plist, [state_of(p) for p in plist],
                               [ids[id(p)] for p in plist], md, self._M_KEY)
                self._plan_created(pl, plist, [state_of(p) for p in plist])
                if self._mirrors is not None:
                    pl.set_peers(*self._mirrors)
                if self.sm_limit is not None:
                    L.check(L.lib().kaon_plan_set_sm_limit(pl.handle, int(self.sm_limit)))
                self._plans[key] = pl
                self._plan_members[key] = sig
            plans.append(pl)
        return plans

    def _run_groups(self, state_of=None) -> None:
        state_of = state_of or (lambda p: self.state[p])
        self._t += 1
        for gi, group in enumerate(self.param_groups):
            if self.before_group is not None:
                self.before_group(gi)
            for pl in self._group_plans(gi, group, state_of):
                with torch.cuda.device(pl.device):
                    stream = torch.cuda.current_stream(pl.device).cuda_stream
                    if pl.set_grads(stream):
                        self._launch(pl, group, self._t, stream)
            if self.after_group is not None:
                self.after_group(gi)

    # ---- checkpoint extras: the stochastic-rounding stream position ----
    def _extra_state(self, sd: dict[str, Any]) -> dict[str, Any]:
        """Adds the one top-level key the fused step needs for bit-exact resume under stochastic rounding
        (the step index and seed that key the noise).  torch's and the reference's loaders ignore it.
        A checkpoint is not written from state a failed kernel left behind: the device status is checked
        first (one stream synchronisation, which reading the state out needs anyway)."""
        self.check_device_status()
        sd["_kaon_b200"] = {"step": self._t, "sr_seed": self.sr_seed}
        return sd

    def _restore_extra(self, sd: dict[str, Any]) -> dict[str, Any]:
        sd = dict(sd)
        extra = sd.pop("_kaon_b200", None)
        if extra is not None:
            self._t = int(extra.get("step", 0))
            self.sr_seed = extra.get("sr_seed")
        else:
            # a checkpoint written by the reference: the noise stream restarts at step 0; the seed in
            # force (``sr_seed``) is kept
            self._t = 0
        return sd

    def check_device_status(self) -> None:
        """Synchronise and raise if a kernel reported a bounded wait that ran out."""
        for pl in self._plans.values():
            pl.status(torch.cuda.current_stream(pl.device).cuda_stream)

    def stats(self) -> dict[str, int]:
        return {"plans": len(self._plans),
                "plan_device_bytes": sum(pl.device_bytes() for pl in self._plans.values()),
                "kernel_launches": sum(pl.launches() for pl in self._plans.values())}
