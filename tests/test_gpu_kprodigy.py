"""Parity of the CUDA KProdigy step (two passes through the C ABI, the distance estimate on the host between
them) with the reference's golden vectors (reference src/kaon/kprodigy.py:299-949) and with the oracle.

Every step starts from the reference's state after the step before (weights, per-tensor state, the group's
d / d_max / d_numerator / k): the estimate feeds on p0 - p, so one stochastic-rounding draw or one
cautious-mask bit that differs moves every later step by a per cent or so, in the reference's own trajectory
as much as here.  The gates are those of the oracle's test (tests/test_oracle_golden.py)."""
import numpy as np
import pytest
import torch

import kaon_oracle as ko
from _golden import Fixture, rel_err
from golden.cases import CASES
from test_oracle_golden import _kprodigy_check, kprodigy_force

pytestmark = pytest.mark.gpu

KP_CASES = [n for n in CASES if n.startswith("kprodigy_")]


def _to_tensor(want: np.ndarray, like: torch.Tensor) -> torch.Tensor:
    if like.dtype == torch.bfloat16:
        t = torch.from_numpy(want.view(np.int16).copy()).view(torch.bfloat16)
    else:
        t = torch.from_numpy(want.copy())
        assert t.dtype == like.dtype, (t.dtype, like.dtype)
    return t.reshape(like.shape).to(like.device)


@pytest.mark.parametrize("name", KP_CASES)
def test_kprodigy_matches_reference_step_by_step(name):
    import kaon_b200
    from _gpu import from_bits, state_np, to_bits
    opt_name, kw, shapes, dtype, steps, seed, o = CASES[name]
    f = Fixture(name)
    params = [torch.nn.Parameter(from_bits(b, s)) for b, s in zip(f.params(), shapes)]
    opt = kaon_b200.KProdigy(params, **kw)
    opt.sr_seed = 0

    def set_weights(i, bits):
        with torch.no_grad():
            params[i].copy_(from_bits(bits, shapes[i]))

    def set_state(i, key, want):
        st = opt.state[params[i]]
        if key == "p0" and want.ndim == 0:
            assert st[key].ndim == 0
            return
        st[key].copy_(_to_tensor(want, st[key]))

    def steps_of():
        for step in range(1, steps + 1):
            if step > 1:
                kprodigy_force(f, step - 1, opt.param_groups[0], len(shapes), set_weights, set_state)
            for p, gb, s in zip(params, f.grads(step), shapes):
                p.grad = from_bits(gb, s)
            opt.step()
            torch.cuda.synchronize()
            opt.check_device_status()
            yield step, f

    def tensor_state(i):
        st = opt.state[params[i]]
        return {k: (state_np(st, k) if torch.is_tensor(v) else v) for k, v in st.items()}

    _kprodigy_check(name, steps_of, lambda: opt.param_groups[0], tensor_state, lambda i: to_bits(params[i]),
                    lambda i: state_np(opt.state[params[i]], "shift"))


BIG = [(640, 2560), (320, 320, 3, 3), (1280,), (333, 77), (3, 16384), (4000, 3), (7,), (50000,)]


@pytest.mark.parametrize("kw", [
    dict(),
    dict(momentum_dtype="int8", second_moment="factored", cautious=True, weight_decay=0.01),
    dict(momentum_dtype="4bit", slice_p=11, bf16_method="none"),
    dict(betas=(0.0, 0.999), weight_decay=0.02, decouple=False),
    dict(betas=(0.0, 0.999), second_moment="factored", weight_decay=0.02),
    dict(momentum_dtype="float32", gradient_centralization=False, use_bias_correction=True, bf16_method="kahan"),
])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_kprodigy_vs_oracle_bigger_shapes(kw, dtype):
    """Ragged and wide shapes, a long 1-D tensor, a steady gradient direction so that d grows; every step both
    sides start from the same weights and state (the CUDA side's), and one step is compared."""
    import kaon_b200
    from _gpu import state_np, to_bits
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(21)
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in BIG]
    base = [torch.randn(s, generator=gen) * 1e-3 for s in BIG]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    # a steady direction at lr = 1 would let d jump by orders of magnitude, and without bias correction the
    # first Adam-style steps are 1/sqrt(1 - beta2) = 32 times lr
    kw = dict(kw, growth_rate=3.0, lr=0.05)
    opt = kaon_b200.KProdigy(params, **kw)
    opt.sr_seed = 4
    orc = ko.OracleKProdigy([to_bits(h) for h in host], BIG, seed=4, **kw)
    md = kw.get("momentum_dtype", "bfloat16") if kw.get("betas", (0.9, 0.999))[0] > 0 else None
    for step in range(1, 7):
        grads = [(b + torch.randn(s, generator=gen) * 3e-4).to(tdt) for b, s in zip(base, BIG)]
        if step > 1:   # the oracle restarts from the CUDA side's state
            grp = opt.param_groups[0]
            orc.group.update(d=grp["d"], d_max=grp["d_max"], d_numerator=grp["d_numerator"], k=grp["k"])
            for i, p in enumerate(params):
                ot, st = orc.tensors[i], opt.state[p]
                ot.p[...] = to_bits(p)
                for key, val in st.items():
                    if torch.is_tensor(val) and val.ndim > 0:
                        ot.state[key][...] = state_np(st, key).reshape(ot.state[key].shape)
        for p, g in zip(params, grads):
            p.grad = g.clone().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        orc.t = opt._t - 1
        orc.step([to_bits(g) for g in grads])
        grp = opt.param_groups[0]
        for key in ("d", "d_max", "d_numerator"):
            assert abs(grp[key] - orc.group[key]) <= 5e-5 * abs(orc.group[key]) + 1e-30, (step, key, grp[key], orc.group[key])
        for i, p in enumerate(params):
            st, ot = opt.state[p], orc.tensors[i]
            for key in ("s", "v", "row", "col"):
                if key in ot.state:
                    want = ot.state[key]
                    np.testing.assert_allclose(state_np(st, key), want, rtol=5e-5, atol=5e-5 * float(np.abs(want).max()),
                                               err_msg=f"{step} {i} {key} {BIG[i]}")
            if md in ("int8", "4bit"):
                assert rel_err(state_np(st, "m_scale"), ot.state["m_scale"]) <= 5e-5, (step, i)
                got_m, want_m = state_np(st, "m"), ot.state["m"]
                if md == "int8":
                    dd = np.abs(got_m.view(np.int8).astype(np.int32) - want_m.view(np.int8).astype(np.int32))
                else:
                    g8, w8 = got_m.view(np.uint8), want_m.view(np.uint8)
                    dd = np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)), np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))
                assert dd.max() <= 1 and np.mean(dd != 0) < 5e-3, (step, i, BIG[i])
            elif md == "bfloat16":
                assert np.mean(state_np(st, "m") != ot.state["m"]) < 2e-3, (step, i, BIG[i])
            elif md == "float32":
                want_m = ot.state["m"]
                np.testing.assert_allclose(state_np(st, "m"), want_m, rtol=5e-5, atol=5e-5 * float(np.abs(want_m).max()))
            got, want = to_bits(p), ot.p
            if dtype == "bf16":
                assert np.mean(got != want) < 3e-2, (step, i, BIG[i], float(np.mean(got != want)))
                a, b = ko.as_f32(got).astype(np.float64), ko.as_f32(want).astype(np.float64)
                assert (np.abs(a - b) <= 2.0 ** -6 * np.maximum(np.abs(b), 1e-3)).all(), (step, i, BIG[i])
            else:
                # an element whose second moment sits at the d*eps floor moves by g*lr/eps: the fp32 noise of a
                # centralised gradient near zero shows there and nowhere else
                bad = np.abs(got - want) > 1e-5 * np.abs(want) + 1e-5 * float(np.abs(want).mean())
                assert bad.sum() <= max(16, 5e-4 * bad.size), (step, i, BIG[i], int(bad.sum()))
                np.testing.assert_allclose(got, want, rtol=1e-3, atol=1e-5 * float(np.abs(want).max()))


def test_kprodigy_constructor_errors_and_resume():
    import copy
    import kaon_b200
    p = [torch.nn.Parameter(torch.zeros(4, 4, device="cuda"))]
    for kw, msg in ((dict(d0=0.0), "d0 must be > 0"), (dict(lr=0.0), "lr must be > 0"), (dict(slice_p=0), "slice_p must be >= 1"),
                    (dict(second_moment="x"), "second_moment must be full/factored"), (dict(d_update_freq=0), "d_update_freq")):
        with pytest.raises(ValueError, match=msg):
            kaon_b200.KProdigy(p, **kw)
    shapes = [(64, 96), (130,), (8, 4, 3, 3)]

    def build():
        gen = torch.Generator().manual_seed(3)
        ps = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).bfloat16().cuda()) for s in shapes]
        o = kaon_b200.KProdigy(ps, momentum_dtype="4bit", second_moment="factored", slice_p=3)
        o.sr_seed = 11
        return ps, o

    gen = torch.Generator().manual_seed(77)
    base = [torch.randn(s, generator=gen) * 1e-3 for s in shapes]
    grads = [[(b + torch.randn(s, generator=gen) * 3e-4).bfloat16().cuda() for b, s in zip(base, shapes)] for _ in range(6)]

    def run(ps, o, ks):
        for k in ks:
            for q, g in zip(ps, grads[k]):
                q.grad = g
            o.step()
        torch.cuda.synchronize()

    pa, oa = build()
    run(pa, oa, range(6))
    pb, ob = build()
    run(pb, ob, range(4))
    sd = copy.deepcopy(ob.state_dict())
    assert {"step", "s", "p0", "m", "m_scale", "row", "col"} <= set(sd["state"][0])
    assert sd["param_groups"][0]["k"] == 4 and sd["param_groups"][0]["d"] == ob.get_d()
    pc, oc = build()
    with torch.no_grad():
        for q, w in zip(pc, pb):
            q.copy_(w)
    oc.load_state_dict(sd)
    run(pc, oc, range(4, 6))
    assert oc.get_d() == oa.get_d()
    for a, c in zip(pa, pc):
        assert torch.equal(a.view(torch.int16), c.view(torch.int16))
