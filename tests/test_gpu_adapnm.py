"""Parity of the CUDA AdaPNM step (through the C ABI) with the reference's golden vectors and the CPU
oracle (reference src/kaon/adapnm.py:599-645, 1039-1273).

The momenta depend on the gradient only (and on the centralisation row mean when that is on): without
centralisation they are compared bit for bit.  Everything downstream of the row / column means and of
the clip rms carries the usual gates: statistics rel <= 1e-5, quantised codes within one level with a
small flip rate, weights within one bf16 ulp ("none") or one ulp per stochastic write."""
import copy

import numpy as np
import pytest
import torch

import kaon_oracle as ko
from _golden import rel_err, sr_close, ulp_diff_bf16
from golden.cases import CASES

pytestmark = pytest.mark.gpu

PNM_CASES = [n for n in CASES if n.startswith("adapnm_")]


def _code_diff(md, got, want):
    if md == "int8":
        return np.abs(got.view(np.int8).astype(np.int32) - want.view(np.int8).astype(np.int32))
    g8, w8 = got.view(np.uint8), want.view(np.uint8)
    return np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)), np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))


def _check_momenta(md, st, want_of, exact, where):
    """Both stored momenta against `want_of(key)`; returns (flipped codes, codes)."""
    from _gpu import state_np
    flips = total = 0
    for mk in ("m_pos", "m_neg"):
        got, want = state_np(st, mk), want_of(mk)
        assert want is not None, (where, mk)
        if md in ("int8", "4bit"):
            gs, ws = state_np(st, f"{mk}_scale"), want_of(f"{mk}_scale").reshape(-1)
            if exact:
                assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), (where, mk)
                assert np.array_equal(gs, ws), (where, mk)
            else:
                assert rel_err(gs, ws) <= 2e-5, (where, mk, rel_err(gs, ws))
                d = _code_diff(md, got, want)
                assert d.max() <= 1, (where, mk, int(d.max()))
                flips += int((d != 0).sum()); total += d.size
        elif md == "bfloat16":
            # one bf16 ulp; an element whose stored value flipped by an ulp one step earlier and whose EMA
            # all but cancels now may be further away in ulps, never in magnitude
            ud = ulp_diff_bf16(got, want)
            if exact:
                assert ud.max() == 0, (where, mk)
            else:
                a, b = ko.as_f32(got).astype(np.float64), ko.as_f32(want).astype(np.float64)
                assert np.mean(ud > 1) < 1e-5, (where, mk, int((ud > 1).sum()))
                assert (np.abs(a - b) <= 2.0 ** -7 * np.maximum(np.abs(b), 1e-4)).all(), (where, mk)
        else:
            if exact:
                assert np.array_equal(got, want.reshape(-1)), (where, mk)
            else:
                np.testing.assert_allclose(got, want.reshape(-1), rtol=1e-5, atol=1e-12)
    return flips, total


@pytest.mark.parametrize("name", PNM_CASES)
def test_adapnm_matches_reference(name):
    from _gpu import run_case_gpu, state_np, to_bits
    kw = CASES[name][1]
    md = kw.get("momentum_dtype", "bfloat16")
    method = kw.get("bf16_method", "stochastic_rounding")
    exact = not kw.get("gradient_centralization", True)
    flips = total = 0
    for step, f, opt, params in run_case_gpu(name):
        assert opt.param_groups[0]["step"] == step
        for i, p in enumerate(params):
            st = opt.state[p]
            for key in ("row", "col", "v", "max_v"):
                want = f.state(step, i, key)
                if want is not None:
                    assert rel_err(state_np(st, key), want) <= 1e-5, (step, i, key, rel_err(state_np(st, key), want))
                    if exact and key in ("v", "max_v"):
                        assert np.array_equal(state_np(st, key), want.reshape(-1)), (step, i, key)
            fl, to = _check_momenta(md, st, lambda k: f.state(step, i, k), exact, (step, i))
            flips += fl; total += to
            got, want = to_bits(p), f.weights(step, i)
            if want.dtype == np.uint16:
                if method == "stochastic_rounding":
                    assert sr_close(got, want, step, 1e-3), (step, i)
                elif method == "kahan":
                    a = ko.as_f32(got).astype(np.float64) + ko.as_f32(state_np(st, "shift"))
                    b = ko.as_f32(want).astype(np.float64) + ko.as_f32(f.state(step, i, "shift"))
                    ulp = np.maximum(np.abs(ko.as_f32(want)), 1e-30) * 2.0 ** -7
                    assert (np.abs(a - b) <= 1.0 * ulp).all(), (step, i)
                else:
                    assert ulp_diff_bf16(got, want).max() <= 1, (step, i)
            else:
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)
    if total:
        assert flips / total < 2e-3, (flips, total)


# ragged and wide shapes, rows longer than a work item, a long 1-D tensor
BIG = [(640, 2560), (320, 320, 3, 3), (1280,), (333, 77), (3, 16384), (4000, 3), (7,), (96, 4100), (50000,),
       (16, 2560, 3, 3)]


@pytest.mark.parametrize("md,wd,method,extra", [
    ("int8", 0.0, "stochastic_rounding", {}),
    ("4bit", 0.1, "none", {"beta0": 1.0}),
    ("bfloat16", 0.01, "stochastic_rounding", {"clip_threshold": 0.0}),
    ("float32", 0.0, "none", {"ams_bound": True, "cautious": False, "gradient_centralization": False}),
    ("int8", 0.05, "kahan", {"betas": (0.9, 0.99)}),
    ("4bit", 0.0, "none", {"momentum_4bit_block": 64}),
    ("4bit", 0.0, "stochastic_rounding", {"momentum_4bit_block": 256}),
])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_adapnm_vs_oracle_bigger_shapes(md, wd, method, extra, dtype):
    import kaon_b200
    from _gpu import state_np, to_bits
    shapes = BIG if dtype == "bf16" else BIG[:-1]   # rows of 23040 elements: bf16 weights only
    if md == "4bit":   # rows of 4100 elements cannot be grouped on 128-element block boundaries within a work item
        shapes = [s for s in shapes if s != (96, 4100)]
    if extra.get("momentum_4bit_block") == 256:   # nor rows of 77 elements on 256-element boundaries
        shapes = [s for s in shapes if s != (333, 77)]
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(9)
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in shapes]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=1e-4, weight_decay=wd, bf16_method=method, momentum_dtype=md, **extra)
    opt = kaon_b200.AdaPNM(params, **kw)
    opt.sr_seed = 4
    orc = ko.OracleAdaPNM([to_bits(h) for h in host], shapes, seed=4, **kw)
    exact = not kw.get("gradient_centralization", True)
    flips = total = 0
    for step in range(1, 5):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(tdt) for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.clone().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        orc.step([to_bits(g) for g in grads])
        (plan,) = opt._plans.values()
        kept = plan.kept_counts(torch.cuda.current_stream().cuda_stream)
        for i, p in enumerate(params):
            st, ot = opt.state[p], orc.tensors[i]
            for key in ("row", "col", "v", "max_v"):
                if key in ot.state:
                    assert rel_err(state_np(st, key), ot.state[key]) <= 1e-5, (step, i, key, shapes[i])
            if kw.get("cautious", True):
                assert abs(kept[i] - orc.kept[i]) <= max(4, 2e-3 * ot.n), (step, i, kept[i], orc.kept[i])
            fl, to = _check_momenta(md, st, lambda k: ot.state[k], exact, (step, i, shapes[i]))
            flips += fl; total += to
            got, want = to_bits(p), ot.p
            if dtype == "bf16":
                if method == "kahan":
                    a = ko.as_f32(got).astype(np.float64) + ko.as_f32(state_np(st, "shift"))
                    b = ko.as_f32(want).astype(np.float64) + ko.as_f32(ot.state["shift"])
                    ulp = np.maximum(np.abs(ko.as_f32(want)), 1e-30) * 2.0 ** -7
                    assert np.mean(np.abs(a - b) > ulp) < 5e-3, (step, i, shapes[i])
                else:
                    assert np.mean(got != want) < 5e-3, (step, i, shapes[i], np.mean(got != want))
            else:
                bad = np.abs(got - want) > 2e-5 * np.abs(want) + 1e-9
                assert bad.mean() < 1e-4 and np.abs(got - want).max() < 3e-4, (step, i, shapes[i], bad.sum())
    if total:
        assert flips / total < 2e-3, (flips, total)


def test_adapnm_resume_is_bit_exact():
    """state_dict -> a fresh optimizer -> the same weights and state as the uninterrupted run
    (reference tests/test_adapnm.py resume tests; the layout is the reference's)."""
    import kaon_b200
    shapes = [(64, 96), (8, 4, 3, 3), (130,), (40, 256)]

    def build(seed=3):
        gen = torch.Generator().manual_seed(seed)
        ps = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).bfloat16().cuda()) for s in shapes]
        o = kaon_b200.AdaPNM(ps, lr=1e-4, momentum_dtype="4bit", weight_decay=0.01)
        o.sr_seed = 11
        return ps, o

    gen = torch.Generator().manual_seed(77)
    grads = [[(torch.randn(s, generator=gen) * 1e-3).bfloat16().cuda() for s in shapes] for _ in range(5)]

    def run(ps, o, ks):
        for k in ks:
            for p, g in zip(ps, grads[k]):
                p.grad = g
            o.step()
        torch.cuda.synchronize()

    pa, oa = build()
    run(pa, oa, range(5))
    pb, ob = build()
    run(pb, ob, range(3))
    sd = copy.deepcopy(ob.state_dict())
    st0 = sd["state"][0]
    assert {"row", "col", "m_pos", "m_pos_scale", "m_pos_numel", "m_pos_block", "m_neg", "m_neg_scale",
            "m_neg_numel", "m_neg_block"} <= set(st0), sorted(st0)
    assert sd["param_groups"][0]["step"] == 3
    pc, oc = build()
    with torch.no_grad():
        for q, p in zip(pc, pb):
            q.copy_(p)
    oc.load_state_dict(sd)
    run(pc, oc, range(3, 5))
    for a, c in zip(pa, pc):
        assert torch.equal(a.view(torch.int16), c.view(torch.int16))
    for a, c in zip(pa, pc):
        for key, va in oa.state[a].items():
            vc = oc.state[c][key]
            assert torch.equal(va, vc) if torch.is_tensor(va) else va == vc, key


def test_adapnm_constructor_errors_match_reference():
    import kaon_b200
    p = [torch.nn.Parameter(torch.zeros(4, 4, device="cuda"))]
    for kw, msg in ((dict(betas=(1.0, 0.9)), r"betas\[0\] must be in \[0, 1\)"), (dict(beta0=1.5), r"beta0 must be in \[0, 1\]"),
                    (dict(eps=-1.0), "eps must be >= 0"), (dict(clip_threshold=-1.0), "clip_threshold must be >= 0"),
                    (dict(momentum_dtype="fp8"), "momentum_dtype must be"), (dict(bf16_method="x"), "bf16_method must be")):
        with pytest.raises(ValueError, match=msg):
            kaon_b200.AdaPNM(p, **kw)
