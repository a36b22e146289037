"""Pin the CPU oracle against vectors produced by the reference itself (tests/golden/*.npz).

Gates (per stage; the reference's order-dependent fp32 reductions cannot be matched bit for bit):
  * codec, SR formula, Lion without GC: bit-exact.
  * anything after a GC row mean / row-col mean / norm: statistics rel <= 1e-5, quantised codes may
    flip by one level on a small fraction, weights within 1 bf16 ulp.
  * Newton-Schulz: the reference's own tolerance rtol=2e-2 (reference tests/test_adamuon.py:109).
"""
import numpy as np
import pytest

import kaon_oracle as ko
from _golden import Fixture, rel_err, sr_close, ulp_diff_bf16
from golden.cases import CASES, SCHEDULES

ORACLES = {"Lion": ko.OracleLion, "Adakaon": ko.OracleAdakaon, "Nekaon": ko.OracleNekaon,
           "AdaMuon": ko.OracleAdaMuon, "AdaPNM": ko.OracleAdaPNM, "KProdigy": ko.OracleKProdigy}


def test_philox_known_answers():
    # Random123 known-answer vectors for Philox4x32-10: they pin the round function and the key schedule;
    # the stochastic-rounding stream runs the same function for seven rounds
    assert [hex(x) for x in ko.philox4x32([0] * 4, [0] * 2)] == ["0x6627e8d5", "0xe169c58d", "0xbc57ac4c", "0x9b00dbd8"]
    assert [hex(x) for x in ko.philox4x32([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2)] == ["0x408f276d", "0x41c83b0e", "0xa20bc7c6", "0x6d5451fd"]
    assert [hex(x) for x in ko.philox4x32([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0])] == ["0xd16cfe09", "0x94fdcceb", "0x5001e420", "0x24126ea1"]


def test_codec_bit_exact():
    f = Fixture("codec")
    for key, rows in (("a", 37), ("b", 0), ("c", 4)):
        codes, scale = ko.encode_int8(f[f"int8_{key}_in"], rows)
        assert np.array_equal(codes, f[f"int8_{key}_codes"])
        assert np.array_equal(scale, f[f"int8_{key}_scale"])
        assert np.array_equal(ko.decode_int8(codes, scale, rows), f[f"int8_{key}_dec"])
        assert codes.min() >= -127
    for n in (1000, 77, 256, 1, 129):
        packed, scale = ko.encode_4bit(f[f"q4_{n}_in"], 128)
        assert np.array_equal(packed, f[f"q4_{n}_packed"])
        assert np.array_equal(scale, f[f"q4_{n}_scale"])
        assert np.array_equal(ko.decode_4bit(packed, scale, n, 128), f[f"q4_{n}_dec"])


def test_fresh_4bit_state_decodes_to_zero():
    t = ko.OracleTensor(np.zeros(300, np.float32), (300,))
    t.init_momentum("4bit", 128)
    assert np.all(t.state["m"] == 0x88) and np.all(t.decoded_m("4bit") == 0.0)


def test_gradient_centralization():
    f = Fixture("gc")
    for key, rows in (("bf16_2d", 24), ("bf16_conv", 6), ("f32_2d", 24)):
        got = ko.centralize(f[f"{key}_in"], rows)
        want = f[f"{key}_out"]
        if want.dtype == np.uint16:
            assert np.array_equal(ko.f32_to_bf16_bits(got), want)
        else:
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)


def test_stochastic_rounding_formula_bit_exact():
    f = Fixture("sr")
    for alpha in (-1.0, 1.0):
        p = f["p_in"].copy()
        ko.write(p, f["delta"], alpha, ko.W_SR_NOISE, noise=f[f"noise_a{alpha:+.0f}"])
        assert np.array_equal(p, f[f"p_out_a{alpha:+.0f}"])


def test_newton_schulz():
    f = Fixture("ns")
    for key, shape in (("sq", (48, 48)), ("tall", (96, 32)), ("wide", (32, 80))):
        got = ko.newton_schulz(f[f"{key}_in"].reshape(shape), 2)
        np.testing.assert_allclose(got, f[f"{key}_out"].reshape(shape), rtol=2e-2, atol=2e-2)


def _run_oracle(name):
    opt_name, kw, shapes, dtype, steps, seed, o = CASES[name]
    f = Fixture(name)
    opt = ORACLES[opt_name](f.params(), shapes, **kw)
    sched = SCHEDULES.get(o.get("lr_sched"))
    for step in range(1, steps + 1):
        if sched is not None:
            opt.hp["lr"] = sched(step - 1)
        opt.step(f.grads(step))
        yield step, f, opt


def _check_state(f, opt, step, *, exact, md, mkeys=("m",)):
    """Compare every tensor's state with the fixture; returns (flipped codes, total codes)."""
    flips = total = 0
    for mk in mkeys:
        fl, to = _check_state_one(f, opt, step, exact=exact, md=md, mk=mk)
        flips += fl
        total += to
    return flips, total


def _check_state_one(f, opt, step, *, exact, md, mk):
    flips = total = 0
    for i, t in enumerate(opt.tensors):
        for key in ("row", "col", "v", "max_v"):
            want = f.state(step, i, key)
            if want is None:
                continue
            if exact:
                assert np.array_equal(t.state[key], want), (step, i, key)
            else:
                assert rel_err(t.state[key], want) <= 1e-5, (step, i, key, rel_err(t.state[key], want))
        want_m = f.state(step, i, mk)
        if want_m is None:
            continue
        got_m = t.state[mk]
        want_sc = f.state(step, i, f"{mk}_scale")
        if md in ("int8", "4bit"):
            if exact:
                assert np.array_equal(got_m.view(np.uint8), want_m.view(np.uint8)), (step, i)
                assert np.array_equal(t.state[f"{mk}_scale"], want_sc.reshape(-1)), (step, i)
            else:
                assert rel_err(t.state[f"{mk}_scale"], want_sc.reshape(-1)) <= 1e-5
                if md == "int8":
                    d = np.abs(got_m.astype(np.int32) - want_m.view(np.int8).astype(np.int32))
                else:
                    g8, w8 = got_m.view(np.uint8), want_m.view(np.uint8)
                    d = np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)),
                                   np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))
                assert d.max() <= 1, (step, i, d.max())
                flips += int((d != 0).sum())
                total += d.size
        elif md == "bfloat16":
            assert ulp_diff_bf16(got_m, want_m).max() <= (0 if exact else 1)
    return flips, total


def test_lion_fp32_grads_with_gc():
    """fp32 grads: the GC mean is not rounded to bf16, so the summation-order difference of ~1 ulp
    reaches the momentum; state agrees to 1e-5, codes flip by at most one level."""
    flips = total = 0
    for step, f, opt in _run_oracle("lion_4bit_f32params"):
        fl, to = _check_state(f, opt, step, exact=False, md="4bit")
        flips, total = flips + fl, total + to
        for i, t in enumerate(opt.tensors):
            np.testing.assert_allclose(t.p, f.weights(step, i), rtol=0, atol=2.1 * 2e-4 / 0.3)
            assert np.mean(t.p != f.weights(step, i)) < 5e-3
    assert flips / total < 2e-3, (flips, total)


@pytest.mark.parametrize("name", ["lion_4bit_nogc_wd", "lion_4bit_none", "lion_int8_none",
                                  "lion_bf16_nocautious", "lion_4bit_block64", "lion_4bit_long"])
def test_lion_bit_exact(name):
    """Lion has no order-dependent reduction except the GC row mean; on these vectors the oracle's
    double-accumulated mean rounds to the same bf16 as torch's, so everything is bit-exact."""
    md = CASES[name][1]["momentum_dtype"]
    for step, f, opt in _run_oracle(name):
        _check_state(f, opt, step, exact=True, md=md)
        for i, t in enumerate(opt.tensors):
            want = f.weights(step, i)
            if want.dtype == np.uint16:
                assert np.array_equal(t.p, want), (step, i)
            else:
                # fp32 params: p - delta is one rounding, same on both sides
                assert np.array_equal(t.p, want), (step, i)


@pytest.mark.parametrize("name", ["lion_4bit_kahan", "lion_int8_kahan_wd_nocautious"])
def test_lion_kahan_bit_exact(name):
    """bf16_method="kahan": weights AND the compensation buffer state["shift"] match the reference bit
    for bit (reference src/kaon/_backend.py:89-94)."""
    md = CASES[name][1]["momentum_dtype"]
    for step, f, opt in _run_oracle(name):
        _check_state(f, opt, step, exact=True, md=md)
        for i, t in enumerate(opt.tensors):
            assert np.array_equal(t.p, f.weights(step, i)), (step, i)
            assert np.array_equal(t.state["shift"], f.state(step, i, "shift")), (step, i)


def _kahan_close(p, shift, want_p, want_shift, tol_ulp=1.0):
    """Weights within one bf16 ulp, and the compensated value p + shift within `tol_ulp` ulps of p."""
    if ulp_diff_bf16(p, want_p).max() > 1:
        return False
    a = ko.as_f32(p).astype(np.float64) + ko.as_f32(shift)
    b = ko.as_f32(want_p).astype(np.float64) + ko.as_f32(want_shift)
    ulp = np.maximum(np.abs(ko.as_f32(want_p)), 1e-30) * 2.0 ** -7
    return bool((np.abs(a - b) <= tol_ulp * ulp).all())


def test_adakaon_kahan():
    flips = total = 0
    for step, f, opt in _run_oracle("adakaon_int8_kahan"):
        fl, to = _check_state(f, opt, step, exact=False, md="int8")
        flips += fl
        total += to
        for i, t in enumerate(opt.tensors):
            assert _kahan_close(t.p, t.state["shift"], f.weights(step, i), f.state(step, i, "shift")), (step, i)
    assert flips / total < 2e-3


def test_adamuon_kahan():
    for step, f, opt in _run_oracle("adamuon_int8_kahan"):
        for i, t in enumerate(opt.tensors):
            np.testing.assert_allclose(ko.as_f32(t.p), ko.as_f32(f.weights(step, i)), rtol=2e-2, atol=2e-3)
            assert "shift" in t.state and f.state(step, i, "shift") is not None


def test_lion_sr_state_is_weight_independent():
    """Under stochastic rounding the weights differ (different RNG) but no state depends on them."""
    for step, f, opt in _run_oracle("lion_4bit_sr"):
        _check_state(f, opt, step, exact=True, md="4bit")
        for i, t in enumerate(opt.tensors):
            assert sr_close(t.p, f.weights(step, i), step, 1e-3)


@pytest.mark.parametrize("name", ["adakaon_int8_none", "adakaon_int8_sr", "adakaon_int8_outlier",
                                  "adakaon_4bit_wd_f32", "adakaon_bf16m_none", "adakaon_4bit_block256_wd",
                                  "adakaon_4bit_block32_f32", "adakaon_int8_long"])
def test_adakaon(name):
    md = CASES[name][1]["momentum_dtype"]
    sr = CASES[name][1].get("bf16_method", "stochastic_rounding") == "stochastic_rounding"
    flips = total = 0
    for step, f, opt in _run_oracle(name):
        fl, to = _check_state(f, opt, step, exact=False, md=md)
        flips += fl
        total += to
        for i, t in enumerate(opt.tensors):
            want = f.weights(step, i)
            if want.dtype == np.uint16:
                if sr:
                    assert sr_close(t.p, want, step, 1e-3), (step, i)
                else:
                    assert ulp_diff_bf16(t.p, want).max() <= 1, (step, i)
            else:
                np.testing.assert_allclose(t.p, want, rtol=1e-5, atol=1e-9)
    if total:
        assert flips / total < 2e-3, (flips, total)


@pytest.mark.parametrize("name", [n for n in CASES if n.startswith("adapnm_") and "kahan" not in n])
def test_adapnm(name):
    """reference src/kaon/adapnm.py: two momenta (only the positive one sees the gradient, the roles
    alternate), Adakaon's factored second moment, RMS clip of the mixed update."""
    kw = CASES[name][1]
    md = kw.get("momentum_dtype", "bfloat16")
    sr = kw.get("bf16_method", "stochastic_rounding") == "stochastic_rounding"
    exact = not kw.get("gradient_centralization", True)   # without a row mean upstream the momenta are exact
    flips = total = 0
    for step, f, opt in _run_oracle(name):
        fl, to = _check_state_one(f, opt, step, exact=False, md=md, mk="m_pos")
        fl2, to2 = _check_state_one(f, opt, step, exact=False, md=md, mk="m_neg")
        flips += fl + fl2
        total += to + to2
        for i, t in enumerate(opt.tensors):
            if exact and "v" in t.state:   # the 1-D second moment (and its running maximum) bit for bit
                assert np.array_equal(t.state["v"], f.state(step, i, "v")), (step, i)
                if "max_v" in t.state:
                    assert np.array_equal(t.state["max_v"], f.state(step, i, "max_v")), (step, i)
            if md == "float32":
                for mk in ("m_pos", "m_neg"):
                    want = f.state(step, i, mk)
                    if exact:
                        assert np.array_equal(t.state[mk], want), (step, i, mk)
                    else:
                        np.testing.assert_allclose(t.state[mk], want, rtol=1e-5, atol=1e-12)
            want = f.weights(step, i)
            if want.dtype == np.uint16:
                if sr:
                    assert sr_close(t.p, want, step, 1e-3), (step, i)
                else:
                    assert ulp_diff_bf16(t.p, want).max() <= 1, (step, i)
            else:
                np.testing.assert_allclose(t.p, want, rtol=1e-5, atol=1e-9)
    if total:
        assert flips / total < 2e-3, (flips, total)


def test_adapnm_kahan():
    flips = total = 0
    for step, f, opt in _run_oracle("adapnm_int8_kahan"):
        fl, to = _check_state(f, opt, step, exact=False, md="int8", mkeys=("m_pos", "m_neg"))
        flips += fl
        total += to
        for i, t in enumerate(opt.tensors):
            assert _kahan_close(t.p, t.state["shift"], f.weights(step, i), f.state(step, i, "shift")), (step, i)
    assert flips / total < 2e-3


def _kprodigy_check(name, steps_of, group_of, tensor_state, weights_of, shift_of):
    """Shared by the oracle test here and the CUDA test: compare a KProdigy run, every step of which starts
    from the reference's state (kprodigy_force), with its fixture."""
    kw = CASES[name][1]
    md = kw.get("momentum_dtype", "bfloat16") if kw.get("betas", (0.9, 0.999))[0] > 0 else None
    method = kw.get("bf16_method", "stochastic_rounding")
    flips = total = 0
    for step, f in steps_of():
        grp = group_of()
        for key in ("d", "d_max", "d_numerator"):
            want = float(f[f"grp_s{step}_{key}"])
            assert abs(grp[key] - want) <= 5e-5 * abs(want) + 1e-30, (step, key, grp[key], want)
        assert grp["k"] == int(f[f"grp_s{step}_k"])
        for i in range(len(f.shapes)):
            st = tensor_state(i)
            for key in ("s", "v", "row", "col"):
                want = f.state(step, i, key)
                if want is not None:
                    # d itself is only good to ~1e-5 (a sum over all tensors), s mixes terms of both signs, and
                    # a centralised fp32 gradient close to zero carries the row mean's rounding
                    np.testing.assert_allclose(st[key], want.reshape(-1), rtol=5e-5,
                                               atol=5e-5 * float(np.abs(want).max()), err_msg=f"{step} {i} {key}")
            assert np.array_equal(np.asarray(st["p0"]).reshape(-1), f.state(step, i, "p0").reshape(-1))
            assert int(st["step"]) == int(f.state(step, i, "step"))
            if md in ("int8", "4bit"):
                want_m, got_m = f.state(step, i, "m"), st["m"]
                assert rel_err(st["m_scale"], f.state(step, i, "m_scale").reshape(-1)) <= 5e-5, (step, i)
                if md == "int8":
                    dd = np.abs(got_m.view(np.int8).astype(np.int32) - want_m.view(np.int8).astype(np.int32))
                else:
                    g8, w8 = got_m.view(np.uint8), want_m.view(np.uint8)
                    dd = np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)),
                                    np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))
                assert dd.max() <= 1, (step, i, int(dd.max()))
                flips += int((dd != 0).sum())
                total += dd.size
            elif md == "bfloat16":
                assert np.mean(ulp_diff_bf16(st["m"], f.state(step, i, "m")) > 1) < 1e-3, (step, i)
            elif md == "float32":
                want_m = f.state(step, i, "m").reshape(-1)
                np.testing.assert_allclose(st["m"], want_m, rtol=5e-5, atol=5e-5 * float(np.abs(want_m).max()))
            got, want = weights_of(i), f.weights(step, i)
            if want.dtype == np.uint16:
                if method == "stochastic_rounding":
                    assert sr_close(got, want, 1, 1e-3), (step, i)   # one write since the forced state
                elif method == "kahan":
                    assert _kahan_close(got, shift_of(i), want, f.state(step, i, "shift"), tol_ulp=2.0), (step, i)
                else:
                    # one ulp, except where a cautious-mask bit flipped (terms of both signs that all but
                    # cancel): such an element is off by one masked update, far below 1e-4; a 4-bit code one level off does the same
                    ud = ulp_diff_bf16(got, want)
                    assert (ud > 1).sum() <= max(2, 5e-3 * ud.size) and (ud > 0).sum() <= max(3, 3e-2 * ud.size), (step, i)
                    assert np.abs(ko.as_f32(got).astype(np.float64) - ko.as_f32(want)).max() < 1e-4, (step, i)
            else:
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-8)
    if total:
        assert flips / total < 5e-3, (flips, total)


def kprodigy_force(f, step, group, n_tensors, set_weights, set_state):
    """Put an implementation into the reference's state after `step` (weights, per-tensor state, the group's
    scalars), so that every step is compared on its own: the distance estimate feeds on p0 - p, so a single
    cautious-mask bit or stochastic rounding draw that differs moves every later step by a per cent or so -
    in the reference's own trajectory as much as here."""
    for key in ("d", "d_max", "d_numerator"):
        group[key] = float(f[f"grp_s{step}_{key}"])
    group["k"] = int(f[f"grp_s{step}_k"])
    for i in range(n_tensors):
        set_weights(i, f.weights(step, i))
        for key in ("s", "p0", "m", "m_scale", "v", "row", "col", "shift"):
            want = f.state(step, i, key)
            if want is not None:
                set_state(i, key, want)


@pytest.mark.parametrize("name", [n for n in CASES if n.startswith("kprodigy_")])
def test_kprodigy(name):
    """reference src/kaon/kprodigy.py: the distance estimate d (a scalar over all tensors) between a pass that
    updates the statistics and the moments and a pass that writes the weights.  Every step starts from the
    reference's state after the step before."""
    opt_name, kw, shapes, dtype, steps, seed, o = CASES[name]
    f = Fixture(name)
    opt = ko.OracleKProdigy(f.params(), shapes, **kw)

    def set_weights(i, bits):
        opt.tensors[i].p[...] = bits

    def set_state(i, key, want):
        st = opt.tensors[i].state
        if key == "p0" and want.ndim == 0:
            st[key] = np.zeros((), np.float32)
        else:
            st[key][...] = want.reshape(st[key].shape).view(st[key].dtype)

    def steps_of():
        for step in range(1, steps + 1):
            if step > 1:
                kprodigy_force(f, step - 1, opt.group, len(shapes), set_weights, set_state)
            opt.step(f.grads(step))
            yield step, f

    _kprodigy_check(name, steps_of, lambda: opt.group, lambda i: opt.tensors[i].state,
                    lambda i: opt.tensors[i].p, lambda i: opt.tensors[i].state["shift"])


def test_nekaon_fp32_params():
    name = "nekaon_f32"
    for step, f, opt in _run_oracle(name):
        _check_state(f, opt, step, exact=False, md="4bit")
        for i, t in enumerate(opt.tensors):
            np.testing.assert_allclose(t.p, f.weights(step, i), rtol=1e-5, atol=1e-9)
    opt.eval()
    for i, t in enumerate(opt.tensors):
        np.testing.assert_allclose(t.p, f[f"p_eval_t{i}"], rtol=1e-5, atol=1e-9)


def test_nekaon_bf16_state():
    for step, f, opt in _run_oracle("nekaon_bf16"):
        _check_state(f, opt, step, exact=False, md="4bit")
        for i, t in enumerate(opt.tensors):
            assert sr_close(t.p, f.weights(step, i), 3 * step, 1e-3)


@pytest.mark.parametrize("name", ["adamuon_int8_none", "adamuon_int8_gc"])
def test_adamuon(name):
    for step, f, opt in _run_oracle(name):
        for i, t in enumerate(opt.tensors):
            got = ko.as_f32(t.p)
            want = ko.as_f32(f.weights(step, i))
            np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-3)
            if t.rows:  # the EMA of the raw (or centralised: bf16 row means agree) grad: bit-exact
                assert np.array_equal(t.state["m"], f.state(step, i, "m").view(np.int8))
                assert np.array_equal(t.state["m_scale"], f.state(step, i, "m_scale").reshape(-1))
                assert rel_err(t.state["row"], f.state(step, i, "row")) < 5e-2
                assert rel_err(t.state["col"], f.state(step, i, "col")) < 5e-2


def test_c1_full_size_state():
    """BASELINE config 1 at full size: Adakaon-int8 + SR on [1024,1024], [320,320,3,3], [1024],
    10 steps.  Inputs are regenerated from the seed with torch's CPU generator."""
    import torch
    opt_name, kw, shapes, dtype, steps, seed, o = CASES["c1_full"]
    f = Fixture("c1_full")
    stride = o["sample"]
    gen = torch.Generator().manual_seed(seed)
    params = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in shapes]
    to_bits = lambda t: t.contiguous().view(torch.int16).numpy().view(np.uint16).reshape(-1)  # noqa: E731
    opt = ko.OracleAdakaon([to_bits(p) for p in params], shapes, **kw)
    flips = total = 0
    for step in range(1, steps + 1):
        gen = torch.Generator().manual_seed(seed + step)
        grads = [to_bits((torch.randn(s, generator=gen) * 1e-3).bfloat16()) for s in shapes]
        opt.step(grads)
        for i, t in enumerate(opt.tensors):
            for key in ("row", "col", "v", "m_scale"):
                want = f.state(step, i, key)
                # m_scale sits downstream of the clip divisor ||u||/sqrt(n): torch's fp32 norm over
                # 1e6 elements is itself ~1e-5 off the exact value (measured 1.1e-5 here), so the
                # momentum scale gets 5e-5; the statistics proper keep 1e-5.
                if want is None:
                    continue
                got = t.state[key].reshape(-1).astype(np.float64)
                err = np.abs(got - want.reshape(-1)) / np.abs(want.reshape(-1))
                if key == "m_scale":
                    # a code that flipped by one level at an earlier step moves that row's next
                    # absmax by up to 1/127: allow it on a small fraction of rows
                    assert np.mean(err > 5e-5) < 0.02 and err.max() < 2e-2, (step, i, err.max())
                else:
                    assert err.max() <= 1e-5, (step, i, key, err.max())
            want_m = f.state(step, i, "m").view(np.int8)
            got_m = t.state["m"][::stride] if t.state["m"].size > 20000 else t.state["m"]
            d = np.abs(got_m.astype(np.int32) - want_m.astype(np.int32))
            assert d.max() <= 1
            flips += int((d != 0).sum())
            total += d.size
    assert flips / total < 2e-3, (flips, total)
