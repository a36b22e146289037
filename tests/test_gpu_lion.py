"""Parity of the CUDA Lion step (through the C ABI) with the reference's golden vectors and with the
CPU oracle.  Bit-exact wherever no order-dependent reduction sits upstream (GC off, or GC means that
round to the same bf16); otherwise the documented tolerances."""
import numpy as np
import pytest
import torch

import kaon_oracle as ko
from _golden import Fixture, rel_err, sr_close, ulp_diff_bf16
from golden.cases import CASES

pytestmark = pytest.mark.gpu


def _inner_state(opt, p):
    return getattr(opt, "base_optimizer", opt).state[p]


@pytest.mark.parametrize("name", ["lion_4bit_nogc_wd", "lion_4bit_none", "lion_int8_none",
                                  "lion_bf16_nocautious", "lion_4bit_block64", "lion_4bit_long"])
def test_lion_matches_reference_bit_exact(name):
    from _gpu import run_case_gpu, state_np, to_bits
    for step, f, opt, params in run_case_gpu(name):
        for i, p in enumerate(params):
            st = _inner_state(opt, p)
            assert np.array_equal(state_np(st, "m").view(np.uint8), f.state(step, i, "m").view(np.uint8)), (step, i, "m")
            if f.state(step, i, "m_scale") is not None:
                assert np.array_equal(state_np(st, "m_scale"), f.state(step, i, "m_scale").reshape(-1)), (step, i, "m_scale")
            assert np.array_equal(to_bits(p), f.weights(step, i)), (step, i, "weights")


def test_lion_fp32_params_with_gc():
    from _gpu import run_case_gpu, state_np, to_bits
    flips = total = 0
    for step, f, opt, params in run_case_gpu("lion_4bit_f32params"):
        for i, p in enumerate(params):
            st = _inner_state(opt, p)
            assert rel_err(state_np(st, "m_scale"), f.state(step, i, "m_scale")) <= 1e-5
            g8, w8 = state_np(st, "m"), f.state(step, i, "m")
            d = np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)), np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))
            assert d.max() <= 1
            flips += int((d != 0).sum()); total += d.size
            got, want = to_bits(p), f.weights(step, i)
            assert np.mean(got != want) < 5e-3
    assert flips / total < 2e-3


def test_lion_sr_matches_oracle_stream_bit_exact():
    """Same Philox stream on both sides: weights under stochastic rounding are bit-identical to the
    oracle's, and the state equals the reference's (it does not depend on the weights)."""
    from _gpu import run_case_gpu, state_np, to_bits
    name = "lion_4bit_sr"
    _, kw, shapes, _, steps, _, _ = CASES[name]
    f0 = Fixture(name)
    orc = ko.OracleLion(f0.params(), shapes, seed=77, **kw)
    for step, f, opt, params in run_case_gpu(name, seed=77):
        orc.step(f.grads(step))
        for i, p in enumerate(params):
            st = opt.state[p]
            assert np.array_equal(state_np(st, "m"), f.state(step, i, "m"))
            assert np.array_equal(state_np(st, "m_scale"), f.state(step, i, "m_scale"))
            assert np.array_equal(to_bits(p), orc.tensors[i].p), (step, i)
            assert sr_close(to_bits(p), f.weights(step, i), step, 1e-3)


def test_kept_counts_match_oracle():
    from _gpu import run_case_gpu
    name = "lion_4bit_none"
    _, kw, shapes, _, _, _, _ = CASES[name]
    orc = ko.OracleLion(Fixture(name).params(), shapes, **kw)
    for step, f, opt, params in run_case_gpu(name):
        orc.step(f.grads(step))
        (plan,) = opt._plans.values()
        kept = plan.kept_counts(torch.cuda.current_stream().cuda_stream)
        assert kept == orc.kept, (step, kept, orc.kept)


SHAPES_BIG = [(640, 2560), (320, 320, 3, 3), (1280,), (5120, 640), (333, 77), (12289,), (3, 16384), (40000, 1)]


@pytest.mark.parametrize("md,gc,method,wd", [("4bit", False, "none", 0.0), ("4bit", True, "stochastic_rounding", 0.0),
                                             ("int8", True, "none", 0.05), ("bfloat16", True, "stochastic_rounding", 0.0),
                                             ("float32", False, "none", 0.0), ("4bit", True, "none", 0.1),
                                             ("4bit/32", False, "none", 0.0), ("4bit/64", True, "stochastic_rounding", 0.0),
                                             ("4bit/256", True, "none", 0.1)])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_lion_vs_oracle_bigger_shapes(md, gc, method, wd, dtype):
    """Shapes with ragged tails, rows that straddle 4-bit blocks (C = 2880, 77), a row of exactly CAP
    elements, a [N,1] column and multi-item tensors, 3 steps, against the oracle on the same inputs."""
    import kaon_b200
    from _gpu import from_bits, state_np, to_bits
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(5)
    shapes = [s for s in SHAPES_BIG if not (md == "int8" and s == (12289,))]
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in shapes]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=2e-4, betas=(0.95, 0.98), weight_decay=wd, momentum_dtype=md, gradient_centralization=gc, bf16_method=method)
    if "/" in md:   # "4bit/64": the 4-bit codec with another block size (reference src/kaon/_momentum_codec.py:192-200)
        md, blk = md.split("/")
        kw.update(momentum_dtype=md, momentum_4bit_block=int(blk))
    opt = kaon_b200.Lion(params, **kw)
    opt.sr_seed = 3
    orc = ko.OracleLion([to_bits(h) for h in host], shapes, seed=3, **kw)
    exact = (not gc) or dtype == "bf16"
    for step in range(1, 4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(tdt) for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.clone().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        orc.step([to_bits(g) for g in grads])
        for i, p in enumerate(params):
            st, ot = opt.state[p], orc.tensors[i]
            gm, om = state_np(st, "m"), ot.state["m"]
            if exact:
                bad = np.mean(gm.view(np.uint8) != om.view(np.uint8))
                # a GC row mean summed in another order can land on the other side of a bf16 rounding
                # boundary for a rare row; everything else must be identical
                assert bad <= (2e-3 if gc else 0.0), (step, i, shapes[i], bad)
                wbad = np.mean(to_bits(p) != ot.p)
                assert wbad <= (2e-3 if gc else 0.0), (step, i, shapes[i], wbad)
            else:
                if md in ("int8", "4bit"):
                    assert rel_err(state_np(st, "m_scale"), ot.state["m_scale"]) <= 1e-5
                assert np.mean(to_bits(p) != ot.p) < 1e-2


LONG_ROWS = [(16, 2560, 3, 3), (96, 4100), (640, 2560), (1280,), (50000,)]


@pytest.mark.parametrize("md,method", [("4bit", "stochastic_rounding"), ("4bit", "none"), ("bfloat16", "none")])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_lion_rows_longer_than_a_work_item(md, method, dtype):
    """A 3x3 convolution over 2560 input channels (rows of 23 040 elements, longer than the 16 384 a work
    item stages) and [96, 4100] (rows that cannot be grouped on 4-bit block boundaries) are cut into flat
    runs whose row means come from a pre-pass; against the oracle on the same inputs."""
    import kaon_b200
    from _gpu import state_np, to_bits
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(15)
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in LONG_ROWS]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype=md, bf16_method=method)
    opt = kaon_b200.Lion(params, **kw)
    opt.sr_seed = 13
    orc = ko.OracleLion([to_bits(h) for h in host], LONG_ROWS, seed=13, **kw)
    for step in range(1, 4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(tdt) for s in LONG_ROWS]
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
            assert abs(kept[i] - orc.kept[i]) <= max(4, 2e-3 * ot.n), (step, i, kept[i], orc.kept[i])
            if dtype == "bf16":
                # a row mean summed in another order can land on the other bf16 neighbour for a rare row
                assert np.mean(state_np(st, "m").view(np.uint8) != ot.state["m"].view(np.uint8)) <= 2e-3, (step, i)
                assert np.mean(to_bits(p) != ot.p) <= 2e-3, (step, i, LONG_ROWS[i])
            else:
                if md == "4bit":
                    assert rel_err(state_np(st, "m_scale"), ot.state["m_scale"]) <= 1e-5
                assert np.mean(to_bits(p) != ot.p) < 1e-2, (step, i, LONG_ROWS[i])


def test_lion_int8_rows_longer_than_a_work_item_are_refused():
    import kaon_b200
    p = torch.nn.Parameter(torch.zeros(4, 2560, 3, 3, dtype=torch.bfloat16, device="cuda"))
    opt = kaon_b200.Lion([p], momentum_dtype="int8")
    p.grad = torch.zeros_like(p)
    with pytest.raises(NotImplementedError, match="cannot be cut into row-aligned work items"):
        opt.step()
