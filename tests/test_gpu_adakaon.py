"""Parity of the CUDA Adakaon / Nekaon step (through the C ABI) with the reference's golden vectors
and the CPU oracle.  Everything here sits downstream of order-dependent fp32 reductions (row/col means,
the clip rms, the GC row mean), so the gates are: statistics rel <= 1e-5, quantised codes within one
level with a small flip rate, weights within one bf16 ulp ("none") or one ulp per stochastic write."""
import numpy as np
import pytest
import torch

import kaon_oracle as ko
from _golden import Fixture, rel_err, sr_close, ulp_diff_bf16
from golden.cases import CASES, SCHEDULES

pytestmark = pytest.mark.gpu


def _code_diff(md, got, want):
    if md == "int8":
        return np.abs(got.view(np.int8).astype(np.int32) - want.view(np.int8).astype(np.int32))
    g8, w8 = got.view(np.uint8), want.view(np.uint8)
    return np.maximum(np.abs((g8 & 15).astype(np.int32) - (w8 & 15)), np.abs((g8 >> 4).astype(np.int32) - (w8 >> 4)))


def _check_against_fixture(name, writes_per_step=1):
    from _gpu import run_case_gpu, state_np, to_bits
    kw = CASES[name][1]
    md = kw.get("momentum_dtype", "bfloat16")
    sr = kw.get("bf16_method", "stochastic_rounding") == "stochastic_rounding"
    flips = total = 0
    last = None
    for step, f, opt, params in run_case_gpu(name):
        inner = getattr(opt, "base_optimizer", opt)
        for i, p in enumerate(params):
            st = inner.state[p]
            for key in ("row", "col", "v"):
                want = f.state(step, i, key)
                if want is not None:
                    assert rel_err(state_np(st, key), want) <= 1e-5, (step, i, key, rel_err(state_np(st, key), want))
            want_m = f.state(step, i, "m")
            if want_m is not None:
                got_m = state_np(st, "m")
                if md in ("int8", "4bit"):
                    assert rel_err(state_np(st, "m_scale"), f.state(step, i, "m_scale").reshape(-1)) <= 1e-5, (step, i)
                    d = _code_diff(md, got_m, want_m)
                    assert d.max() <= 1, (step, i, int(d.max()))
                    flips += int((d != 0).sum()); total += d.size
                elif md == "bfloat16":
                    assert ulp_diff_bf16(got_m, want_m).max() <= 1
            got, want = to_bits(p), f.weights(step, i)
            if want.dtype == np.uint16:
                if sr or writes_per_step > 1:
                    assert sr_close(got, want, writes_per_step * step, 1e-3), (step, i)
                else:
                    assert ulp_diff_bf16(got, want).max() <= 1, (step, i)
            else:
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-9)
        last = (f, opt, params)
    if total:
        assert flips / total < 2e-3, (flips, total)
    return last


@pytest.mark.parametrize("name", ["adakaon_int8_none", "adakaon_int8_sr", "adakaon_int8_outlier",
                                  "adakaon_4bit_wd_f32", "adakaon_bf16m_none", "adakaon_4bit_block256_wd",
                                  "adakaon_4bit_block32_f32", "adakaon_int8_long"])
def test_adakaon_matches_reference(name):
    _check_against_fixture(name)


def test_nekaon_fp32_matches_reference_including_eval():
    from _gpu import to_bits
    f, opt, params = _check_against_fixture("nekaon_f32")
    opt.eval()
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        np.testing.assert_allclose(to_bits(p), f[f"p_eval_t{i}"], rtol=1e-5, atol=1e-9)
    with pytest.raises(RuntimeError, match="outside train mode"):
        opt.step()
    opt.train()
    torch.cuda.synchronize()
    for i, p in enumerate(params):
        np.testing.assert_allclose(to_bits(p), f.weights(5, i), rtol=1e-5, atol=1e-9)


def test_nekaon_bf16_matches_reference():
    _check_against_fixture("nekaon_bf16", writes_per_step=3)


def test_nekaon_fused_equals_three_pass_path():
    """The fused removal+update+climb and the three separate passes draw the same noise and must give
    identical weights (bf16, stochastic rounding)."""
    import kaon_b200
    from _gpu import from_bits, to_bits
    name = "nekaon_bf16"
    _, kw, shapes, _, steps, _, _ = CASES[name]
    f = Fixture(name)
    results = []
    for mode in ("fused", "three_pass"):
        params = [torch.nn.Parameter(from_bits(b, s)) for b, s in zip(f.params(), shapes)]
        opt = kaon_b200.Nekaon(params, **kw)
        opt.sr_seed = 5
        if mode == "three_pass":
            opt._all_momentum_tensors_have_grads = lambda: False
        for step in range(1, steps + 1):
            for g in opt.param_groups:
                g["lr"] = SCHEDULES["cosine5"](step - 1)
            for p, gb, s in zip(params, f.grads(step), shapes):
                p.grad = from_bits(gb, s)
            opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        results.append([to_bits(p) for p in params])
    for a, b in zip(*results):
        assert np.array_equal(a, b)


def test_c1_full_size():
    """BASELINE config 1: Adakaon-int8 + SR, [1024,1024] + [320,320,3,3] + [1024], 10 steps."""
    import kaon_b200
    from _gpu import state_np
    _, kw, shapes, _, steps, seed, o = CASES["c1_full"]
    f = Fixture("c1_full")
    stride = o["sample"]
    gen = torch.Generator().manual_seed(seed)
    params = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).bfloat16().cuda()) for s in shapes]
    opt = kaon_b200.Adakaon(params, **kw)
    opt.sr_seed = 0
    flips = total = 0
    for step in range(1, steps + 1):
        gen = torch.Generator().manual_seed(seed + step)
        for p, s in zip(params, shapes):
            p.grad = (torch.randn(s, generator=gen) * 1e-3).bfloat16().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        for i, p in enumerate(params):
            st = opt.state[p]
            for key in ("row", "col", "v", "m_scale"):
                want = f.state(step, i, key)
                if want is None:
                    continue
                got = state_np(st, key).astype(np.float64)
                err = np.abs(got - want.reshape(-1)) / np.abs(want.reshape(-1))
                if key == "m_scale":
                    assert np.mean(err > 5e-5) < 0.02 and err.max() < 2e-2, (step, i, err.max())
                else:
                    assert err.max() <= 1e-5, (step, i, key, err.max())
            want_m = f.state(step, i, "m").view(np.int8)
            got_m = state_np(st, "m")
            got_m = got_m[::stride] if got_m.size > 20000 else got_m
            d = np.abs(got_m.astype(np.int32) - want_m.astype(np.int32))
            assert d.max() <= 1
            flips += int((d != 0).sum()); total += d.size
    assert flips / total < 2e-3, (flips, total)


BIG_ALL = [(640, 2560), (320, 320, 3, 3), (1280,), (5120, 640), (333, 77), (3, 16384), (4000, 1), (7,), (96, 4100)]
# every row a multiple of 16 elements: the plan takes the streaming stages and the separate COUNT / APPLY launches
BIG_STREAM = [(640, 2560), (320, 320, 4, 4), (1280,), (5120, 640), (336, 80), (3, 16384), (4000, 16), (7,), (96, 4096)]


@pytest.mark.parametrize("md,wd,method", [("int8", 0.0, "stochastic_rounding"), ("4bit", 0.1, "none"),
                                          ("bfloat16", 0.0, "none"), ("float32", 0.01, "stochastic_rounding"),
                                          (None, 0.0, "none")])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("kind", ["ragged", "stream"])
def test_adakaon_vs_oracle_bigger_shapes(md, wd, method, dtype, kind):
    # rows of 4100 elements cannot start every work item on a 128-element 4-bit block boundary within
    # the shared-memory budget: the plan refuses that shape for 4-bit momentum (tested below)
    BIG = [s for s in BIG_ALL if not (md == "4bit" and s == (96, 4100))] if kind == "ragged" else BIG_STREAM
    _adakaon_vs_oracle(BIG, md, wd, method, dtype)


# rows of 23040 elements exceed a work item: stepped by the streaming launches only
LONG_ROWS = [(16, 2560, 3, 3), (640, 2560), (1280,), (9, 16640)]


@pytest.mark.parametrize("md,wd,method", [("int8", 0.0, "stochastic_rounding"), ("4bit", 0.1, "none"),
                                          ("bfloat16", 0.01, "stochastic_rounding")])
def test_adakaon_vs_oracle_rows_longer_than_a_work_item(md, wd, method):
    _adakaon_vs_oracle(LONG_ROWS, md, wd, method, "bf16")


# 1-D tensors above a work item's 16384 elements: one FLAT item streamed from global memory
LONG_FLAT = [(50000,), (640, 320), (16385,), (131, 7), (300001,)]


@pytest.mark.parametrize("md,wd,method", [("int8", 0.0, "stochastic_rounding"), ("4bit", 0.1, "none"),
                                          ("bfloat16", 0.01, "stochastic_rounding"), ("float32", 0.0, "none"),
                                          (None, 0.0, "none")])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_adakaon_vs_oracle_long_1d_tensors(md, wd, method, dtype):
    _adakaon_vs_oracle(LONG_FLAT, md, wd, method, dtype)


@pytest.mark.parametrize("block", [32, 64, 256, 0])
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_adakaon_vs_oracle_other_4bit_block_sizes(block, dtype):
    """momentum_4bit_block other than 128 (reference src/kaon/_momentum_codec.py:192-200): powers of two, and
    0 = one block per tensor, which the library takes for 1-D tensors of any length and for tensors of at
    most 128 elements."""
    shapes = BIG_ALL[:-1] if block else [(1280,), (7,), (50000,), (8, 16), (100,)]
    if block == 256:   # rows of 77 elements cannot be grouped on 256-element block boundaries within a work item
        shapes = [s for s in shapes if s != (333, 77)]
    _adakaon_vs_oracle(shapes, "4bit", 0.01, "stochastic_rounding", dtype, momentum_4bit_block=block)


def test_one_4bit_block_over_a_big_matrix_is_refused():
    import kaon_b200
    p = torch.nn.Parameter(torch.zeros(64, 128, dtype=torch.bfloat16, device="cuda"))
    opt = kaon_b200.Adakaon([p], momentum_dtype="4bit", momentum_4bit_block=0)
    p.grad = torch.zeros_like(p)
    with pytest.raises(NotImplementedError, match="4-bit block size"):
        opt.step()


def test_rows_longer_than_a_work_item_need_the_streaming_form():
    import kaon_b200
    p = torch.nn.Parameter(torch.zeros(16, 2560, 3, 3, dtype=torch.float32, device="cuda"))
    opt = kaon_b200.Adakaon([p], momentum_dtype="4bit")
    p.grad = torch.zeros_like(p)
    with pytest.raises(NotImplementedError, match="streaming launches"):
        opt.step()
    q = torch.nn.Parameter(torch.zeros(4, 16388, dtype=torch.bfloat16, device="cuda"))
    opt = kaon_b200.Adakaon([q], momentum_dtype="bfloat16")
    q.grad = torch.zeros_like(q)
    with pytest.raises(NotImplementedError, match="cannot be cut into row-aligned work items"):
        opt.step()


def _adakaon_vs_oracle(BIG, md, wd, method, dtype, **more):
    import kaon_b200
    from _gpu import state_np, to_bits
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(9)
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in BIG]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=1e-4, betas=(0.9 if md else 0.0, 0.999), weight_decay=wd, bf16_method=method)
    if md:
        kw["momentum_dtype"] = md
    kw.update(more)
    opt = kaon_b200.Adakaon(params, **kw)
    opt.sr_seed = 4
    orc = ko.OracleAdakaon([to_bits(h) for h in host], BIG, seed=4, **kw)
    flips = total = 0
    for step in range(1, 4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(tdt) for s in BIG]
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
            for key in ("row", "col", "v"):
                if key in ot.state:
                    assert rel_err(state_np(st, key), ot.state[key]) <= 1e-5, (step, i, key, BIG[i])
            assert abs(kept[i] - orc.kept[i]) <= max(4, 2e-3 * ot.n), (step, i, kept[i], orc.kept[i])
            if md in ("int8", "4bit"):
                assert rel_err(state_np(st, "m_scale"), ot.state["m_scale"]) <= 2e-5, (step, i, BIG[i])
                d = _code_diff(md, state_np(st, "m"), ot.state["m"])
                assert d.max() <= 1, (step, i, BIG[i])
                flips += int((d != 0).sum()); total += d.size
            got, want = to_bits(p), ot.p
            if dtype == "bf16":
                assert np.mean(got != want) < 5e-3, (step, i, BIG[i], np.mean(got != want))
            else:
                # a cautious-mask bit can flip where delta*g is within rounding of zero: such an
                # element moves by at most one update (~lr); everything else agrees to 2e-5
                bad = np.abs(got - want) > 2e-5 * np.abs(want) + 1e-9
                assert bad.mean() < 1e-4 and np.abs(got - want).max() < 3e-4, (step, i, BIG[i], bad.sum())
    if total:
        assert flips / total < 2e-3, (flips, total)


def test_unsupported_shape_is_refused_loudly():
    import kaon_b200
    p = torch.nn.Parameter(torch.zeros(96, 4100, dtype=torch.bfloat16, device="cuda"))
    opt = kaon_b200.Adakaon([p], momentum_dtype="4bit")
    p.grad = torch.zeros_like(p)
    with pytest.raises(NotImplementedError, match="cannot be cut into row-aligned work items"):
        opt.step()


@pytest.mark.parametrize("md", ["4bit", "int8"])
def test_nekaon_vs_oracle_rows_longer_than_a_work_item(md):
    _nekaon_vs_oracle(LONG_ROWS, md, "bf16")


@pytest.mark.parametrize("md", ["4bit", "int8"])
def test_nekaon_vs_oracle_long_1d_tensors(md):
    _nekaon_vs_oracle(LONG_FLAT, md, "bf16")


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("md", ["4bit", "int8"])
def test_nekaon_vs_oracle_streaming_shapes(md, dtype):
    """Nekaon (removal + update + climb on one weight access) on shapes that take the streaming stages
    and the separate COUNT / APPLY launches, against the oracle with the same Philox stream."""
    _nekaon_vs_oracle(BIG_STREAM, md, dtype)


def _nekaon_vs_oracle(BIG_STREAM, md, dtype):
    import kaon_b200
    from _gpu import state_np, to_bits
    tdt = torch.bfloat16 if dtype == "bf16" else torch.float32
    gen = torch.Generator().manual_seed(19)
    host = [(torch.randn(s, generator=gen) * 0.02).to(tdt) for s in BIG_STREAM]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    kw = dict(lr=1e-4, betas=(0.2, 0.999), momentum_dtype=md)
    opt = kaon_b200.Nekaon(params, **kw)
    opt.sr_seed = 6
    orc = ko.OracleNekaon([to_bits(h) for h in host], BIG_STREAM, seed=6, **kw)
    flips = total = 0
    for step in range(1, 4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).to(tdt) for s in BIG_STREAM]
        for p, g in zip(params, grads):
            p.grad = g.clone().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        orc.step([to_bits(g) for g in grads])
        for i, p in enumerate(params):
            st, ot = opt.base_optimizer.state[p], orc.tensors[i]
            for key in ("row", "col", "v"):
                if key in ot.state:
                    assert rel_err(state_np(st, key), ot.state[key]) <= 1e-5, (step, i, key)
            # a code that flipped by one level at the previous step moves that row's (block's) next scale
            # by up to one level: a few scales may be off by <= 1/7 (4-bit) or 1/127 (int8) of themselves
            gs, ws = state_np(st, "m_scale").astype(np.float64), ot.state["m_scale"].astype(np.float64)
            err = np.abs(gs - ws) / np.abs(ws)
            assert np.mean(err > 5e-5) < 0.02 and err.max() < (0.16 if md == "4bit" else 2e-2), (step, i, err.max())
            d = _code_diff(md, state_np(st, "m"), ot.state["m"])
            assert d.max() <= 1, (step, i)
            flips += int((d != 0).sum()); total += d.size
            got, want = to_bits(p), ot.p
            if dtype == "bf16":
                assert np.mean(got != want) < 1e-2, (step, i, np.mean(got != want))
            else:
                bad = np.abs(got - want) > 2e-5 * np.abs(want) + 1e-9
                assert bad.mean() < 2e-4 and np.abs(got - want).max() < 1e-3, (step, i, bad.sum())
    assert flips / total < 2e-3, (flips, total)
