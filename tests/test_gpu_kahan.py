"""bf16_method="kahan" on the CUDA path: the compensated write with the per-tensor shift buffer
(reference src/kaon/_backend.py:89-94; the reference runs it per parameter, tests/test_lion.py:321-330)."""
import io

import numpy as np
import pytest
import torch

import kaon_oracle as ko
from _golden import rel_err, ulp_diff_bf16

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["lion_4bit_kahan", "lion_int8_kahan_wd_nocautious"])
def test_lion_kahan_matches_reference_bit_exact(name):
    from _gpu import run_case_gpu, state_np, to_bits
    for step, f, opt, params in run_case_gpu(name):
        for i, p in enumerate(params):
            st = opt.state[p]
            assert np.array_equal(state_np(st, "m").view(np.uint8), f.state(step, i, "m").view(np.uint8)), (step, i)
            assert np.array_equal(to_bits(p), f.weights(step, i)), (step, i, "weights")
            assert np.array_equal(state_np(st, "shift"), f.state(step, i, "shift")), (step, i, "shift")


def _kahan_close(p, shift, want_p, want_shift):
    if ulp_diff_bf16(p, want_p).max() > 1:
        return False
    a = ko.as_f32(p).astype(np.float64) + ko.as_f32(shift)
    b = ko.as_f32(want_p).astype(np.float64) + ko.as_f32(want_shift)
    ulp = np.maximum(np.abs(ko.as_f32(want_p)), 1e-30) * 2.0 ** -7
    return bool((np.abs(a - b) <= ulp).all())


def test_adakaon_kahan_matches_reference():
    from _gpu import run_case_gpu, state_np, to_bits
    for step, f, opt, params in run_case_gpu("adakaon_int8_kahan"):
        for i, p in enumerate(params):
            st = opt.state[p]
            for key in ("row", "col", "v"):
                want = f.state(step, i, key)
                if want is not None:
                    assert rel_err(state_np(st, key), want) <= 1e-5, (step, i, key)
            assert _kahan_close(to_bits(p), state_np(st, "shift"), f.weights(step, i), f.state(step, i, "shift")), (step, i)


def test_adamuon_kahan_matches_reference():
    from _gpu import run_case_gpu, state_np, to_bits
    for step, f, opt, params in run_case_gpu("adamuon_int8_kahan"):
        for i, p in enumerate(params):
            np.testing.assert_allclose(ko.as_f32(to_bits(p)), ko.as_f32(f.weights(step, i)), rtol=2e-2, atol=2e-3)
            assert state_np(opt.state[p], "shift") is not None


def test_kahan_keeps_updates_that_nearest_rounding_loses():
    """The point of the buffer: with updates far below a bf16 ulp, nearest rounding never moves the
    weights; the compensated write accumulates them."""
    import kaon_b200
    runs = {}
    for method in ("none", "kahan"):
        p = torch.nn.Parameter(torch.ones(64, 64, dtype=torch.bfloat16, device="cuda"))
        opt = kaon_b200.Lion([p], lr=1e-4, betas=(0.0, 0.0), momentum_dtype="bfloat16", cautious=False,
                             gradient_centralization=False, bf16_method=method)
        for _ in range(100):
            p.grad = torch.ones_like(p)
            opt.step()
        torch.cuda.synchronize()
        runs[method] = p.detach().float().mean().item()
    assert runs["none"] == 1.0                      # 1e-4 is below half a bf16 ulp at 1.0: lost every time
    assert abs(runs["kahan"] - (1.0 - 100 * 1e-4)) < 4e-3


def test_kahan_fp32_weights_have_no_shift_and_checkpoint_round_trips():
    import kaon_b200
    p32 = torch.nn.Parameter(torch.randn(16, 16, device="cuda"))
    o32 = kaon_b200.Adakaon([p32], bf16_method="kahan")
    p32.grad = torch.randn_like(p32)
    o32.step()
    assert "shift" not in o32.state[p32]
    gen = torch.Generator().manual_seed(0)
    def mk():
        return torch.nn.Parameter((torch.randn(32, 48, generator=torch.Generator().manual_seed(1)) * 0.1).bfloat16().cuda())
    pa = mk()
    oa = kaon_b200.Adakaon([pa], momentum_dtype="int8", bf16_method="kahan")
    grads = [(torch.randn(32, 48, generator=gen) * 1e-2).bfloat16().cuda() for _ in range(6)]
    for g in grads[:3]:
        pa.grad = g
        oa.step()
    buf = io.BytesIO()
    torch.save({"sd": oa.state_dict(), "p": pa.detach().clone()}, buf)
    for g in grads[3:]:
        pa.grad = g
        oa.step()
    buf.seek(0)
    ck = torch.load(buf)
    pb = mk()
    pb.data.copy_(ck["p"])
    ob = kaon_b200.Adakaon([pb], momentum_dtype="int8", bf16_method="kahan")
    ob.load_state_dict(ck["sd"])
    for g in grads[3:]:
        pb.grad = g
        ob.step()
    torch.cuda.synchronize()
    assert torch.equal(pa.detach().view(torch.int16), pb.detach().view(torch.int16))
    assert torch.equal(oa.state[pa]["shift"].view(torch.int16), ob.state[pb]["shift"].view(torch.int16))


@pytest.mark.parametrize("cls_name,okls,kw", [
    ("Adakaon", "OracleAdakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="kahan")),
    ("Adakaon", "OracleAdakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="4bit", weight_decay=0.1, bf16_method="kahan")),
    ("Lion", "OracleLion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", bf16_method="kahan")),
])
def test_kahan_vs_oracle_on_streaming_shapes(cls_name, okls, kw):
    """The compensated write on shapes whose plan takes the streaming stages and the separate COUNT / APPLY
    launches (Adakaon) or the 4-bit fast path (Lion), against the oracle."""
    import kaon_b200
    from _gpu import state_np, to_bits
    shapes = [(640, 256), (64, 32, 4, 4), (1280,), (336, 80), (3, 4096), (7,)]
    gen = torch.Generator().manual_seed(23)
    host = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in shapes]
    params = [torch.nn.Parameter(h.clone().cuda()) for h in host]
    opt = getattr(kaon_b200, cls_name)(params, **kw)
    orc = getattr(ko, okls)([to_bits(h) for h in host], shapes, **kw)
    for step in range(1, 4):
        grads = [(torch.randn(s, generator=gen) * 1e-3).bfloat16() for s in shapes]
        for p, g in zip(params, grads):
            p.grad = g.clone().cuda()
        opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        orc.step([to_bits(g) for g in grads])
        for i, p in enumerate(params):
            st, ot = opt.state[p], orc.tensors[i]
            got_p, got_s = to_bits(p), state_np(st, "shift")
            if cls_name == "Lion":
                # the only reduction upstream is the centralization mean: a handful of elements may differ
                assert np.mean(got_p != ot.p) < 5e-3 and np.mean(got_s != ot.state["shift"]) < 5e-3, (step, i)
            else:
                # weights within one ulp almost everywhere; the compensated value p + shift within one ulp of p
                a = ko.as_f32(got_p).astype(np.float64) + ko.as_f32(got_s)
                b = ko.as_f32(ot.p).astype(np.float64) + ko.as_f32(ot.state["shift"])
                ulp = np.maximum(np.abs(ko.as_f32(ot.p)), 1e-30) * 2.0 ** -7
                bad = np.abs(a - b) > ulp
                assert bad.mean() < 2e-3, (step, i, bad.mean())
                assert ulp_diff_bf16(got_p, ot.p).max() <= 2, (step, i)
