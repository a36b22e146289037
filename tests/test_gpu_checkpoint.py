"""Checkpoint / resume through state_dict, and the state layout against the reference's.

The reference tests bit-exact resume on fp32 parameters for every momentum dtype
(reference tests/test_adakaon.py:346-385, tests/test_lion.py:271-304, tests/test_adamuon.py:175-208).
Here resume is also bit-exact for bf16 parameters under stochastic rounding, because the noise stream's
position (step index, seed) travels in the checkpoint."""
import io

import numpy as np
import pytest
import torch

from _golden import Fixture

pytestmark = pytest.mark.gpu

SHAPES = [(96, 128), (16, 12, 3, 3), (200,), (40, 72)]


def _make(cls_name, dtype, seed, **kw):
    import kaon_b200
    gen = torch.Generator().manual_seed(seed)
    params = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).to(dtype).cuda()) for s in SHAPES]
    opt = getattr(kaon_b200, cls_name)(params, **kw)
    opt.sr_seed = 17
    return params, opt


def _step(params, opt, dtype, step):
    gen = torch.Generator().manual_seed(1000 + step)
    for p, s in zip(params, SHAPES):
        p.grad = (torch.randn(s, generator=gen) * 1e-3).to(dtype).cuda()
    opt.step()


@pytest.mark.parametrize("cls_name,kw", [
    ("Lion", dict(lr=2e-4, momentum_dtype="4bit")),
    ("Lion", dict(lr=2e-4, momentum_dtype="int8", weight_decay=0.1)),
    ("Adakaon", dict(lr=1e-4, momentum_dtype="int8")),
    ("Adakaon", dict(lr=1e-4, momentum_dtype="4bit", weight_decay=0.1)),
    ("Adakaon", dict(lr=1e-4, momentum_dtype="bfloat16")),
    ("AdaMuon", dict(lr=1e-3, momentum_dtype="int8")),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_resume_is_bit_exact(cls_name, kw, dtype):
    pa, oa = _make(cls_name, dtype, 3, **kw)
    for s in range(1, 4):
        _step(pa, oa, dtype, s)
    buf = io.BytesIO()
    torch.save({"opt": oa.state_dict(), "params": [p.detach().clone() for p in pa]}, buf)
    for s in range(4, 7):
        _step(pa, oa, dtype, s)
    torch.cuda.synchronize()
    # resume in a fresh optimizer
    buf.seek(0)
    ck = torch.load(buf)
    pb, ob = _make(cls_name, dtype, 99, **kw)
    for p, q in zip(pb, ck["params"]):
        p.data.copy_(q)
    ob.load_state_dict(ck["opt"])
    for s in range(4, 7):
        _step(pb, ob, dtype, s)
    torch.cuda.synchronize()
    ob.check_device_status()
    for i, (p, q) in enumerate(zip(pa, pb)):
        assert torch.equal(p.detach().view(torch.int16) if dtype == torch.bfloat16 else p.detach(),
                           q.detach().view(torch.int16) if dtype == torch.bfloat16 else q.detach()), i
        sa, sb = oa.state[p], ob.state[q]
        assert sa.keys() == sb.keys()
        for k in sa:
            if torch.is_tensor(sa[k]):
                assert sa[k].dtype == sb[k].dtype and torch.equal(sa[k], sb[k]), (i, k)
            else:
                assert sa[k] == sb[k]


def test_nekaon_checkpoint_in_eval_mode_round_trips():
    """reference tests/test_msam.py:250-268: save in eval mode (unperturbed weights), resume, keep going."""
    dtype = torch.float32
    kw = dict(lr=1e-4, betas=(0.2, 0.999))
    pa, oa = _make("Nekaon", dtype, 5, **kw)
    for s in range(1, 4):
        _step(pa, oa, dtype, s)
    oa.eval()
    sd = oa.state_dict()
    assert sd["msam"] == {} and set(sd) >= {"state", "param_groups", "msam"}
    buf = io.BytesIO()
    torch.save(sd, buf)  # a snapshot: state_dict() hands out the live state tensors
    buf.seek(0)
    sd = torch.load(buf)
    weights = [p.detach().clone() for p in pa]
    oa.train()
    for s in range(4, 6):
        _step(pa, oa, dtype, s)
    pb, ob = _make("Nekaon", dtype, 6, **kw)
    for p, q in zip(pb, weights):
        p.data.copy_(q)
    ob.load_state_dict(sd)
    # the reference resumes without a climb in place; its first step after load therefore differs from
    # the uninterrupted run by that climb only: check the state instead of the live weights
    for s in range(4, 6):
        _step(pb, ob, dtype, s)
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        sa, sb = oa.base_optimizer.state[p], ob.base_optimizer.state[q]
        for k in ("row", "col", "v"):
            if k in sa:
                assert torch.equal(sa[k], sb[k]), k  # second-moment statistics depend on the gradients only


@pytest.mark.parametrize("name", ["lion_4bit_none", "lion_int8_none", "adakaon_int8_none", "adakaon_4bit_wd_f32",
                                  "adakaon_bf16m_none", "nekaon_bf16", "adamuon_int8_none", "lion_4bit_kahan",
                                  "adakaon_int8_kahan"])
def test_state_layout_matches_reference(name):
    """Same per-tensor state keys, dtypes and element counts as the reference's state_dict."""
    from _gpu import run_case_gpu
    last = None
    for step, f, opt, params in run_case_gpu(name):
        last = (f, opt, params)
        break
    f, opt, params = last
    inner = getattr(opt, "base_optimizer", opt)
    for i, p in enumerate(params):
        st = inner.state[p]
        ref_keys = {k.split(f"st_s1_t{i}_", 1)[1] for k in f.z.files if k.startswith(f"st_s1_t{i}_")}
        assert set(st.keys()) == ref_keys, (i, set(st.keys()), ref_keys)
        for k in ref_keys:
            want = f.state(1, i, k)
            if torch.is_tensor(st[k]):
                assert st[k].numel() == want.size, (i, k)
                np_dtype = {torch.int8: np.int8, torch.uint8: np.uint8, torch.float32: np.float32,
                            torch.bfloat16: np.uint16}[st[k].dtype]
                assert want.dtype == np_dtype, (i, k, want.dtype, st[k].dtype)
            else:
                assert int(st[k]) == int(want)
    sd = opt.state_dict()
    assert {"state", "param_groups"} <= set(sd)
    ref_group_keys = {"Lion": {"lr", "betas", "weight_decay", "momentum_dtype", "momentum_4bit_block", "cautious",
                               "gradient_centralization", "bf16_method", "params"}}
    if type(opt).__name__ == "Lion":
        assert set(sd["param_groups"][0]) == ref_group_keys["Lion"]
