"""Stochastic-rounding weight write on its own (kaon_sr_add): unbiased, and only ever one of the two
bf16 neighbours of the fp32 result (reference src/kaon/_stochastic_rounding.py:88-96; the reference's
own unbiasedness test is tests/test_fused_triton.py:843-864)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

N = 4096
ROUNDS = 10_000


def _sr_add(p, delta, step, seed=99, tensor_id=3):
    from kaon_b200 import _lib as L
    L.check(L.lib().kaon_sr_add(C.c_void_p(p.data_ptr()), L.DT_BF16, C.c_void_p(delta.data_ptr()),
                                C.c_int64(p.numel()), C.c_float(1.0), 1, C.c_uint64(seed), C.c_uint32(step),
                                C.c_uint32(tensor_id), C.c_uint32(0),
                                C.c_void_p(torch.cuda.current_stream().cuda_stream)))


def _targets(kind):
    gen = torch.Generator().manual_seed(1)
    if kind == "reference_value":        # the reference's own probe: 1.0 + 0.003
        base = torch.ones(N)
        delta = torch.full((N,), 0.003)
    elif kind == "mixed":                 # both signs, six decades of magnitude
        base = torch.randn(N, generator=gen) * torch.logspace(-3, 3, N)
        delta = base * (torch.rand(N, generator=gen) - 0.5) * 2e-2
    elif kind == "tiny":                  # next to the smallest normal numbers
        base = (torch.rand(N, generator=gen) + 1.0) * 2e-37 * torch.where(torch.rand(N, generator=gen) < 0.5, -1.0, 1.0)
        delta = base * (torch.rand(N, generator=gen) - 0.5) * 1e-2
    else:
        raise ValueError(kind)
    base = base.bfloat16()
    return base.cuda(), delta.float().cuda()


@pytest.mark.parametrize("kind", ["reference_value", "mixed", "tiny"])
def test_sr_is_unbiased_and_stays_between_the_neighbours(kind):
    base, delta = _targets(kind)
    target = base.float() + delta                      # the fp32 value the kernel rounds (one fp32 add)
    lo = (target.view(torch.int32) & -65536).view(torch.float32)          # truncation toward zero
    hi = ((target.view(torch.int32) & -65536) + 65536).view(torch.float32)  # next bf16 away from zero
    ulp = (hi - lo).abs().double()
    acc = torch.zeros(N, dtype=torch.float64, device="cuda")
    p = torch.empty_like(base)
    seen_other = torch.zeros((), dtype=torch.int64, device="cuda")
    for k in range(1, ROUNDS + 1):
        p.copy_(base)
        _sr_add(p, delta, k)
        pf = p.float()
        acc += pf.double()
        if k % 97 == 0:
            seen_other += ((pf != lo) & (pf != hi)).sum()
    torch.cuda.synchronize()
    assert seen_other.item() == 0
    err_ulp = ((acc / ROUNDS - target.double()) / ulp)
    # 4096 elements x 10^4 rounds: the standard error of the mean is ~8e-5 ulp
    assert abs(err_ulp.mean().item()) <= 1e-3, err_ulp.mean().item()
    # and no single element is off by more than sampling noise allows (sigma <= 0.005 ulp per element)
    assert err_ulp.abs().max().item() < 0.03


def test_exact_bf16_values_never_move():
    base = (torch.randn(N, generator=torch.Generator().manual_seed(2)) * 3).bfloat16().cuda()
    delta = torch.zeros(N, device="cuda")
    p = base.clone()
    for k in range(1, 200):
        _sr_add(p, delta, k)
    torch.cuda.synchronize()
    assert torch.equal(p.view(torch.int16), base.view(torch.int16))


def test_stream_is_a_function_of_seed_step_tensor_and_element():
    base, delta = _targets("mixed")
    outs = []
    for seed, step, tid in [(5, 1, 0), (5, 1, 0), (6, 1, 0), (5, 2, 0), (5, 1, 1)]:
        p = base.clone()
        _sr_add(p, delta, step, seed=seed, tensor_id=tid)
        outs.append(p.view(torch.int16).clone())
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1])
    for o in outs[2:]:
        assert not torch.equal(outs[0], o)
