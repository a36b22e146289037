"""The device status word: a bounded wait that runs out is reported, the plan drains, nothing hangs.

The wait is made to run out on purpose with the library's test hook (one tensor expects one more finished
MAIN work item than its work list holds, and the completion-counter poll limit is cut to 1000), which
neither faults nor hangs the GPU: the waiting thread gives up, records its code and every CTA leaves."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(seed=0):
    import kaon_b200
    gen = torch.Generator().manual_seed(seed)
    shapes = [(256, 384), (64, 640), (1000,)]
    params = [torch.nn.Parameter((torch.randn(s, generator=gen) * 0.02).bfloat16().cuda()) for s in shapes]
    grads = [[(torch.randn(s, generator=gen) * 1e-3).bfloat16().cuda() for s in shapes] for _ in range(3)]
    opt = kaon_b200.Lion(params, lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True)
    opt.sr_seed = 5
    return params, grads, opt


def _step(opt, params, grads):
    for p, g in zip(params, grads):
        p.grad = g
    opt.step()
    torch.cuda.synchronize()


def test_wait_that_runs_out_sets_status_and_drains_the_plan():
    from kaon_b200 import _lib as L
    lib = L.lib()
    # an undisturbed run of three steps
    ref_params, grads, ref_opt = _make()
    for k in range(3):
        _step(ref_opt, ref_params, grads[k])
    ref_opt.check_device_status()

    params, grads, opt = _make()
    _step(opt, params, grads[0])
    opt.check_device_status()
    (plan,) = opt._plans.values()
    L.check(lib.kaon_plan_debug_stall(plan.handle, 0, C.c_uint32(1000)))
    before = [p.detach().clone() for p in params]
    _step(opt, params, grads[1])           # returns: the wait gave up after 1000 polls
    with pytest.raises(L.KaonError, match="bounded wait ran out"):
        opt.check_device_status()
    with pytest.raises(L.KaonError, match="bounded wait ran out"):
        opt.state_dict()                   # no checkpoint from state a failed kernel left behind
    assert lib.kaon_plan_status(plan.handle, C.c_void_p(torch.cuda.current_stream().cuda_stream)) == -4
    assert torch.equal(params[0].detach().view(torch.int16), before[0].view(torch.int16))  # APPLY never ran
    # the status is sticky: later steps of this plan do nothing and keep reporting
    mid = [p.detach().clone() for p in params]
    _step(opt, params, grads[2])
    for p, q in zip(params, mid):
        assert torch.equal(p.detach().view(torch.int16), q.view(torch.int16))
    with pytest.raises(L.KaonError):
        opt.check_device_status()

    # the context is intact: a fresh optimizer steps normally and reproduces the undisturbed run
    params2, grads2, opt2 = _make()
    for k in range(3):
        _step(opt2, params2, grads2[k])
    opt2.check_device_status()
    for p, q in zip(params2, ref_params):
        assert np.array_equal(p.detach().cpu().view(torch.int16).numpy(), q.detach().cpu().view(torch.int16).numpy())
