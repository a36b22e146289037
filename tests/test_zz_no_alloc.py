"""The allocation-free Lion entry point against the plan-based one, through the C ABI.

kaon_lion_step_noalloc serves callers that may not allocate device memory at the point where they step
(a host that owns every allocation, a launch-only path): its table, work list and scratch sit in an
array built into the library instead of coming from cudaMalloc.  It must produce exactly what
kaon_lion_step produces on the same inputs (same kernel, same arithmetic: the comparison is bit for
bit), also on a second call that finds the previous call's contents in the shared array.
This file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _desc(L, p, g, m, m_scale, tensor_id, block):
    d = L.TensorDesc()
    d.p, d.g, d.m, d.m_scale = p.data_ptr(), (g.data_ptr() if g is not None else 0), m.data_ptr(), m_scale.data_ptr()
    d.stat_a = d.stat_b = None
    d.numel = p.numel()
    d.rows = p.shape[0] if p.ndim >= 2 else 0
    d.tensor_id = tensor_id
    d.block = block
    return d


@pytest.mark.parametrize("shape,dtype,cautious,method", [
    ((640, 2560), torch.bfloat16, 1, "sr"), ((320, 320, 3, 3), torch.bfloat16, 1, "sr"),
    ((5000,), torch.bfloat16, 1, "sr"), ((77,), torch.bfloat16, 1, "sr"), ((333, 77), torch.float32, 1, "sr"),
    # cautious off: MAIN items write the weights themselves and the work list has no APPLY items
    ((640, 2560), torch.bfloat16, 0, "sr"), ((333, 77), torch.bfloat16, 0, "none"),
    # nearest rounding; rows that are not a multiple of 8 elements over several work items
    ((1000, 77), torch.bfloat16, 1, "none")])
def test_noalloc_matches_plan_path_two_calls_in_a_row(shape, dtype, cautious, method):
    from kaon_b200 import _lib as L
    lib = L.lib()
    dev = torch.device("cuda", 0)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    gen = torch.Generator().manual_seed(123)
    n = int(np.prod(shape))
    block = min(128, n)
    pdt = L.DT_BF16 if dtype == torch.bfloat16 else L.DT_F32
    p0 = (torch.randn(shape, generator=gen) * 0.02).to(dtype)
    grads = [(torch.randn(shape, generator=gen) * 1e-3).to(dtype).to(dev) for _ in range(2)]

    def fresh():
        return (p0.clone().to(dev), torch.full(((n + 1) // 2,), 0x88, dtype=torch.uint8, device=dev),
                torch.ones((n + block - 1) // block, dtype=torch.float32, device=dev))

    hp = L.LionHParams(lr=2e-4, beta1=0.95, beta2=0.98, weight_decay=0.01, cautious=cautious,
                       gradient_centralization=1, bf16_method=L.W_SR if method == "sr" else L.W_NONE, reserved=0)
    seed, tid = 99, 7

    # existing entry point: a plan over the one tensor
    pa, ma, sa = fresh()
    descs = (L.TensorDesc * 1)(_desc(L, pa, None, ma, sa, tid, block))
    plan = C.c_void_p()
    L.check(lib.kaon_plan_create(C.byref(plan), L.OPT_LION, pdt, L.M_4BIT, descs, 1))
    # new entry point: no plan, no allocation
    pb, mb, sb = fresh()
    try:
        for step, g in enumerate(grads, start=1):
            arr = (C.c_void_p * 1)(g.data_ptr())
            L.check(lib.kaon_plan_set_grads(plan, arr, 1, stream))
            L.check(lib.kaon_lion_step(plan, C.byref(hp), C.c_uint64(seed), C.c_uint32(step), stream))
            d = _desc(L, pb, g, mb, sb, tid, block)
            if step == 2:
                # the first call on a device resolves the array's address and loads the kernel; from the
                # second call on, the free device memory the driver reports (cudaMemGetInfo: it sees every
                # cudaMalloc and cudaFree of the process, the library's own too) must not move
                torch.cuda.synchronize()
                free_before = torch.cuda.mem_get_info(dev)[0]
            L.check(lib.kaon_lion_step_noalloc(C.byref(d), pdt, C.byref(hp), C.c_uint64(seed), C.c_uint32(step), stream))
            torch.cuda.synchronize()
            if step == 2:
                assert torch.cuda.mem_get_info(dev)[0] == free_before
            L.check(lib.kaon_plan_status(plan, stream))
            assert torch.equal(ma, mb), (step, "momentum codes")
            assert torch.equal(sa, sb), (step, "momentum scales")
            assert torch.equal(pa.view(torch.int16) if dtype == torch.bfloat16 else pa,
                               pb.view(torch.int16) if dtype == torch.bfloat16 else pb), (step, "weights")
        assert not torch.equal(pa, p0.to(dev))  # the steps did move the weights
        assert lib.kaon_lion_noalloc_status(stream) == 0
    finally:
        lib.kaon_plan_destroy(plan)


def test_noalloc_rejects_sizes_beyond_the_built_in_scratch():
    from kaon_b200 import _lib as L
    lib = L.lib()
    n = (1 << 22) + 128
    dev = torch.device("cuda", 0)
    p = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    m = torch.full((n // 2,), 0x88, dtype=torch.uint8, device=dev)
    s = torch.ones(n // 128, dtype=torch.float32, device=dev)
    d = _desc(L, p, p, m, s, 0, 128)
    hp = L.LionHParams(lr=1e-4, beta1=0.9, beta2=0.99, weight_decay=0.0, cautious=1,
                       gradient_centralization=1, bf16_method=L.W_SR, reserved=0)
    rc = lib.kaon_lion_step_noalloc(C.byref(d), L.DT_BF16, C.byref(hp), C.c_uint64(0), C.c_uint32(1),
                                    C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == -2 and b"KAON_NOALLOC_MAX_NUMEL" in lib.kaon_last_error()
    with pytest.raises(NotImplementedError):
        L.check(rc)


def test_noalloc_refuses_the_kahan_write():
    """The compensated write needs the per-tensor shift buffer of a plan: KAON_E_UNSUPPORTED (-2)."""
    from kaon_b200 import _lib as L
    lib = L.lib()
    dev = torch.device("cuda", 0)
    n = 1024
    p = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    m = torch.full((n // 2,), 0x88, dtype=torch.uint8, device=dev)
    s = torch.ones(n // 128, dtype=torch.float32, device=dev)
    d = _desc(L, p, p, m, s, 0, 128)
    hp = L.LionHParams(lr=1e-4, beta1=0.9, beta2=0.99, weight_decay=0.0, cautious=1,
                       gradient_centralization=1, bf16_method=L.W_KAHAN, reserved=0)
    rc = lib.kaon_lion_step_noalloc(C.byref(d), L.DT_BF16, C.byref(hp), C.c_uint64(0), C.c_uint32(1),
                                    C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    assert rc == -2 and b"bf16_method" in lib.kaon_last_error()
