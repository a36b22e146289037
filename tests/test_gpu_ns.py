"""Newton-Schulz on tcgen05 against the CPU oracle (small shapes) and against the same iteration written
with plain torch ops on the GPU (larger shapes).  Tolerance: the reference's own, rtol=2e-2 atol=2e-2
on the bf16 result (reference tests/test_adamuon.py:101-109); singular values inside (0.5, 1.3)
(reference tests/test_adamuon.py:112-118)."""
import ctypes as C

import numpy as np
import pytest
import torch

import kaon_oracle as ko

pytestmark = pytest.mark.gpu


def ns_gpu(x_bf16: torch.Tensor, steps: int) -> torch.Tensor:
    from kaon_b200 import _lib as L
    lib = L.lib()
    lib.kaon_newton_schulz_workspace_bytes.restype = C.c_int64
    R, Cc = x_bf16.shape
    nbytes = lib.kaon_newton_schulz_workspace_bytes(C.c_int64(R), C.c_int64(Cc))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=x_bf16.device)
    out = torch.empty_like(x_bf16)
    L.check(lib.kaon_newton_schulz(C.c_void_p(x_bf16.data_ptr()), C.c_int64(R), C.c_int64(Cc), steps,
                                   C.c_void_p(out.data_ptr()), C.c_void_p(ws.data_ptr()), C.c_int64(nbytes),
                                   C.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    assert int(ws[:4].view(torch.int32).item()) == 0, "device status: a bounded wait ran out"
    return out


def ns_torch(x: torch.Tensor, steps: int) -> torch.Tensor:
    """The iteration of reference src/kaon/adamuon.py:97-118 in plain torch ops."""
    a, b, c = 3.4445, -4.7750, 2.0315
    x = x.bfloat16()
    t = x.size(0) > x.size(1)
    if t:
        x = x.mT
    x = x / (x.norm() + 1e-7)
    for _ in range(steps):
        aa = x @ x.mT
        bb = b * aa + c * (aa @ aa)
        x = a * x + bb @ x
    return x.mT if t else x


@pytest.mark.parametrize("shape", [(64, 64), (48, 32), (32, 80), (128, 256), (256, 128), (200, 328), (77, 50), (130, 64)])
def test_ns_small_shapes_vs_oracle(shape):
    gen = torch.Generator().manual_seed(21)
    x = (torch.randn(shape, generator=gen) * 1e-3).bfloat16()
    got = ns_gpu(x.cuda(), 2).float().cpu().numpy()
    want = ko.newton_schulz(x.float().numpy(), 2)
    np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
    assert np.abs(got - want).mean() < 2e-3


@pytest.mark.parametrize("shape", [(512, 512), (384, 1280), (1536, 512), (1024, 2048), (3072, 1024)])
@pytest.mark.parametrize("steps", [1, 2, 3])
def test_ns_larger_shapes_vs_torch(shape, steps):
    gen = torch.Generator().manual_seed(22)
    x = (torch.randn(shape, generator=gen) * 1e-3).bfloat16().cuda()
    got = ns_gpu(x, steps).float()
    want = ns_torch(x, steps).float()
    torch.testing.assert_close(got, want, rtol=2e-2, atol=2e-2)
    rel = (got - want).norm() / want.norm()
    assert rel < 1e-2, rel
    if steps >= 2:
        # the quintic pushes every singular value towards ~0.9 and never overshoots 1.3
        assert torch.linalg.svdvals(got).max() < 1.3
