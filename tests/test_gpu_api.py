"""Behaviour of the classes around the step (what the reference's own class tests check), on the GPU,
plus the stand-alone codec entry points against the oracle's codec (bit-exact)."""
import ctypes as C

import numpy as np
import pytest
import torch

import kaon_oracle as ko

pytestmark = pytest.mark.gpu

SHAPES = [(48, 64), (8, 6, 3, 3), (130,), (33, 77)]


def _mk(dtype=torch.float32, seed=0, shapes=SHAPES):
    g = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter((torch.randn(s, generator=g) * 0.05).to(dtype).cuda()) for s in shapes]


def _grads(params, seed):
    g = torch.Generator().manual_seed(100 + seed)
    for p in params:
        p.grad = (torch.randn(p.shape, generator=g) * 1e-2).to(p.dtype).cuda()


def _run(params, opt, steps=3):
    for s in range(steps):
        _grads(params, s)
        opt.step()
    torch.cuda.synchronize()
    opt.check_device_status()


# ------------------------------------------------------------------------------- codec entry points

def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("shape", [(5, 300), (1, 7), (64, 1), (1000,), (3, 4, 5)])
def test_int8_codec_bit_exact_and_in_range(shape):
    """reference tests/test_momentum_codec.py: codes stay in [-127, 127], zero encodes to zero"""
    from kaon_b200 import _lib as L
    rows = shape[0] if len(shape) >= 2 else 0
    g = torch.Generator().manual_seed(3)
    m = torch.randn(shape, generator=g) * torch.logspace(-4, 2, int(np.prod(shape))).reshape(shape)
    m.view(-1)[::7] = 0.0
    md = m.cuda().contiguous()
    codes = torch.empty(shape, dtype=torch.int8, device="cuda")
    scale = torch.empty(max(rows, 1), dtype=torch.float32, device="cuda")
    L.check(L.lib().kaon_codec_encode_int8(C.c_void_p(md.data_ptr()), C.c_int64(m.numel()), C.c_int64(rows),
                                           C.c_void_p(codes.data_ptr()), C.c_void_p(scale.data_ptr()), _stream()))
    out = torch.empty_like(md)
    L.check(L.lib().kaon_codec_decode_int8(C.c_void_p(codes.data_ptr()), C.c_void_p(scale.data_ptr()),
                                           C.c_int64(m.numel()), C.c_int64(rows), C.c_void_p(out.data_ptr()), _stream()))
    torch.cuda.synchronize()
    want_codes, want_scale = ko.encode_int8(m.numpy(), rows)
    assert np.array_equal(codes.cpu().numpy().reshape(-1), want_codes)
    assert np.array_equal(scale.cpu().numpy(), want_scale)
    assert np.array_equal(out.cpu().numpy().reshape(-1), ko.decode_int8(want_codes, want_scale, rows))
    assert codes.min().item() >= -127
    assert (codes.view(-1)[::7] == 0).all()


@pytest.mark.parametrize("n", [128, 129, 255, 4096 + 37, 5, 1])
def test_4bit_codec_bit_exact_and_never_uses_the_reserved_code(n):
    """reference tests/test_momentum_codec.py: nibbles live in 1..15 (0 is reserved), odd lengths pack"""
    from kaon_b200 import _lib as L
    g = torch.Generator().manual_seed(n)
    m = torch.randn(n, generator=g) * torch.logspace(-3, 1, n)
    bs = ko.fourbit_block(n, 128)
    md = m.cuda()
    packed = torch.zeros((n + 1) // 2, dtype=torch.uint8, device="cuda")
    scale = torch.empty((n + bs - 1) // bs, dtype=torch.float32, device="cuda")
    L.check(L.lib().kaon_codec_encode_4bit(C.c_void_p(md.data_ptr()), C.c_int64(n), C.c_int64(bs),
                                           C.c_void_p(packed.data_ptr()), C.c_void_p(scale.data_ptr()), _stream()))
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    L.check(L.lib().kaon_codec_decode_4bit(C.c_void_p(packed.data_ptr()), C.c_void_p(scale.data_ptr()), C.c_int64(n),
                                           C.c_int64(bs), C.c_void_p(out.data_ptr()), _stream()))
    torch.cuda.synchronize()
    want_packed, want_scale = ko.encode_4bit(m.numpy(), 128)
    got = packed.cpu().numpy()
    assert np.array_equal(scale.cpu().numpy(), want_scale)
    nib = np.stack([got & 15, got >> 4], axis=1).reshape(-1)[:n]
    want_nib = np.stack([want_packed & 15, want_packed >> 4], axis=1).reshape(-1)[:n]
    assert np.array_equal(nib, want_nib)
    assert nib.min() >= 1
    assert np.array_equal(out.cpu().numpy(), ko.decode_4bit(want_packed, want_scale, n, 128))


# ------------------------------------------------------------------------------- around the step

@pytest.mark.parametrize("cls_name", ["Lion", "Adakaon", "AdaMuon"])
def test_tensors_without_gradient_are_left_alone(cls_name):
    import kaon_b200
    params = _mk()
    before = [p.detach().clone() for p in params]
    opt = getattr(kaon_b200, cls_name)(params, momentum_dtype="int8")
    for s in range(2):
        _grads(params, s)
        params[1].grad = None
        opt.step()
    torch.cuda.synchronize()
    opt.check_device_status()
    assert torch.equal(params[1].detach(), before[1]) and params[1] not in opt.state
    for i in (0, 2, 3):
        assert not torch.equal(params[i].detach(), before[i])
    # the skipped tensor joins later: state appears, the others carry on
    _grads(params, 5)
    opt.step()
    torch.cuda.synchronize()
    assert params[1] in opt.state and not torch.equal(params[1].detach(), before[1])


@pytest.mark.parametrize("cls_name", ["Lion", "Adakaon"])
def test_empty_tensor_is_harmless(cls_name):
    import kaon_b200
    params = _mk() + [torch.nn.Parameter(torch.zeros(0, 16, device="cuda"))]
    opt = getattr(kaon_b200, cls_name)(params, momentum_dtype="4bit")
    for s in range(2):
        _grads(params, s)
        opt.step()
    torch.cuda.synchronize()
    opt.check_device_status()
    assert params[-1].numel() == 0


@pytest.mark.parametrize("cls_name", ["Lion", "Adakaon"])
def test_param_groups_step_with_their_own_hyperparameters(cls_name):
    """Two groups in one optimizer == two optimizers (fp32 weights: bit-identical)."""
    import kaon_b200
    cls = getattr(kaon_b200, cls_name)
    pa, pb = _mk(), _mk()
    one = cls([{"params": pa[:2], "lr": 3e-3, "weight_decay": 0.2}, {"params": pa[2:]}], lr=1e-3, momentum_dtype="int8")
    two = [cls(pb[:2], lr=3e-3, weight_decay=0.2, momentum_dtype="int8"), cls(pb[2:], lr=1e-3, momentum_dtype="int8")]
    for s in range(3):
        _grads(pa, s)
        _grads(pb, s)
        one.step()
        for o in two:
            o.step()
    torch.cuda.synchronize()
    for a, b in zip(pa, pb):
        assert torch.equal(a.detach(), b.detach())


def test_sparse_gradient_is_rejected():
    """reference tests/test_lion.py:333-339"""
    import kaon_b200
    p = torch.nn.Parameter(torch.randn(4, 4, device="cuda"))
    opt = kaon_b200.Lion([p])
    p.grad = torch.zeros(4, 4, device="cuda").to_sparse()
    with pytest.raises(RuntimeError, match="sparse"):
        opt.step()


def test_nekaon_k_zero_is_plain_adakaon():
    """reference tests/test_nekaon.py:42-52"""
    import kaon_b200
    pa, pb = _mk(), _mk()
    a = kaon_b200.Nekaon(pa, lr=1e-3, k=0.0, betas=(0.9, 0.999), momentum_dtype="float32")
    b = kaon_b200.Adakaon(pb, lr=1e-3, weight_decay=0.1, betas=(0.9, 0.999), momentum_dtype="float32")
    _run(pa, a)
    _run(pb, b)
    for x, y in zip(pa, pb):
        assert torch.equal(x.detach(), y.detach())


def test_nekaon_eval_shows_true_weights_and_train_restores():
    """reference tests/test_nekaon.py:69-75"""
    import kaon_b200
    pa = _mk()
    opt = kaon_b200.Nekaon(pa, lr=1e-3, k=1.5, betas=(0.9, 0.999), momentum_dtype="float32")
    _run(pa, opt, steps=1)
    live = [p.detach().clone() for p in pa]
    opt.eval()
    torch.cuda.synchronize()
    assert any(not torch.equal(a.detach(), w) for a, w in zip(pa, live))
    opt.train()
    torch.cuda.synchronize()
    for a, w in zip(pa, live):
        torch.testing.assert_close(a.detach(), w, rtol=1e-6, atol=1e-9)


def test_nekaon_low_vram_above_routes_big_tensors_to_a_momentum_free_group():
    """reference tests/test_nekaon.py:78-90; here also: each group steps exactly like a stand-alone
    optimizer with that group's settings."""
    import kaon_b200
    pa, pb = _mk(), _mk()
    thr = 3000  # (48,64)=3072 and (33,77)=2541: one above, three below
    opt = kaon_b200.Nekaon(pa, lr=1e-3, k=1.5, betas=(0.9, 0.999), momentum_dtype="float32", low_vram_above=thr)
    big = [p for p in pb if p.numel() > thr]
    small = [p for p in pb if p.numel() <= thr]
    ref_small = kaon_b200.Nekaon(small, lr=1e-3, k=1.5, betas=(0.9, 0.999), momentum_dtype="float32")
    ref_big = kaon_b200.Adakaon(big, lr=5e-4, betas=(0.0, 0.999), weight_decay=0.1, momentum_dtype="float32")
    for s in range(3):
        _grads(pa, s)
        _grads(pb, s)
        opt.step()
        ref_small.step()
        ref_big.step()
    torch.cuda.synchronize()
    opt.check_device_status()
    st = opt.base_optimizer.state
    for p in pa:
        assert ("m" in st[p]) == (p.numel() <= thr)
    for a, b in zip(pa, pb):
        assert torch.equal(a.detach(), b.detach())


def test_lr_schedule_between_steps_is_honoured():
    """Hyper-parameters are read from the param group at every step (schedulers mutate them)."""
    import kaon_b200
    pa, pb = _mk(), _mk()
    a = kaon_b200.Lion(pa, lr=1e-3, momentum_dtype="4bit")
    b = kaon_b200.Lion(pb, lr=1e-3, momentum_dtype="4bit")
    _run(pa, a, steps=1)
    _run(pb, b, steps=1)
    for g in a.param_groups:
        g["lr"] = 0.0
    before = [p.detach().clone() for p in pa]
    _grads(pa, 9)
    a.step()
    torch.cuda.synchronize()
    for p, q in zip(pa, before):
        assert torch.equal(p.detach(), q)        # lr = 0: weights stay, state still moves
    _grads(pb, 9)
    b.step()
    torch.cuda.synchronize()
    for p, q in zip(pa, pb):
        assert torch.equal(a.state[p]["m"], b.state[q]["m"])


@pytest.mark.parametrize("cls_name,kw", [("Lion", dict(lr=2e-4, momentum_dtype="4bit")),
                                         ("Adakaon", dict(lr=1e-4, momentum_dtype="int8")),
                                         ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999)))])
def test_results_do_not_depend_on_how_the_list_is_split(cls_name, kw):
    """A 41 M-parameter UNet-shaped list stepped by one optimizer, and by two optimizers over interleaved
    halves of it (what sharding does): weights and state are bit-identical, stochastic rounding
    included - work-item scheduling, grid size and list composition do not leak into the results."""
    import kaon_b200
    from kaon_b200 import workloads as W
    shapes = W.WORKLOADS["unet_sample"]()
    gen = torch.Generator(device="cuda").manual_seed(3)
    base = [(torch.randn(s, generator=gen, device="cuda") * 0.02).bfloat16() for s in shapes]
    grads = [[(torch.randn(s, generator=gen, device="cuda") * 1e-3).bfloat16() for s in shapes] for _ in range(2)]

    def run(split):
        params = [torch.nn.Parameter(b.clone()) for b in base]
        for i, p in enumerate(params):
            p.kaon_tensor_id = i
        groups = [params] if not split else [params[0::2], params[1::2]]
        opts = [getattr(kaon_b200, cls_name)(g, **kw) for g in groups]
        for o in opts:
            o.sr_seed = 9
        for step in range(2):
            for p, g in zip(params, grads[step]):
                p.grad = g
            for o in opts:
                o.step()
        torch.cuda.synchronize()
        for o in opts:
            o.check_device_status()
        state = {}
        for o in opts:
            inner = getattr(o, "base_optimizer", o)
            for p in inner.state:
                state[p.kaon_tensor_id] = inner.state[p]
        return params, state

    pa, sa = run(False)
    pb, sb = run(True)
    for i, (a, b) in enumerate(zip(pa, pb)):
        assert torch.equal(a.detach().view(torch.int16), b.detach().view(torch.int16)), i
        for k, v in sa[i].items():
            if torch.is_tensor(v):
                assert torch.equal(v, sb[i][k]), (i, k)


@pytest.mark.parametrize("cls_name", ["Adakaon", "AdaMuon"])
def test_plans_with_different_row_widths_coexist(cls_name):
    """The kernels' shared-memory need grows with the widest row of a plan; a later, narrower plan must
    not take the room away from an earlier, wider one that keeps stepping."""
    import kaon_b200
    wide = [torch.nn.Parameter(torch.randn(24, 12288, device="cuda").bfloat16() * 0.02)]
    narrow = [torch.nn.Parameter(torch.randn(64, 64, device="cuda").bfloat16() * 0.02)]
    ow = getattr(kaon_b200, cls_name)(wide, momentum_dtype="int8")
    on = getattr(kaon_b200, cls_name)(narrow, momentum_dtype="int8")
    for step in range(3):
        for p in wide + narrow:
            p.grad = (torch.randn_like(p.float()) * 1e-3).bfloat16()
        ow.step()
        on.step()
    torch.cuda.synchronize()
    ow.check_device_status()
    on.check_device_status()
    assert torch.isfinite(wide[0].float()).all() and torch.isfinite(narrow[0].float()).all()
